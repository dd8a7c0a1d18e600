// C ABI of the library (include/qipack_b200.h): argument checks, tensor-map encoding, tile
// selection and launches. One translation unit so that every kernel shares one status word.
#include "../../include/qipack_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "quantize.cuh"
#include "w4a16_gemm.cuh"
#include "w4a16_gemv.cuh"
#include "w4a16_gemv_stream.cuh"
#include "w4a16_pair_gemm.cuh"
#include "w4a4_gemm.cuh"
#include "w4a4_wide_gemm.cuh"
#include "w4a4_pair_gemm.cuh"
#include "probe.cuh"

namespace qi {
namespace {

constexpr int INVALID = static_cast<int>(cudaErrorInvalidValue);

bool aligned16(const void *pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15) == 0; }

// ---- per-device facts ------------------------------------------------------------------------

constexpr int MAX_DEVICES = 64;

int current_device() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return -1;
    return device;
}

// The lazily filled tables below are atomics: two host threads that meet in a first call both do the
// (idempotent) query or cudaFuncSetAttribute, and neither reads a half-written entry.
int sm_count(int device) {
    static std::atomic<int> cached[MAX_DEVICES];
    int count = cached[device].load(std::memory_order_relaxed);
    if (count == 0) {
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            return 148;
        cached[device].store(count, std::memory_order_relaxed);
    }
    return count;
}

// Opts a kernel into its dynamic shared memory once per device; `done` is that kernel's per-device flag.
template <typename Kernel>
cudaError_t configure_once(Kernel kernel, int smem_bytes, std::atomic<bool> &done) {
    if (done.load(std::memory_order_acquire)) return cudaSuccess;
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (error == cudaSuccess) done.store(true, std::memory_order_release);
    return error;
}

// ---- TMA descriptors ---------------------------------------------------------------------------

typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static std::atomic<EncodeTiled> cached{nullptr};
    EncodeTiled function = cached.load(std::memory_order_acquire);
    if (function == nullptr) {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            function = reinterpret_cast<EncodeTiled>(entry);
            cached.store(function, std::memory_order_release);
        }
    }
    return function;
}

// A row-major [rows, row_bytes / element] matrix seen as a 2-D tensor; box = box_inner elements
// x box_rows rows. Out-of-range rows read as zero.
bool make_map(CUtensorMap *map, CUtensorMapDataType type, int element_bytes, const void *base, uint64_t inner,
              uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows,
              CUtensorMapSwizzle swizzle) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    (void)element_bytes;
    return encode(map, type, 2, const_cast<void *>(base), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- tile selection -----------------------------------------------------------------------------

// W4A16 tiles: 0 = choose by shape; 1 = 128x128, 2 = 256x128, 3 = 128x256, 4 = 256x256, 5 = 256x256 on a pair of CTAs.

template <int NUM_M, int BN, int STAGES>
int launch_w4a16(const void *x_half, const void *codes, const void *scales, const void *minimums, const float *bias,
                 void *y, const GemmShape &shape, cudaStream_t stream, int device) {
    using T = w4a16::Tile<NUM_M, BN, STAGES>;
    CUtensorMap map_x, map_codes;
    if (!make_map(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x_half, shape.k, shape.m,
                  static_cast<uint64_t>(shape.k) * 2, 64, T::BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return INVALID;
    if (!make_map(&map_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, shape.k / 2, shape.n,
                  static_cast<uint64_t>(shape.k) / 2, 32, BN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return INVALID;
    auto kernel = w4a16::gemm_kernel<NUM_M, BN, STAGES>;
    static std::atomic<bool> configured[MAX_DEVICES];
    if (const cudaError_t error = configure_once(kernel, T::SMEM_BYTES, configured[device])) return static_cast<int>(error);
    const int tiles = ((shape.m + T::BM - 1) / T::BM) * ((shape.n + BN - 1) / BN);
    const int grid = tiles < sm_count(device) ? tiles : sm_count(device);
    kernel<<<grid, w4a16::THREADS, T::SMEM_BYTES, stream>>>(map_x, map_codes, static_cast<const __half *>(scales),
                                                            static_cast<const __half *>(minimums), bias, y, shape);
    return static_cast<int>(cudaGetLastError());
}

template <int STAGES>
int launch_w4a16_pair(const void *x_half, const void *codes, const void *scales, const void *minimums, const float *bias,
                      void *y, const GemmShape &shape, cudaStream_t stream, int device) {
    namespace wp = w4a16_pair;
    using T = wp::Tile<STAGES>;
    CUtensorMap map_x, map_codes;
    if (!make_map(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x_half, shape.k, shape.m,
                  static_cast<uint64_t>(shape.k) * 2, 64, wp::BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return INVALID;
    if (!make_map(&map_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, shape.k / 2, shape.n,
                  static_cast<uint64_t>(shape.k) / 2, 32, wp::BN / 2, CU_TENSOR_MAP_SWIZZLE_NONE))
        return INVALID;
    auto kernel = wp::gemm_kernel<STAGES>;
    static std::atomic<bool> configured[MAX_DEVICES];
    if (const cudaError_t error = configure_once(kernel, T::SMEM_BYTES, configured[device])) return static_cast<int>(error);
    const int tiles = ((shape.m + 2 * wp::BM - 1) / (2 * wp::BM)) * ((shape.n + wp::BN - 1) / wp::BN);
    const int pairs = sm_count(device) / 2;
    const int grid = 2 * (tiles < pairs ? tiles : pairs);  // the kernel carries __cluster_dims__(2, 1, 1)
    kernel<<<grid, wp::THREADS, T::SMEM_BYTES, stream>>>(map_x, map_codes, static_cast<const __half *>(scales),
                                                         static_cast<const __half *>(minimums), bias, y, shape);
    return static_cast<int>(cudaGetLastError());
}

template <int BN, int STAGES>
int launch_w4a4(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                const float *bias, void *y, int32_t *dots, const GemmShape &shape, cudaStream_t stream, int device) {
    using T = w4a4::Tile<BN, STAGES>;
    CUtensorMap map_a, map_w;
    if (!make_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_codes, shape.k / 2, shape.m,
                  static_cast<uint64_t>(shape.k) / 2, 64, T::BM, CU_TENSOR_MAP_SWIZZLE_NONE))
        return INVALID;
    if (!make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_codes, shape.k / 2, shape.n,
                  static_cast<uint64_t>(shape.k) / 2, 64, BN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return INVALID;
    auto kernel = dots != nullptr ? w4a4::gemm_kernel<BN, STAGES, true> : w4a4::gemm_kernel<BN, STAGES, false>;
    static std::atomic<bool> configured[MAX_DEVICES][2];
    if (const cudaError_t error = configure_once(kernel, T::SMEM_BYTES, configured[device][dots != nullptr]))
        return static_cast<int>(error);
    const int tiles = ((shape.m + T::BM - 1) / T::BM) * ((shape.n + BN - 1) / BN);
    const int grid = tiles < sm_count(device) ? tiles : sm_count(device);
    kernel<<<grid, w4a4::THREADS, T::SMEM_BYTES, stream>>>(map_a, map_w, static_cast<const __half *>(a_scales),
                                                           static_cast<const __half *>(w_scales), bias, y, dots, shape);
    return static_cast<int>(cudaGetLastError());
}

template <int STAGES>
int launch_w4a4_wide(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                     const float *bias, void *y, int32_t *dots, const GemmShape &shape, cudaStream_t stream, int device) {
    using T = w4a4_wide::Tile<STAGES>;
    CUtensorMap map_a, map_w;
    if (!make_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_bytes, shape.k, shape.m, static_cast<uint64_t>(shape.k),
                  w4a4_wide::STAGE_K, w4a4_wide::BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return INVALID;
    if (!make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_bytes, shape.k, shape.n, static_cast<uint64_t>(shape.k),
                  w4a4_wide::STAGE_K, w4a4_wide::BN, CU_TENSOR_MAP_SWIZZLE_128B))
        return INVALID;
    auto kernel = dots != nullptr ? w4a4_wide::gemm_kernel<STAGES, true> : w4a4_wide::gemm_kernel<STAGES, false>;
    static std::atomic<bool> configured[MAX_DEVICES][2];
    if (const cudaError_t error = configure_once(kernel, T::SMEM_BYTES, configured[device][dots != nullptr]))
        return static_cast<int>(error);
    const int tiles = ((shape.m + w4a4_wide::BM - 1) / w4a4_wide::BM) * ((shape.n + w4a4_wide::BN - 1) / w4a4_wide::BN);
    const int grid = tiles < sm_count(device) ? tiles : sm_count(device);
    kernel<<<grid, w4a4_wide::THREADS, T::SMEM_BYTES, stream>>>(map_a, map_w, static_cast<const __half *>(a_scales),
                                                                static_cast<const __half *>(w_scales), bias, y, dots, shape);
    return static_cast<int>(cudaGetLastError());
}

int launch_w4a4_pair(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                     const float *bias, void *y, int32_t *dots, const GemmShape &shape, cudaStream_t stream, int device,
                     const w4a4_pair::PeerOutputs *peers = nullptr) {
    namespace wp = w4a4_pair;
    CUtensorMap map_a, map_w;
    if (!make_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_bytes, shape.k, shape.m, static_cast<uint64_t>(shape.k),
                  128, wp::BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return INVALID;
    if (!make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_bytes, shape.k, shape.n, static_cast<uint64_t>(shape.k),
                  128, wp::B_BOX_ROWS, CU_TENSOR_MAP_SWIZZLE_128B))
        return INVALID;
    if (peers != nullptr && dots != nullptr) return INVALID;
    const int variant = peers != nullptr ? 2 : (dots != nullptr ? 1 : 0);
    auto kernel = variant == 2 ? wp::gemm_kernel<false, true>
                               : (variant == 1 ? wp::gemm_kernel<true, false> : wp::gemm_kernel<false, false>);
    static std::atomic<bool> configured[MAX_DEVICES][3];
    if (const cudaError_t error = configure_once(kernel, wp::SMEM_BYTES, configured[device][variant]))
        return static_cast<int>(error);
    const wp::PeerOutputs outputs = peers != nullptr ? *peers : wp::PeerOutputs{};
    const int tiles = ((shape.m + 2 * wp::BM - 1) / (2 * wp::BM)) * ((shape.n + wp::BN - 1) / wp::BN);
    const int pairs = sm_count(device) / 2;
    const int grid = 2 * (tiles < pairs ? tiles : pairs);  // the kernel carries __cluster_dims__(2, 1, 1)
    kernel<<<grid, wp::THREADS, wp::SMEM_BYTES, stream>>>(map_a, map_w, static_cast<const __half *>(a_scales),
                                                          static_cast<const __half *>(w_scales), bias, y, dots, shape,
                                                          outputs);
    return static_cast<int>(cudaGetLastError());
}

bool output_ok(const void *y, int y_dtype, long long ldy, int n) {
    if (y == nullptr || !aligned16(y) || ldy < n) return false;
    if (y_dtype == QI_DTYPE_F32) return ldy % 4 == 0;
    if (y_dtype == QI_DTYPE_F16) return ldy % 8 == 0;
    return false;
}

__global__ void dequantize_kernel(const uint8_t *__restrict__ codes, const __half *__restrict__ scales,
                                  const __half *__restrict__ minimums, __half *__restrict__ out, int n, int k) {
    // one thread per 16 code bytes (32 inputs, half a group)
    const long long chunks = static_cast<long long>(n) * (k / 32);
    const long long chunk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (chunk >= chunks) return;
    const long long row = chunk / (k / 32);
    const int in_row = static_cast<int>(chunk % (k / 32));
    const int group = in_row / 2;
    const uint4 packed = __ldg(reinterpret_cast<const uint4 *>(codes + row * (k / 2)) + in_row);
    const __half2 scale2 = __half2half2(__ldg(scales + row * (k / 64) + group));
    const __half2 minimum2 = __half2half2(__ldg(minimums + row * (k / 64) + group));
    uint4 values[4];
    w4a16::unpack32(packed, scale2, minimum2, values);
    uint4 *destination = reinterpret_cast<uint4 *>(out + row * k + in_row * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) destination[j] = values[j];
}

int w4a16_gemv(const void *x_half, const void *codes, const void *scales, const void *minimums, const float *bias,
               void *y, int y_dtype, long long ldy, int m, int n, int k, cudaStream_t stream) {
    if (m < 1 || m > 8 || n <= 0 || k <= 0 || n % 16 != 0 || k % 64 != 0) return INVALID;
    if (!x_half || !codes || !scales || !minimums || !y) return INVALID;
    if (!aligned16(x_half) || !aligned16(codes) || (k % 8) != 0) return INVALID;
    if (ldy < n || (y_dtype != QI_DTYPE_F32 && y_dtype != QI_DTYPE_F16)) return INVALID;
    // Rows short enough for 16 of them to fit a stage, and regions that bulk copies can take: the streaming kernel.
    if (k <= w4a16::STREAM_MAX_K && aligned16(scales) && aligned16(minimums)) {
        const int device = current_device();
        if (device < 0) return INVALID;
        // two CTAs per SM: as many stages (at most three) as fit 110 KB beside the activations
        constexpr int CTA_BYTES = 110 * 1024;
        int stages = (CTA_BYTES - 128 - w4a16::stream_x_bytes(m, k)) / w4a16::stream_stage_bytes(k);
        stages = stages > w4a16::STREAM_MAX_STAGES ? w4a16::STREAM_MAX_STAGES : stages;
        static std::atomic<bool> configured[MAX_DEVICES];
        if (const cudaError_t error = configure_once(w4a16::gemv_stream_kernel, CTA_BYTES, configured[device]))
            return static_cast<int>(error);
        if (stages >= 1) {
            const int smem_bytes = stages * w4a16::stream_stage_bytes(k) + w4a16::stream_x_bytes(m, k) + 128;
            const int tiles = n / w4a16::STREAM_ROWS, resident = 2 * sm_count(device);
            w4a16::gemv_stream_kernel<<<tiles < resident ? tiles : resident, w4a16::STREAM_THREADS, smem_bytes, stream>>>(
                static_cast<const __half *>(x_half), static_cast<const uint8_t *>(codes), static_cast<const __half *>(scales),
                static_cast<const __half *>(minimums), bias, y, m, n, k, ldy, y_dtype == QI_DTYPE_F16, stages);
            return static_cast<int>(cudaGetLastError());
        }
    }
    const int quads = (k / 64 + 3) / 4;
    int k_splits = 1;
    for (int candidate = 8; candidate >= 1; candidate /= 2)
        if (quads % candidate == 0) { k_splits = candidate; break; }
    const int row_tiles = w4a16::GEMV_WARPS / k_splits;
    const int blocks = (n / 16 + row_tiles - 1) / row_tiles;
    w4a16::gemv_kernel<<<blocks, w4a16::GEMV_THREADS, 0, stream>>>(
        static_cast<const __half *>(x_half), static_cast<const uint8_t *>(codes), static_cast<const __half *>(scales),
        static_cast<const __half *>(minimums), bias, y, m, n, k, ldy, y_dtype == QI_DTYPE_F16, k_splits);
    return static_cast<int>(cudaGetLastError());
}

// Several matrices of one shape against the same activations: launches of up to STREAM_GROUP matrices each.
int w4a16_gemv_grouped(const void *x_half, const qi_gemv_item *items, int count, int y_dtype, long long ldy, int m, int n,
                       int k, cudaStream_t stream) {
    if (m < 1 || m > 8 || n <= 0 || k <= 0 || n % 16 != 0 || k % 64 != 0 || count < 1 || items == nullptr) return INVALID;
    if (!x_half || !aligned16(x_half) || k > w4a16::STREAM_MAX_K) return INVALID;
    if (ldy < n || (y_dtype != QI_DTYPE_F32 && y_dtype != QI_DTYPE_F16)) return INVALID;
    for (int i = 0; i < count; ++i) {
        const qi_gemv_item &item = items[i];
        if (!item.codes || !item.scales || !item.minimums || !item.y) return INVALID;
        if (!aligned16(item.codes) || !aligned16(item.scales) || !aligned16(item.minimums)) return INVALID;
    }
    const int device = current_device();
    if (device < 0) return INVALID;
    constexpr int CTA_BYTES = 110 * 1024;  // two CTAs per SM, as for the single matrix
    int stages = (CTA_BYTES - 128 - w4a16::stream_x_bytes(m, k)) / w4a16::stream_stage_bytes(k);
    stages = stages > w4a16::STREAM_MAX_STAGES ? w4a16::STREAM_MAX_STAGES : stages;
    if (stages < 1) return INVALID;
    static std::atomic<bool> configured[MAX_DEVICES];
    if (const cudaError_t error = configure_once(w4a16::gemv_stream_grouped_kernel, CTA_BYTES, configured[device]))
        return static_cast<int>(error);
    const int smem_bytes = stages * w4a16::stream_stage_bytes(k) + w4a16::stream_x_bytes(m, k) + 128;
    const int resident = 2 * sm_count(device);
    for (int first = 0; first < count; first += w4a16::STREAM_GROUP) {
        const int now = count - first < w4a16::STREAM_GROUP ? count - first : w4a16::STREAM_GROUP;
        w4a16::StreamItems group;
        for (int i = 0; i < now; ++i) {
            const qi_gemv_item &item = items[first + i];
            group.item[i] = {static_cast<const uint8_t *>(item.codes), static_cast<const __half *>(item.scales),
                             static_cast<const __half *>(item.minimums), item.bias, item.y};
        }
        for (int i = now; i < w4a16::STREAM_GROUP; ++i) group.item[i] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        const long long tiles = static_cast<long long>(now) * (n / w4a16::STREAM_ROWS);
        w4a16::gemv_stream_grouped_kernel<<<tiles < resident ? static_cast<int>(tiles) : resident, w4a16::STREAM_THREADS, smem_bytes, stream>>>(
            static_cast<const __half *>(x_half), group, now, m, n, k, ldy, y_dtype == QI_DTYPE_F16, stages);
        const cudaError_t launched = cudaGetLastError();
        if (launched != cudaSuccess) return static_cast<int>(launched);
    }
    return 0;
}

int w4a16_gemm(const void *x_half, const void *codes, const void *scales, const void *minimums, const float *bias,
               void *y, int y_dtype, long long ldy, int m, int n, int k, int tile, cudaStream_t stream) {
    if (m <= 0 || n <= 0 || k <= 0 || n % 32 != 0 || k % 64 != 0) return INVALID;
    if (!x_half || !codes || !scales || !minimums) return INVALID;
    if (!aligned16(x_half) || !aligned16(codes) || !output_ok(y, y_dtype, ldy, n)) return INVALID;
    const int device = current_device();
    if (device < 0) return INVALID;
    const GemmShape shape = {m, n, k, ldy, y_dtype == QI_DTYPE_F16};
    if (tile == 0) {
        // Measured on B200 (4096 x {3072, 9216, 12288} x {3072, 12288}, 1024 and 256 rows): per tile the
        // 256x256 tile on one CTA is about 4 % faster than the same tile on a CTA pair, but a pair wave is
        // 74 tiles instead of 148, which wastes less of the last wave; below two single-CTA waves the pair
        // (half the unpacking per CTA, overlapped epilogue) wins outright; 128x128 wins when even pairs
        // would leave most of the machine idle.
        const int sms = sm_count(device);
        const long long tiles_256 = static_cast<long long>((m + 255) / 256) * ((n + 255) / 256);
        const long long pairs = sms / 2;
        const double single_waves = static_cast<double>((tiles_256 + sms - 1) / sms) / 1.04;
        const double pair_waves = static_cast<double>((tiles_256 + pairs - 1) / pairs) / 2.0;
        if (tiles_256 >= 2LL * sms) tile = single_waves <= pair_waves ? 4 : 5;
        else if (tiles_256 * 4 >= sms) tile = 5;
        else tile = 1;
    }
    switch (tile) {
        case 1: return launch_w4a16<1, 128, 6>(x_half, codes, scales, minimums, bias, y, shape, stream, device);
        case 2: return launch_w4a16<2, 128, 4>(x_half, codes, scales, minimums, bias, y, shape, stream, device);
        case 3: return launch_w4a16<1, 256, 4>(x_half, codes, scales, minimums, bias, y, shape, stream, device);
        case 4: return launch_w4a16<2, 256, 3>(x_half, codes, scales, minimums, bias, y, shape, stream, device);
        case 5: return launch_w4a16_pair<6>(x_half, codes, scales, minimums, bias, y, shape, stream, device);
        default: return INVALID;
    }
}

// single_cta: always the one-CTA kernel (128 x 128 tiles); otherwise CTA pairs where the shape and pointers allow.
int w4a4_gemm_wide(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                   const float *bias, void *y, int y_dtype, long long ldy, int32_t *dots, int m, int n, int k,
                   bool single_cta, cudaStream_t stream) {
    if (m <= 0 || n <= 0 || k <= 0 || n % 32 != 0 || k % 128 != 0) return INVALID;
    if (!a_bytes || !a_scales || !w_bytes || !w_scales) return INVALID;
    if (!aligned16(a_bytes) || !aligned16(w_bytes) || (reinterpret_cast<uintptr_t>(a_scales) & 3) ||
        (reinterpret_cast<uintptr_t>(w_scales) & 3) || !output_ok(y, y_dtype, ldy, n))
        return INVALID;
    const int device = current_device();
    if (device < 0) return INVALID;
    const GemmShape shape = {m, n, k, ldy, y_dtype == QI_DTYPE_F16};
    // The pair kernel's stage is four groups, and it stages both scale arrays eight bytes at a time; anything
    // else goes to the one-CTA kernel, which takes two groups per stage and four-byte-aligned scales.
    const bool scales_aligned8 = ((reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(w_scales)) & 7) == 0;
    if (single_cta || k % w4a4_pair::STAGE_K != 0 || !scales_aligned8)
        return launch_w4a4_wide<6>(a_bytes, a_scales, w_bytes, w_scales, bias, y, dots, shape, stream, device);
    return launch_w4a4_pair(a_bytes, a_scales, w_bytes, w_scales, bias, y, dots, shape, stream, device);
}

// The W4A4 GEMM on nibble-packed codes (the reference's operand format). `path`: 1 = the int8 kernel that widens the
// nibbles in shared memory; 2 = both operands widened to one byte per code in scratch memory of the stream's pool
// (two small kernels), then the byte-operand kernel on CTA pairs, which is the faster GEMM by more than the
// widening costs once the matrices are large; 0 = 2 where the pair kernel takes the shape, else 1. Same bits on
// every path. The scratch is (m + n) * k bytes from the library's own memory pool (cudaMallocFromPoolAsync) and goes
// back with cudaFreeAsync, both in stream order; if the pool refuses, path 0 falls back to 1.
constexpr int W4A4_PATHS = 3;

// The library's own memory pool for that scratch, one per device, made at first use. The device's default pool gives
// its memory back to the system at every synchronisation (release threshold 0), so a caller that synchronises
// between calls would pay a round trip to the driver per call (measured: 1.0-1.7 ms instead of 0.32 ms for the
// 4096 x 9216 x 3072 linear); this pool keeps what it has handed out until qi_w4a4_scratch_trim.
cudaMemPool_t scratch_pool(int device) {
    static std::atomic<cudaMemPool_t> pools[MAX_DEVICES];
    cudaMemPool_t pool = pools[device].load(std::memory_order_acquire);
    if (pool != nullptr) return pool;
    cudaMemPoolProps properties = {};
    properties.allocType = cudaMemAllocationTypePinned;
    properties.handleTypes = cudaMemHandleTypeNone;
    properties.location.type = cudaMemLocationTypeDevice;
    properties.location.id = device;
    if (cudaMemPoolCreate(&pool, &properties) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    unsigned long long keep = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    cudaMemPool_t expected = nullptr;
    if (!pools[device].compare_exchange_strong(expected, pool, std::memory_order_acq_rel)) {
        cudaMemPoolDestroy(pool);  // another host thread was first
        pool = expected;
    }
    return pool;
}
int w4a4_gemm(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales, const float *bias,
              void *y, int y_dtype, long long ldy, int32_t *dots, int m, int n, int k, int path, cudaStream_t stream) {
    if (m <= 0 || n <= 0 || k <= 0 || n % 32 != 0 || k % 128 != 0 || path < 0 || path >= W4A4_PATHS) return INVALID;
    if (!a_codes || !a_scales || !w_codes || !w_scales) return INVALID;
    if (!aligned16(a_codes) || !aligned16(w_codes) || (reinterpret_cast<uintptr_t>(a_scales) & 3) ||
        (reinterpret_cast<uintptr_t>(w_scales) & 3) || !output_ok(y, y_dtype, ldy, n))
        return INVALID;
    const int device = current_device();
    if (device < 0) return INVALID;
    const GemmShape shape = {m, n, k, ldy, y_dtype == QI_DTYPE_F16};
    const bool scales_aligned8 = ((reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(w_scales)) & 7) == 0;
    const bool pair_takes_it = dots == nullptr && k % w4a4_pair::STAGE_K == 0 && scales_aligned8;
    if (path == 2 && !pair_takes_it) return INVALID;
    if (path == 2 || (path == 0 && pair_takes_it && m >= 256 && n >= 256)) {
        const size_t a_bytes = (static_cast<size_t>(m) * k + 255) & ~static_cast<size_t>(255);
        const size_t w_bytes = static_cast<size_t>(n) * k;
        uint8_t *scratch = nullptr;
        const cudaMemPool_t pool = scratch_pool(device);
        const cudaError_t allocated = pool == nullptr ? cudaErrorMemoryAllocation
                                                      : cudaMallocFromPoolAsync(reinterpret_cast<void **>(&scratch), a_bytes + w_bytes, pool, stream);
        if (allocated == cudaSuccess) {
            int status = qi_w4a4_widen_codes_ex(a_codes, scratch, m, k, stream);
            if (status == 0) status = qi_w4a4_widen_codes_ex(w_codes, scratch + a_bytes, n, k, stream);
            if (status == 0)
                status = launch_w4a4_pair(scratch, a_scales, scratch + a_bytes, w_scales, bias, y, nullptr, shape, stream, device);
            const cudaError_t freed = cudaFreeAsync(scratch, stream);
            return status != 0 ? status : static_cast<int>(freed);
        }
        (void)cudaGetLastError();  // the refusal is not the caller's error
        if (path == 2) return static_cast<int>(allocated);
    }
    return launch_w4a4<128, 4>(a_codes, a_scales, w_codes, w_scales, bias, y, dots, shape, stream, device);
}

}  // namespace
}  // namespace qi

using namespace qi;

extern "C" {

int qi_w4a4_quantize_activations_ex(const void *x, int x_dtype, void *codes, void *scales, int m, int k, void *stream) {
    if (m < 0 || k <= 0 || k % 256 != 0) return INVALID;
    if (x_dtype != QI_DTYPE_F32 && x_dtype != QI_DTYPE_F16) return INVALID;
    if (m == 0) return 0;
    if (!x || !codes || !scales || !aligned16(x) || (reinterpret_cast<uintptr_t>(codes) & 7) ||
        (reinterpret_cast<uintptr_t>(scales) & 1))
        return INVALID;
    return static_cast<int>(launch_quantize_activations(x, x_dtype == QI_DTYPE_F16, codes, scales, nullptr, m, k,
                                                        static_cast<cudaStream_t>(stream)));
}

int qi_w4a4_quantize_activations_wide_ex(const void *x, int x_dtype, void *codes, void *scales, void *bytes, int m,
                                         int k, void *stream) {
    if (m < 0 || k <= 0 || k % 256 != 0) return INVALID;
    if (x_dtype != QI_DTYPE_F32 && x_dtype != QI_DTYPE_F16) return INVALID;
    if (m == 0) return 0;
    if (!x || !scales || !bytes || !aligned16(x) || !aligned16(bytes) || (reinterpret_cast<uintptr_t>(codes) & 7) ||
        (reinterpret_cast<uintptr_t>(scales) & 1))
        return INVALID;
    return static_cast<int>(launch_quantize_activations(x, x_dtype == QI_DTYPE_F16, codes, scales, bytes, m, k,
                                                        static_cast<cudaStream_t>(stream)));
}

static int fused_quantize(int producer, const float *first, const float *second, void *codes, void *scales, void *bytes,
                          int m, int k, void *stream) {
    if (m < 0 || k <= 0 || k % 256 != 0) return INVALID;
    if (m == 0) return 0;
    if (!first || (producer == 1 && !second) || !scales || (!codes && !bytes)) return INVALID;
    if (!aligned16(first) || (second && !aligned16(second)) || (bytes && !aligned16(bytes)) ||
        (reinterpret_cast<uintptr_t>(codes) & 7) || (reinterpret_cast<uintptr_t>(scales) & 1))
        return INVALID;
    return static_cast<int>(launch_fused_quantize(producer, first, second, codes, scales, bytes, m, k, static_cast<cudaStream_t>(stream)));
}

int qi_w4a4_swiglu_quantize_ex(const float *gate, const float *up, void *codes, void *scales, void *bytes, int m, int k,
                               void *stream) {
    return fused_quantize(1, gate, up, codes, scales, bytes, m, k, stream);
}

int qi_w4a4_gelu_quantize_ex(const float *x, void *codes, void *scales, void *bytes, int m, int k, void *stream) {
    return fused_quantize(2, x, nullptr, codes, scales, bytes, m, k, stream);
}

int qi_w4a4_widen_codes_ex(const void *codes, void *bytes, long long rows, int k, void *stream) {
    if (rows < 0 || k <= 0 || k % 32 != 0) return INVALID;
    if (rows == 0) return 0;
    if (!codes || !bytes || !aligned16(codes) || !aligned16(bytes)) return INVALID;
    const long long chunks = rows * (k / 32);
    const long long blocks = (chunks + 255) / 256;
    if (blocks > 0x7fffffffLL) return INVALID;
    w4a4_wide::widen_codes_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(codes), static_cast<uint8_t *>(bytes), chunks);
    return static_cast<int>(cudaGetLastError());
}

int qi_w4a4_gemm_wide_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                         const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream) {
    return w4a4_gemm_wide(a_bytes, a_scales, w_bytes, w_scales, bias, y, y_dtype, ldy, nullptr, m, n, k, false,
                          static_cast<cudaStream_t>(stream));
}

int qi_w4a4_gemm_wide_single_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                                const float *bias, void *y, int y_dtype, long long ldy, int32_t *dots, int m, int n,
                                int k, void *stream) {
    return w4a4_gemm_wide(a_bytes, a_scales, w_bytes, w_scales, bias, y, y_dtype, ldy, dots, m, n, k, true,
                          static_cast<cudaStream_t>(stream));
}

int qi_w4a4_gemm_wide_scatter_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                                 const float *bias, void *const *y_copies, int copies, int first_copy, int y_dtype,
                                 long long ldy, int column, int m, int n, int k, void *stream) {
    namespace wp = w4a4_pair;
    if (y_copies == nullptr || copies < 1 || copies > wp::MAX_PEERS || first_copy < 0 || first_copy >= copies)
        return INVALID;
    if (m <= 0 || n <= 0 || k <= 0 || n % 32 != 0 || k % wp::STAGE_K != 0 || column < 0 || column % 32 != 0) return INVALID;
    if (!a_bytes || !a_scales || !w_bytes || !w_scales) return INVALID;
    // this entry point always runs on CTA pairs, whose scale staging copies eight bytes at a time
    if (!aligned16(a_bytes) || !aligned16(w_bytes) || (reinterpret_cast<uintptr_t>(a_scales) & 7) ||
        (reinterpret_cast<uintptr_t>(w_scales) & 7))
        return INVALID;
    if (y_dtype != QI_DTYPE_F16 && y_dtype != QI_DTYPE_F32) return INVALID;
    if (ldy < static_cast<long long>(column) + n) return INVALID;
    const size_t element = y_dtype == QI_DTYPE_F16 ? 2 : 4;
    wp::PeerOutputs outputs = {};
    outputs.count = copies;
    outputs.first = first_copy;
    for (int i = 0; i < copies; ++i) {
        if (y_copies[i] == nullptr) return INVALID;
        outputs.y[i] = static_cast<char *>(y_copies[i]) + static_cast<size_t>(column) * element;
        if (!output_ok(outputs.y[i], y_dtype, ldy, n) || (reinterpret_cast<uintptr_t>(outputs.y[i]) & 31)) return INVALID;
    }
    if ((ldy * static_cast<long long>(element)) % 32 != 0) return INVALID;  // the epilogue stores whole 32-byte sectors
    const int device = current_device();
    if (device < 0) return INVALID;
    const GemmShape shape = {m, n, k, ldy, y_dtype == QI_DTYPE_F16};
    return launch_w4a4_pair(a_bytes, a_scales, w_bytes, w_scales, bias, outputs.y[first_copy], nullptr, shape,
                            static_cast<cudaStream_t>(stream), device, &outputs);
}

int qi_w4a4_group_dots_wide_ex(const void *a_bytes, const void *a_scales, const void *w_bytes, const void *w_scales,
                               float *y, int32_t *dots, int m, int n, int k, void *stream) {
    if (dots == nullptr) return INVALID;
    return w4a4_gemm_wide(a_bytes, a_scales, w_bytes, w_scales, nullptr, y, QI_DTYPE_F32, n, dots, m, n, k, false,
                          static_cast<cudaStream_t>(stream));
}

int qi_w4a4_quantize_activations(const float *x, void *codes, void *scales, int m, int k) {
    return qi_w4a4_quantize_activations_ex(x, QI_DTYPE_F32, codes, scales, m, k, nullptr);
}

int qi_w4a4_gemm_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                    const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream) {
    return w4a4_gemm(a_codes, a_scales, w_codes, w_scales, bias, y, y_dtype, ldy, nullptr, m, n, k, 0,
                     static_cast<cudaStream_t>(stream));
}

int qi_w4a4_scratch_trim(void) {
    const int device = current_device();
    if (device < 0) return INVALID;
    const cudaMemPool_t pool = scratch_pool(device);
    if (pool == nullptr) return static_cast<int>(cudaErrorMemoryAllocation);
    return static_cast<int>(cudaMemPoolTrimTo(pool, 0));
}

int qi_w4a4_gemm_path_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                         const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, int path, void *stream) {
    return w4a4_gemm(a_codes, a_scales, w_codes, w_scales, bias, y, y_dtype, ldy, nullptr, m, n, k, path,
                     static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ---- the packed W4A4 GEMM for callers that must not allocate ------------------------------------------------------
// The widened operands of qi_w4a4_gemm_noalloc_ex live in this array instead of pool memory. One array per device
// (the runtime gives every device its own instance of a __device__ variable), shared by every call on that device:
// calls that overlap in time - two streams, two host threads - write over each other's operands. Nothing in it has
// to start at zero: a call writes every byte it later reads, so there is nothing to clear between calls.
constexpr size_t NOALLOC_SCRATCH_BYTES = static_cast<size_t>(QI_NOALLOC_SCRATCH_BYTES);
static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

extern "C" {

int qi_w4a4_gemm_noalloc_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                            const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream) {
    if (m <= 0 || n <= 0 || k <= 0 || n % 32 != 0 || k % w4a4_pair::STAGE_K != 0) return INVALID;
    if (!a_codes || !a_scales || !w_codes || !w_scales) return INVALID;
    if (!aligned16(a_codes) || !aligned16(w_codes) || !output_ok(y, y_dtype, ldy, n)) return INVALID;
    if (((reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(w_scales)) & 7) != 0) return INVALID;
    const size_t a_bytes = (static_cast<size_t>(m) * k + 255) & ~static_cast<size_t>(255);
    const size_t w_bytes = static_cast<size_t>(n) * k;
    if (a_bytes + w_bytes > NOALLOC_SCRATCH_BYTES) return QI_NOALLOC_TOO_LARGE;
    const int device = current_device();
    if (device < 0) return INVALID;
    // Set-up, once per device, with that device current: where this device's instance of the array is. It happens in
    // the first call on the device, which may also be what makes the runtime load this library's device code; make
    // that call before any stream capture begins.
    static std::atomic<uint8_t *> address[MAX_DEVICES];
    uint8_t *scratch = address[device].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        const cudaError_t found = cudaGetSymbolAddress(reinterpret_cast<void **>(&scratch), g_noalloc_scratch);
        if (found != cudaSuccess) return static_cast<int>(found);
        if (scratch == nullptr) return INVALID;
        address[device].store(scratch, std::memory_order_release);
    }
    const cudaStream_t on = static_cast<cudaStream_t>(stream);
    int status = qi_w4a4_widen_codes_ex(a_codes, scratch, m, k, stream);
    if (status == 0) status = qi_w4a4_widen_codes_ex(w_codes, scratch + a_bytes, n, k, stream);
    if (status != 0) return status;
    const GemmShape shape = {m, n, k, ldy, y_dtype == QI_DTYPE_F16};
    return launch_w4a4_pair(scratch, a_scales, scratch + a_bytes, w_scales, bias, y, nullptr, shape, on, device);
}

int qi_w4a4_gemm(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales, float *y,
                 int m, int n, int k) {
    if (m % 128 != 0 || n % 128 != 0 || k % 256 != 0) return INVALID;  // gemm.cu:185
    return w4a4_gemm(a_codes, a_scales, w_codes, w_scales, nullptr, y, QI_DTYPE_F32, n, nullptr, m, n, k, 0, nullptr);
}

int qi_w4a4_group_dots_ex(const void *a_codes, const void *a_scales, const void *w_codes, const void *w_scales,
                          float *y, int32_t *dots, int m, int n, int k, void *stream) {
    if (dots == nullptr) return INVALID;
    return w4a4_gemm(a_codes, a_scales, w_codes, w_scales, nullptr, y, QI_DTYPE_F32, n, dots, m, n, k, 1,
                     static_cast<cudaStream_t>(stream));
}

int qi_w4a16_gemv_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                     const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream) {
    return w4a16_gemv(x_half, codes, scales, minimums, bias, y, y_dtype, ldy, m, n, k, static_cast<cudaStream_t>(stream));
}

int qi_w4a16_gemv_grouped_ex(const void *x_half, const qi_gemv_item *items, int count, int y_dtype, long long ldy, int m,
                             int n, int k, void *stream) {
    return w4a16_gemv_grouped(x_half, items, count, y_dtype, ldy, m, n, k, static_cast<cudaStream_t>(stream));
}

int qi_w4a16_gemm_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                     const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, void *stream) {
    if (m >= 1 && m <= 8 && n % 16 == 0)
        return w4a16_gemv(x_half, codes, scales, minimums, bias, y, y_dtype, ldy, m, n, k, static_cast<cudaStream_t>(stream));
    return w4a16_gemm(x_half, codes, scales, minimums, bias, y, y_dtype, ldy, m, n, k, 0, static_cast<cudaStream_t>(stream));
}

int qi_w4a16_gemm_tile_ex(const void *x_half, const void *codes, const void *scales, const void *minimums,
                          const float *bias, void *y, int y_dtype, long long ldy, int m, int n, int k, int tile,
                          void *stream) {
    if (tile < 0 || tile > 5) return INVALID;
    return w4a16_gemm(x_half, codes, scales, minimums, bias, y, y_dtype, ldy, m, n, k, tile, static_cast<cudaStream_t>(stream));
}

int qi_w4a16_gemm(const void *x_half, const void *codes, const void *scales, const void *minimums, float *y, int m,
                  int n, int k) {
    if (m % 128 != 0 || n % 128 != 0 || k % 64 != 0) return INVALID;  // gemm.cu:264
    return w4a16_gemm(x_half, codes, scales, minimums, nullptr, y, QI_DTYPE_F32, n, m, n, k, 0, nullptr);
}

int qi_f32_to_f16(const float *source, void *out, unsigned long long count) {
    if (count == 0) return 0;
    if (!source || !out) return INVALID;
    return static_cast<int>(launch_f32_to_f16(source, out, count, nullptr));
}

int qi_f32_to_f16_ex(const float *source, void *out, unsigned long long count, void *stream) {
    if (count == 0) return 0;
    if (!source || !out) return INVALID;
    return static_cast<int>(launch_f32_to_f16(source, out, count, static_cast<cudaStream_t>(stream)));
}

int qi_w4a16_dequantize_ex(const void *codes, const void *scales, const void *minimums, void *w_half, int n, int k,
                           void *stream) {
    if (n <= 0 || k <= 0 || k % 64 != 0) return INVALID;
    if (!codes || !scales || !minimums || !w_half || !aligned16(codes) || !aligned16(w_half)) return INVALID;
    const long long chunks = static_cast<long long>(n) * (k / 32);
    const long long blocks = (chunks + 255) / 256;
    if (blocks > 0x7fffffffLL) return INVALID;
    dequantize_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(codes), static_cast<const __half *>(scales), static_cast<const __half *>(minimums),
        static_cast<__half *>(w_half), n, k);
    return static_cast<int>(cudaGetLastError());
}

int qi_linear(const qi_packed_linear *record, const qi_linear_work *work, const void *input, int input_dtype,
              void *output, int output_dtype, long long ld_output, int rows, int reuse_input, void *stream) {
    if (!record || !work || !input || !output || rows <= 0) return INVALID;
    if (record->group_size != 64) return INVALID;
    if (input_dtype != QI_DTYPE_F32 && input_dtype != QI_DTYPE_F16) return INVALID;
    const int n = record->n, k = record->k;
    if (record->scheme == QI_SCHEME_W4A4_H256) {  // transformer.cplus:702-708
        if (!work->code_scales) return INVALID;
        if (record->weights_wide != nullptr && work->wide != nullptr) {
            // one byte per code on both sides: no unpacking inside the GEMM
            if (!reuse_input) {
                const int status = qi_w4a4_quantize_activations_wide_ex(input, input_dtype, work->codes, work->code_scales,
                                                                        work->wide, rows, k, stream);
                if (status != 0) return status;
            }
            return qi_w4a4_gemm_wide_ex(work->wide, work->code_scales, record->weights_wide, record->scales, record->bias,
                                        output, output_dtype, ld_output, rows, n, k, stream);
        }
        if (!work->codes) return INVALID;
        if (!reuse_input) {
            const int status = qi_w4a4_quantize_activations_ex(input, input_dtype, work->codes, work->code_scales, rows, k, stream);
            if (status != 0) return status;
        }
        return qi_w4a4_gemm_ex(work->codes, work->code_scales, record->weights, record->scales, record->bias, output,
                               output_dtype, ld_output, rows, n, k, stream);
    }
    if (record->scheme == QI_SCHEME_W4A16) {  // transformer.cplus:709-712
        const void *x_half = input;
        if (input_dtype == QI_DTYPE_F32) {
            if (!work->halves) return INVALID;
            if (!reuse_input) {
                const int status = static_cast<int>(launch_f32_to_f16(static_cast<const float *>(input), work->halves,
                                                                      static_cast<unsigned long long>(rows) * k,
                                                                      static_cast<cudaStream_t>(stream)));
                if (status != 0) return status;
            }
            x_half = work->halves;
        }
        return qi_w4a16_gemm_ex(x_half, record->weights, record->scales, record->zeros, record->bias, output,
                                output_dtype, ld_output, rows, n, k, stream);
    }
    return INVALID;
}

int qi_kernel_status(unsigned int *status) {
    if (!status) return INVALID;
    cudaError_t error = cudaDeviceSynchronize();
    if (error != cudaSuccess) return static_cast<int>(error);
    uint32_t value = 0;
    error = cudaMemcpyFromSymbol(&value, g_status, sizeof(value));
    if (error != cudaSuccess) return static_cast<int>(error);
    if (value != 0) {
        const uint32_t zero = 0;
        error = cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    }
    *status = value;
    return static_cast<int>(error);
}

int qi_probe_tensor_rate(int kind, double seconds, double *tera_ops_per_second) {
    if (kind < 0 || kind > 2 || !(seconds > 0.0) || seconds > 2.0 || !tera_ops_per_second) return INVALID;
    const int device = current_device();
    if (device < 0) return INVALID;
    void (*kernel)(int) = kind == 0 ? probe::mma_rate_kernel<0> : kind == 1 ? probe::mma_rate_kernel<1> : probe::mma_rate_kernel<2>;
    cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, probe::SMEM_BYTES);
    if (error != cudaSuccess) return static_cast<int>(error);
    const int sms = sm_count(device);
    const double ops_per_batch = 2.0 * 128 * 256 * (kind == 0 ? 16 : 32) * probe::BATCH * sms;
    cudaEvent_t begin, end;
    if ((error = cudaEventCreate(&begin)) != cudaSuccess) return static_cast<int>(error);
    if ((error = cudaEventCreate(&end)) != cudaSuccess) { cudaEventDestroy(begin); return static_cast<int>(error); }
    // a short launch sizes the long one: the rate under the power limit differs from the rate of a burst
    int batches = 64;
    float ms = 0.0f;
    for (int round = 0; round < 2 && error == cudaSuccess; ++round) {
        cudaEventRecord(begin, nullptr);
        kernel<<<sms, probe::THREADS, probe::SMEM_BYTES>>>(batches);
        cudaEventRecord(end, nullptr);
        error = cudaEventSynchronize(end);
        if (error == cudaSuccess) error = cudaEventElapsedTime(&ms, begin, end);
        if (round == 0 && error == cudaSuccess && ms > 0.0f) {
            const double wanted = seconds * 1e3 / ms * batches;
            batches = wanted > 4e6 ? 4000000 : (wanted < 64 ? 64 : static_cast<int>(wanted));
        }
    }
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
    if (error != cudaSuccess) return static_cast<int>(error);
    *tera_ops_per_second = ops_per_batch * batches / (ms * 1e-3) / 1e12;
    return 0;
}

int qi_probe_wait_timeout(unsigned long long limit_ns, void *stream) {
    if (limit_ns == 0 || limit_ns > 100000000ull) return INVALID;  // at most a tenth of a second
    probe::wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
    return static_cast<int>(cudaGetLastError());
}

const char *qi_b200_version(void) { return "qipack_b200 0.1 sm_100a"; }

}  // extern "C"

#include "shard.cuh"
#include "pack_file.cuh"
