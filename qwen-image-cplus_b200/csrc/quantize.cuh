// W4A4 activation quantiser: block-diagonal H256 rotation of every row, then symmetric
// per-64-group int4 codes with an fp16 scale. Replaces quantize_activations_kernel of the
// reference (qwen_image_cuda/cuda/gemm.cu:22-57; fp16-input twin in
// qwen_image_cuda/cuda/bench/bench_w4a4.cu:33-66) and produces the same bytes.
//
// Layout in HBM (all row-major, caller-owned):
//   x      [m, k]     float32 or float16
//   codes  [m, k/2]   one byte per two inputs, even input in the low nibble, two's complement
//   scales [m, k/64]  float16
//
// One half-warp owns one 256-chunk of one row; each lane holds 16 values in registers.
// The radix-4 butterflies for strides 1 and 4 act on a lane's own 16 contiguous values;
// a transpose through shared memory brings strides 16 and 64 into the lane as well, and a
// second transpose restores the contiguous order for the group reductions and for packing.
// Every sum keeps the reference's association order ((a+b)+c)-d etc. The four halvings are
// applied as one exact scaling (by 16 on the divisor side), which gives the same bits as
// four multiplications by 0.5 for every |x| below 2^120.
//
// rint(v / scale) is evaluated as a fused multiply by the reciprocal plus a magic-number
// rounding; a lane whose quotient lies within 2^-16 of a rounding tie redoes it with the
// IEEE division the reference uses, so the codes are identical.
#pragma once
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace qi {

namespace {

constexpr int QUANT_THREADS = 256;
constexpr int PITCH = 20;                  // floats per transposed row: 128-bit reads stay conflict-free
constexpr int REGION = 16 * PITCH + 16;    // second half-warp lands 16 banks away from the first
constexpr float MAGIC = 12582912.0f;       // 1.5 * 2^23: adding it rounds to an integer, ties to even
constexpr int MAGIC_BITS = 0x4B400000;
constexpr float SCALE_FLOOR = 5.9604645e-08f;  // 2^-24, gemm.cu:45

__device__ __forceinline__ void load16(const float *source, float (&v)[16]) {
    const float4 *p = reinterpret_cast<const float4 *>(source);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 q = __ldg(p + i);
        v[4 * i] = q.x, v[4 * i + 1] = q.y, v[4 * i + 2] = q.z, v[4 * i + 3] = q.w;
    }
}

__device__ __forceinline__ void load16(const __half *source, float (&v)[16]) {
    const uint4 *p = reinterpret_cast<const uint4 *>(source);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 q = __ldg(p + i);
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 pair = __half22float2(*reinterpret_cast<const __half2 *>(&words[j]));
            v[8 * i + 2 * j] = pair.x, v[8 * i + 2 * j + 1] = pair.y;
        }
    }
}

// gemm.cu:33-36 without the halving.
__device__ __forceinline__ void butterfly(float &a, float &b, float &c, float &d) {
    const float sum = a + b, difference = a - b, reversed = b - a;  // b - a == (-a) + b exactly
    const float o0 = (sum + c) - d;
    const float o1 = (sum - c) + d;
    const float o2 = (difference + c) + d;
    const float o3 = (reversed + c) + d;
    a = o0, b = o1, c = o2, d = o3;
}

// Strides 1 and 4 of a 16-value array (also strides 16 and 64 after the transpose).
__device__ __forceinline__ void two_passes(float (&v)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) butterfly(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
#pragma unroll
    for (int o = 0; o < 4; ++o) butterfly(v[o], v[o + 4], v[o + 8], v[o + 12]);
}

// WIDE: also (or only, when codes is null) write every code as one FP8 E4M3 byte, [m, k], the
// operand layout of w4a4_wide_gemm.cuh.
template <typename T, bool WIDE>
__global__ void __launch_bounds__(QUANT_THREADS)
quantize_activations_kernel(const T *__restrict__ x, uint8_t *__restrict__ codes, __half *__restrict__ scales,
                            uint8_t *__restrict__ bytes, long long chunks) {
    __shared__ __align__(16) float transpose[(QUANT_THREADS / 32) * 2 * REGION];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half_warp = lane >> 4, l = lane & 15;
    float *region = transpose + (warp * 2 + half_warp) * REGION;
    const long long chunk = (static_cast<long long>(blockIdx.x) * (QUANT_THREADS / 32) + warp) * 2 + half_warp;
    const bool active = chunk < chunks;

    float v[16];
    if (active) {
        load16(x + chunk * 256 + l * 16, v);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.0f;
    }
    two_passes(v);  // strides 1, 4

    // contiguous -> strided: lane l ends up with elements 16 * r + l, r = 0..15
#pragma unroll
    for (int c = 0; c < 16; ++c) region[c * PITCH + l] = v[c];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 q = *reinterpret_cast<const float4 *>(region + l * PITCH + 4 * j);
        v[4 * j] = q.x, v[4 * j + 1] = q.y, v[4 * j + 2] = q.z, v[4 * j + 3] = q.w;
    }
    two_passes(v);  // strides 16, 64

    // strided -> contiguous (each lane rewrites only the row it has just read)
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<float4 *>(region + l * PITCH + 4 * j) =
            make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 16; ++c) v[c] = region[c * PITCH + l];

    // v holds 16 * (rotated value); four lanes share one 64-group (gemm.cu:40-51)
    float peak16 = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) peak16 = fmaxf(peak16, fabsf(v[i]));
    peak16 = fmaxf(peak16, __shfl_xor_sync(0xffffffffu, peak16, 1));
    peak16 = fmaxf(peak16, __shfl_xor_sync(0xffffffffu, peak16, 2));
    const float peak = peak16 * 0.0625f;
    const __half scale_half = __float2half_rn(fmaxf(peak / 7.0f, SCALE_FLOOR));
    const float scale16 = __half2float(scale_half) * 16.0f;  // v / scale == (16 v) / (16 scale)
    const float reciprocal = 1.0f / scale16;

    uint32_t packed[2] = {0u, 0u};
    uint32_t wide[4] = {0u, 0u, 0u, 0u};
    float previous = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float rounded = fmaf(v[i], reciprocal, MAGIC);
        const float integer = rounded - MAGIC;
        const float residual = fmaf(v[i], reciprocal, -integer);
        int bits = __float_as_int(rounded);
        if (!(fabsf(residual) < 0.5f - 1.52587890625e-05f)) {
            // near a tie (or not finite): the reference's own expression
            const float exact = fminf(fmaxf(rintf(v[i] / scale16), -7.0f), 7.0f);
            bits = MAGIC_BITS + static_cast<int>(exact);
        }
        bits = min(max(bits, MAGIC_BITS - 7), MAGIC_BITS + 7);
        packed[i >> 3] |= static_cast<uint32_t>(bits & 0xF) << (4 * (i & 7));
        if (WIDE) {
            const float code = __int_as_float(bits) - MAGIC;  // exact
            if (i & 1) {
                const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(previous, code), __NV_SATFINITE, __NV_E4M3);
                wide[i >> 2] |= pair << (8 * (i & 2));
            }
            previous = code;
        }
    }
    if (active) {
        if (!WIDE || codes != nullptr)
            *reinterpret_cast<uint2 *>(codes + chunk * 128 + l * 8) = make_uint2(packed[0], packed[1]);
        if (WIDE) *reinterpret_cast<uint4 *>(bytes + chunk * 256 + l * 16) = make_uint4(wide[0], wide[1], wide[2], wide[3]);
        if ((l & 3) == 0) scales[chunk * 4 + (l >> 2)] = scale_half;
    }
}

__global__ void f32_to_f16_kernel(const float *__restrict__ source, __half *__restrict__ out,
                                  unsigned long long count) {
    // eight values per thread when both pointers allow 16-byte accesses, scalar tail otherwise
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    const unsigned long long thread = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(source) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    const unsigned long long vectors = aligned ? count / 8 : 0;
    for (unsigned long long i = thread; i < vectors; i += stride) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(source) + 2 * i);
        const float4 b = __ldg(reinterpret_cast<const float4 *>(source) + 2 * i + 1);
        uint4 o;
        __half2 h;
        h = __floats2half2_rn(a.x, a.y), o.x = *reinterpret_cast<uint32_t *>(&h);
        h = __floats2half2_rn(a.z, a.w), o.y = *reinterpret_cast<uint32_t *>(&h);
        h = __floats2half2_rn(b.x, b.y), o.z = *reinterpret_cast<uint32_t *>(&h);
        h = __floats2half2_rn(b.z, b.w), o.w = *reinterpret_cast<uint32_t *>(&h);
        reinterpret_cast<uint4 *>(out)[i] = o;
    }
    for (unsigned long long i = vectors * 8 + thread; i < count; i += stride) out[i] = __float2half_rn(source[i]);
}

}  // namespace

inline cudaError_t launch_quantize_activations(const void *x, int x_is_half, void *codes, void *scales, void *bytes,
                                               int m, int k, cudaStream_t stream) {
    const long long chunks = static_cast<long long>(m) * (k / 256);
    if (chunks == 0) return cudaSuccess;
    const int chunks_per_block = QUANT_THREADS / 16;
    const long long blocks = (chunks + chunks_per_block - 1) / chunks_per_block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    const unsigned grid = static_cast<unsigned>(blocks);
    uint8_t *c = static_cast<uint8_t *>(codes), *b = static_cast<uint8_t *>(bytes);
    __half *s = static_cast<__half *>(scales);
    if (bytes != nullptr) {
        if (x_is_half)
            quantize_activations_kernel<__half, true><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const __half *>(x), c, s, b, chunks);
        else
            quantize_activations_kernel<float, true><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const float *>(x), c, s, b, chunks);
    } else {
        if (x_is_half)
            quantize_activations_kernel<__half, false><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const __half *>(x), c, s, b, chunks);
        else
            quantize_activations_kernel<float, false><<<grid, QUANT_THREADS, 0, stream>>>(static_cast<const float *>(x), c, s, b, chunks);
    }
    return cudaGetLastError();
}

inline cudaError_t launch_f32_to_f16(const float *source, void *out, unsigned long long count, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    unsigned long long blocks = (count / 8 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148ull * 16) blocks = 148ull * 16;
    f32_to_f16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(source, static_cast<__half *>(out), count);
    return cudaGetLastError();
}

}  // namespace qi
