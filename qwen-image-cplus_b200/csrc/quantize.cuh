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
//
// Two forms. The older one (one chunk per half-warp, scalar arithmetic) issues 34 instructions per value and
// is bound by that, at 0.37-0.42 of the HBM rate. The paired form gives a half-warp TWO chunks and keeps value
// i of both in one 64-bit register, so that the butterflies, the rounding and its check are packed fp32 pair
// instructions (add / sub / fma .f32x2: the same IEEE results, half the issue slots), moves the pairs through
// the transposes with 8- and 16-byte accesses, checks for rounding ties once per thread instead of once per
// value, and emits only the code formats asked for. It is used whenever there are at least two chunks.
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

// What the quantiser reads. Plain: the activations themselves. The other two compute the activation on the
// fly from what its producer would have read, with the producer's own expression, so that the [m, k] float32
// matrix between the two kernels of the reference is never written or read:
//   SwiGLU (qwen_image_cuda/cuda/ops.cu:133-138):    g / (1 + expf(-g)) * up
//   GELU-tanh (qwen_image_cuda/cuda/ops.cu:155-160): 0.5 v (1 + tanhf(0.7978845608028654 (v + 0.044715 v v v)))
template <typename T>
struct PlainSource {
    const T *x;
    __device__ __forceinline__ void load(long long offset, float (&v)[16]) const { load16(x + offset, v); }
};
struct SwigluSource {
    const float *gate, *up;
    __device__ __forceinline__ void load(long long offset, float (&v)[16]) const {
        float u[16];
        load16(gate + offset, v);
        load16(up + offset, u);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.0f + expf(-v[i])) * u[i];
    }
};
struct GeluSource {
    const float *x;
    __device__ __forceinline__ void load(long long offset, float (&v)[16]) const {
        load16(x + offset, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.5f * v[i] * (1.0f + tanhf(0.7978845608028654f * (v[i] + 0.044715f * v[i] * v[i] * v[i])));
    }
};

// WIDE: also (or only, when codes is null) write every code as one FP8 E4M3 byte, [m, k], the
// operand layout of w4a4_wide_gemm.cuh.
template <typename Source, bool WIDE>
__global__ void __launch_bounds__(QUANT_THREADS)
quantize_activations_kernel(const Source source, uint8_t *__restrict__ codes, __half *__restrict__ scales,
                            uint8_t *__restrict__ bytes, long long chunks) {
    __shared__ __align__(16) float transpose[(QUANT_THREADS / 32) * 2 * REGION];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half_warp = lane >> 4, l = lane & 15;
    float *region = transpose + (warp * 2 + half_warp) * REGION;
    const long long chunk = (static_cast<long long>(blockIdx.x) * (QUANT_THREADS / 32) + warp) * 2 + half_warp;
    const bool active = chunk < chunks;

    float v[16];
    if (active) {
        source.load(chunk * 256 + l * 16, v);
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

// ---- the paired form -------------------------------------------------------------------------------------

constexpr int PAIR_PITCH = 18;                      // 64-bit elements per transposed row: 16-byte reads stay conflict-free
constexpr int PAIR_REGION = 16 * PAIR_PITCH + 8;    // the second half-warp lands 16 banks away from the first

__device__ __forceinline__ uint64_t sub_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// gemm.cu:33-36 without the halving, on (chunk A, chunk B) pairs: the same association order per component.
__device__ __forceinline__ void butterfly2(uint64_t &a, uint64_t &b, uint64_t &c, uint64_t &d) {
    const uint64_t sum = add_f32x2(a, b), difference = sub_f32x2(a, b), reversed = sub_f32x2(b, a);
    const uint64_t o0 = sub_f32x2(add_f32x2(sum, c), d);
    const uint64_t o1 = add_f32x2(sub_f32x2(sum, c), d);
    const uint64_t o2 = add_f32x2(add_f32x2(difference, c), d);
    const uint64_t o3 = add_f32x2(add_f32x2(reversed, c), d);
    a = o0, b = o1, c = o2, d = o3;
}

__device__ __forceinline__ void two_passes2(uint64_t (&v)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) butterfly2(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
#pragma unroll
    for (int o = 0; o < 4; ++o) butterfly2(v[o], v[o + 4], v[o + 8], v[o + 12]);
}

// Scale of one 64-group from 16 x its peak, and what the rounding needs: 1 / (16 scale) and whether the short
// cut is safe at all (a scale in fp16's denormal range may be far from peak / 7, so quotients can pass 7.5 and
// must be clamped; a peak that is not finite leaves nothing to trust).
struct GroupScale {
    __half scale_half;
    float scale16, reciprocal;
    bool plain;
};

__device__ __forceinline__ GroupScale group_scale(float peak16) {
    GroupScale g;
    const float peak = peak16 * 0.0625f;
    g.scale_half = __float2half_rn(fmaxf(peak / 7.0f, SCALE_FLOOR));
    const float scale = __half2float(g.scale_half);
    g.scale16 = scale * 16.0f;  // v / scale == (16 v) / (16 scale)
    g.reciprocal = 1.0f / g.scale16;
    g.plain = scale >= 6.103515625e-05f && peak16 < 3.0e38f;  // fp16 normal, finite input
    return g;
}

// The reference's own expression for one value (gemm.cu:46-48), as 1.5 * 2^23 + code.
__device__ __forceinline__ float exact_code(float value16, float scale16) {
    return MAGIC + fminf(fmaxf(rintf(value16 / scale16), -7.0f), 7.0f);
}

// A lane's 16 values of one chunk as they come from memory, and their conversion to fp32.
template <typename T>
struct Raw16;
template <>
struct Raw16<__half> {
    uint4 q[2];
    __device__ __forceinline__ void load(const __half *source, bool active) {
        const uint4 *p = reinterpret_cast<const uint4 *>(source);
        q[0] = active ? __ldg(p) : make_uint4(0u, 0u, 0u, 0u), q[1] = active ? __ldg(p + 1) : make_uint4(0u, 0u, 0u, 0u);
    }
    __device__ __forceinline__ void convert(float (&v)[16]) const {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t words[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 pair = __half22float2(*reinterpret_cast<const __half2 *>(&words[j]));
                v[8 * i + 2 * j] = pair.x, v[8 * i + 2 * j + 1] = pair.y;
            }
        }
    }
};
template <>
struct Raw16<float> {
    float4 q[4];
    __device__ __forceinline__ void load(const float *source, bool active) {
        const float4 *p = reinterpret_cast<const float4 *>(source);
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = active ? __ldg(p + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    __device__ __forceinline__ void convert(float (&v)[16]) const {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[4 * i] = q[i].x, v[4 * i + 1] = q[i].y, v[4 * i + 2] = q[i].z, v[4 * i + 3] = q[i].w;
    }
};

// CODES: write nibble-packed codes [m, k/2]; WIDE: write one FP8 E4M3 byte per code [m, k]. At least one of them.
// A half-warp walks over pairs of chunks with the stride of the grid; the loads of its next pair are in flight
// while it works on the current one (the kernel holds 16 warps per SM: without that, too few bytes are under way
// to keep HBM busy).
template <typename T, bool CODES, bool WIDE>
__global__ void __launch_bounds__(QUANT_THREADS)
quantize_pairs_kernel(const T *__restrict__ x, uint8_t *__restrict__ codes, __half *__restrict__ scales,
                      uint8_t *__restrict__ bytes, long long chunks) {
    __shared__ __align__(16) uint64_t transpose[(QUANT_THREADS / 32) * 2 * PAIR_REGION];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half_warp = lane >> 4, l = lane & 15;
    uint64_t *region = transpose + (warp * 2 + half_warp) * PAIR_REGION;
    const long long pairs = (chunks + 1) / 2, stride = static_cast<long long>(gridDim.x) * (QUANT_THREADS / 16);
    long long pair = (static_cast<long long>(blockIdx.x) * (QUANT_THREADS / 32) + warp) * 2 + half_warp;
    Raw16<T> next_a, next_b;
    next_a.load(x + (2 * pair) * 256 + l * 16, 2 * pair < chunks);
    next_b.load(x + (2 * pair + 1) * 256 + l * 16, 2 * pair + 1 < chunks);
    // every half-warp of a warp runs the same number of rounds (the shuffles and __syncwarp below are warp-wide)
    const long long first_of_warp = (static_cast<long long>(blockIdx.x) * (QUANT_THREADS / 32) + warp) * 2;
    for (long long base = first_of_warp; base < pairs; base += stride, pair += stride) {
    const long long chunk_a = 2 * pair, chunk_b = chunk_a + 1;
    const bool active_a = chunk_a < chunks, active_b = chunk_b < chunks;

    uint64_t v[16];  // v[i] = (value i of this lane's 16 in chunk A, the same in chunk B)
    {
        float a[16], b[16];
        next_a.convert(a);
        next_b.convert(b);
        const long long after = pair + stride;
        next_a.load(x + (2 * after) * 256 + l * 16, 2 * after < chunks);
        next_b.load(x + (2 * after + 1) * 256 + l * 16, 2 * after + 1 < chunks);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = pack_f32x2(a[i], b[i]);
    }
    two_passes2(v);  // strides 1, 4

    // contiguous -> strided: lane l ends up with elements 16 * r + l, r = 0..15
#pragma unroll
    for (int c = 0; c < 16; ++c) region[c * PAIR_PITCH + l] = v[c];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const ulonglong2 q = *reinterpret_cast<const ulonglong2 *>(region + l * PAIR_PITCH + 2 * j);
        v[2 * j] = q.x, v[2 * j + 1] = q.y;
    }
    two_passes2(v);  // strides 16, 64

    // strided -> contiguous (each lane rewrites only the row it has just read)
#pragma unroll
    for (int j = 0; j < 8; ++j)
        *reinterpret_cast<ulonglong2 *>(region + l * PAIR_PITCH + 2 * j) = make_ulonglong2(v[2 * j], v[2 * j + 1]);
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 16; ++c) v[c] = region[c * PAIR_PITCH + l];

    // v holds 16 * (rotated value); four lanes share one 64-group of each chunk (gemm.cu:40-51)
    float peak_a = 0.0f, peak_b = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float a, b;
        unpack_f32x2(v[i], a, b);
        peak_a = fmaxf(peak_a, fabsf(a)), peak_b = fmaxf(peak_b, fabsf(b));
    }
    peak_a = fmaxf(peak_a, __shfl_xor_sync(0xffffffffu, peak_a, 1));
    peak_b = fmaxf(peak_b, __shfl_xor_sync(0xffffffffu, peak_b, 1));
    peak_a = fmaxf(peak_a, __shfl_xor_sync(0xffffffffu, peak_a, 2));
    peak_b = fmaxf(peak_b, __shfl_xor_sync(0xffffffffu, peak_b, 2));
    // every rotated value depends on all 256 inputs of its chunk: one value that is not finite means none can be trusted
    float first_a, first_b;
    unpack_f32x2(v[0], first_a, first_b);
    GroupScale ga = group_scale(peak_a), gb = group_scale(peak_b);
    ga.plain = ga.plain && fabsf(first_a) < 3.0e38f;
    gb.plain = gb.plain && fabsf(first_b) < 3.0e38f;

    const uint64_t reciprocal2 = pack_f32x2(ga.reciprocal, gb.reciprocal);
    const uint64_t negative2 = pack_f32x2(-ga.reciprocal, -gb.reciprocal), magic2 = pack_f32x2(MAGIC, MAGIC);
    uint64_t rounded[16];  // (1.5 * 2^23 + code) for both chunks: the code is the low nibble of the bits, two's complement
    float worst = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        rounded[i] = fma_f32x2(v[i], reciprocal2, magic2);
        const uint64_t integer = sub_f32x2(rounded[i], magic2);
        float ra, rb;
        unpack_f32x2(fma_f32x2(v[i], negative2, integer), ra, rb);  // integer - quotient: the distance from the rounding
        worst = fmaxf(worst, fmaxf(fabsf(ra), fabsf(rb)));
    }
    if (!(worst < 0.5f - 1.52587890625e-05f) || !ga.plain || !gb.plain) {
        // somewhere a quotient is near a tie, or the short cut does not hold for this group: the reference's expression
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float a, b;
            unpack_f32x2(v[i], a, b);
            rounded[i] = pack_f32x2(exact_code(a, ga.scale16), exact_code(b, gb.scale16));
        }
    }

    float code_a[16], code_b[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) unpack_f32x2(rounded[i], code_a[i], code_b[i]);
    if (CODES) {
        uint32_t packed_a[2] = {0u, 0u}, packed_b[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            packed_a[i >> 3] |= (__float_as_uint(code_a[i]) & 0xFu) << (4 * (i & 7));
            packed_b[i >> 3] |= (__float_as_uint(code_b[i]) & 0xFu) << (4 * (i & 7));
        }
        if (active_a) *reinterpret_cast<uint2 *>(codes + chunk_a * 128 + l * 8) = make_uint2(packed_a[0], packed_a[1]);
        if (active_b) *reinterpret_cast<uint2 *>(codes + chunk_b * 128 + l * 8) = make_uint2(packed_b[0], packed_b[1]);
    }
    if (WIDE) {
        uint32_t wide_a[4], wide_b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // values 4 j .. 4 j + 3 as four E4M3 bytes; the codes are exact small integers
            const uint32_t a_low = __nv_cvt_float2_to_fp8x2(make_float2(code_a[4 * j] - MAGIC, code_a[4 * j + 1] - MAGIC), __NV_SATFINITE, __NV_E4M3);
            const uint32_t a_high = __nv_cvt_float2_to_fp8x2(make_float2(code_a[4 * j + 2] - MAGIC, code_a[4 * j + 3] - MAGIC), __NV_SATFINITE, __NV_E4M3);
            const uint32_t b_low = __nv_cvt_float2_to_fp8x2(make_float2(code_b[4 * j] - MAGIC, code_b[4 * j + 1] - MAGIC), __NV_SATFINITE, __NV_E4M3);
            const uint32_t b_high = __nv_cvt_float2_to_fp8x2(make_float2(code_b[4 * j + 2] - MAGIC, code_b[4 * j + 3] - MAGIC), __NV_SATFINITE, __NV_E4M3);
            wide_a[j] = __byte_perm(a_low, a_high, 0x5410), wide_b[j] = __byte_perm(b_low, b_high, 0x5410);
        }
        if (active_a) *reinterpret_cast<uint4 *>(bytes + chunk_a * 256 + l * 16) = make_uint4(wide_a[0], wide_a[1], wide_a[2], wide_a[3]);
        if (active_b) *reinterpret_cast<uint4 *>(bytes + chunk_b * 256 + l * 16) = make_uint4(wide_b[0], wide_b[1], wide_b[2], wide_b[3]);
    }
    if ((l & 3) == 0) {
        if (active_a) scales[chunk_a * 4 + (l >> 2)] = ga.scale_half;
        if (active_b) scales[chunk_b * 4 + (l >> 2)] = gb.scale_half;
    }
    __syncwarp();  // the region is rewritten by the next round
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
    if (chunks >= 2) {
        // a half-warp takes two chunks
        long long pair_blocks = (chunks + 2 * chunks_per_block - 1) / (2 * chunks_per_block);
        int device = 0, sms = 148;
        if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (pair_blocks > 2LL * sms) pair_blocks = 2LL * sms;  // two CTAs per SM stay resident and walk over the rest
        const unsigned pairs_grid = static_cast<unsigned>(pair_blocks);
        const int variant = (bytes != nullptr ? 2 : 0) | (codes != nullptr ? 1 : 0);  // 1: codes, 2: bytes, 3: both
        if (x_is_half) {
            const __half *xs = static_cast<const __half *>(x);
            if (variant == 1) quantize_pairs_kernel<__half, true, false><<<pairs_grid, QUANT_THREADS, 0, stream>>>(xs, c, s, b, chunks);
            else if (variant == 2) quantize_pairs_kernel<__half, false, true><<<pairs_grid, QUANT_THREADS, 0, stream>>>(xs, c, s, b, chunks);
            else quantize_pairs_kernel<__half, true, true><<<pairs_grid, QUANT_THREADS, 0, stream>>>(xs, c, s, b, chunks);
        } else {
            const float *xs = static_cast<const float *>(x);
            if (variant == 1) quantize_pairs_kernel<float, true, false><<<pairs_grid, QUANT_THREADS, 0, stream>>>(xs, c, s, b, chunks);
            else if (variant == 2) quantize_pairs_kernel<float, false, true><<<pairs_grid, QUANT_THREADS, 0, stream>>>(xs, c, s, b, chunks);
            else quantize_pairs_kernel<float, true, true><<<pairs_grid, QUANT_THREADS, 0, stream>>>(xs, c, s, b, chunks);
        }
        return cudaGetLastError();
    }
    const PlainSource<__half> from_half = {static_cast<const __half *>(x)};
    const PlainSource<float> from_float = {static_cast<const float *>(x)};
    if (bytes != nullptr) {
        if (x_is_half) quantize_activations_kernel<PlainSource<__half>, true><<<grid, QUANT_THREADS, 0, stream>>>(from_half, c, s, b, chunks);
        else quantize_activations_kernel<PlainSource<float>, true><<<grid, QUANT_THREADS, 0, stream>>>(from_float, c, s, b, chunks);
    } else {
        if (x_is_half) quantize_activations_kernel<PlainSource<__half>, false><<<grid, QUANT_THREADS, 0, stream>>>(from_half, c, s, b, chunks);
        else quantize_activations_kernel<PlainSource<float>, false><<<grid, QUANT_THREADS, 0, stream>>>(from_float, c, s, b, chunks);
    }
    return cudaGetLastError();
}

// producer: 1 = SwiGLU of (first, second), 2 = GELU-tanh of first
inline cudaError_t launch_fused_quantize(int producer, const float *first, const float *second, void *codes, void *scales,
                                         void *bytes, int m, int k, cudaStream_t stream) {
    const long long chunks = static_cast<long long>(m) * (k / 256);
    if (chunks == 0) return cudaSuccess;
    const int chunks_per_block = QUANT_THREADS / 16;
    const long long blocks = (chunks + chunks_per_block - 1) / chunks_per_block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    const unsigned grid = static_cast<unsigned>(blocks);
    uint8_t *c = static_cast<uint8_t *>(codes), *b = static_cast<uint8_t *>(bytes);
    __half *s = static_cast<__half *>(scales);
    const SwigluSource swiglu = {first, second};
    const GeluSource gelu = {first};
    if (producer == 1) {
        if (bytes != nullptr) quantize_activations_kernel<SwigluSource, true><<<grid, QUANT_THREADS, 0, stream>>>(swiglu, c, s, b, chunks);
        else quantize_activations_kernel<SwigluSource, false><<<grid, QUANT_THREADS, 0, stream>>>(swiglu, c, s, b, chunks);
    } else {
        if (bytes != nullptr) quantize_activations_kernel<GeluSource, true><<<grid, QUANT_THREADS, 0, stream>>>(gelu, c, s, b, chunks);
        else quantize_activations_kernel<GeluSource, false><<<grid, QUANT_THREADS, 0, stream>>>(gelu, c, s, b, chunks);
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
