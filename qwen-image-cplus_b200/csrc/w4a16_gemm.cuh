// W4A16 g64 dequant-GEMM for sm_100a: y[m,n] = x_fp16[m,:] . W^[n,:] (+ bias[n]) with
// W^[n,k] = fp16(code[n,k] * scale[n,k/64] + minimum[n,k/64]), fp32 accumulation.
// Replaces w4a16_gemm_kernel of the reference (qwen_image_cuda/cuda/gemm.cu:191-268).
//
// Layout in HBM (row-major, caller-owned): x [m,k] fp16; codes [n,k/2] bytes, even input in
// the low nibble, values 0..15; scales, minimums [n,k/64] fp16; y [m,ldy] fp32 or fp16.
//
// One persistent CTA per SM walks output tiles of (NUM_M*128) x BN. Per 64-wide K block
// (one quantisation group):
//   warp 0     TMA: the x tile (128-byte swizzled, K-major) and the packed code tile
//   warps 8-15 unpack the codes to fp16 into the same swizzled K-major layout
//   warp 1     one thread issues tcgen05.mma kind::f16 (M=128, N=BN, K=16) x 4 per M block,
//              accumulating in TMEM; tcgen05.commit releases the shared-memory stage
//   warps 4-7  epilogue: tcgen05.ld the finished accumulator, add bias, store y; the
//              accumulator is double-buffered where TMEM allows, so this overlaps the next tile
//
// Dequantisation: a nibble becomes the fp16 numbers 1024+c (low) / 64+c (high) by one byte
// permute and one logic op, loses the offset by an exact subtraction, and goes through one
// half2 fused multiply-add. That is a single rounding of code*scale+minimum; the reference
// rounds the same exact value to fp32 first, which changes nothing whenever
// |code*scale+minimum| <= 1 (the sum of two multiples of 2^-24 below 1 is exact in fp32).
#pragma once
#include "ptx.cuh"

namespace qi {

__device__ uint32_t g_status = 0;  // first failed wait of any kernel of this library (0 = none)


struct GemmShape {
    int m, n, k;
    long long ldy;    // elements between rows of y
    int y_is_half;    // 0: float32, 1: float16
};

namespace w4a16 {

constexpr int THREADS = 512;
constexpr int BK = 64;                       // one quantisation group = one 128-byte swizzle row of fp16
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, EPILOGUE_WARP0 = 4, UNPACK_WARP0 = 8;
constexpr int UNPACK_WARPS = 8;

template <int NUM_M, int BN, int STAGES>
struct Tile {
    static constexpr int BM = NUM_M * 128;
    static constexpr int ACC_COLUMNS = NUM_M * BN;                   // TMEM columns of one accumulator
    static constexpr int ACC_STAGES = (2 * ACC_COLUMNS <= 512) ? 2 : 1;
    static constexpr int TMEM_COLUMNS = ACC_COLUMNS * ACC_STAGES;    // 128, 256 or 512: a power of two
    static constexpr int A_BYTES = BM * 128;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int C_BYTES = BN * 32;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + C_BYTES;
    static constexpr int BARRIER_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BARRIER_BYTES + 1024;  // + alignment slack
    static_assert(TMEM_COLUMNS == 128 || TMEM_COLUMNS == 256 || TMEM_COLUMNS == 512, "TMEM allocation size");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
    static_assert((3 * STAGES + 2 * ACC_STAGES) * 8 + 8 <= BARRIER_BYTES, "barrier block");
};

// 32 packed nibbles (16 bytes) -> 32 fp16 values in input order.
// Byte b of a word holds codes 2b (low nibble) and 2b + 1. The fast path puts each code into mantissa bits 4..7 of
// an fp16 with a zero exponent field, i.e. the subnormal code * 2^-20, and lets ONE fused multiply-add per pair do
// the rest: fma(code * 2^-20, scale * 2^20, minimum) = fp16(code * scale + minimum), the product exact and the
// sum rounded once like the reference's (gemm.cu:223-230). It needs scale * 2^20 to be an fp16 number: |scale| < 1/16.
// Any other scale (a NaN included) takes the path that first makes each code an fp16 integer.
__device__ __forceinline__ void unpack32(const uint4 packed, const __half2 scale2, const __half2 minimum2,
                                         uint4 (&out)[4]) {
    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
    uint32_t values[16];
    const __half sixteenth = __ushort_as_half(0x2C00), two_to_10 = __ushort_as_half(0x6400);
    if (__hlt(__habs(__low2half(scale2)), sixteenth)) {
        const __half2 up = __half2half2(two_to_10);
        const __half2 scale_up = __hmul2(__hmul2(scale2, up), up);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t low_nibbles_up = words[w] << 4;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                // [byte b of the shifted word, -, byte b of the word, -], then the two nibbles in bits 4..7 and 20..23
                uint32_t pair = __byte_perm(low_nibbles_up, words[w], 0x4400u + 0x1111u * b) & 0x00F000F0u;
                const __half2 weight = __hfma2(*reinterpret_cast<__half2 *>(&pair), scale_up, minimum2);
                values[4 * w + b] = *reinterpret_cast<const uint32_t *>(&weight);
            }
        }
    } else {
        const __half2 offsets = __halves2half2(__ushort_as_half(0x6400), __ushort_as_half(0x5400));  // (1024, 64)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t spread = __byte_perm(words[w], 0u, 0x4040u + 0x0101u * b);  // [byte b, 0, byte b, 0]
                uint32_t magic = (spread & 0x00F0000Fu) | 0x54006400u;
                const __half2 code = __hsub2(*reinterpret_cast<__half2 *>(&magic), offsets);
                const __half2 weight = __hfma2(code, scale2, minimum2);
                values[4 * w + b] = *reinterpret_cast<const uint32_t *>(&weight);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = make_uint4(values[4 * j], values[4 * j + 1], values[4 * j + 2], values[4 * j + 3]);
}

template <int NUM_M, int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_codes,
            const __half *__restrict__ scales, const __half *__restrict__ minimums,
            const float *__restrict__ bias, void *__restrict__ y, const GemmShape shape) {
    using T = Tile<NUM_M, BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + STAGES * T::A_BYTES;
    uint8_t *smem_c = smem_b + STAGES * T::B_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_c + STAGES * T::C_BYTES);
    uint64_t *ready = full + STAGES;
    uint64_t *empty = ready + STAGES;
    uint64_t *tmem_full = empty + STAGES;
    uint64_t *tmem_empty = tmem_full + T::ACC_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + T::ACC_STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (shape.m + T::BM - 1) / T::BM, tiles_n = (shape.n + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n, k_blocks = shape.k / BK, groups = shape.k / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full[s], 1);
            mbarrier_init(&ready[s], UNPACK_WARPS);
            mbarrier_init(&empty[s], 1);
        }
        for (int a = 0; a < T::ACC_STAGES; ++a) {
            mbarrier_init(&tmem_full[a], 1);
            mbarrier_init(&tmem_empty[a], 4);
        }
        fence_barrier_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(tmem_slot, T::TMEM_COLUMNS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            prefetch_tensormap(&map_x);
            prefetch_tensormap(&map_codes);
            uint32_t iteration = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * T::BM, n0 = (tile / tiles_m) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | s)) { alive = false; break; }
                    mbarrier_arrive_expect_tx(&full[s], T::A_BYTES + T::C_BYTES);
                    tma_load_2d(smem_a + s * T::A_BYTES, &map_x, &full[s], kb * BK, m0);
                    tma_load_2d(smem_c + s * T::C_BYTES, &map_codes, &full[s], kb * (BK / 2), n0);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16_f32(128, BN);
            uint32_t iteration = 0, tile_count = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++tile_count) {
                const uint32_t acc = tile_count % T::ACC_STAGES, acc_phase = (tile_count / T::ACC_STAGES) & 1;
                if (!mbarrier_wait(&tmem_empty[acc], acc_phase ^ 1, &g_status, STATUS_WAIT_TMEM_EMPTY | acc)) break;
                tcgen05_fence_after();
                const uint32_t tmem_acc = tmem_base + acc * T::ACC_COLUMNS;
                for (int kb = 0; kb < k_blocks; ++kb, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&full[s], phase, &g_status, STATUS_WAIT_FULL | s) ||
                        !mbarrier_wait(&ready[s], phase, &g_status, STATUS_WAIT_READY | s)) { alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_address = smem_u32(smem_a + s * T::A_BYTES);
                    const uint32_t b_address = smem_u32(smem_b + s * T::B_BYTES);
#pragma unroll
                    for (int mi = 0; mi < NUM_M; ++mi) {
#pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk) {
                            umma_f16(tmem_acc + mi * BN, umma_desc_k_sw128(a_address + mi * 16384 + kk * 32),
                                     umma_desc_k_sw128(b_address + kk * 32), idesc, (kb | kk) != 0 ? 1u : 0u);
                        }
                    }
                    tcgen05_commit(&empty[s]);
                }
                if (alive) tcgen05_commit(&tmem_full[acc]);
            }
        }
    } else if (warp >= UNPACK_WARP0) {
        const int d = threadIdx.x - UNPACK_WARP0 * 32;  // 0..255
        const int half_row = d & 1;
        uint32_t iteration = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int n0 = (tile / tiles_m) * BN;
            // scale and minimum of this thread's rows for the first K block
            __half scale_next[BN / 128], minimum_next[BN / 128];
#pragma unroll
            for (int p = 0; p < BN / 128; ++p) {
                const int row = n0 + p * 128 + (d >> 1);
                const bool inside = row < shape.n;
                scale_next[p] = inside ? __ldg(scales + static_cast<size_t>(row) * groups) : __ushort_as_half(0);
                minimum_next[p] = inside ? __ldg(minimums + static_cast<size_t>(row) * groups) : __ushort_as_half(0);
            }
            for (int kb = 0; kb < k_blocks; ++kb, ++iteration) {
                const int s = iteration % STAGES;
                const uint32_t phase = (iteration / STAGES) & 1;
                __half scale_now[BN / 128], minimum_now[BN / 128];
#pragma unroll
                for (int p = 0; p < BN / 128; ++p) {
                    scale_now[p] = scale_next[p], minimum_now[p] = minimum_next[p];
                    const int row = n0 + p * 128 + (d >> 1);
                    if (kb + 1 < k_blocks && row < shape.n) {
                        scale_next[p] = __ldg(scales + static_cast<size_t>(row) * groups + kb + 1);
                        minimum_next[p] = __ldg(minimums + static_cast<size_t>(row) * groups + kb + 1);
                    }
                }
                if (!mbarrier_wait(&full[s], phase, &g_status, STATUS_WAIT_FULL | 0x100 | s)) { alive = false; break; }
                const uint8_t *codes_tile = smem_c + s * T::C_BYTES;
                uint8_t *b_tile = smem_b + s * T::B_BYTES;
#pragma unroll
                for (int p = 0; p < BN / 128; ++p) {
                    const int row = p * 128 + (d >> 1);
                    const uint4 packed = *reinterpret_cast<const uint4 *>(codes_tile + row * 32 + half_row * 16);
                    uint4 out[4];
                    unpack32(packed, __half2half2(scale_now[p]), __half2half2(minimum_now[p]), out);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4 *>(b_tile + row * 128 + (((half_row * 4 + j) ^ (row & 7)) << 4)) = out[j];
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbarrier_arrive(&ready[s]);
            }
        }
    } else if (warp >= EPILOGUE_WARP0 && warp < EPILOGUE_WARP0 + 4) {
        const int quadrant = warp & 3;  // TMEM lanes 32*quadrant .. +31 belong to this warp
        uint32_t tile_count = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tile_count) {
            const int m0 = (tile % tiles_m) * T::BM, n0 = (tile / tiles_m) * BN;
            const uint32_t acc = tile_count % T::ACC_STAGES, acc_phase = (tile_count / T::ACC_STAGES) & 1;
            if (!mbarrier_wait(&tmem_full[acc], acc_phase, &g_status, STATUS_WAIT_TMEM_FULL | acc)) break;
            tcgen05_fence_after();
#pragma unroll
            for (int mi = 0; mi < NUM_M; ++mi) {
                const int row = m0 + mi * 128 + quadrant * 32 + lane;
                const uint32_t tmem_row = tmem_base + acc * T::ACC_COLUMNS + mi * BN + (static_cast<uint32_t>(quadrant * 32) << 16);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_load_32x32(tmem_row + c * 32, r);
                    tmem_load_wait();
                    const int col = n0 + c * 32;
                    if (row < shape.m && col < shape.n) {
                        if (bias != nullptr) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(bias + col + j));
                        }
                        if (shape.y_is_half) {
                            __half *out = static_cast<__half *>(y) + static_cast<size_t>(row) * shape.ldy + col;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint32_t h[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const __half2 pair = __floats2half2_rn(__uint_as_float(r[8 * j + 2 * i]), __uint_as_float(r[8 * j + 2 * i + 1]));
                                    h[i] = *reinterpret_cast<const uint32_t *>(&pair);
                                }
                                reinterpret_cast<uint4 *>(out)[j] = make_uint4(h[0], h[1], h[2], h[3]);
                            }
                        } else {
                            float *out = static_cast<float *>(y) + static_cast<size_t>(row) * shape.ldy + col;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4 *>(out)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbarrier_arrive(&tmem_empty[acc]);
        }
    }

    // teardown: nothing of this CTA may still be in flight when TMEM and shared memory go away
    tcgen05_fence_before();
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t *>(&g_status) != 0) {
        // a wait gave up: let bulk copies that were already issued land before the CTA exits
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == MMA_WARP) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, T::TMEM_COLUMNS);
    }
}

}  // namespace w4a16
}  // namespace qi
