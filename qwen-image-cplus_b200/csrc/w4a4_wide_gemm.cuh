// W4A4 (H256, g64) GEMM on operands already widened to one byte per code:
//   y[m,n] = sum_g fma(dot_g[m,n], sa[m,g] * sw[n,g], y[m,n])   (+ bias[n]),  g ascending,
//   dot_g[m,n] = exact dot of the 64 signed 4-bit codes of group g.
// Same operator and the same fp32 arithmetic as w4a4_gemm.cuh / the reference's w4a4_gemm_kernel
// (qwen_image_cuda/cuda/gemm.cu:65-189); only the container of the codes differs.
//
// Layout in HBM (row-major, caller-owned): a_bytes [m,k], w_bytes [n,k]: code c in -7..7 stored as
// the FP8 E4M3 number c (exactly representable); a_scales [m,k/64], w_scales [n,k/64] fp16;
// y [m,ldy] fp32 or fp16. The byte matrices come from widen_codes_kernel below (weights: once,
// when the pack is loaded) or straight from the wide form of the activation quantiser.
//
// Why E4M3 and not int8: a product of two codes is at most 49 and a 64-term sum at most 3136, so
// tcgen05.mma kind::f8f6f4 with fp32 accumulation returns every group dot exactly — already as
// the float the fold needs. An int32 dot would first have to be converted, and int->float
// conversion issues at a quarter of the fp32 rate on this chip, which made it the bottleneck of
// the int8 kernel. With the codes pre-widened there is also nothing left to unpack in the
// kernel: TMA delivers both tiles in the 128-byte-swizzled K-major layout the tensor core reads.
//
// One persistent CTA per SM, 128 x 128 output tiles, 128 inputs (two groups) per stage:
//   warp 0      TMA for the A and B byte tiles
//   warp 1      one thread issues two tcgen05.mma (K = 32) per group into one of four TMEM
//               buffers of 128 fp32 columns, commits the buffer, and after two groups the stage
//   warps 2-3   stage sw of the two groups as fp32 in shared memory
//   warps 4-19  fold: thread = one row x 32 columns; tcgen05.ld the group's dots, release the
//               buffer, then per pair of columns one packed multiply (sa*sw) and one packed fused
//               multiply-add into register accumulators; after the last group add bias, store y
#pragma once
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace w4a4_wide {

constexpr int THREADS = 640;
constexpr int BM = 128, BN = 128;
constexpr int STAGE_K = 128;
constexpr int BUFFERS = 4;  // TMEM buffers of BN fp32 columns: 512 columns in all
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, SCALE_WARP0 = 2, SCALE_WARPS = 2, FOLD_WARP0 = 4, FOLD_WARPS = 16;
constexpr int COLUMNS = BN / (FOLD_WARPS / 4);  // 32 per fold thread
// setmaxnreg can only hand out what the launch allocated: floor8(65536 / 640) = 96 registers per thread.
// Asking for more than that pool blocks the warpgroup for ever, so the split is checked here.
constexpr int LAUNCH_REGISTERS = 96, CONTROL_REGISTERS = 64, FOLD_REGISTERS = 104;
static_assert(128 * CONTROL_REGISTERS + FOLD_WARPS * 32 * FOLD_REGISTERS <= THREADS * LAUNCH_REGISTERS,
              "setmaxnreg.inc would wait for registers that do not exist");
constexpr int SCALE_AHEAD = 6;                  // stages of weight scales in flight (global-load latency >> one stage)
constexpr int SCALE_RING = 8;

template <int STAGES>
struct Tile {
    static constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128;
    static constexpr int SCALE_BYTES = 2 * BN * 4;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SCALE_BYTES;
    static constexpr int BARRIER_BYTES = 512;
    static constexpr int RING_BYTES = SCALE_RING * BN * 4;  // fp16 pairs on their way in (cp.async)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RING_BYTES + BARRIER_BYTES + 1024;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
    static_assert((3 * STAGES + 2 * BUFFERS) * 8 + 8 <= BARRIER_BYTES, "barrier block");
};

// Packed nibbles -> one E4M3 byte per code, same element order. One thread per 16 input bytes.
__global__ void widen_codes_kernel(const uint8_t *__restrict__ codes, uint8_t *__restrict__ bytes, long long chunks) {
    const long long chunk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (chunk >= chunks) return;
    const uint4 packed = __ldg(reinterpret_cast<const uint4 *>(codes) + chunk);
    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
    uint32_t out[8];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t four = 0;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const int nibble = h * 4 + p * 2;
                const float lo = static_cast<float>((static_cast<int32_t>(words[w] << (28 - 4 * nibble))) >> 28);
                const float hi = static_cast<float>((static_cast<int32_t>(words[w] << (24 - 4 * nibble))) >> 28);
                const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
                four |= pair << (16 * p);
            }
            out[2 * w + h] = four;
        }
    }
    uint4 *destination = reinterpret_cast<uint4 *>(bytes) + 2 * chunk;
    destination[0] = make_uint4(out[0], out[1], out[2], out[3]);
    destination[1] = make_uint4(out[4], out[5], out[6], out[7]);
}

template <int STAGES, bool DUMP_DOTS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
            const __half *__restrict__ a_scales, const __half *__restrict__ w_scales,
            const float *__restrict__ bias, void *__restrict__ y, int32_t *__restrict__ dots_out,
            const GemmShape shape) {
    using T = Tile<STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tile_a = smem;
    uint8_t *tile_b = tile_a + STAGES * T::A_BYTES;
    float *sw_tile = reinterpret_cast<float *>(tile_b + STAGES * T::B_BYTES);
    __half2 *sw_ring = reinterpret_cast<__half2 *>(reinterpret_cast<uint8_t *>(sw_tile) + STAGES * T::SCALE_BYTES);
    uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sw_ring) + T::RING_BYTES);
    uint64_t *scale_ready = full + STAGES;
    uint64_t *empty = scale_ready + STAGES;
    uint64_t *dot_full = empty + STAGES;
    uint64_t *dot_empty = dot_full + BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(dot_empty + BUFFERS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (shape.m + BM - 1) / BM, tiles_n = (shape.n + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n, k_stages = shape.k / STAGE_K, groups = shape.k / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full[s], 1);
            mbarrier_init(&scale_ready[s], SCALE_WARPS);
            mbarrier_init(&empty[s], 1 + FOLD_WARPS);  // tensor core done with the tiles + fold done with sw
        }
        for (int b = 0; b < BUFFERS; ++b) {
            mbarrier_init(&dot_full[b], 1);
            mbarrier_init(&dot_empty[b], FOLD_WARPS);
        }
        fence_barrier_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(tmem_slot, BUFFERS * BN);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < FOLD_WARP0) {
      setmaxnreg_dec<CONTROL_REGISTERS>();  // warpgroup 0 (TMA, MMA, scale staging) gives registers to the fold warps
      if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_w);
            uint32_t iteration = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                for (int ks = 0; ks < k_stages; ++ks, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x3000 | s)) { alive = false; break; }
                    mbarrier_arrive_expect_tx(&full[s], T::A_BYTES + T::B_BYTES);
                    tma_load_2d(tile_a + s * T::A_BYTES, &map_a, &full[s], ks * STAGE_K, m0);
                    tma_load_2d(tile_b + s * T::B_BYTES, &map_w, &full[s], ks * STAGE_K, n0);
                }
            }
        }
      } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_e4m3_f32(BM, BN);
            uint32_t iteration = 0, group_count = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                for (int ks = 0; ks < k_stages && alive; ++ks, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&full[s], phase, &g_status, STATUS_WAIT_FULL | 0x3000 | s)) { alive = false; break; }
                    const uint32_t a_address = smem_u32(tile_a + s * T::A_BYTES);
                    const uint32_t b_address = smem_u32(tile_b + s * T::B_BYTES);
#pragma unroll
                    for (int gl = 0; gl < 2; ++gl, ++group_count) {
                        const uint32_t buffer = group_count % BUFFERS, buffer_phase = (group_count / BUFFERS) & 1;
                        if (!mbarrier_wait(&dot_empty[buffer], buffer_phase ^ 1, &g_status, STATUS_WAIT_TMEM_EMPTY | 0x3000 | buffer)) { alive = false; break; }
                        tcgen05_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 2; ++kk)
                            umma_f8(tmem_base + buffer * BN, umma_desc_k_sw128(a_address + gl * 64 + kk * 32),
                                    umma_desc_k_sw128(b_address + gl * 64 + kk * 32), idesc, kk);
                        tcgen05_commit(&dot_full[buffer]);
                    }
                    if (alive) tcgen05_commit(&empty[s]);
                }
            }
        }
      } else {
        // Weight scales of each stage's two groups, converted to fp32 once for all fold threads.
        // The fp16 pairs travel global -> shared with cp.async, SCALE_AHEAD stages ahead of their
        // use, because one global-load latency is longer than the tensor core needs for a stage.
        const int t = threadIdx.x - SCALE_WARP0 * 32;  // 0..63
        const int my_tiles = blockIdx.x < tiles ? (tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
        const uint32_t total = static_cast<uint32_t>(my_tiles) * k_stages;
        auto fetch = [&](uint32_t it) {
            if (it < total) {
                const int tile = blockIdx.x + static_cast<int>(it / k_stages) * gridDim.x;
                const int ks = it % k_stages, n0 = (tile / tiles_m) * BN;
#pragma unroll
                for (int p = 0; p < BN / 64; ++p) {
                    const int col = n0 + p * 64 + t;
                    __half2 *slot = sw_ring + (it % SCALE_RING) * BN + p * 64 + t;
                    if (col < shape.n) cp_async_4(slot, w_scales + static_cast<size_t>(col) * groups + 2 * ks);
                    else *slot = __halves2half2(__ushort_as_half(0), __ushort_as_half(0));
                }
            }
            cp_async_commit();
        };
        for (uint32_t it = 0; it < SCALE_AHEAD; ++it) fetch(it);
        for (uint32_t it = 0; it < total; ++it) {
            const int s = it % STAGES;
            const uint32_t phase = (it / STAGES) & 1;
            fetch(it + SCALE_AHEAD);
            cp_async_wait<SCALE_AHEAD>();  // this thread's copies for stage `it` have landed
            float2 values[BN / 64];
#pragma unroll
            for (int p = 0; p < BN / 64; ++p) values[p] = __half22float2(sw_ring[(it % SCALE_RING) * BN + p * 64 + t]);
            if (!mbarrier_wait_warp(&empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x4000 | s, lane)) break;
            float *sw_stage = sw_tile + s * 2 * BN;
#pragma unroll
            for (int p = 0; p < BN / 64; ++p) {
                sw_stage[p * 64 + t] = values[p].x;
                sw_stage[BN + p * 64 + t] = values[p].y;
            }
            __syncwarp();
            if (lane == 0) mbarrier_arrive(&scale_ready[s]);
        }
        cp_async_wait<0>();
      }
    } else {
        setmaxnreg_inc<FOLD_REGISTERS>();
        const int quadrant = warp & 3, slice = (warp - FOLD_WARP0) >> 2;
        uint32_t iteration = 0, group_count = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const int row = m0 + quadrant * 32 + lane;
            const bool row_inside = row < shape.m;
            const __half *sa_row = a_scales + static_cast<size_t>(row_inside ? row : 0) * groups;
            uint64_t acc[COLUMNS / 2];
#pragma unroll
            for (int j = 0; j < COLUMNS / 2; ++j) acc[j] = 0ull;  // two +0.0f
            __half2 sa_next = __ldg(reinterpret_cast<const __half2 *>(sa_row));
            for (int ks = 0; ks < k_stages && alive; ++ks, ++iteration) {
                const int s = iteration % STAGES;
                const uint32_t phase = (iteration / STAGES) & 1;
                const float2 sa_pair = __half22float2(sa_next);
                if (ks + 1 < k_stages) sa_next = __ldg(reinterpret_cast<const __half2 *>(sa_row + 2 * ks + 2));
                if (!mbarrier_wait_warp(&scale_ready[s], phase, &g_status, STATUS_WAIT_READY | 0x3000 | s, lane)) { alive = false; break; }
                const float *sw_stage = sw_tile + s * 2 * BN + slice * COLUMNS;
#pragma unroll
                for (int gl = 0; gl < 2; ++gl, ++group_count) {
                    const uint32_t buffer = group_count % BUFFERS, buffer_phase = (group_count / BUFFERS) & 1;
                    const float sa = gl == 0 ? sa_pair.x : sa_pair.y;
                    const uint64_t sa2 = pack_f32x2(sa, sa);
                    if (!mbarrier_wait_warp(&dot_full[buffer], buffer_phase, &g_status, STATUS_WAIT_TMEM_FULL | 0x3000 | buffer, lane)) { alive = false; break; }
                    tcgen05_fence_after();
                    uint32_t r[32];
                    tmem_load_32x32(tmem_base + buffer * BN + slice * COLUMNS + (static_cast<uint32_t>(quadrant * 32) << 16), r);
                    tmem_load_wait();
                    // the dots are in registers: hand the buffer back to the tensor core
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbarrier_arrive(&dot_empty[buffer]);
                    if (DUMP_DOTS && row_inside) {
                        const int group = ks * 2 + gl;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = n0 + slice * COLUMNS + j;
                            if (col < shape.n)
                                dots_out[(static_cast<size_t>(row) * shape.n + col) * groups + group] =
                                    static_cast<int32_t>(__uint_as_float(r[j]));
                        }
                    }
                    const float *sw_group = sw_stage + gl * BN;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 sw4 = *reinterpret_cast<const float4 *>(sw_group + j);
                        const uint64_t p01 = mul_f32x2(sa2, pack_f32x2(sw4.x, sw4.y));
                        const uint64_t p23 = mul_f32x2(sa2, pack_f32x2(sw4.z, sw4.w));
                        acc[j / 2] = fma_f32x2(pack_u32x2(r[j], r[j + 1]), p01, acc[j / 2]);
                        acc[j / 2 + 1] = fma_f32x2(pack_u32x2(r[j + 2], r[j + 3]), p23, acc[j / 2 + 1]);
                    }
                }
                if (alive) {
                    __syncwarp();
                    if (lane == 0) mbarrier_arrive(&empty[s]);  // done reading this stage's sw
                }
            }
            if (!alive) break;
            const int col = n0 + slice * COLUMNS;
            if (row_inside && col < shape.n) {
                float v[COLUMNS];
#pragma unroll
                for (int j = 0; j < COLUMNS / 2; ++j) unpack_f32x2(acc[j], v[2 * j], v[2 * j + 1]);
                if (bias != nullptr) {
#pragma unroll
                    for (int j = 0; j < COLUMNS; ++j) v[j] += __ldg(bias + col + j);
                }
                if (shape.y_is_half) {
                    __half *out = static_cast<__half *>(y) + static_cast<size_t>(row) * shape.ldy + col;
#pragma unroll
                    for (int j = 0; j < COLUMNS / 8; ++j) {
                        uint32_t h[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const __half2 pair = __floats2half2_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
                            h[i] = *reinterpret_cast<const uint32_t *>(&pair);
                        }
                        reinterpret_cast<uint4 *>(out)[j] = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                } else {
                    float *out = static_cast<float *>(y) + static_cast<size_t>(row) * shape.ldy + col;
#pragma unroll
                    for (int j = 0; j < COLUMNS / 4; ++j)
                        reinterpret_cast<float4 *>(out)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t *>(&g_status) != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let bulk copies already issued land
    }
    if (warp == MMA_WARP) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, BUFFERS * BN);
    }
}

}  // namespace w4a4_wide
}  // namespace qi
