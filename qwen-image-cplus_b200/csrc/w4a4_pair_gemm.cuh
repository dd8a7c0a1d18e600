// W4A4 (H256, g64) GEMM on byte-wide (E4M3) codes, one 256 x 256 output tile per PAIR of CTAs
// (thread-block cluster of two, tcgen05 cta_group::2). Same operator, arithmetic and bits as
// w4a4_wide_gemm.cuh and the reference's w4a4_gemm_kernel (qwen_image_cuda/cuda/gemm.cu:65-189).
//
// Why pairs: with one byte per code a 128 x 128 tile moves 32 KB from L2 per 2.1 M multiply-adds,
// and the L2 -> SM path (about 8 TB/s over the chip) saturates long before the tensor cores do.
// In a pair each CTA loads its own 128 rows of A and only HALF of the tile's B rows; the MMA
// (M = 256 across the pair, N = 256) reads both halves of B from both CTAs' shared memory. That is
// 32 KB per 4.2 M multiply-adds per CTA: half the traffic, with no TMA multicast.
//
// Per CTA (rank 0 = leader issues the MMAs for both):
//   warp 0      TMA: own A rows and own half of B; completion bytes are counted on the leader's barrier
//   warp 1      leader only: per group two tcgen05.mma.cta_group::2 kind::f8f6f4 (K = 32) into one of
//               two TMEM buffers of 256 fp32 columns; commits arrive on both CTAs' barriers
//   warps 2-3   stage sw of the stage's two groups (256 columns) as fp32
//   warps 4-11  fold this CTA's 128 rows x 256 columns, 32 rows x 128 columns per warp; after its last
//               load of a group the warp releases the TMEM buffer on the LEADER's barrier
#pragma once
#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace w4a4_pair {

constexpr int THREADS = 384;
constexpr int BM = 128;        // rows per CTA; the pair covers 256
constexpr int BN = 256;        // columns of the pair's tile; each CTA loads 128 of the B rows
constexpr int STAGE_K = 128;
constexpr int BUFFERS = 2;     // TMEM buffers of BN fp32 columns
constexpr int STAGES = 6;
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, SCALE_WARP0 = 2, SCALE_WARPS = 2, FOLD_WARP0 = 4, FOLD_WARPS = 8;
constexpr int COLUMNS = BN / (FOLD_WARPS / 4);  // columns per fold warp: 128
constexpr bool DOUBLE_BUFFER = true;            // a second register set for the dots in flight
// setmaxnreg can only hand out what the launch allocated: floor8(65536 / 384) = 168 registers per thread.
// Two fold warps per scheduler, each with 128 accumulators and two sets of 32 fetched dots. Measured
// against four warps per scheduler with 64 accumulators and one set (112 registers, spills): 1.7x faster.
constexpr int LAUNCH_REGISTERS = 168, CONTROL_REGISTERS = 40, FOLD_REGISTERS = 232;
static_assert(128 * CONTROL_REGISTERS + FOLD_WARPS * 32 * FOLD_REGISTERS <= THREADS * LAUNCH_REGISTERS,
              "setmaxnreg.inc would wait for registers that do not exist");
constexpr int SCALE_AHEAD = 6, SCALE_RING = 8;

constexpr int A_BYTES = BM * 128, B_BYTES = (BN / 2) * 128;
constexpr int SCALE_BYTES = 2 * BN * 4;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SCALE_BYTES;
constexpr int RING_BYTES = SCALE_RING * BN * 4;
constexpr int BARRIER_BYTES = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RING_BYTES + BARRIER_BYTES + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
static_assert((3 * STAGES + 2 * BUFFERS) * 8 + 8 <= BARRIER_BYTES, "barrier block");


// Everything a role needs to find its way around the CTA's shared memory and the problem.
struct View {
    float *sw_tile;
    __half2 *sw_ring;
    uint64_t *scale_ready, *empty, *dot_full, *dot_empty;
    uint32_t tmem_base, cta;
    int pair, pairs, tiles, tiles_m, k_stages, groups;
};

// Warps 2-3: weight scales of each stage's two groups for the tile's 256 columns, converted to fp32
// once for all fold threads; fetched SCALE_AHEAD stages early with cp.async (one global-load latency
// is longer than the tensor core needs for a stage).
__device__ __forceinline__ void scale_role(const View &v, const __half *__restrict__ w_scales, const GemmShape &shape,
                                           int t, int lane) {
    const int my_tiles = v.pair < v.tiles ? (v.tiles - 1 - v.pair) / v.pairs + 1 : 0;
    const uint32_t total = static_cast<uint32_t>(my_tiles) * v.k_stages;
    auto fetch = [&](uint32_t it) {
        if (it < total) {
            const int tile = v.pair + static_cast<int>(it / v.k_stages) * v.pairs;
            const int ks = it % v.k_stages, n0 = (tile / v.tiles_m) * BN;
#pragma unroll
            for (int p = 0; p < BN / 64; ++p) {
                const int col = n0 + p * 64 + t;
                __half2 *slot = v.sw_ring + (it % SCALE_RING) * BN + p * 64 + t;
                if (col < shape.n) cp_async_4(slot, w_scales + static_cast<size_t>(col) * v.groups + 2 * ks);
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
        for (int p = 0; p < BN / 64; ++p) values[p] = __half22float2(v.sw_ring[(it % SCALE_RING) * BN + p * 64 + t]);
        if (!mbarrier_wait_warp(&v.empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x6000 | s, lane)) break;
        float *sw_stage = v.sw_tile + s * 2 * BN;
#pragma unroll
        for (int p = 0; p < BN / 64; ++p) {
            sw_stage[p * 64 + t] = values[p].x;
            sw_stage[BN + p * 64 + t] = values[p].y;
        }
        __syncwarp();
        if (lane == 0) mbarrier_arrive(&v.scale_ready[s]);
    }
    cp_async_wait<0>();
}

// Warps 4-11: a warp folds 32 rows x 128 columns of this CTA's half of the tile.
// The dots are fetched with tcgen05.ld.16x256b, whose register layout is that of an MMA accumulator
// fragment: a thread holds 4 rows x 32 columns (column pairs 8 apart), not 1 row x 128 columns.
// With a whole row per thread every lane needs the SAME weight scale for a column, i.e. one
// shared-memory broadcast per column and warp - more load wavefronts than the fp32 pipe has
// cycles. In the fragment layout a thread's columns never change, so a group costs 16 eight-byte
// loads of sw and 4 values of sa per thread.
// With DOUBLE_BUFFER two register sets alternate (the tcgen05.ld of the next 32-column batch is in flight
// during the arithmetic of this one).
template <bool DUMP_DOTS>
__device__ __forceinline__ void fold_role(const View &v, const __half *__restrict__ a_scales,
                                          const float *__restrict__ bias, void *__restrict__ y,
                                          int32_t *__restrict__ dots_out, const GemmShape &shape, int warp, int lane) {
    constexpr int BATCHES = COLUMNS / 32;  // 4 per group
    const int quadrant = warp & 3, slice = (warp - FOLD_WARP0) >> 2;
    const int pair_column = 2 * (lane & 3), fragment_row = lane >> 2;
    const uint32_t leader_dot_empty = map_to_cta(smem_u32(v.dot_empty), 0);
    const uint32_t tmem_lane = v.tmem_base + slice * COLUMNS + (static_cast<uint32_t>(quadrant * 32) << 16);
    const int my_tiles = v.pair < v.tiles ? (v.tiles - 1 - v.pair) / v.pairs + 1 : 0;
    const uint32_t total_groups = static_cast<uint32_t>(my_tiles) * v.groups;
    uint32_t set[DOUBLE_BUFFER ? 2 : 1][32] = {};  // [16 * half + 4 * x + 2 * a + e]: rows fragment_row + 16 half + 8 a, columns 8 x + pair_column + e
    bool alive = true;

    // Starts the load of batch `batch` of group `group_count`; the first batch of a group waits for its dots.
    auto issue = [&](uint32_t group_count, int batch, uint32_t (&destination)[32], bool blocking) -> bool {
        const uint32_t buffer = group_count % BUFFERS, phase = (group_count / BUFFERS) & 1;
        if (batch == 0) {
            if (!blocking) {
                uint32_t ready = 0;
                if (lane == 0) ready = mbarrier_try_wait(&v.dot_full[buffer], phase) ? 1u : 0u;
                if (__shfl_sync(0xffffffffu, ready, 0) == 0) return false;
            } else if (!mbarrier_wait_warp(&v.dot_full[buffer], phase, &g_status, STATUS_WAIT_TMEM_FULL | 0x5000 | buffer, lane)) {
                alive = false;
                return false;
            }
            tcgen05_fence_after();
        }
        const uint32_t address = tmem_lane + buffer * BN + batch * 32;
        if (shape.ablate & 8) return true;  // tuning: leave the registers as they are
        tmem_load_16x256_x4(address, &destination[0]);
        tmem_load_16x256_x4(address + (16u << 16), &destination[16]);
        return true;
    };

    uint32_t iteration = 0, group_count = 0;
    if (total_groups > 0) issue(0, 0, set[0], true);
    for (int tile = v.pair; tile < v.tiles && alive; tile += v.pairs) {
        const int m0 = (tile % v.tiles_m) * 2 * BM + v.cta * BM + quadrant * 32, n0 = (tile / v.tiles_m) * BN + slice * COLUMNS;
        // this thread's four rows: m0 + fragment_row + 8 * index, index = 2 * half + a
        const __half *sa_rows[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = m0 + fragment_row + 8 * i;
            sa_rows[i] = a_scales + static_cast<size_t>(row < shape.m ? row : 0) * v.groups;
        }
        float acc[4][COLUMNS / 4];  // [row index][2 * column pair + element]
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < COLUMNS / 4; ++j) acc[i][j] = 0.0f;
        __half2 sa_next[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) sa_next[i] = __ldg(reinterpret_cast<const __half2 *>(sa_rows[i]));
        for (int ks = 0; ks < v.k_stages && alive; ++ks, ++iteration) {
            const int s = iteration % STAGES;
            const uint32_t phase = (iteration / STAGES) & 1;
            float2 sa_pair[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                sa_pair[i] = __half22float2(sa_next[i]);
                if (ks + 1 < v.k_stages) sa_next[i] = __ldg(reinterpret_cast<const __half2 *>(sa_rows[i] + 2 * ks + 2));
            }
            if (!mbarrier_wait_warp(&v.scale_ready[s], phase, &g_status, STATUS_WAIT_READY | 0x5000 | s, lane)) { alive = false; break; }
            const float *sw_stage = v.sw_tile + s * 2 * BN + slice * COLUMNS + pair_column;
#pragma unroll
            for (int gl = 0; gl < 2; ++gl, ++group_count) {
                const uint32_t buffer = group_count % BUFFERS;
                float sa[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) sa[i] = gl == 0 ? sa_pair[i].x : sa_pair[i].y;
                const float *sw_group = sw_stage + gl * BN;
#pragma unroll
                for (int b = 0; b < BATCHES; ++b) {
                    uint32_t(&current)[32] = set[DOUBLE_BUFFER ? (b & 1) : 0];
                    uint32_t(&following)[32] = set[DOUBLE_BUFFER ? ((b + 1) & 1) : 0];
                    tmem_load_wait();  // `current` has landed; nothing else is in flight
                    const bool last_batch = b == BATCHES - 1;
                    const uint32_t next_group = group_count + (last_batch ? 1 : 0);
                    const bool has_next = next_group < total_groups;
                    bool issued = false;
                    if (last_batch) {
                        // every dot of this buffer is in registers: hand it back to the leader's MMA thread
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbarrier_arrive_cluster(leader_dot_empty + buffer * 8);
                        if (DOUBLE_BUFFER && has_next) issued = issue(next_group, 0, following, false);  // only if its dots are already there
                    } else if (DOUBLE_BUFFER) {
                        issued = issue(group_count, b + 1, following, true);
                    }
                    if (DUMP_DOTS) {
                        const int group = ks * 2 + gl;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int row = m0 + fragment_row + 8 * i;
#pragma unroll
                            for (int x = 0; x < 4; ++x)
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int col = n0 + b * 32 + 8 * x + pair_column + e;
                                    if (row < shape.m && col < shape.n)
                                        dots_out[(static_cast<size_t>(row) * shape.n + col) * v.groups + group] =
                                            static_cast<int32_t>(__uint_as_float(current[16 * (i >> 1) + 4 * x + 2 * (i & 1) + e]));
                                }
                        }
                    }
                    if (!(shape.ablate & 2)) {
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            // scalar FMUL + FFMA: as fast on the fp32 pipe as the packed f32x2 forms and free of
                            // their 64-bit register-pair constraints; the eight scale products come first
                            const float2 sw = *reinterpret_cast<const float2 *>(sw_group + b * 32 + 8 * x);
                            float product[4][2];
#pragma unroll
                            for (int i = 0; i < 4; ++i) product[i][0] = sa[i] * sw.x, product[i][1] = sa[i] * sw.y;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int r = 16 * (i >> 1) + 4 * x + 2 * (i & 1);
                                const int c = 2 * (b * 4 + x);
                                acc[i][c] = fmaf(__uint_as_float(current[r]), product[i][0], acc[i][c]);
                                acc[i][c + 1] = fmaf(__uint_as_float(current[r + 1]), product[i][1], acc[i][c + 1]);
                            }
                        }
                    }
                    if (last_batch) {
                        if (has_next && !issued && alive) issue(next_group, 0, following, true);
                    } else if (!DOUBLE_BUFFER) {
                        issue(group_count, b + 1, following, true);
                    }
                }
                if (!alive) break;
            }
            if (alive) {
                __syncwarp();
                if (lane == 0) mbarrier_arrive(&v.empty[s]);  // done reading this stage's sw
            }
        }
        if (!alive) break;
        if (shape.ablate & 4) continue;
        // y: per row 16 pairs of adjacent columns, 8 columns apart
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = m0 + fragment_row + 8 * i;
            if (row >= shape.m) continue;
#pragma unroll
            for (int j = 0; j < COLUMNS / 8; ++j) {
                const int col = n0 + 8 * j + pair_column;
                if (col >= shape.n) continue;
                float lo = acc[i][2 * j], hi = acc[i][2 * j + 1];
                if (bias != nullptr) {
                    const float2 add = __ldg(reinterpret_cast<const float2 *>(bias + col));
                    lo += add.x, hi += add.y;
                }
                if (shape.y_is_half)
                    *reinterpret_cast<__half2 *>(static_cast<__half *>(y) + static_cast<size_t>(row) * shape.ldy + col) = __floats2half2_rn(lo, hi);
                else
                    *reinterpret_cast<float2 *>(static_cast<float *>(y) + static_cast<size_t>(row) * shape.ldy + col) = make_float2(lo, hi);
            }
        }
    }
    tmem_load_wait();  // nothing of this warp may still be in flight at teardown
}

template <bool DUMP_DOTS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
            const __half *__restrict__ a_scales, const __half *__restrict__ w_scales,
            const float *__restrict__ bias, void *__restrict__ y, int32_t *__restrict__ dots_out,
            const GemmShape shape) {
    extern __shared__ uint8_t smem_raw[];
    // the same offsets in both CTAs: the dynamic shared window starts at the same address in each
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tile_a = smem;
    uint8_t *tile_b = tile_a + STAGES * A_BYTES;
    float *sw_tile = reinterpret_cast<float *>(tile_b + STAGES * B_BYTES);
    __half2 *sw_ring = reinterpret_cast<__half2 *>(reinterpret_cast<uint8_t *>(sw_tile) + STAGES * SCALE_BYTES);
    uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sw_ring) + RING_BYTES);
    uint64_t *scale_ready = full + STAGES;
    uint64_t *empty = scale_ready + STAGES;
    uint64_t *dot_full = empty + STAGES;
    uint64_t *dot_empty = dot_full + BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(dot_empty + BUFFERS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();  // 0 = leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (shape.m + 2 * BM - 1) / (2 * BM), tiles_n = (shape.n + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n, k_stages = shape.k / STAGE_K, groups = shape.k / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full[s], 1);                 // the leader's is the one in use
            mbarrier_init(&scale_ready[s], SCALE_WARPS);
            mbarrier_init(&empty[s], 1 + FOLD_WARPS);   // pair commit + this CTA's fold warps
        }
        for (int b = 0; b < BUFFERS; ++b) {
            mbarrier_init(&dot_full[b], 1);             // pair commit
            mbarrier_init(&dot_empty[b], 2 * FOLD_WARPS);  // the leader's: fold warps of both CTAs
        }
        fence_barrier_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(tmem_slot, BUFFERS * BN);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before anything arrives on them from the other side
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const View view = {sw_tile, sw_ring, scale_ready, empty, dot_full, dot_empty, tmem_base, cta,
                       pair, pairs, tiles, tiles_m, k_stages, groups};

    if (warp < FOLD_WARP0) {
      setmaxnreg_dec<CONTROL_REGISTERS>();
      if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_w);
            uint32_t iteration = 0;
            bool alive = true;
            for (int tile = pair; tile < tiles && alive; tile += pairs) {
                const int m0 = (tile % tiles_m) * 2 * BM + cta * BM, n0 = (tile / tiles_m) * BN + cta * (BN / 2);
                for (int ks = 0; ks < k_stages; ++ks, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x5000 | s)) { alive = false; break; }
                    // the leader expects the bytes of both CTAs' loads on its barrier
                    if (cta == 0) mbarrier_arrive_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
                    tma_load_2d_pair(tile_a + s * A_BYTES, &map_a, &full[s], ks * STAGE_K, m0);
                    tma_load_2d_pair(tile_b + s * B_BYTES, &map_w, &full[s], ks * STAGE_K, n0);
                }
            }
        }
      } else if (warp == MMA_WARP) {
        if (lane == 0 && cta == 0) {
            constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * BM, BN);
            uint32_t iteration = 0, group_count = 0;
            bool alive = true;
            for (int tile = pair; tile < tiles && alive; tile += pairs) {
                for (int ks = 0; ks < k_stages && alive; ++ks, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&full[s], phase, &g_status, STATUS_WAIT_FULL | 0x5000 | s)) { alive = false; break; }
                    const uint32_t a_address = smem_u32(tile_a + s * A_BYTES);
                    const uint32_t b_address = smem_u32(tile_b + s * B_BYTES);
#pragma unroll
                    for (int gl = 0; gl < 2; ++gl, ++group_count) {
                        const uint32_t buffer = group_count % BUFFERS, buffer_phase = (group_count / BUFFERS) & 1;
                        if (!mbarrier_wait(&dot_empty[buffer], buffer_phase ^ 1, &g_status, STATUS_WAIT_TMEM_EMPTY | 0x5000 | buffer)) { alive = false; break; }
                        tcgen05_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 2; ++kk)
                            if (!(shape.ablate & 16))
                                umma_f8_pair(tmem_base + buffer * BN, umma_desc_k_sw128(a_address + gl * 64 + kk * 32),
                                             umma_desc_k_sw128(b_address + gl * 64 + kk * 32), idesc, kk);
                        tcgen05_commit_pair(&dot_full[buffer]);
                    }
                    if (alive) tcgen05_commit_pair(&empty[s]);
                }
            }
        }
      } else {
        scale_role(view, w_scales, shape, static_cast<int>(threadIdx.x) - SCALE_WARP0 * 32, lane);
      }
    } else {
        setmaxnreg_inc<FOLD_REGISTERS>();
        fold_role<DUMP_DOTS>(view, a_scales, bias, y, dots_out, shape, warp, lane);
    }

    tcgen05_fence_before();
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t *>(&g_status) != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let bulk copies already issued land
    }
    __syncwarp();
    cluster_sync();  // neither CTA may leave while the other can still reach its shared memory or barriers
    if (warp == MMA_WARP) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, BUFFERS * BN);
    }
}

}  // namespace w4a4_pair
}  // namespace qi
