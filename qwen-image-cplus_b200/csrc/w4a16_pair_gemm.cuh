// W4A16 g64 dequant-GEMM on PAIRS of CTAs (thread-block cluster of two, tcgen05 cta_group::2):
// one 256 x 256 output tile per pair. Same operator and unpacking as w4a16_gemm.cuh
// (reference: qwen_image_cuda/cuda/gemm.cu:191-268).
//
// Each CTA loads its own 128 rows of x and the packed codes of HALF of the tile's 256 weight rows,
// unpacks those 128 rows to fp16 in its own shared memory, and the leader's MMA (M = 256 across the
// pair, N = 256, K = 16) reads both halves. Compared with a 256 x 256 tile on one CTA this halves
// the unpacking work per CTA, leaves 256 TMEM columns per accumulator so that two fit (the epilogue
// of one tile overlaps the main loop of the next), and puts 74 tiles in a wave instead of 148 half
// as often full.
//
//   warp 0     TMA: own x rows (completion counted on the LEADER's barrier) and own code rows (own barrier)
//   warps 8-23 unpack own code rows, two groups of eight warps taking the K blocks in turn (measured on the block's
//              four shapes at M = 4096: 1081 -> 1127 TFLOP/s against one group; same bits); when done, arrive on the
//              LEADER's `ready` barrier
//   warp 1     leader only: 4 tcgen05.mma.cta_group::2 kind::f16 per K block; commits arrive in both CTAs
//   warps 4-7  epilogue of this CTA's 128 rows; release the accumulator on the LEADER's barrier
#pragma once
#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace w4a16_pair {

using w4a16::unpack32;
constexpr int UNPACK_GROUPS = 2;  // groups of eight unpack warps that take the K blocks in turn
constexpr int THREADS = 256 + UNPACK_GROUPS * 256;
constexpr int BK = 64;
constexpr int BM = 128, BN = 256;  // per CTA rows; pair tile is 256 x 256, each CTA unpacks 128 weight rows
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, MMA_WARPS = 2, EPILOGUE_WARP0 = 4, UNPACK_WARP0 = 8, UNPACK_WARPS = 8;  // per group
constexpr int ACC_STAGES = 2;
constexpr int A_BYTES = BM * 128, B_BYTES = (BN / 2) * 128, C_BYTES = (BN / 2) * 32;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + C_BYTES;
constexpr int BARRIER_BYTES = 512;

template <int STAGES>
struct Tile {
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BARRIER_BYTES + 1024;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
    static_assert((4 * STAGES + 2 * ACC_STAGES + MMA_WARPS) * 8 + 8 <= BARRIER_BYTES, "barrier block");
};

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_codes,
            const __half *__restrict__ scales, const __half *__restrict__ minimums,
            const float *__restrict__ bias, void *__restrict__ y, const GemmShape shape) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + STAGES * A_BYTES;
    uint8_t *smem_c = smem_b + STAGES * B_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_c + STAGES * C_BYTES);  // own code tile
    uint64_t *a_full = full + STAGES;                                          // the leader's: both CTAs' x tiles
    uint64_t *ready = a_full + STAGES;                                         // the leader's: both CTAs' unpack warps
    uint64_t *empty = ready + STAGES;
    uint64_t *tmem_full = empty + STAGES;
    uint64_t *tmem_empty = tmem_full + ACC_STAGES;
    uint64_t *token = tmem_empty + ACC_STAGES;  // passes the turn between the two MMA-issuing threads
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(token + MMA_WARPS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();  // 0 = leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (shape.m + (2 * BM) - 1) / (2 * BM), tiles_n = (shape.n + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n, k_blocks = shape.k / BK, groups = shape.k / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full[s], 1);
            mbarrier_init(&a_full[s], 1);
            mbarrier_init(&ready[s], 2 * UNPACK_WARPS);
            mbarrier_init(&empty[s], 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbarrier_init(&tmem_full[a], k_blocks < MMA_WARPS ? k_blocks : MMA_WARPS);  // one commit per issuing thread
            mbarrier_init(&tmem_empty[a], 2 * 4);
        }
        for (int t = 0; t < MMA_WARPS; ++t) mbarrier_init(&token[t], 1);
        fence_barrier_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(tmem_slot, (ACC_STAGES * BN));
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before anything arrives on them from the other side
    tcgen05_fence_after();
    const uint32_t leader_ready = map_to_cta(smem_u32(ready), 0), leader_tmem_empty = map_to_cta(smem_u32(tmem_empty), 0);
    const uint32_t tmem_base = *tmem_slot;

    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            prefetch_tensormap(&map_x);
            prefetch_tensormap(&map_codes);
            uint32_t iteration = 0;
            bool alive = true;
            for (int tile = pair; tile < tiles && alive; tile += pairs) {
                const int m0 = (tile % tiles_m) * (2 * BM) + cta * BM, n0 = (tile / tiles_m) * BN + cta * (BN / 2);
                for (int kb = 0; kb < k_blocks; ++kb, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x7000 | s)) { alive = false; break; }
                    if (cta == 0) mbarrier_arrive_expect_tx(&a_full[s], 2 * A_BYTES);  // both CTAs' x tiles
                    mbarrier_arrive_expect_tx(&full[s], C_BYTES);
                    tma_load_2d_pair(smem_a + s * A_BYTES, &map_x, &a_full[s], kb * BK, m0);
                    tma_load_2d(smem_c + s * C_BYTES, &map_codes, &full[s], kb * (BK / 2), n0);
                }
            }
        }
    } else if (warp >= MMA_WARP && warp < MMA_WARP + MMA_WARPS) {
        // Two threads in two warps of the leader issue the MMAs, K block by K block in turn. A tcgen05.commit
        // holds up the later tcgen05 instructions of the thread that issued it for about 440 cycles, as long
        // as the 512 tensor cycles of a K block here: one thread alone leaves bubbles, and the other thread's
        // instructions are not held up. A token passed between the two keeps the MMAs in K order, so the
        // accumulation order - and every bit of y - is fixed.
        if (lane == 0 && cta == 0) {
            constexpr uint32_t idesc = umma_idesc_f16_f32(2 * BM, BN);
            const uint32_t mine = warp - MMA_WARP;
            uint32_t iteration = mine, tile_count = 0;
            int kb = mine, tile = pair;
            while (true) {
                while (kb >= k_blocks) {
                    kb -= k_blocks;
                    tile += pairs;
                    ++tile_count;
                }
                if (tile >= tiles) break;
                const uint32_t acc = tile_count % ACC_STAGES, acc_phase = (tile_count / ACC_STAGES) & 1;
                const uint32_t tmem_acc = tmem_base + acc * BN;
                const int s = iteration % STAGES;
                const uint32_t phase = (iteration / STAGES) & 1;
                if (!mbarrier_wait(&a_full[s], phase, &g_status, STATUS_WAIT_FULL | 0x7000 | s) ||
                    !mbarrier_wait(&ready[s], phase, &g_status, STATUS_WAIT_READY | 0x7000 | s))
                    break;
                // the other thread has issued K block `iteration - 1` (thread 0 starts with the token)
                const uint32_t round = (iteration / MMA_WARPS) & 1;
                if (!mbarrier_wait(&token[mine], mine == 0 ? round ^ 1 : round, &g_status, STATUS_WAIT_READY | 0x7200 | mine)) break;
                if (kb == 0 && !mbarrier_wait(&tmem_empty[acc], acc_phase ^ 1, &g_status, STATUS_WAIT_TMEM_EMPTY | 0x7000 | acc)) break;
                tcgen05_fence_after();
                const uint32_t a_address = smem_u32(smem_a + s * A_BYTES);
                const uint32_t b_address = smem_u32(smem_b + s * B_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)
                    umma_f16_pair(tmem_acc, umma_desc_k_sw128(a_address + kk * 32), umma_desc_k_sw128(b_address + kk * 32),
                                  idesc, (kb | kk) != 0 ? 1u : 0u);
                mbarrier_arrive(&token[mine ^ 1]);
                tcgen05_commit_pair(&empty[s]);
                // the last K block of each thread closes the tile: together the commits cover every MMA of the tile
                if (kb + MMA_WARPS >= k_blocks) tcgen05_commit_pair(&tmem_full[acc]);
                iteration += MMA_WARPS;
                kb += MMA_WARPS;
            }
        }
    } else if (warp >= UNPACK_WARP0) {
        // Eight warps unpack one K block (a thread: half a weight row, 32 codes); with more than one group of eight
        // the groups take the K blocks in turn, so that one group's waits and fences overlap the other's arithmetic.
        const int unpacker = threadIdx.x - UNPACK_WARP0 * 32;
        const int d = unpacker & 255, group = unpacker >> 8;
        const int half_row = d & 1, local_row = d >> 1;
        uint32_t iteration = group;
        int kb = group, tile = pair;
        int row_global = (tile / tiles_m) * BN + cta * (BN / 2) + local_row;
        while (true) {
            if (kb >= k_blocks) {
                do {
                    kb -= k_blocks;
                    tile += pairs;
                } while (kb >= k_blocks);
                row_global = (tile / tiles_m) * BN + cta * (BN / 2) + local_row;
            }
            if (tile >= tiles) break;
            const bool inside = row_global < shape.n;
            const __half scale = inside ? __ldg(scales + static_cast<size_t>(row_global) * groups + kb) : __ushort_as_half(0);
            const __half minimum = inside ? __ldg(minimums + static_cast<size_t>(row_global) * groups + kb) : __ushort_as_half(0);
            const int s = iteration % STAGES;
            const uint32_t phase = (iteration / STAGES) & 1;
            if (!mbarrier_wait_warp(&full[s], phase, &g_status, STATUS_WAIT_FULL | 0x7100 | s, lane)) break;
            const uint8_t *codes_tile = smem_c + s * C_BYTES;
            uint8_t *b_tile = smem_b + s * B_BYTES;
            const uint4 packed = *reinterpret_cast<const uint4 *>(codes_tile + local_row * 32 + half_row * 16);
            uint4 out[4];
            unpack32(packed, __half2half2(scale), __half2half2(minimum), out);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4 *>(b_tile + local_row * 128 + (((half_row * 4 + j) ^ (local_row & 7)) << 4)) = out[j];
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbarrier_arrive_cluster(leader_ready + s * 8);
            iteration += UNPACK_GROUPS;
            kb += UNPACK_GROUPS;
        }
    } else if (warp >= EPILOGUE_WARP0 && warp < EPILOGUE_WARP0 + 4) {
        const int quadrant = warp & 3;  // TMEM lanes 32*quadrant .. +31 belong to this warp
        uint32_t tile_count = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++tile_count) {
            const int m0 = (tile % tiles_m) * (2 * BM) + cta * BM, n0 = (tile / tiles_m) * BN;
            const uint32_t acc = tile_count % ACC_STAGES, acc_phase = (tile_count / ACC_STAGES) & 1;
            if (!mbarrier_wait_warp(&tmem_full[acc], acc_phase, &g_status, STATUS_WAIT_TMEM_FULL | 0x7000 | acc, lane)) break;
            tcgen05_fence_after();
            {
                const int row = m0 + quadrant * 32 + lane;
                const uint32_t tmem_row = tmem_base + acc * BN + (static_cast<uint32_t>(quadrant * 32) << 16);
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
            if (lane == 0) mbarrier_arrive_cluster(leader_tmem_empty + acc * 8);
        }
    }

    // teardown: nothing of this CTA may still be in flight when TMEM and shared memory go away
    tcgen05_fence_before();
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t *>(&g_status) != 0) {
        // a wait gave up: let bulk copies that were already issued land before the CTA exits
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    __syncwarp();
    cluster_sync();  // neither CTA may leave while the other can still reach its shared memory or barriers
    if (warp == MMA_WARP) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, (ACC_STAGES * BN));
    }
}

}  // namespace w4a16_pair
}  // namespace qi
