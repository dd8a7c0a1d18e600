// W4A4 (H256, g64) GEMM for sm_100a:
//   y[m,n] = sum_g fma((float)dot_g[m,n], sa[m,g] * sw[n,g], y[m,n])   (+ bias[n]),  g ascending,
//   dot_g[m,n] = exact int32 dot of the 64 signed 4-bit codes of group g.
// Replaces w4a4_gemm_kernel of the reference (qwen_image_cuda/cuda/gemm.cu:65-189) and keeps its
// arithmetic: exact integer group dots, one fp32 fused multiply-add per group in the same order.
//
// Layout in HBM (row-major, caller-owned): a_codes [m,k/2], w_codes [n,k/2] bytes, even input in
// the low nibble, two's complement -7..7; a_scales [m,k/64], w_scales [n,k/64] fp16; y [m,ldy].
//
// tcgen05 has no 4-bit integer MMA, so codes are widened to int8 in shared memory. A nibble
// moved to the top of its byte is the int8 value 16*code (no sign extension needed); with both
// operands widened this way the tensor core returns 256*dot, which is undone exactly by
// scaling sa by 2^-8. Even and odd nibbles of a word go to two separate words, i.e. the k
// order inside every 8 inputs becomes 0,2,4,6,1,3,5,7 for both operands alike, which leaves the
// dot product unchanged.
//
// One persistent CTA per SM walks 128 x BN output tiles; a shared-memory stage holds 128
// inputs (two groups):
//   warp 0      TMA: packed A and B code tiles
//   warps 4-7   widen both tiles into the 128-byte-swizzled K-major int8 layout; stage sw as fp32
//   warp 1      one thread issues, per group, two tcgen05.mma kind::i8 (K = 32) into one of two
//               TMEM buffers of BN int32 columns and commits it
//   warps 8-15  fold: tcgen05.ld the group's dots, fp32 fused multiply-add into register
//               accumulators (thread = one row x BN/2 columns), release the TMEM buffer; after
//               the last group add bias and store y
#pragma once
#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace w4a4 {

constexpr int THREADS = 512;
constexpr int STAGE_K = 128;  // int8 inputs per swizzle row = two 64-groups
constexpr int PRODUCER_WARP = 0, MMA_WARP = 1, WIDEN_WARP0 = 4, WIDEN_WARPS = 4, FOLD_WARP0 = 8, FOLD_WARPS = 8;

// setmaxnreg can only hand out what the launch allocated: 65536 / 512 = 128 registers per thread.
// Asking for more than that pool blocks the warpgroup for ever, so the split is checked here.
constexpr int LAUNCH_REGISTERS = 128, CONTROL_REGISTERS = 56, WIDEN_REGISTERS = 80, FOLD_REGISTERS = 184;
static_assert(128 * (CONTROL_REGISTERS + WIDEN_REGISTERS + 2 * FOLD_REGISTERS) <= THREADS * LAUNCH_REGISTERS,
              "setmaxnreg.inc would wait for registers that do not exist");

template <int BN, int STAGES>
struct Tile {
    static constexpr int BM = 128;
    static constexpr int TMEM_COLUMNS = 2 * BN;  // two group-dot buffers
    static constexpr int PACKED_A_BYTES = BM * 64, PACKED_B_BYTES = BN * 64;
    static constexpr int WIDE_A_BYTES = BM * 128, WIDE_B_BYTES = BN * 128;
    static constexpr int SCALE_BYTES = 2 * BN * 4;  // sw of the two groups as fp32
    static constexpr int STAGE_BYTES = PACKED_A_BYTES + PACKED_B_BYTES + WIDE_A_BYTES + WIDE_B_BYTES + SCALE_BYTES;
    static constexpr int BARRIER_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BARRIER_BYTES + 1024;
    static_assert(TMEM_COLUMNS == 256 || TMEM_COLUMNS == 512, "TMEM allocation size");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
    static_assert((3 * STAGES + 4) * 8 + 8 <= BARRIER_BYTES, "barrier block");
};

// 32 packed nibbles -> 32 int8 values 16*code: out[0..1] = first 16 inputs, out[2..3] = next 16.
__device__ __forceinline__ void widen32(const uint4 packed, uint4 (&out)[2]) {
    const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
    uint32_t v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = (w[i] << 4) & 0xF0F0F0F0u;  // inputs 0,2,4,6 of the word
        v[2 * i + 1] = w[i] & 0xF0F0F0F0u;     // inputs 1,3,5,7
    }
    out[0] = make_uint4(v[0], v[1], v[2], v[3]);
    out[1] = make_uint4(v[4], v[5], v[6], v[7]);
}

template <int BN, int STAGES, bool DUMP_DOTS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
            const __half *__restrict__ a_scales, const __half *__restrict__ w_scales,
            const float *__restrict__ bias, void *__restrict__ y, int32_t *__restrict__ dots_out,
            const GemmShape shape) {
    using T = Tile<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *wide_a = smem;
    uint8_t *wide_b = wide_a + STAGES * T::WIDE_A_BYTES;
    uint8_t *packed_a = wide_b + STAGES * T::WIDE_B_BYTES;
    uint8_t *packed_b = packed_a + STAGES * T::PACKED_A_BYTES;
    float *sw_tile = reinterpret_cast<float *>(packed_b + STAGES * T::PACKED_B_BYTES);
    uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sw_tile) + STAGES * T::SCALE_BYTES);
    uint64_t *ready = full + STAGES;
    uint64_t *empty = ready + STAGES;
    uint64_t *dot_full = empty + STAGES;
    uint64_t *dot_empty = dot_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(dot_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (shape.m + T::BM - 1) / T::BM, tiles_n = (shape.n + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n, k_stages = shape.k / STAGE_K, groups = shape.k / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full[s], 1);
            mbarrier_init(&ready[s], WIDEN_WARPS);
            mbarrier_init(&empty[s], 1 + FOLD_WARPS);  // tensor core done with the tiles + fold done with sw
        }
        for (int b = 0; b < 2; ++b) {
            mbarrier_init(&dot_full[b], 1);
            mbarrier_init(&dot_empty[b], FOLD_WARPS);
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

    // Warpgroup 0 = control, 1 = widen, 2-3 = fold. The fold warps hold the fp32 accumulators
    // of the whole tile, so registers move to them from the other two warpgroups.
    if (warp < WIDEN_WARP0) {
      setmaxnreg_dec<CONTROL_REGISTERS>();
      if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_w);
            uint32_t iteration = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * T::BM, n0 = (tile / tiles_m) * BN;
                for (int ks = 0; ks < k_stages; ++ks, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x1000 | s)) { alive = false; break; }
                    mbarrier_arrive_expect_tx(&full[s], T::PACKED_A_BYTES + T::PACKED_B_BYTES);
                    tma_load_2d(packed_a + s * T::PACKED_A_BYTES, &map_a, &full[s], ks * 64, m0);
                    tma_load_2d(packed_b + s * T::PACKED_B_BYTES, &map_w, &full[s], ks * 64, n0);
                }
            }
        }
      } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_s8_s32(128, BN);
            uint32_t iteration = 0, group_count = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                for (int ks = 0; ks < k_stages && alive; ++ks, ++iteration) {
                    const int s = iteration % STAGES;
                    const uint32_t phase = (iteration / STAGES) & 1;
                    if (!mbarrier_wait(&ready[s], phase, &g_status, STATUS_WAIT_READY | 0x1000 | s)) { alive = false; break; }
                    const uint32_t a_address = smem_u32(wide_a + s * T::WIDE_A_BYTES);
                    const uint32_t b_address = smem_u32(wide_b + s * T::WIDE_B_BYTES);
#pragma unroll
                    for (int gl = 0; gl < 2; ++gl, ++group_count) {
                        const uint32_t buffer = group_count & 1, buffer_phase = (group_count >> 1) & 1;
                        if (!mbarrier_wait(&dot_empty[buffer], buffer_phase ^ 1, &g_status, STATUS_WAIT_TMEM_EMPTY | 0x1000 | buffer)) { alive = false; break; }
                        tcgen05_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 2; ++kk)
                            umma_i8(tmem_base + buffer * BN, umma_desc_k_sw128(a_address + gl * 64 + kk * 32),
                                    umma_desc_k_sw128(b_address + gl * 64 + kk * 32), idesc, kk);
                        tcgen05_commit(&dot_full[buffer]);
                    }
                    if (alive) tcgen05_commit(&empty[s]);
                }
            }
        }
      }
    } else if (warp < FOLD_WARP0) {
        setmaxnreg_dec<WIDEN_REGISTERS>();
        const int t = threadIdx.x - WIDEN_WARP0 * 32;  // 0..127
        uint32_t iteration = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int n0 = (tile / tiles_m) * BN;
            for (int ks = 0; ks < k_stages; ++ks, ++iteration) {
                const int s = iteration % STAGES;
                const uint32_t phase = (iteration / STAGES) & 1;
                // weight scales of the two groups of this stage, as fp32, for the fold warps
                float sw_pair[BN / 128][2];
#pragma unroll
                for (int p = 0; p < BN / 128; ++p) {
                    const int col = n0 + p * 128 + t;
                    __half2 pair = __halves2half2(__ushort_as_half(0), __ushort_as_half(0));
                    if (col < shape.n)
                        pair = __ldg(reinterpret_cast<const __half2 *>(w_scales + static_cast<size_t>(col) * groups + 2 * ks));
                    sw_pair[p][0] = __low2float(pair), sw_pair[p][1] = __high2float(pair);
                }
                if (!mbarrier_wait(&full[s], phase, &g_status, STATUS_WAIT_FULL | 0x1000 | s)) { alive = false; break; }
                float *sw_stage = sw_tile + s * 2 * BN;
#pragma unroll
                for (int p = 0; p < BN / 128; ++p) {
                    sw_stage[p * 128 + t] = sw_pair[p][0];
                    sw_stage[BN + p * 128 + t] = sw_pair[p][1];
                }
                // 16 bytes (32 nibbles) per task: task -> (row, quarter of the 64-byte packed row)
                const uint8_t *pa = packed_a + s * T::PACKED_A_BYTES;
                uint8_t *qa = wide_a + s * T::WIDE_A_BYTES;
#pragma unroll
                for (int i = 0; i < T::BM * 4 / 128; ++i) {
                    const int task = i * 128 + t, row = task >> 2, quarter = task & 3;
                    uint4 out[2];
                    widen32(*reinterpret_cast<const uint4 *>(pa + task * 16), out);
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        *reinterpret_cast<uint4 *>(qa + row * 128 + (((quarter * 2 + j) ^ (row & 7)) << 4)) = out[j];
                }
                const uint8_t *pb = packed_b + s * T::PACKED_B_BYTES;
                uint8_t *qb = wide_b + s * T::WIDE_B_BYTES;
#pragma unroll
                for (int i = 0; i < BN * 4 / 128; ++i) {
                    const int task = i * 128 + t, row = task >> 2, quarter = task & 3;
                    uint4 out[2];
                    widen32(*reinterpret_cast<const uint4 *>(pb + task * 16), out);
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        *reinterpret_cast<uint4 *>(qb + row * 128 + (((quarter * 2 + j) ^ (row & 7)) << 4)) = out[j];
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbarrier_arrive(&ready[s]);
            }
        }
    } else {
        setmaxnreg_inc<FOLD_REGISTERS>();
        constexpr int COLUMNS = BN / 2;  // per thread
        const int quadrant = warp & 3, column_half = (warp - FOLD_WARP0) >> 2;
        uint32_t iteration = 0, group_count = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * T::BM, n0 = (tile / tiles_m) * BN;
            const int row = m0 + quadrant * 32 + lane;
            const bool row_inside = row < shape.m;
            const __half *sa_row = a_scales + static_cast<size_t>(row_inside ? row : 0) * groups;
            float acc[COLUMNS];
#pragma unroll
            for (int j = 0; j < COLUMNS; ++j) acc[j] = 0.0f;
            for (int ks = 0; ks < k_stages && alive; ++ks, ++iteration) {
                const int s = iteration % STAGES;
                const uint32_t phase = (iteration / STAGES) & 1;
                const __half2 sa_pair = __ldg(reinterpret_cast<const __half2 *>(sa_row + 2 * ks));
                if (!mbarrier_wait(&ready[s], phase, &g_status, STATUS_WAIT_READY | 0x2000 | s)) { alive = false; break; }
                const float *sw_stage = sw_tile + s * 2 * BN + column_half * COLUMNS;
#pragma unroll
                for (int gl = 0; gl < 2; ++gl, ++group_count) {
                    const uint32_t buffer = group_count & 1, buffer_phase = (group_count >> 1) & 1;
                    // 2^-8 undoes the 16 x 16 of the widened operands; exact
                    const float sa = (gl == 0 ? __low2float(sa_pair) : __high2float(sa_pair)) * 0.00390625f;
                    if (!mbarrier_wait(&dot_full[buffer], buffer_phase, &g_status, STATUS_WAIT_TMEM_FULL | 0x1000 | buffer)) { alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t tmem_row = tmem_base + buffer * BN + column_half * COLUMNS + (static_cast<uint32_t>(quadrant * 32) << 16);
                    const float *sw_group = sw_stage + gl * BN;
#pragma unroll
                    for (int c = 0; c < COLUMNS / 32; ++c) {
                        uint32_t r[32];
                        tmem_load_32x32(tmem_row + c * 32, r);
                        tmem_load_wait();
                        if (c == COLUMNS / 32 - 1) {
                            // every dot of this buffer is in registers: hand it back to the tensor core
                            tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) mbarrier_arrive(&dot_empty[buffer]);
                        }
                        if (DUMP_DOTS && row_inside) {
                            const int group = ks * 2 + gl;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int col = n0 + column_half * COLUMNS + c * 32 + j;
                                if (col < shape.n)
                                    dots_out[(static_cast<size_t>(row) * shape.n + col) * groups + group] = static_cast<int32_t>(r[j]) >> 8;
                            }
                        }
                        // int32 -> fp32 without the conversion unit (it issues at a quarter of the fp32 rate):
                        // adding the bits of 1.5 * 2^23 to an integer below 2^22 in magnitude gives the float
                        // 1.5 * 2^23 + value exactly; one fp32 subtraction takes the offset away again.
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 sw4 = *reinterpret_cast<const float4 *>(sw_group + c * 32 + j);
                            const float f0 = __int_as_float(static_cast<int32_t>(r[j]) + 0x4B400000) - 12582912.0f;
                            const float f1 = __int_as_float(static_cast<int32_t>(r[j + 1]) + 0x4B400000) - 12582912.0f;
                            const float f2 = __int_as_float(static_cast<int32_t>(r[j + 2]) + 0x4B400000) - 12582912.0f;
                            const float f3 = __int_as_float(static_cast<int32_t>(r[j + 3]) + 0x4B400000) - 12582912.0f;
                            acc[c * 32 + j] = fmaf(f0, sa * sw4.x, acc[c * 32 + j]);
                            acc[c * 32 + j + 1] = fmaf(f1, sa * sw4.y, acc[c * 32 + j + 1]);
                            acc[c * 32 + j + 2] = fmaf(f2, sa * sw4.z, acc[c * 32 + j + 2]);
                            acc[c * 32 + j + 3] = fmaf(f3, sa * sw4.w, acc[c * 32 + j + 3]);
                        }
                    }
                }
                if (alive) {
                    __syncwarp();
                    if (lane == 0) mbarrier_arrive(&empty[s]);  // done reading this stage's sw
                }
            }
            if (!alive) break;
            // epilogue straight from the register accumulators
            const int col0 = n0 + column_half * COLUMNS;
            if (row_inside) {
#pragma unroll
                for (int c = 0; c < COLUMNS / 32; ++c) {
                    const int col = col0 + c * 32;
                    if (col >= shape.n) continue;
                    if (bias != nullptr) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[c * 32 + j] += __ldg(bias + col + j);
                    }
                    if (shape.y_is_half) {
                        __half *out = static_cast<__half *>(y) + static_cast<size_t>(row) * shape.ldy + col;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t h[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const __half2 pair = __floats2half2_rn(acc[c * 32 + 8 * j + 2 * i], acc[c * 32 + 8 * j + 2 * i + 1]);
                                h[i] = *reinterpret_cast<const uint32_t *>(&pair);
                            }
                            reinterpret_cast<uint4 *>(out)[j] = make_uint4(h[0], h[1], h[2], h[3]);
                        }
                    } else {
                        float *out = static_cast<float *>(y) + static_cast<size_t>(row) * shape.ldy + col;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            reinterpret_cast<float4 *>(out)[j] =
                                make_float4(acc[c * 32 + 4 * j], acc[c * 32 + 4 * j + 1], acc[c * 32 + 4 * j + 2], acc[c * 32 + 4 * j + 3]);
                    }
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
        tmem_dealloc(tmem_base, T::TMEM_COLUMNS);
    }
}

}  // namespace w4a4
}  // namespace qi
