// W4A16 g64 GEMV for 1..8 activation rows, streaming form: same operator and arithmetic as w4a16_gemv.cuh
// (the reference's w4a16_gemm_kernel, qwen_image_cuda/cuda/gemm.cu:191-268, without its padding of the rows
// to 128), for matrices whose rows are short enough that 16 of them fit a shared-memory stage (K <= 4096).
//
// The older kernel loads everything a warp will need, waits, and then unpacks: on a 32 MB matrix the memory
// system idles while the SMs unpack and the SMs idle while it streams. Here a CTA walks over several tiles of
// 16 weight rows. A tile's codes, scales and minimums are three contiguous ranges of the pack (16 whole rows
// each), so one thread fetches them with three bulk asynchronous copies (cp.async.bulk, completion counted on
// an mbarrier) into a ring of stages, and the copies of the next tiles are in flight while the warps unpack
// the current one. Within a tile the eight warps split K: lane (r, q) = (lane / 4, lane % 4) takes 32 codes
// (half a group) of rows r and r + 8 per step, unpacks them, and feeds them as the A operand of
// mma.sync.m16n8k16 (fp32 accumulate) whose B operand carries up to 8 activation rows; the order of k inside
// an MMA is free as long as both operands agree. The K slices are summed through shared memory in a fixed order.
//
// Unpacking is what the SMs spend their time on (measured on 18432 x 3072: copies alone 6 us, unpacking alone
// 10 us, the tensor-core step nothing), so it is cut to three instructions per two weights. A nibble moved to
// bits 6..9 of a 16-bit lane is the fp16 denormal code * 2^-18; one half2 fused multiply-add with the scale
// times 2^18 and the minimum gives fp16(code * scale + minimum) with a single rounding, which is what the
// reference's __float2half(fmaf(code, scale, minimum)) gives whenever |w| <= 1 (gemm.cu:229-230; see
// w4a16_gemm.cuh). A word of eight nibbles yields the pairs (0,4), (1,5), (2,6), (3,7) by one shift and one
// mask each; the activations are stored once per CTA in shared memory in that order. A scale of 1/4 or more,
// whose 2^18-fold is no fp16 number, sends the warp's step down a slower path with the same pairing.
#pragma once
#include "ptx.cuh"
#include "w4a16_gemv.cuh"

namespace qi {
namespace w4a16 {

constexpr int STREAM_THREADS = 256, STREAM_WARPS = STREAM_THREADS / 32, STREAM_MAX_STAGES = 3, STREAM_ROWS = 16;
constexpr int STREAM_MAX_K = 4096;  // 16 rows of codes, scales and minimums: 36 KB per stage

__host__ __device__ constexpr int stream_stage_bytes(int k) { return STREAM_ROWS * (k / 2) + 2 * STREAM_ROWS * (k / 64) * 2; }
__host__ __device__ constexpr int stream_x_bytes(int m, int k) { return m * k * 2; }

// global -> shared, any multiple of 16 bytes, both addresses 16-byte aligned; completion on an mbarrier of this CTA
__device__ __forceinline__ void bulk_load(void *smem, const void *global, uint32_t bytes, uint64_t *barrier) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem)),
                 "l"(global), "r"(bytes), "r"(smem_u32(barrier))
                 : "memory");
}

// Eight nibbles of one row -> four half2 of dequantised weights, pairs (0,4), (1,5), (2,6), (3,7).
// scale_up = scale * 2^18 in both lanes.
__device__ __forceinline__ void unpack_word(uint32_t word, __half2 scale_up, __half2 minimum2, uint32_t (&out)[4]) {
    uint32_t moved[4] = {(word << 6) & 0x03C003C0u, (word << 2) & 0x03C003C0u, (word >> 2) & 0x03C003C0u,
                         (word >> 6) & 0x03C003C0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 weight = __hfma2(*reinterpret_cast<__half2 *>(&moved[j]), scale_up, minimum2);
        out[j] = *reinterpret_cast<const uint32_t *>(&weight);
    }
}

// The same pairs for any scale: each code as an fp16 integer, then the same fused multiply-add.
__device__ __forceinline__ void unpack_word_any_scale(uint32_t word, __half2 scale2, __half2 minimum2, uint32_t (&out)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 code = __halves2half2(__ushort2half_rn(static_cast<unsigned short>((word >> (4 * j)) & 15u)),
                                            __ushort2half_rn(static_cast<unsigned short>((word >> (4 * j + 16)) & 15u)));
        const __half2 weight = __hfma2(code, scale2, minimum2);
        out[j] = *reinterpret_cast<const uint32_t *>(&weight);
    }
}

// Several matrices of one shape for one launch: the grouped form walks the tiles of all of them as one list, so
// that the launch, the first copies and the staging of the activations are paid once. The table travels in the
// kernel's parameters (40 bytes per matrix).
constexpr int STREAM_GROUP = 64;
struct StreamItem {
    const uint8_t *codes;
    const __half *scales, *minimums;
    const float *bias;
    void *y;
};
struct StreamItems {
    StreamItem item[STREAM_GROUP];
};

// Dynamic shared memory: `stages` stages of stream_stage_bytes(k), then the activations (m * k * 2 bytes).
// GROUPED: `count` matrices [n, k] from `group`, tile t of the launch is tile t % (n / 16) of matrix t / (n / 16);
// otherwise the one matrix given by the pointer arguments.
template <bool GROUPED>
__device__ __forceinline__ void gemv_stream_body(const __half *__restrict__ x, const uint8_t *__restrict__ codes, const __half *__restrict__ scales,
                   const __half *__restrict__ minimums, const float *__restrict__ bias, void *__restrict__ y,
                   int m, int n, int k, long long ldy, int y_is_half, int stages, const StreamItems *group, int count) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    __shared__ uint64_t full[STREAM_MAX_STAGES];
    __shared__ float partial[STREAM_WARPS][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, q = lane & 3;
    const int groups = k / 64, steps = (groups + 1) / 2;  // a step: two groups, a quarter of the lanes on each half group
    const int code_bytes = STREAM_ROWS * (k / 2), scale_bytes = STREAM_ROWS * groups * 2;
    const int stage_bytes = code_bytes + 2 * scale_bytes;
    const int tiles_each = n / STREAM_ROWS, tiles = GROUPED ? tiles_each * count : tiles_each;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) mbarrier_init(&full[s], 1);
        fence_barrier_init();
    }
    // the activations, once per CTA, every eight inputs in the order (0,4,1,5,2,6,3,7) the unpacked pairs have
    uint4 *x_pairs = reinterpret_cast<uint4 *>(smem + static_cast<size_t>(stages) * stage_bytes);  // [m][k / 8]
    for (int item = threadIdx.x; item < m * (k / 8); item += STREAM_THREADS) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x) + item);
        x_pairs[item] = make_uint4(__byte_perm(v.x, v.z, 0x5410), __byte_perm(v.x, v.z, 0x7632), __byte_perm(v.y, v.w, 0x5410),
                                   __byte_perm(v.y, v.w, 0x7632));
    }
    __syncthreads();
    auto fetch = [&](int tile, int s) {  // thread 0 only
        uint8_t *stage = smem + static_cast<size_t>(s) * stage_bytes;
        const uint8_t *from_codes = codes;
        const __half *from_scales = scales, *from_minimums = minimums;
        if (GROUPED) {
            const StreamItem &item = group->item[tile / tiles_each];
            from_codes = item.codes, from_scales = item.scales, from_minimums = item.minimums;
            tile %= tiles_each;
        }
        const size_t row0 = static_cast<size_t>(tile) * STREAM_ROWS;
        mbarrier_arrive_expect_tx(&full[s], static_cast<uint32_t>(stage_bytes));
        bulk_load(stage, from_codes + row0 * (k / 2), code_bytes, &full[s]);
        bulk_load(stage + code_bytes, from_scales + row0 * groups, scale_bytes, &full[s]);
        bulk_load(stage + code_bytes + scale_bytes, from_minimums + row0 * groups, scale_bytes, &full[s]);
    };
    if (threadIdx.x == 0) {
        int tile = blockIdx.x;
        for (int s = 0; s < stages && tile < tiles; ++s, tile += gridDim.x) fetch(tile, s);
    }

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const __half nothing = __ushort_as_half(0), quarter = __float2half(0.25f), two_to_9 = __ushort_as_half(0x6000);
    const bool has_x = r < m;
    uint32_t s = 0, phase = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const bool arrived = mbarrier_wait(&full[s], phase, &g_status, STATUS_WAIT_FULL | 0xB000 | s);
        const uint8_t *stage = smem + static_cast<size_t>(s) * stage_bytes;
        const __half *stage_scales = reinterpret_cast<const __half *>(stage + code_bytes);
        const __half *stage_minimums = reinterpret_cast<const __half *>(stage + code_bytes + scale_bytes);
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (arrived) {
            for (int step = warp; step < steps; step += STREAM_WARPS) {
                const int g = 2 * step + (q >> 1), half_group = q & 1;
                const bool valid = g < groups;  // every lane runs the same mma.sync; a lane past a ragged end feeds zeros
                const int column = g * 32 + half_group * 16;  // byte offset of this lane's 32 codes in a row
                const uint4 code_a = valid ? *reinterpret_cast<const uint4 *>(stage + r * (k / 2) + column) : zero;
                const uint4 code_b = valid ? *reinterpret_cast<const uint4 *>(stage + (r + 8) * (k / 2) + column) : zero;
                const __half scale_a = valid ? stage_scales[r * groups + g] : nothing;
                const __half scale_b = valid ? stage_scales[(r + 8) * groups + g] : nothing;
                const __half2 ma = __half2half2(valid ? stage_minimums[r * groups + g] : nothing);
                const __half2 mb = __half2half2(valid ? stage_minimums[(r + 8) * groups + g] : nothing);
                const uint32_t wa[4] = {code_a.x, code_a.y, code_a.z, code_a.w};
                const uint32_t wb[4] = {code_b.x, code_b.y, code_b.z, code_b.w};
                // activation row (lane / 4) supplies the B operand for the same 32 inputs
                const uint4 *px = x_pairs + static_cast<size_t>(r) * (k / 8) + g * 8 + half_group * 4;
                const bool has_operand = has_x && valid;
                // scale * 2^18 stays an fp16 number below 1/4 (a NaN fails the test and takes the other path too)
                const bool small = __hlt(__habs(scale_a), quarter) && __hlt(__habs(scale_b), quarter);
                if (__all_sync(0xffffffffu, small)) {
                    const __half2 sa = __half2half2(__hmul(__hmul(scale_a, two_to_9), two_to_9));
                    const __half2 sb = __half2half2(__hmul(__hmul(scale_b, two_to_9), two_to_9));
#pragma unroll
                    for (int w = 0; w < 4; ++w) {  // 8 inputs of each row per word, two MMA steps
                        const uint4 xv = has_operand ? px[w] : zero;
                        uint32_t pa[4], pb[4];
                        unpack_word(wa[w], sa, ma, pa);
                        unpack_word(wb[w], sb, mb, pb);
                        const uint32_t first[4] = {pa[0], pb[0], pa[1], pb[1]}, second[4] = {pa[2], pb[2], pa[3], pb[3]};
                        mma_m16n8k16(c, first, xv.x, xv.y);
                        mma_m16n8k16(c, second, xv.z, xv.w);
                    }
                } else {
                    const __half2 sa = __half2half2(scale_a), sb = __half2half2(scale_b);
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const uint4 xv = has_operand ? px[w] : zero;
                        uint32_t pa[4], pb[4];
                        unpack_word_any_scale(wa[w], sa, ma, pa);
                        unpack_word_any_scale(wb[w], sb, mb, pb);
                        const uint32_t first[4] = {pa[0], pb[0], pa[1], pb[1]}, second[4] = {pa[2], pb[2], pa[3], pb[3]};
                        mma_m16n8k16(c, first, xv.x, xv.y);
                        mma_m16n8k16(c, second, xv.z, xv.w);
                    }
                }
            }
        }
        // c[0], c[1]: weight row r, activation rows 2q, 2q+1; c[2], c[3]: weight row r + 8
        partial[warp][r][2 * q] = c[0], partial[warp][r][2 * q + 1] = c[1];
        partial[warp][r + 8][2 * q] = c[2], partial[warp][r + 8][2 * q + 1] = c[3];
        __syncthreads();  // every warp is done with the stage, and the partial sums are complete
        if (threadIdx.x == 0) {
            const int next = tile + stages * gridDim.x;
            if (next < tiles) fetch(next, s);
        }
        if (threadIdx.x < 16 * 8) {  // fixed-order sum over the K slices: thread -> (weight row, activation row)
            const int row = threadIdx.x >> 3, b = threadIdx.x & 7;
            const float *to_bias = bias;
            void *to_y = y;
            int local_tile = tile;
            if (GROUPED) {
                const StreamItem &item = group->item[tile / tiles_each];
                to_bias = item.bias, to_y = item.y;
                local_tile = tile % tiles_each;
            }
            const int out_row = local_tile * STREAM_ROWS + row;
            if (b < m) {
                float total = 0.0f;
#pragma unroll
                for (int slice = 0; slice < STREAM_WARPS; ++slice) total += partial[slice][row][b];
                if (to_bias != nullptr) total += __ldg(to_bias + out_row);
                if (y_is_half) static_cast<__half *>(to_y)[static_cast<size_t>(b) * ldy + out_row] = __float2half_rn(total);
                else static_cast<float *>(to_y)[static_cast<size_t>(b) * ldy + out_row] = total;
            }
        }
        __syncthreads();  // the partial sums have been read before the next tile overwrites them
        if (++s == static_cast<uint32_t>(stages)) s = 0, phase ^= 1;
    }
}

__global__ void __launch_bounds__(STREAM_THREADS, 2)
gemv_stream_kernel(const __half *__restrict__ x, const uint8_t *__restrict__ codes, const __half *__restrict__ scales,
                   const __half *__restrict__ minimums, const float *__restrict__ bias, void *__restrict__ y,
                   int m, int n, int k, long long ldy, int y_is_half, int stages) {
    gemv_stream_body<false>(x, codes, scales, minimums, bias, y, m, n, k, ldy, y_is_half, stages, nullptr, 1);
}

__global__ void __launch_bounds__(STREAM_THREADS, 2)
gemv_stream_grouped_kernel(const __half *__restrict__ x, const __grid_constant__ StreamItems group, int count,
                           int m, int n, int k, long long ldy, int y_is_half, int stages) {
    gemv_stream_body<true>(x, nullptr, nullptr, nullptr, nullptr, nullptr, m, n, k, ldy, y_is_half, stages, &group, count);
}

}  // namespace w4a16
}  // namespace qi
