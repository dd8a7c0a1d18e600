// W4A16 g64 GEMV for 1..8 activation rows (the adaLN modulation linears run at M = 1):
// y[b,n] = x_fp16[b,:] . W^[n,:] (+ bias[n]), W^ as in w4a16_gemm.cuh, fp32 accumulation.
// Same operator as w4a16_gemm_kernel of the reference (qwen_image_cuda/cuda/gemm.cu:191-268)
// without its padding of the rows to 128.
//
// HBM-bound: every weight byte is read once with 16-byte loads. A warp owns 16 weight rows
// and a slice of K; lane (r, q) = (lane / 4, lane % 4) streams the 32 code bytes of one
// 64-group of rows r and r + 8 per step, unpacks them with the half2 fused multiply-add of
// the GEMM, and feeds them as the A operand of mma.sync.m16n8k16 (fp32 accumulate) whose B
// operand carries up to 8 activation rows. The order of k inside an MMA is free as long as
// both operands agree, so no shuffle is needed. The K slices of a block are summed through
// shared memory in a fixed order (deterministic split-K).
#pragma once
#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace w4a16 {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_AHEAD = 3;  // steps whose loads are in flight together

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One byte (two nibbles) -> half2 (even input, odd input) of dequantised weights.
__device__ __forceinline__ uint32_t unpack_byte(uint32_t word, int byte, __half2 scale2, __half2 minimum2) {
    const __half2 offsets = __halves2half2(__ushort_as_half(0x6400), __ushort_as_half(0x5400));
    const uint32_t spread = __byte_perm(word, 0u, 0x4040u + 0x0101u * byte);
    uint32_t magic = (spread & 0x00F0000Fu) | 0x54006400u;
    const __half2 weight = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&magic), offsets), scale2, minimum2);
    return *reinterpret_cast<const uint32_t *>(&weight);
}

// k_splits * row_tiles == GEMV_WARPS. Block b owns weight rows [16 * row_tiles * b, ...).
__global__ void __launch_bounds__(GEMV_THREADS, 2)
gemv_kernel(const __half *__restrict__ x, const uint8_t *__restrict__ codes, const __half *__restrict__ scales,
            const __half *__restrict__ minimums, const float *__restrict__ bias, void *__restrict__ y,
            int m, int n, int k, long long ldy, int y_is_half, int k_splits) {
    __shared__ float partial[GEMV_WARPS][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, q = lane & 3;
    const int row_tiles = GEMV_WARPS / k_splits;
    const int k_split = warp % k_splits, row_tile = warp / k_splits;
    const int n0 = (blockIdx.x * row_tiles + row_tile) * 16;
    const int groups = k / 64, quads = (groups + 3) / 4;
    const bool rows_inside = n0 < n;  // n is a multiple of 16

    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (rows_inside) {
        const size_t row_a = static_cast<size_t>(n0 + r), row_b = row_a + 8;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const __half nothing = __ushort_as_half(0);
        // Latency, not arithmetic, is what this kernel pays for: a warp has only a few steps, and a step
        // that waits for its own loads costs a full trip to HBM. So the loads of up to GEMV_AHEAD steps
        // (2 KB of codes per warp and step) are all issued before the first one is used.
        for (int quad0 = k_split; quad0 < quads; quad0 += k_splits * GEMV_AHEAD) {
            uint4 code_a[GEMV_AHEAD][2], code_b[GEMV_AHEAD][2];
            __half scale_a[GEMV_AHEAD], minimum_a[GEMV_AHEAD], scale_b[GEMV_AHEAD], minimum_b[GEMV_AHEAD];
#pragma unroll
            for (int i = 0; i < GEMV_AHEAD; ++i) {
                // every lane runs the same mma.sync; a lane past a ragged end feeds zeros
                const int g = (quad0 + i * k_splits) * 4 + q;
                const bool valid = g < groups;
                const uint4 *pa = reinterpret_cast<const uint4 *>(codes + row_a * (k / 2) + g * 32);
                const uint4 *pb = reinterpret_cast<const uint4 *>(codes + row_b * (k / 2) + g * 32);
                code_a[i][0] = valid ? __ldg(pa) : zero, code_a[i][1] = valid ? __ldg(pa + 1) : zero;
                code_b[i][0] = valid ? __ldg(pb) : zero, code_b[i][1] = valid ? __ldg(pb + 1) : zero;
                scale_a[i] = valid ? __ldg(scales + row_a * groups + g) : nothing;
                minimum_a[i] = valid ? __ldg(minimums + row_a * groups + g) : nothing;
                scale_b[i] = valid ? __ldg(scales + row_b * groups + g) : nothing;
                minimum_b[i] = valid ? __ldg(minimums + row_b * groups + g) : nothing;
            }
#pragma unroll
            for (int i = 0; i < GEMV_AHEAD; ++i) {
                const int g = (quad0 + i * k_splits) * 4 + q;
                if ((quad0 + i * k_splits) >= quads) break;  // uniform over the warp
                const bool valid = g < groups;
                const __half2 sa = __half2half2(scale_a[i]), ma = __half2half2(minimum_a[i]);
                const __half2 sb = __half2half2(scale_b[i]), mb = __half2half2(minimum_b[i]);
                const uint32_t wa[8] = {code_a[i][0].x, code_a[i][0].y, code_a[i][0].z, code_a[i][0].w,
                                        code_a[i][1].x, code_a[i][1].y, code_a[i][1].z, code_a[i][1].w};
                const uint32_t wb[8] = {code_b[i][0].x, code_b[i][0].y, code_b[i][0].z, code_b[i][0].w,
                                        code_b[i][1].x, code_b[i][1].y, code_b[i][1].z, code_b[i][1].w};
                // activation row (lane / 4) supplies the B operand for the same 64 inputs
                const uint4 *px = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(r) * k + g * 64);
                const bool has_x = valid && r < m;
#pragma unroll
                for (int w = 0; w < 8; ++w) {  // 8 inputs (4 bytes of each row) per word, two MMA steps
                    const uint4 xv = has_x ? __ldg(px + w) : zero;
                    uint32_t a[4];
                    a[0] = unpack_byte(wa[w], 0, sa, ma), a[1] = unpack_byte(wb[w], 0, sb, mb);
                    a[2] = unpack_byte(wa[w], 1, sa, ma), a[3] = unpack_byte(wb[w], 1, sb, mb);
                    mma_m16n8k16(c, a, xv.x, xv.y);
                    a[0] = unpack_byte(wa[w], 2, sa, ma), a[1] = unpack_byte(wb[w], 2, sb, mb);
                    a[2] = unpack_byte(wa[w], 3, sa, ma), a[3] = unpack_byte(wb[w], 3, sb, mb);
                    mma_m16n8k16(c, a, xv.z, xv.w);
                }
            }
        }
    }
    // c[0], c[1]: weight row r, activation rows 2q, 2q+1; c[2], c[3]: weight row r + 8
    partial[warp][r][2 * q] = c[0], partial[warp][r][2 * q + 1] = c[1];
    partial[warp][r + 8][2 * q] = c[2], partial[warp][r + 8][2 * q + 1] = c[3];
    __syncthreads();
    // fixed-order sum over the K slices: thread -> (row tile, weight row, activation row)
    for (int item = threadIdx.x; item < row_tiles * 16 * 8; item += GEMV_THREADS) {
        const int tile = item / 128, row = (item / 8) % 16, b = item % 8;
        const int out_row = (blockIdx.x * row_tiles + tile) * 16 + row;
        if (b < m && out_row < n) {
            float total = 0.0f;
            for (int s = 0; s < k_splits; ++s) total += partial[tile * k_splits + s][row][b];
            if (bias != nullptr) total += __ldg(bias + out_row);
            if (y_is_half) static_cast<__half *>(y)[static_cast<size_t>(b) * ldy + out_row] = __float2half_rn(total);
            else static_cast<float *>(y)[static_cast<size_t>(b) * ldy + out_row] = total;
        }
    }
}

}  // namespace w4a16
}  // namespace qi
