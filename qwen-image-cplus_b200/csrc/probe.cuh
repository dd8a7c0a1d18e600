// Measures what the tensor cores of this GPU deliver when nothing else is in the way: every SM issues
// dense tcgen05.mma instructions (M = 128, N = 256, one instruction = 128 x 256 x K multiply-adds) on
// operands that stay in shared memory, into accumulators that stay in TMEM. The bench uses the figure
// as the denominator of its tensor rooflines, since no 8-bit peak is published for a given board, clock
// and power limit. Same bounded waits as the GEMM kernels.
#pragma once
#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace probe {

constexpr int THREADS = 128;
constexpr int OPERAND_BYTES = 2 * 32768;  // A: 128 rows, B: 256 rows of 128 bytes, swizzled layout, all zero
constexpr int SMEM_BYTES = OPERAND_BYTES + 2048;
constexpr int BATCH = 64;                 // instructions between commits

// kind: 0 = f16 (K = 16), 1 = e4m3 (K = 32), 2 = s8 (K = 32)
template <int KIND>
__global__ void __launch_bounds__(THREADS, 1) mma_rate_kernel(int batches) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_slot;
    __shared__ uint64_t done;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < OPERAND_BYTES / 4; i += THREADS) reinterpret_cast<uint32_t *>(smem)[i] = 0;
    if (threadIdx.x == 0) {
        mbarrier_init(&done, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 32) {
        const uint32_t a = smem_u32(smem), b = smem_u32(smem + 32768);
        constexpr uint32_t idesc = KIND == 0 ? umma_idesc_f16_f32(128, 256) : KIND == 1 ? umma_idesc_e4m3_f32(128, 256)
                                                                                      : umma_idesc_s8_s32(128, 256);
        for (int batch = 0; batch < batches; ++batch) {
#pragma unroll 4
            for (int i = 0; i < BATCH; ++i) {
                const uint32_t offset = (i & 3) * 32;                 // the four K steps of a 128-byte row
                const uint32_t accumulator = tmem_base + (i & 1) * 256;  // two accumulators in turn
                if (KIND == 0) umma_f16(accumulator, umma_desc_k_sw128(a + offset), umma_desc_k_sw128(b + offset), idesc, 1);
                if (KIND == 1) umma_f8(accumulator, umma_desc_k_sw128(a + offset), umma_desc_k_sw128(b + offset), idesc, 1);
                if (KIND == 2) umma_i8(accumulator, umma_desc_k_sw128(a + offset), umma_desc_k_sw128(b + offset), idesc, 1);
            }
            tcgen05_commit(&done);
            if (!mbarrier_wait(&done, batch & 1, &g_status, STATUS_WAIT_TMEM_FULL | 0x9000)) break;
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// A wait that nothing ends: one thread waits on an mbarrier nobody arrives on until `limit_ns` have passed, then
// does what every wait of this library does when it runs out of time: records the code and returns. Lets a test
// see the status path (code set, read clears it, the next launch is healthy) without anything going wrong.
__global__ void __launch_bounds__(32, 1) wait_timeout_kernel(unsigned long long limit_ns) {
    __shared__ uint64_t never;
    if (threadIdx.x == 0) {
        mbarrier_init(&never, 1);
        fence_barrier_init();
        mbarrier_wait_spin(&never, 0, &g_status, STATUS_WAIT_FULL | 0xA000, 0, limit_ns);
    }
}

}  // namespace probe
}  // namespace qi
