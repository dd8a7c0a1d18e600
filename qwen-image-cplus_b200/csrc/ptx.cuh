// Thin wrappers over the sm_100a PTX this library is built from: mbarriers, TMA
// (cp.async.bulk.tensor, never multicast), tcgen05 (TMEM allocation, MMA, commit, load)
// and the proxy / thread-sync fences between them. Every wait is bounded: a wait that
// runs out records where it gave up in a status word and returns false, so that a logic
// error ends in an error code and never in a hung device.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qi {

// Status word written by a kernel that gave up on a wait (0 = healthy). The high half
// says which wait, the low half carries block / stage detail.
enum : uint32_t {
    STATUS_OK = 0,
    STATUS_WAIT_FULL = 0x00010000u,       // consumer waited for TMA data
    STATUS_WAIT_EMPTY = 0x00020000u,      // producer waited for a free smem stage
    STATUS_WAIT_READY = 0x00030000u,      // MMA warp waited for the unpacked operand
    STATUS_WAIT_TMEM_FULL = 0x00040000u,  // epilogue waited for an accumulator
    STATUS_WAIT_TMEM_EMPTY = 0x00050000u, // MMA warp waited for a drained accumulator
    STATUS_BAD_ARGUMENT = 0x00060000u,
};

// Fast spins first, then 128 ns sleeps until two seconds of wall clock have passed.
constexpr uint32_t WAIT_FAST_SPINS = 1u << 12;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    return now;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t predicate = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(predicate));
    return predicate != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------

__device__ __forceinline__ void mbarrier_init(uint64_t *barrier, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(barrier)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbarrier_arrive(uint64_t *barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(barrier)) : "memory");
}

__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint64_t *barrier, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(barrier)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint64_t *barrier, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(barrier)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait. On time-out writes `code` to *status (first writer wins) and returns false;
// also gives up as soon as another thread has reported a failure. The caller must then drain
// and leave without touching the data.
// A wait whose phase is already complete is the common case in a pipeline that runs ahead, and it
// must cost no more than the one try_wait (about 25 cycles; a loop around it triples that).
__device__ __forceinline__ bool mbarrier_wait_spin(uint64_t *barrier, uint32_t parity, uint32_t *status, uint32_t code,
                                                   uint32_t backoff_ns = 0, uint64_t limit_ns = WAIT_LIMIT_NS) {
    for (uint32_t spin = 0; spin < WAIT_FAST_SPINS; ++spin) {
        if (mbarrier_try_wait(barrier, parity)) return true;
        // A role that runs far ahead of its consumers spends its life here. Without a pause its polling
        // takes issue slots from the warps that share its scheduler (measured: a fold warp next to a
        // spinning warp fell four groups behind the others and set the pace of the whole CTA).
        if (backoff_ns != 0) __nanosleep(backoff_ns);
    }
    const uint64_t start = global_timer_ns();
    while (true) {
        if (mbarrier_try_wait(barrier, parity)) return true;
        __nanosleep(128);
        if (*reinterpret_cast<volatile uint32_t *>(status) != 0) return false;
        if (global_timer_ns() - start > limit_ns) break;
    }
    atomicCAS(status, 0u, code);
    return false;
}

__device__ __forceinline__ bool mbarrier_wait(uint64_t *barrier, uint32_t parity, uint32_t *status,
                                              uint32_t code, uint32_t backoff_ns = 0) {
    if (mbarrier_try_wait(barrier, parity)) return true;
    return mbarrier_wait_spin(barrier, parity, status, code, backoff_ns);
}

// The same for a whole converged warp. Every lane makes the first attempt (one instruction, one
// shared-memory access for the warp). Only if that fails does lane 0 poll alone while the others
// wait for it at a shuffle: 32 lanes spinning on one barrier word only multiply the traffic.
__device__ __forceinline__ bool mbarrier_wait_warp(uint64_t *barrier, uint32_t parity, uint32_t *status,
                                                   uint32_t code, int lane, uint32_t backoff_ns = 0) {
    if (__all_sync(0xffffffffu, mbarrier_try_wait(barrier, parity))) return true;
    uint32_t ok = 1;
    if (lane == 0) ok = mbarrier_wait_spin(barrier, parity, status, code, backoff_ns) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---- TMA ---------------------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load global -> shared, completion on an mbarrier of this CTA. x is the
// innermost (contiguous) coordinate in elements and must keep x * element size a multiple
// of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *smem, const CUtensorMap *map, uint64_t *barrier, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(barrier)), "r"(x), "r"(y)
        : "memory");
}

// Generic-proxy writes to shared memory become visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 -----------------------------------------------------------------------------

// One whole warp allocates `columns` (power of two, >= 32) TMEM columns; the base address
// lands in *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrives once on `barrier` when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void tcgen05_commit(uint64_t *barrier) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(barrier))
                 : "memory");
}

// Shared-memory operand descriptor for a K-major tile in the 128-byte-swizzled canonical
// layout: rows of 128 bytes, 8-row groups 1024 bytes apart, 16-byte chunk c of row r stored
// at chunk position c ^ (r % 8). `address` may point inside the first 128 bytes of a row
// to step along K.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t address) {
    uint64_t descriptor = 0;
    descriptor |= static_cast<uint64_t>((address & 0x3FFFFu) >> 4);  // start address, 16-byte units
    descriptor |= static_cast<uint64_t>(1) << 16;                    // leading byte offset (unused when swizzled)
    descriptor |= static_cast<uint64_t>(1024 >> 4) << 32;            // stride byte offset between 8-row groups
    descriptor |= static_cast<uint64_t>(1) << 46;                    // descriptor version for sm_100
    descriptor |= static_cast<uint64_t>(2) << 61;                    // layout type: 128-byte swizzle
    return descriptor;
}

// Instruction descriptors: D format, A/B formats, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32(int m, int n) {
    return (1u << 4) /* D = f32 */ | (0u << 7) /* A = f16 */ | (0u << 10) /* B = f16 */ |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__host__ __device__ constexpr uint32_t umma_idesc_s8_s32(int m, int n) {
    return (2u << 4) /* D = s32 */ | (1u << 7) /* A = s8 */ | (1u << 10) /* B = s8 */ |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(int m, int n) {
    return (1u << 4) /* D = f32 */ | (0u << 7) /* A = e4m3 */ | (0u << 10) /* B = e4m3 */ |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread. accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns; thread t gets
// lane (warp % 4) * 32 + t, register j gets column `address.column + j`.
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(address)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Warpgroup-wide register reallocation (all four warps of the warpgroup execute it).
template <uint32_t REGISTERS>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}
template <uint32_t REGISTERS>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}

// ---- packed fp32 pairs (one instruction, two IEEE-rounded results) ------------------------------

__device__ __forceinline__ uint64_t pack_f32x2(float low, float high) {
    uint64_t packed;
    asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "f"(low), "f"(high));
    return packed;
}

__device__ __forceinline__ uint64_t pack_u32x2(uint32_t low, uint32_t high) {
    uint64_t packed;
    asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "r"(low), "r"(high));
    return packed;
}

__device__ __forceinline__ void unpack_f32x2(uint64_t packed, float &low, float &high) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(packed));
}

__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// ---- cp.async (4- or 8-byte, global -> shared, per thread) --------------------------------------------

__device__ __forceinline__ void cp_async_4(void *smem, const void *global) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem)), "l"(global) : "memory");
}

__device__ __forceinline__ void cp_async_8(void *smem, const void *global) {  // both addresses 8-byte aligned
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem)), "l"(global) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int PENDING>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// ---- thread-block clusters and cta_group::2 (one MMA over a pair of CTAs) ------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

// All threads of both CTAs; orders shared-memory and barrier initialisation before remote use.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_address, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    return remote;
}

__device__ __forceinline__ void mbarrier_arrive_cluster(uint32_t cluster_address) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}

// Shared-memory addresses of the even CTA of a pair: bit 24 of a shared::cluster address is the
// rank within the pair.
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;

// TMA load whose completion bytes are counted on the pair leader's mbarrier (no multicast: each CTA
// fetches its own tile into its own shared memory).
__device__ __forceinline__ void tma_load_2d_pair(void *smem, const CUtensorMap *map, uint64_t *barrier, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(barrier) & PAIR_LEADER_MASK), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t *slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

// Arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t *barrier) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(barrier)),
                 "h"(both)
                 : "memory");
}

__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 16 TMEM lanes x 32 columns in the fragment layout of an m16n8 accumulator, repeated 4 times along
// the columns: with i = thread index, register 4x+0, 4x+1 = lane i/4, columns 8x + 2(i%4) + {0,1};
// register 4x+2, 4x+3 = lane i/4 + 8, same columns. `address` carries the first of the 16 lanes.
__device__ __forceinline__ void tmem_load_16x256_x4(uint32_t address, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_load_32x16(uint32_t address, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address)
        : "memory");
}

// 32-byte store (sm_100): a thread that owns 32 adjacent bytes of a row writes a whole sector at once.
// The address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void *address, const uint32_t (&r)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// ---- small utilities -----------------------------------------------------------------------

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace qi
