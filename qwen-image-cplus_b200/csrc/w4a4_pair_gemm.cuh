// W4A4 (H256, g64) GEMM on byte-wide (E4M3) codes, one 256 x 128 output tile per PAIR of CTAs
// (thread-block cluster of two, tcgen05 cta_group::2). Same operator, arithmetic and bits as
// w4a4_wide_gemm.cuh and the reference's w4a4_gemm_kernel (qwen_image_cuda/cuda/gemm.cu:65-189).
//
// Per group of 64 inputs the tensor cores leave a tile of EXACT integer dots (as fp32) in TMEM and
// the fp32 pipe folds them: y += dot * (sa * sw). That fold is two fp32 operations per output and
// group - at full tensor rate more than the fp32 pipe can do - so the kernel is built around
// keeping sixteen fold warps busy and everything else out of their way. What was measured on the
// way, and what the design does about it:
//
//   * In a pair each CTA loads its own 128 rows of A and HALF of the B rows; the MMAs (M = 256
//     across the pair) read B from both CTAs' shared memory. No TMA multicast.
//   * Warps that wait on the same barrier run in lock step: all copy dots out of TMEM at the same
//     time (queueing at the TMEM read port), then all multiply at the same time. So the tile's 128
//     columns are split into two TEAMS of 64, each a pipeline of its own: own MMAs (N = 64), own
//     two TMEM buffers, own barriers, own eight fold warps per CTA. The teams drift apart and one
//     fills the other's gaps.
//   * The fold warps set the pace (a count of their waits: the dots are ready at the first look in
//     every one of 768 groups, while the MMA threads wait for a free buffer 99 % of the time), so
//     what a fold warp does per hand-off counts: a TMEM buffer holds the dots of TWO groups (one
//     128-byte slab of K: four MMAs, one commit), which halves the looks at the barrier and the
//     hand-backs (760 -> 807 TOP/s on the block), and a look is one try_wait by every lane
//     without a vote around it (-> 823).
//   * A tcgen05.commit holds up the later tcgen05 instructions of the THREAD that issued it for
//     some 440 cycles, however deep the pipeline, but not those of other threads. So each team has
//     two issuing threads (in different warps) that take turns group by group.
//   * A fold warp copies its 32 x 32 dots of a group with one tcgen05.ld.32x32b.x32 (about 360
//     B/clk/SM with eight warps; the 16x256b fragment shape reaches 230), computes half of the
//     group's scale products while the copy is in flight, hands the buffer back and then does
//     the rest of the arithmetic from registers.
//   * A wait on a barrier whose phase is complete must cost one try_wait. A polling loop with a
//     lane-0 / shuffle wrapper around it cost 230 cycles, a try_wait with a vote about 100.
//   * Integer division costs a warp over a hundred cycles: the per-stage roles walk the
//     (tile, stage) sequence incrementally. Scales reach the fold threads as fp32 in shared memory,
//     staged by two warps with cp.async several stages ahead. The TMA has a thread of its own: when
//     it shared a warp with the scale staging, the MMA threads waited for `full` most of the time.
//   * A thread owns one output row: it stores whole 32-byte sectors (st.global.v8).
//   * A stage is four groups (256 bytes of K, two TMA boxes per operand): the per-stage hand-offs (scale
//     barrier, stage release) cost a fold warp some 270 cycles, so they are paid every fourth group.
//
// Per CTA (rank 0 = leader issues the MMAs for both), 24 warps:
//   warp 0      one thread: TMA for own A rows and own B rows
//   warps 1, 2  stage the scales (sw: the tile's 128 columns; sa: this CTA's 128 rows; four groups per stage)
//   warps 4-7   leader only, one thread each: tcgen05.mma.cta_group::2 kind::f8f6f4 (two K = 32 steps
//               per group, two groups per buffer) and the commit that arrives on both CTAs' barriers
//   warps 8-23  fold this CTA's 128 rows x 128 columns, 32 rows x 32 columns per warp
//   (warp 3 only gives up its registers: setmaxnreg works on groups of four warps)
#pragma once
#include "ptx.cuh"
#include "w4a16_gemm.cuh"

namespace qi {
namespace w4a4_pair {

// Shared-window (32-bit) forms of the barrier and load helpers for the fold warps: their loop is short on
// registers, and a generic 64-bit pointer costs two of them and an address conversion per use (measured on the
// block workload: 660 -> 731 TOP/s from this change alone).
__device__ __forceinline__ bool try_wait_u32(uint32_t barrier, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\tselp.u32 %0, 1, 0, P;\n\t}\n"
                 : "=r"(done) : "r"(barrier), "r"(parity) : "memory");
    return done != 0;
}
__device__ __noinline__ bool wait_slow_u32(uint32_t barrier, uint32_t parity, uint32_t code, uint32_t backoff_ns) {
    for (uint32_t spin = 0; spin < WAIT_FAST_SPINS; ++spin) {
        if (try_wait_u32(barrier, parity)) return true;
        if (backoff_ns != 0) __nanosleep(backoff_ns);
    }
    const uint64_t start = global_timer_ns();
    while (true) {
        if (try_wait_u32(barrier, parity)) return true;
        __nanosleep(128);
        if (*reinterpret_cast<volatile uint32_t *>(&g_status) != 0) return false;
        if (global_timer_ns() - start > WAIT_LIMIT_NS) break;
    }
    atomicCAS(&g_status, 0u, code);
    return false;
}
__device__ __forceinline__ bool wait_warp_u32(uint32_t barrier, uint32_t parity, uint32_t code, int lane, uint32_t backoff_ns) {
    if (__all_sync(0xffffffffu, try_wait_u32(barrier, parity))) return true;
    uint32_t ok = 1;
    if (lane == 0) ok = wait_slow_u32(barrier, parity, code, backoff_ns) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ ulonglong2 lds_pairs(uint32_t address) {
    ulonglong2 value;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(value.x), "=l"(value.y) : "r"(address));
    return value;
}
__device__ __forceinline__ float lds_f32(uint32_t address) {
    float value;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(value) : "r"(address));
    return value;
}
__device__ __forceinline__ void arrive_u32(uint32_t barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barrier) : "memory");
}
// The wait for a 32-register copy out of TMEM, with the registers tied to it: nothing that uses them can be
// scheduled before it, while work that does not need them may sit between the copy and the wait.
__device__ __forceinline__ void tmem_load_wait_32(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
          "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
          "+r"(r[30]), "+r"(r[31])
        :: "memory");
}

constexpr int TEAMS = 2;       // independent fold pipelines, each with its own half of the columns
constexpr int THREADS = 768;
constexpr int BM = 128;        // rows per CTA; the pair covers 256
constexpr int BN = 128;        // columns of the pair's tile; each CTA loads 64 of the B rows
constexpr int STAGE_K = 256;   // bytes (= codes) of K per pipeline stage: four groups, as two 128-byte swizzle rows
constexpr int STAGE_GROUPS = STAGE_K / 64, K_HALVES = STAGE_K / 128;
constexpr int TEAM_COLUMNS = BN / TEAMS;
constexpr int BUFFERS = 2;     // TMEM buffers per team, each the dots of TWO groups (one 128-byte slab of K): 2 x TEAM_COLUMNS columns
constexpr int BUFFER_COLUMNS = 2 * TEAM_COLUMNS;
constexpr int STAGES = 4;
constexpr int TURNS = 2;       // MMA-issuing threads per team, taking turns group by group
constexpr int PRODUCER_WARP = 0, SW_WARP = 1, SA_WARP = 2, MMA_WARP0 = 4, MMA_WARPS = TURNS * TEAMS, FOLD_WARP0 = 8, FOLD_WARPS = 16;  // warp 3 idle
static_assert(MMA_WARP0 + MMA_WARPS <= FOLD_WARP0, "the issuing threads sit in control warps");
constexpr int COLUMNS = BN / (FOLD_WARPS / 4);  // columns per fold warp: 32
// Registers live in the four schedulers' own files (16384 each), and warp w runs on scheduler w % 4:
// six warps per scheduler here, 80 registers per thread at launch. setmaxnreg moves registers
// between the warps of ONE scheduler, and it is executed by whole warpgroups (four consecutive
// warps) - hence eight control warps although three of them have nothing to do. Per scheduler
// afterwards: two control warps and four fold warps.
// A fold thread keeps 32 accumulators and 32 fetched dots.
constexpr int LAUNCH_REGISTERS = 80, CONTROL_REGISTERS = 48, FOLD_REGISTERS = 96;
static_assert(THREADS % 128 == 0 && FOLD_WARP0 % 4 == 0, "setmaxnreg is a warpgroup instruction");
static_assert(THREADS / 128 * LAUNCH_REGISTERS * 32 <= 16384, "registers of one scheduler at launch");
static_assert(FOLD_WARP0 / 4 * CONTROL_REGISTERS + FOLD_WARPS / 4 * FOLD_REGISTERS <= THREADS / 128 * LAUNCH_REGISTERS,
              "setmaxnreg.inc would wait for registers that do not exist");
// Pause between polls of the roles that run stages ahead and therefore wait most of the time: a warp that spins
// takes issue slots from the fold warps of its scheduler.
constexpr uint32_t AHEAD_BACKOFF_NS = 256;
// The fold warps and the MMA threads wait for each other group by group. Sixteen warps polling one barrier
// word with all their lanes slow down every other barrier operation of the CTA, the passing waits of the
// warps that are behind included (measured: 588 -> 660 TOP/s on the block when the waiting is done by one
// lane per warp with a pause between polls; a try_wait with a suspend-time hint instead was slower, 572).
constexpr uint32_t FOLD_BACKOFF_NS = 200, MMA_BACKOFF_NS = 64;
// Columns whose scale products sa * sw a fold thread computes while its copy of the dots out of TMEM is still in
// flight (measured on 4096 x 9216 x 3072: 0 -> 295 us, 16 -> 293 .. 288, more than 16 no better: registers).
constexpr int HOIST = 16;
constexpr int SCALE_AHEAD = 3, SCALE_RING = 4;  // stages of scales in flight; ring slots

constexpr int A_HALF_BYTES = BM * 128, B_HALF_BYTES = (BN / 2) * 128;  // one 128-byte-wide slab of a stage
constexpr int A_BYTES = K_HALVES * A_HALF_BYTES, B_BYTES = K_HALVES * B_HALF_BYTES;
constexpr int SW_BYTES = STAGE_GROUPS * BN * 4;   // fp32 [group of the stage][column]
constexpr int SA_BYTES = BM * 16;                 // float4 [row] = the stage's four groups
constexpr int RING_BYTES = SCALE_RING * (BN + BM) * 8;  // four fp16 per column / row and slot
constexpr int BARRIER_BYTES = 512;
constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES + SW_BYTES + SA_BYTES) + RING_BYTES + BARRIER_BYTES + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
static_assert((3 * STAGES + 2 * TEAMS * BUFFERS) * 8 + 8 <= BARRIER_BYTES, "barrier block");
constexpr int B_BOX_ROWS = TEAM_COLUMNS / 2;  // rows of B per TMA load: one CTA's half of one team's columns
static_assert(BN == 128 && BM == 128, "the staging warp handles four columns and four rows per lane");

// Where a column-sharded linear puts its slice: the same [m, ldy] matrix on every GPU of the box,
// each one's copy reached through a peer mapping of its memory. The epilogue stores the tile into
// every copy (plain st.global; the stores to the other GPUs travel over NVLink while the next
// tiles are computed), so that no separate all-gather follows the kernel. `first` is the copy a
// CTA starts with: each rank starts with another GPU, so that they do not all write to one at once.
constexpr int MAX_PEERS = 8;
struct PeerOutputs {
    void *y[MAX_PEERS];
    int count, first;
};

// Everything a role needs to find its way around the CTA's shared memory and the problem.
struct View {
    uint8_t *tile_a, *tile_b;
    float *sw_tile;
    float4 *sa_tile;
    uint2 *ring;
    uint64_t *full, *scale_ready, *empty, *dot_full, *dot_empty;
    uint32_t tmem_base, cta;
    int pair, pairs, tiles, tiles_m, k_stages, groups;
};

// A walk over this pair's (tile, stage) sequence without divisions in the loop: integer division
// costs a warp more than a hundred cycles, and a role that pays several per stage becomes the
// pace-setter of the whole kernel.
struct StageWalk {
    int tile, ks, m_index, n_index;
    __device__ __forceinline__ StageWalk(const View &v) : tile(v.pair), ks(0), m_index(v.pair % v.tiles_m), n_index(v.pair / v.tiles_m) {}
    __device__ __forceinline__ bool done(const View &v) const { return tile >= v.tiles; }
    __device__ __forceinline__ void next(const View &v) {
        if (++ks == v.k_stages) {
            ks = 0;
            tile += v.pairs;
            m_index += v.pairs;  // pairs may exceed tiles_m: reduce by repeated subtraction of the few wraps
            while (m_index >= v.tiles_m) {
                m_index -= v.tiles_m;
                ++n_index;
            }
        }
    }
};

// Warp 0, one thread: TMA of this CTA's A rows and of its half of each team's B rows, stage by stage.
// It does nothing else: a clock trace showed the MMA threads waiting 700 cycles per stage for `full`
// when the thread that issues the TMA also staged the scales (about 1450 cycles of serial work per stage).
__device__ __forceinline__ void producer_role(const View &v, const CUtensorMap *map_a, const CUtensorMap *map_w) {
    prefetch_tensormap(map_a);
    prefetch_tensormap(map_w);
    uint32_t s = 0, phase = 0;
    for (StageWalk walk(v); !walk.done(v); walk.next(v)) {
        if (!mbarrier_wait(&v.empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x5000 | s, AHEAD_BACKOFF_NS)) break;
        const int m0 = walk.m_index * 2 * BM + static_cast<int>(v.cta) * BM;
        const int n0 = walk.n_index * BN + static_cast<int>(v.cta) * B_BOX_ROWS;
        // the leader expects the bytes of both CTAs' loads on its barrier
        if (v.cta == 0) mbarrier_arrive_expect_tx(&v.full[s], 2 * (A_BYTES + B_BYTES));
#pragma unroll
        for (int half = 0; half < K_HALVES; ++half) {
            const int k0 = walk.ks * STAGE_K + half * 128;
            tma_load_2d_pair(v.tile_a + s * A_BYTES + half * A_HALF_BYTES, map_a, &v.full[s], k0, m0);
#pragma unroll
            for (int team = 0; team < TEAMS; ++team)  // this CTA's half of each team's columns
                tma_load_2d_pair(v.tile_b + s * B_BYTES + half * B_HALF_BYTES + team * (B_BOX_ROWS * 128), map_w, &v.full[s], k0,
                                 n0 + team * TEAM_COLUMNS);
        }
        if (++s == STAGES) s = 0, phase ^= 1;
    }
}

// Warps 1 and 2. Warp 1 stages the weight scales of the tile's 128 columns, warp 2 the activation scales of
// this CTA's 128 rows: per stage the four groups' values (8 bytes per column or row) are fetched
// SCALE_AHEAD stages early with 4-byte cp.async and, when the stage is free again, written out as
// fp32: sw[group][column] and sa[row] = (groups 0..3).
template <bool ROWS>
__device__ __forceinline__ void scale_role(const View &v, const __half *__restrict__ values, int limit, int lane) {
    constexpr int RING_OFFSET = ROWS ? BN : 0;
    StageWalk ahead(v);
    uint32_t ahead_slot = 0;
    auto fetch = [&]() {
        if (!ahead.done(v)) {
            const int first = ROWS ? ahead.m_index * 2 * BM + static_cast<int>(v.cta) * BM : ahead.n_index * BN;
            uint2 *slot = v.ring + ahead_slot * (BN + BM) + RING_OFFSET + lane;
            const __half *source = values + static_cast<size_t>(first + lane) * v.groups + STAGE_GROUPS * ahead.ks;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                if (first + p * 32 + lane < limit) cp_async_8(slot + p * 32, source + static_cast<size_t>(p * 32) * v.groups);
                else slot[p * 32] = make_uint2(0u, 0u);
            }
            ahead.next(v);
        }
        if (++ahead_slot == SCALE_RING) ahead_slot = 0;
        cp_async_commit();
    };
    for (int i = 0; i < SCALE_AHEAD; ++i) fetch();
    uint32_t s = 0, phase = 0, slot_index = 0;
    for (StageWalk walk(v); !walk.done(v); walk.next(v)) {
        fetch();
        cp_async_wait<SCALE_AHEAD>();  // this thread's copies for this stage have landed
        const uint2 *slot = v.ring + slot_index * (BN + BM) + RING_OFFSET + lane;
        float4 quad[4];  // [p] = the four groups' scales of column / row p * 32 + lane
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint2 raw = slot[p * 32];
            const float2 low = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
            const float2 high = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
            quad[p] = make_float4(low.x, low.y, high.x, high.y);
        }
        if (!mbarrier_wait_warp(&v.empty[s], phase ^ 1, &g_status, STATUS_WAIT_EMPTY | 0x6000 | s, lane, AHEAD_BACKOFF_NS)) break;
        if (ROWS) {
            float4 *sa_stage = v.sa_tile + s * BM + lane;
#pragma unroll
            for (int p = 0; p < 4; ++p) sa_stage[p * 32] = quad[p];
        } else {
            float *sw_stage = v.sw_tile + s * STAGE_GROUPS * BN + lane;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                sw_stage[p * 32] = quad[p].x;
                sw_stage[BN + p * 32] = quad[p].y;
                sw_stage[2 * BN + p * 32] = quad[p].z;
                sw_stage[3 * BN + p * 32] = quad[p].w;
            }
        }
        __syncwarp();
        if (lane == 0) mbarrier_arrive(&v.scale_ready[s]);
        if (++s == STAGES) s = 0, phase ^= 1;
        if (++slot_index == SCALE_RING) slot_index = 0;
    }
    cp_async_wait<0>();
}

// Warps 4-7 of the leader, one thread each. Thread `mine` serves team (mine % TEAMS) and multiplies the
// slabs (128 bytes of K = two groups) whose running number is (mine / TEAMS) modulo TURNS into that team's TMEM
// buffers: N = 64 columns per MMA, the slab's first group into the buffer's first 64 columns, the second into the
// other 64. A slab's number fixes everything else: its pipeline stage (two slabs per stage) and its buffer.
__device__ __forceinline__ void mma_role(const View &v, uint32_t mine) {
    constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * BM, TEAM_COLUMNS);
    const int my_tiles = v.pair < v.tiles ? (v.tiles - 1 - v.pair) / v.pairs + 1 : 0;
    const uint32_t total_slabs = static_cast<uint32_t>(my_tiles) * v.groups / 2;  // a slab: 128 bytes of K = two groups
    const uint32_t team = mine % TEAMS, turn = mine / TEAMS;
    uint64_t *dot_full = v.dot_full + team * BUFFERS, *dot_empty = v.dot_empty + team * BUFFERS;
    for (uint32_t slab = turn; slab < total_slabs; slab += TURNS) {
        const uint32_t iteration = slab / K_HALVES, half = slab % K_HALVES;
        const uint32_t s = iteration % STAGES, phase = (iteration / STAGES) & 1;
        const uint32_t buffer = slab % BUFFERS, buffer_phase = (slab / BUFFERS) & 1;
        if (!mbarrier_wait(&v.full[s], phase, &g_status, STATUS_WAIT_FULL | 0x5000 | s, MMA_BACKOFF_NS)) break;
        if (!mbarrier_wait(&dot_empty[buffer], buffer_phase ^ 1, &g_status, STATUS_WAIT_TMEM_EMPTY | 0x5000 | buffer, MMA_BACKOFF_NS)) break;
        tcgen05_fence_after();
        const uint32_t a_address = smem_u32(v.tile_a + s * A_BYTES + half * A_HALF_BYTES);
        const uint32_t b_address = smem_u32(v.tile_b + s * B_BYTES + half * B_HALF_BYTES + team * (B_BOX_ROWS * 128));
        const uint32_t accumulator = v.tmem_base + (team * BUFFERS + buffer) * BUFFER_COLUMNS;
#pragma unroll
        for (int gl = 0; gl < 2; ++gl)
#pragma unroll
            for (int kk = 0; kk < 2; ++kk)
                umma_f8_pair(accumulator + gl * TEAM_COLUMNS, umma_desc_k_sw128(a_address + gl * 64 + kk * 32),
                             umma_desc_k_sw128(b_address + gl * 64 + kk * 32), idesc, kk);
        tcgen05_commit_pair(&dot_full[buffer]);
    }
}

// Warps 8-23: a warp folds 32 rows x 32 columns of this CTA's half of the tile; a thread owns one
// row (its TMEM lane) and 32 accumulators.
// Per slab a warp looks at the barrier once; per group it starts the copy of its 32 x 32 dots into registers (one
// tcgen05.ld.32x32b.x32, the shape with the highest TMEM read rate), computes the scale products
// of its first HOIST columns meanwhile and does the arithmetic once the copy has landed; the buffer goes back
// when the copy of the slab's second group has landed. The other three warps of its scheduler fill the waits.
// All lanes need the same weight scales: one 16-byte broadcast load per four columns.
// The arithmetic is the packed fp32 pair form of  acc = fma(dot, sa * sw, acc): each half is
// IEEE-rounded exactly like the scalar instruction, so the result has the reference's bits.
template <bool DUMP_DOTS, bool SCATTER>
__device__ __forceinline__ void fold_role(const View &v, const float *__restrict__ bias, void *__restrict__ y,
                                          const PeerOutputs &peers,
                                          int32_t *__restrict__ dots_out, const GemmShape &shape, int warp, int lane) {
    static_assert(COLUMNS == 32, "one tcgen05.ld.32x32b.x32 per warp and group");
    // The hardware ties a warp to the TMEM lanes 32 * (warp % 4); four consecutive warps make one column slice.
    const int quadrant = warp & 3, slice = (warp - FOLD_WARP0) >> 2, team = slice / (TEAM_COLUMNS / COLUMNS);
    const uint32_t dot_full = smem_u32(v.dot_full + team * BUFFERS);
    const uint32_t leader_dot_empty = map_to_cta(smem_u32(v.dot_empty + team * BUFFERS), 0);
    const uint32_t tmem_lane = v.tmem_base + team * BUFFERS * BUFFER_COLUMNS + (slice % (TEAM_COLUMNS / COLUMNS)) * COLUMNS +
                               (static_cast<uint32_t>(quadrant * 32) << 16);
    const uint32_t sw_base = smem_u32(v.sw_tile) + slice * COLUMNS * 4;
    const uint32_t sa_base = smem_u32(v.sa_tile) + (quadrant * 32 + lane) * 16;
    const uint32_t scale_ready = smem_u32(v.scale_ready), empty = smem_u32(v.empty);
    uint32_t dots[COLUMNS];  // dots[j] = dot of this thread's row and column j of the warp's 32
    // A look at a barrier is one try_wait by every lane; a lane that finds the phase incomplete polls on its own, with
    // pauses (the fold warps are the pace-setters: that path is for the first groups and for errors). A wait that ran
    // out of time sets `failed` in its lane; the warp looks at the flags once per stage.
    bool alive = true, failed = false;
    uint32_t s = 0, phase = 0, group_count = 0;
    for (int tile = v.pair; tile < v.tiles && alive; tile += v.pairs) {
        const int row = (tile % v.tiles_m) * 2 * BM + static_cast<int>(v.cta) * BM + quadrant * 32 + lane;
        const int n0 = (tile / v.tiles_m) * BN + slice * COLUMNS;
        uint64_t acc[COLUMNS / 2];  // acc[j] = columns 2 j, 2 j + 1
#pragma unroll
        for (int j = 0; j < COLUMNS / 2; ++j) acc[j] = 0;
        for (int ks = 0; ks < v.k_stages && alive; ++ks) {
            if (__any_sync(0xffffffffu, failed)) { alive = false; break; }
            failed = false;
            if (!try_wait_u32(scale_ready + s * 8, phase)) failed = !wait_slow_u32(scale_ready + s * 8, phase, STATUS_WAIT_READY | 0x5000 | s, FOLD_BACKOFF_NS);
            __syncwarp();
            const uint32_t sw_stage = sw_base + s * SW_BYTES;
#pragma unroll
            for (int gl = 0; gl < STAGE_GROUPS; ++gl, ++group_count) {
                const uint32_t slab = group_count >> 1, buffer = slab % BUFFERS, slab_parity = (slab / BUFFERS) & 1;
                if ((gl & 1) == 0) {
                    if (!try_wait_u32(dot_full + buffer * 8, slab_parity))
                        failed |= !wait_slow_u32(dot_full + buffer * 8, slab_parity, STATUS_WAIT_TMEM_FULL | 0x5000 | buffer, FOLD_BACKOFF_NS);
                    __syncwarp();
                    tcgen05_fence_after();
                }
                tmem_load_32x32(tmem_lane + buffer * BUFFER_COLUMNS + (gl & 1) * TEAM_COLUMNS, dots);
                // while the copy is in flight: the scale products of the first HOIST columns
                const float scale = lds_f32(sa_base + s * SA_BYTES + gl * 4);
                const uint64_t sa2 = pack_f32x2(scale, scale);
                const uint32_t sw_group = sw_stage + gl * BN * 4;
                uint64_t p[HOIST / 2];
#pragma unroll
                ulonglong2 sw4;
                for (int q = 0; q < HOIST / 4; ++q) {
                    sw4 = lds_pairs(sw_group + 16 * q);
                    p[2 * q] = mul_f32x2(sa2, sw4.x);
                    p[2 * q + 1] = mul_f32x2(sa2, sw4.y);
                }
                tmem_load_wait_32(dots);
                if ((gl & 1) == 1) {  // both groups of the slab are in registers or folded: hand the buffer back
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbarrier_arrive_cluster(leader_dot_empty + buffer * 8);
                }
                if (DUMP_DOTS && row < shape.m) {
#pragma unroll
                    for (int j = 0; j < COLUMNS; ++j)
                        if (n0 + j < shape.n)
                            dots_out[(static_cast<size_t>(row) * shape.n + n0 + j) * v.groups + ks * STAGE_GROUPS + gl] =
                                static_cast<int32_t>(__uint_as_float(dots[j]));
                }
#pragma unroll
                for (int q = 0; q < HOIST / 4; ++q) {
                    acc[2 * q] = fma_f32x2(pack_u32x2(dots[4 * q], dots[4 * q + 1]), p[2 * q], acc[2 * q]);
                    acc[2 * q + 1] = fma_f32x2(pack_u32x2(dots[4 * q + 2], dots[4 * q + 3]), p[2 * q + 1], acc[2 * q + 1]);
                }
#pragma unroll
                for (int q = HOIST / 4; q < COLUMNS / 4; ++q) {
                    sw4 = lds_pairs(sw_group + 16 * q);  // four columns, as two pairs
                    acc[2 * q] = fma_f32x2(pack_u32x2(dots[4 * q], dots[4 * q + 1]), mul_f32x2(sa2, sw4.x), acc[2 * q]);
                    acc[2 * q + 1] = fma_f32x2(pack_u32x2(dots[4 * q + 2], dots[4 * q + 3]), mul_f32x2(sa2, sw4.y), acc[2 * q + 1]);
                }
                        }
            __syncwarp();
            if (lane == 0) arrive_u32(empty + s * 8);  // done with this stage's scales; its codes were consumed before the dots arrived
            if (++s == STAGES) s = 0, phase ^= 1;
        }
        if (!alive) break;
        if (row >= shape.m) continue;
        // y: this thread's row, 32 adjacent columns
        float out[COLUMNS];
#pragma unroll
        for (int j = 0; j < COLUMNS / 2; ++j) unpack_f32x2(acc[j], out[2 * j], out[2 * j + 1]);
        if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < COLUMNS; ++j)
                if (n0 + j < shape.n) out[j] += __ldg(bias + n0 + j);
        }
        const size_t element = static_cast<size_t>(row) * shape.ldy + n0;
        if constexpr (SCATTER) {
            // The launcher admits only outputs that take whole 32-byte sectors (32-byte aligned copies,
            // n a multiple of 32, ldy a multiple of a sector): a warp's 32 columns lie wholly inside the
            // matrix or wholly outside it (n not a multiple of the tile's 128 columns).
            if (n0 >= shape.n) continue;
            if (shape.y_is_half) {
                uint32_t packed[COLUMNS / 2];
#pragma unroll
                for (int j = 0; j < COLUMNS / 2; ++j) {
                    const __half2 h = __floats2half2_rn(out[2 * j], out[2 * j + 1]);
                    packed[j] = *reinterpret_cast<const uint32_t *>(&h);
                }
                int index = peers.first;
                for (int copy = 0; copy < peers.count; ++copy) {
                    __half *target = static_cast<__half *>(peers.y[index]) + element;
#pragma unroll
                    for (int j = 0; j < COLUMNS / 16; ++j)
                        st_global_v8(target + 16 * j, *reinterpret_cast<const uint32_t(*)[8]>(&packed[8 * j]));
                    if (++index == peers.count) index = 0;
                }
            } else {
                int index = peers.first;
                for (int copy = 0; copy < peers.count; ++copy) {
                    float *target = static_cast<float *>(peers.y[index]) + element;
#pragma unroll
                    for (int j = 0; j < COLUMNS / 8; ++j)
                        st_global_v8(target + 8 * j, *reinterpret_cast<const uint32_t(*)[8]>(&out[8 * j]));
                    if (++index == peers.count) index = 0;
                }
            }
            continue;
        }
        // whole 32-byte sectors when the row segment is aligned for them, else element by element
        const bool sectors = n0 + COLUMNS <= shape.n &&
                             (reinterpret_cast<uintptr_t>(y) & 31) == 0 && shape.ldy % (shape.y_is_half ? 16 : 8) == 0;
        if (shape.y_is_half) {
            uint32_t packed[COLUMNS / 2];
#pragma unroll
            for (int j = 0; j < COLUMNS / 2; ++j) {
                const __half2 h = __floats2half2_rn(out[2 * j], out[2 * j + 1]);
                packed[j] = *reinterpret_cast<const uint32_t *>(&h);
            }
            __half *target = static_cast<__half *>(y) + element;
            if (sectors) {
#pragma unroll
                for (int j = 0; j < COLUMNS / 16; ++j)
                    st_global_v8(target + 16 * j, *reinterpret_cast<const uint32_t(*)[8]>(&packed[8 * j]));
            } else {
#pragma unroll
                for (int j = 0; j < COLUMNS; ++j)
                    if (n0 + j < shape.n) target[j] = __float2half_rn(out[j]);
            }
        } else {
            float *target = static_cast<float *>(y) + element;
            if (sectors) {
#pragma unroll
                for (int j = 0; j < COLUMNS / 8; ++j)
                    st_global_v8(target + 8 * j, *reinterpret_cast<const uint32_t(*)[8]>(&out[8 * j]));
            } else {
#pragma unroll
                for (int j = 0; j < COLUMNS; ++j)
                    if (n0 + j < shape.n) target[j] = out[j];
            }
        }
    }
    tmem_load_wait();  // nothing of this warp may still be in flight at teardown
}

template <bool DUMP_DOTS, bool SCATTER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
            const __half *__restrict__ a_scales, const __half *__restrict__ w_scales,
            const float *__restrict__ bias, void *__restrict__ y, int32_t *__restrict__ dots_out,
            const GemmShape shape, const __grid_constant__ PeerOutputs peers) {
    extern __shared__ uint8_t smem_raw[];
    // the same offsets in both CTAs: the dynamic shared window starts at the same address in each
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tile_a = smem;
    uint8_t *tile_b = tile_a + STAGES * A_BYTES;
    float *sw_tile = reinterpret_cast<float *>(tile_b + STAGES * B_BYTES);
    float4 *sa_tile = reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(sw_tile) + STAGES * SW_BYTES);
    uint2 *ring = reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(sa_tile) + STAGES * SA_BYTES);
    uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(ring) + RING_BYTES);
    uint64_t *scale_ready = full + STAGES;
    uint64_t *empty = scale_ready + STAGES;
    uint64_t *dot_full = empty + STAGES;
    uint64_t *dot_empty = dot_full + TEAMS * BUFFERS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(dot_empty + TEAMS * BUFFERS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();  // 0 = leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (shape.m + 2 * BM - 1) / (2 * BM), tiles_n = (shape.n + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n, k_stages = shape.k / STAGE_K, groups = shape.k / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full[s], 1);                 // the leader's is the one in use
            mbarrier_init(&scale_ready[s], 2);          // the two scale-staging warps
            // This CTA's fold warps. They arrive after they have seen the dots of both groups of the
            // stage, and a tcgen05.commit arrives only when the MMAs before it have read their operands:
            // so the codes of the stage are free as well, in both CTAs, without a commit of their own.
            mbarrier_init(&empty[s], FOLD_WARPS);
        }
        for (int b = 0; b < TEAMS * BUFFERS; ++b) {
            mbarrier_init(&dot_full[b], 1);                        // pair commit
            mbarrier_init(&dot_empty[b], 2 * FOLD_WARPS / TEAMS);  // the leader's: the team's fold warps of both CTAs
        }
        fence_barrier_init();
    }
    if (warp == MMA_WARP0) {
        tmem_alloc_pair(tmem_slot, TEAMS * BUFFERS * BUFFER_COLUMNS);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before anything arrives on them from the other side
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const View view = {tile_a, tile_b, sw_tile, sa_tile, ring, full, scale_ready, empty, dot_full, dot_empty,
                       tmem_base, cta, pair, pairs, tiles, tiles_m, k_stages, groups};

    if (warp < FOLD_WARP0) {
        setmaxnreg_dec<CONTROL_REGISTERS>();
        if (warp == PRODUCER_WARP) {
            if (lane == 0) producer_role(view, &map_a, &map_w);
        } else if (warp == SW_WARP) {
            scale_role<false>(view, w_scales, shape.n, lane);
        } else if (warp == SA_WARP) {
            scale_role<true>(view, a_scales, shape.m, lane);
        } else if (lane == 0 && cta == 0 && warp >= MMA_WARP0 && warp < MMA_WARP0 + MMA_WARPS) {
            mma_role(view, static_cast<uint32_t>(warp - MMA_WARP0));
        }
    } else {
        setmaxnreg_inc<FOLD_REGISTERS>();
        fold_role<DUMP_DOTS, SCATTER>(view, bias, y, peers, dots_out, shape, warp, lane);
    }

    tcgen05_fence_before();
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t *>(&g_status) != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let bulk copies already issued land
    }
    __syncwarp();
    cluster_sync();  // neither CTA may leave while the other can still reach its shared memory or barriers
    if (warp == MMA_WARP0) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, TEAMS * BUFFERS * BUFFER_COLUMNS);
    }
}

}  // namespace w4a4_pair
}  // namespace qi
