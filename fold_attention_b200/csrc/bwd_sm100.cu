// The deterministic attention backward on Blackwell tensor cores: tcgen05.mma
// with TMEM accumulators, TMA-fed 128-byte-swizzled shared tiles, mbarrier
// pipelines between specialised warps. Head dim 128, bf16 or fp16, dense or packed.
//
// One CTA owns one block of 128 keys of one (request, KV head) and walks query
// tiles of 128 rows, for each of the group's G query heads in turn. Every MMA is
// M=128, N=128, K=16 (the shape the tensor pipe runs at its full rate whatever
// else the SM does; N=64 runs at half of it). Per query tile i:
//     S^T  = K Q^T            SS  keys x queries                          -> T_S
//     dP^T = V dO^T           SS                                          -> T_DP
//     P~^T = exp2(S^T c - (L - s))      compute warps; 16-bit, over S^T in TMEM
//     dS~^T = P~^T (dP^T - Delta)       compute warps; to shared, swizzled
//     dV  += P~^T dO          TS  A from TMEM
//     dQ~^T = K^T dS~^T       SS  A = K^T (MN-major), B = dS~^T (MN-major) -> T_DP
//     dK  += dS~^T Q          SS  A = dS~^T (K-major), B = Q (MN-major)
// TMEM holds exactly S^T, dP^T/dQ~^T, dK and dV (4 x 128 columns), so nothing is
// double-buffered; the one MMA thread keeps the pipe fed by interleaving two
// tiles: dP(i) | dV(i) S(i+1) | dQ(i) dK(i) dP(i+1) | ..., so that the exponentials
// of tile i+1 run under dQ(i), dK(i), dP(i+1) and its dS~ under dV(i+1). A thread's
// MMAs execute in issue order, which is what lets S(i+1) overwrite P~(i) right
// behind dV(i).
// dK and dV stay in TMEM for the CTA's whole life, summed in one fixed order;
// dQ~ leaves the GEMM on the request's integer grid (the softmax carries the
// grid exponent s; for fp16 it is applied at the drain), is rounded to
// nearest-even int32 and added to the accumulator with integer reductions, which
// commute exactly.
//
// Warps: 0 TMA producer, 1 MMA issuer (owns the TMEM allocation), then NWG
// compute warpgroups (128 / NWG queries of the tile each; a thread is one key
// row = one TMEM lane), then the dQ drain's four warps (TMEM -> int32 -> shared
// -> cp.reduce.async.bulk add into the accumulator). The compute phases are
// chains of TMEM load -> arithmetic -> store whose latency, not throughput,
// sets their length, so four warpgroups of 32 queries (four compute warps per
// scheduler) finish a tile's exponentials and dS~ sooner than two of 64.
// Every mbarrier wait is bounded: on expiry the kernel raises a status word,
// stops waiting everywhere, frees its TMEM and returns.
// Reference arithmetic: src/fold_attention/backward/kernel.py:1191-1330.
#include <cuda.h>

#include <algorithm>

#include "bwd_common.cuh"

namespace fold {

namespace sm100 {

constexpr int BN = 128;   // keys per CTA
constexpr int BM = 128;   // queries per tile
constexpr int HD = 128;   // head dim
constexpr int STAGES = 2;
constexpr int ISLOTS = 2;   // work items the producer may run ahead of the slowest role
#ifndef FOLD_BWD_NWG
#define FOLD_BWD_NWG 2
#endif
constexpr int NWG = FOLD_BWD_NWG;            // compute warpgroups
constexpr int QPW = BM / NWG;                // queries per compute warpgroup
constexpr int NCOMPUTE = 128 * NWG;          // compute threads
constexpr int W_DRAIN = 2 + 4 * NWG;         // first warp of the dQ drain
constexpr int NTHREADS = 32 * (W_DRAIN + 4);
static_assert(NWG == 2 || NWG == 4, "two or four compute warpgroups");
constexpr long long WAIT_CYCLES = 1ll << 31;   // about a second of SM clocks
// nanoseconds a waiting thread sleeps between polls of its barrier: a polling warp takes issue
// slots from the working warps of its scheduler
#ifndef FOLD_PACKED_MATH
#define FOLD_PACKED_MATH 1
#endif
#ifndef FOLD_DRAIN_PACKED
#define FOLD_DRAIN_PACKED 1
#endif
#ifndef FOLD_SLEEP_WORKER
#define FOLD_SLEEP_WORKER 64
#endif
#ifndef FOLD_SLEEP_ISSUER
#define FOLD_SLEEP_ISSUER 0
#endif
// 1: dQ~ leaves the GEMM with queries on the TMEM lanes (dQ~ = dS~ K instead of its transpose), so a
// drain thread holds 32 consecutive channels of one query: it stages them with eight 16-byte
// stores into a 128-byte-swizzled block and the block is added to the accumulator by a tiled TMA
// reduction. 0: channels on the lanes, 4-byte stores into a row-major block, untiled bulk reduction.
#ifndef FOLD_BWD_DRAIN_T
#define FOLD_BWD_DRAIN_T 1
#endif
// 1: the drain adds its rounding constant's bits to the accumulator along with the value and the
// preprocess starts the accumulator at minus their sum (int32 wraps, so the total is exact):
// one integer subtract per element less
#ifndef FOLD_BWD_BIAS
#define FOLD_BWD_BIAS 1
#endif
constexpr int SLEEP_WORKER = FOLD_SLEEP_WORKER, SLEEP_PRODUCER = 100, SLEEP_ISSUER = FOLD_SLEEP_ISSUER;

// shared memory map (bytes from a 1024-aligned base)
constexpr int SM_K = 0;                         // [2 boxes][128 keys][64 ch] 16-bit, SW128
constexpr int SM_V = 32768;
constexpr int SM_Q = 65536;                     // [2 stages][2 boxes][128 queries][64 ch]
constexpr int SM_DO = SM_Q + 2 * 32768;         // one buffer: dO(i+1) lands between dV(i) and dP(i+1)
constexpr int SM_DS = SM_DO + 32768;            // [2 boxes][128 keys][64 queries] 16-bit, SW128
constexpr int SM_STG = SM_DS + 32768;           // [2][32 queries][128 ch] int32: dQ~ on its way to the accumulator
constexpr int SM_L = SM_STG + 2 * 16384;        // L [2 stages][128] f32, then Delta [2][128] f32
constexpr int SM_DL = SM_L + 2 * 512;
constexpr int SM_BAR = SM_DL + 2 * 512;
constexpr int SM_TOTAL = SM_BAR + 256;
constexpr int SMEM_BYTES = 232448;              // all an SM gives one CTA; the base may use what is left to align
constexpr int ALIGN_SLACK = SMEM_BYTES - SM_TOTAL;

// barrier indices
enum {
    B_KV = 0,
    B_QFULL = 1,                 // [STAGES] Q and L of the stage have landed
    B_QEMPTY = B_QFULL + STAGES, // [STAGES] dK has read Q
    B_OFULL = B_QEMPTY + STAGES, // dO and Delta have landed
    B_OEMPTY,                    // dV has read dO
    B_S,                         // S^T in TMEM
    B_DP,                        // dP^T in TMEM (and dS~^T's shared buffer free: dQ, dK of the tile before retired)
    B_P,                         // P~^T in TMEM (256 arrivals)
    B_DS,                        // dS~^T in shared (256 arrivals)
    B_DQF,                       // dQ~^T in TMEM
    B_DQE,                       // dQ~^T read out (128 arrivals)
    B_DONE,                      // every MMA of the item retired
    B_KVFREE,                    // the item's last dQ~ (its last read of K) retired
    B_ACCFREE,                   // the item's dK, dV have been read out of TMEM (NCOMPUTE arrivals)
    B_IFULL,                     // [ISLOTS] the producer has published a work item
    B_IEMPTY = B_IFULL + 2,      // [ISLOTS] every consumer has taken it
    B_COUNT = B_IEMPTY + 2,
};

// TMEM columns
constexpr uint32_t T_S = 0, T_DP = 128, T_DK = 256, T_DV = 384;

struct Shared {
    uint32_t base;
    __device__ uint32_t bar(int i) const { return base + SM_BAR + 8 * i; }
};

// ---- PTX ----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// one poll that never suspends the thread, for a thread that watches several barriers
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. `abort` (shared) is raised by whoever runs out first; once it
// is up nobody waits any more, so every role runs to its end.
template <int SLEEP_NS = 0>
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          long long limit = WAIT_CYCLES) {
    if (mbar_try(bar, parity)) return;
    if (*abort_flag) return;
    const long long t0 = clock64();
    for (int i = 0;; ++i) {
        if (mbar_try(bar, parity)) return;
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);   // a waiting warp group must not take the issue slots of a working one
        if ((i & 63) == 63) {
            if (*abort_flag) return;
            if (clock64() - t0 > limit) break;
        }
    }
    *abort_flag = 1;
    atomicExch(status, FOLD_ERR_TIMEOUT);
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
                 ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 floats of shared memory as eight 16-byte reads issued back to back (volatile: they stay where
// they are written, ahead of the wait they are meant to overlap; under the MMAs' operand traffic a
// shared load takes a couple of hundred cycles)
__device__ __forceinline__ void lds32(uint32_t addr, float (&v)[32]) {
#pragma unroll
    for (int u = 0; u < 8; ++u)
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[4 * u]), "=f"(v[4 * u + 1]), "=f"(v[4 * u + 2]), "=f"(v[4 * u + 3]) : "r"(addr + 16 * u));
}
__device__ __forceinline__ void lds16(uint32_t addr, float (&v)[16]) {
#pragma unroll
    for (int u = 0; u < 4; ++u)
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[4 * u]), "=f"(v[4 * u + 1]), "=f"(v[4 * u + 2]), "=f"(v[4 * u + 3]) : "r"(addr + 16 * u));
}
// Packed fp32 arithmetic (two IEEE operations per instruction, the results bit for bit those of
// the scalar forms): the compute warps are short of issue slots and of nothing else.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, uint64_t b, float c0, float c1) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack2(a0, a1)), "l"(b), "l"(pack2(c0, c1)));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
// (a - b) * c
__device__ __forceinline__ void submul2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    uint64_t t, d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(t) : "l"(pack2(a0, a1)), "l"(pack2(b0, b1)));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(t), "l"(pack2(c0, c1)));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- descriptors ----------------------------------------------------------------
// shared-memory matrix descriptor, 128-byte swizzle; offsets in bytes
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;   // descriptor version (Blackwell)
    d |= 2ull << 61;   // SWIZZLE_128B
    return d;
}
// instruction descriptor: 16-bit x 16-bit -> f32 (format 1 bf16, 0 fp16), M x N, operand majors (0 K, 1 MN)
__host__ __device__ constexpr uint32_t instr_desc(int fmt, int M, int N, int a_mn, int b_mn) {
    return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) | (static_cast<uint32_t>(a_mn) << 15) |
           (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
           (static_cast<uint32_t>(M >> 4) << 24);
}

struct Maps {
    CUtensorMap q, dout, k, v;   // (channel, row, head, batch), boxes (64, 128, 1, 1)
    CUtensorMap dk, dv;          // the same view of the outputs, for the private exit's tile stores
    CUtensorMap dq;              // the int32 accumulator as (channel, head * padded row), boxes (32, 128)
};

// The bounded wait by itself: one warp waits on a barrier nobody will arrive at, for `limit`
// cycles, through the same mbar_wait the main loop's roles use. The wait runs out, raises the
// status word and the abort flag, and the kernel returns normally: what a host-side check of
// the status word has to see, without a fault and without touching TMEM or the tensor pipe.
__global__ void __launch_bounds__(32) wait_probe_kernel(long long limit, int* status, int* flag_out) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = static_cast<uint32_t>(__cvta_generic_to_shared(&bar));
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (threadIdx.x == 0) mbar_wait<SLEEP_WORKER>(b, 0, &abort_flag, status, limit);
    __syncwarp();
    // every other role sees the flag and stops waiting at once
    if (threadIdx.x == 1) mbar_wait<SLEEP_WORKER>(b, 0, &abort_flag, status, 1ll << 40);
    __syncwarp();
    if (threadIdx.x == 0 && flag_out) *flag_out = abort_flag;
}

// ---- optional cycle counters (-DFOLD_BWD_COUNTERS): where each role's time goes -----------
// Sums over every CTA of a launch, taken by one thread per role: slots are
//  0 CTAs, 1 tiles, 2 CTA lifetime, 3 prologue (until K and V have landed), 4 epilogue,
//  5 compute: wait for S^T, 6 exponential phase, 7 wait for dP^T, 8 dS~ phase,
//  9 MMA thread: cycles with nothing ready to issue, 10 drain: wait for dQ~^T, 11 drain busy,
// 12 drain: from dQ~^T ready to its columns released; the MMA thread's waits in the fixed issue
// order: 13 for P~, 14 for Q, 15 for dS~, 16 for dO, 17 for the drain's release.
#ifdef FOLD_BWD_COUNTERS
__device__ unsigned long long g_counters[24];
#define CNT_ADD(slot, v) atomicAdd(&g_counters[slot], static_cast<unsigned long long>(v))
#define CNT_T(var) const long long var = clock64()
#define CNT_WAIT(acc, ...) do { const long long _t = clock64(); mbar_wait<SLEEP_ISSUER>(__VA_ARGS__); acc += clock64() - _t; } while (0)
#else
#define CNT_ADD(slot, v) do { } while (0)
#define CNT_T(var) do { } while (0)
#define CNT_WAIT(acc, ...) mbar_wait<SLEEP_ISSUER>(__VA_ARGS__)
#endif

// One work item: a key block of one (request, KV head), `nh` of the group's query heads from
// `h0`, and the query blocks [m_first, m_first + per_head) that can see it.
struct Item {
    int nb, hkv, b, h0, nh, n0, m_first, per_head, total;
    SeqInfo sq;
};
__device__ __forceinline__ Item load_item(const BwdParams& p, int idx) {
    const int4* w = reinterpret_cast<const int4*>(p.work) + 2 * static_cast<int64_t>(idx);
    const int4 a = __ldg(w), c = __ldg(w + 1);
    Item it;
    it.nb = a.x; it.hkv = a.y; it.b = a.z; it.h0 = a.w; it.nh = c.x;
    it.sq = seq_info(p, it.b);
    it.n0 = it.nb * BN;
    const int nm = (it.sq.len + BM - 1) / BM;
    const int m_min = p.causal ? (it.n0 / BM) : 0;
    it.m_first = max(m_min, c.y);
    it.per_head = (it.n0 < it.sq.len) ? max(min(nm, c.z) - it.m_first, 0) : 0;
    it.total = it.per_head * it.nh;
    return it;
}

// Whether any of the `count` threads meeting at named barrier `id` wants to stop. The threads of
// a role leave their item loop together or not at all: they share named barriers inside it, and a
// thread that left alone (it saw the abort flag a moment before its neighbours did) would leave the
// others waiting at one for ever.
__device__ __forceinline__ bool any_stops(bool stop, int id, int count) {
    uint32_t r;
    asm volatile("{ .reg .pred p, q; setp.ne.b32 p, %1, 0; barrier.cta.red.or.pred q, %2, %3, p; selp.u32 %0, 1, 0, q; }"
                 : "=r"(r) : "r"(static_cast<uint32_t>(stop)), "r"(id), "r"(count) : "memory");
    return r != 0;
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// x * 2^e for any e in [-250, 250] without leaving fp32's exponent range half way
__device__ __forceinline__ float scale_pow2(float x, int e) {
    const int e1 = max(-120, min(120, e));
    return x * pow2f(e1) * pow2f(e - e1);
}

// A persistent CTA: every role loops over the work items its producer thread claims from the
// list (an atomic counter), longest first, so the grid ends on short items and a CTA's fixed
// costs (TMEM allocation, barrier set-up, the wait for the first loads) are paid once. The
// roles run asynchronously across item boundaries: while the drain finishes an item's last
// tile and the compute warps write its dK and dV out, K and V of the next item are already
// on their way. Barrier phases count tiles (or items) since the CTA started.
template <bool F16>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_main_sm100_kernel(const BwdParams p, const __grid_constant__ Maps maps) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    const uint32_t base = (raw + 1023u) & ~1023u;
    if (base - raw > static_cast<uint32_t>(ALIGN_SLACK)) {   // the map below would not fit: refuse, loudly
        if (threadIdx.x == 0) atomicExch(p.status, FOLD_ERR_LAUNCH);
        return;
    }
    uint8_t* smem = smem_raw + (base - raw);
    Shared sh{base};
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 8 * B_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 8 * B_COUNT + 8);
    volatile int* item_slot = reinterpret_cast<volatile int*>(smem + SM_BAR + 8 * B_COUNT + 16);   // [ISLOTS]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    CNT_T(cta_t0);

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(sh.bar(B_KV), 1);
        mbar_init(sh.bar(B_KVFREE), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sh.bar(B_QFULL + s), 1);
            mbar_init(sh.bar(B_QEMPTY + s), 1);
        }
        mbar_init(sh.bar(B_OFULL), 1);
        mbar_init(sh.bar(B_OEMPTY), 1);
        mbar_init(sh.bar(B_S), 1);
        mbar_init(sh.bar(B_DP), 1);
        mbar_init(sh.bar(B_P), NCOMPUTE);
        mbar_init(sh.bar(B_DS), NCOMPUTE);
        mbar_init(sh.bar(B_DQF), 1);
        mbar_init(sh.bar(B_DQE), 128);
        mbar_init(sh.bar(B_DONE), 1);
        mbar_init(sh.bar(B_ACCFREE), NCOMPUTE);
        for (int s = 0; s < ISLOTS; ++s) {
            mbar_init(sh.bar(B_IFULL + s), 1);
            mbar_init(sh.bar(B_IEMPTY + s), 1 + NCOMPUTE + 128);   // the MMA thread, the compute warps, the drain
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;"
                     ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(tmem_slot))) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // The j-th item this CTA works on, as the producer published it (-1: the list is exhausted).
    // Every consumer takes each slot once, in order.
    auto next_item = [&](int j) -> int {
        const int s = j % ISLOTS;
        mbar_wait<SLEEP_WORKER>(sh.bar(B_IFULL + s), (j / ISLOTS) & 1, abort_flag, p.status);
        const int idx = item_slot[s];
        mbar_arrive(sh.bar(B_IEMPTY + s));
        return (*abort_flag || static_cast<unsigned>(idx) >= static_cast<unsigned>(p.n_items)) ? -1 : idx;
    };

    if (warp == 0) {
        // ================= work claims and TMA loads =================
        if (lane == 0) {
            int t = 0;   // tiles loaded so far
            for (int j = 0;; ++j) {
                // claim until an item has work (the list keeps a slot for every key block up to the
                // longest sequence: the ones past a shorter request's end are empty) or the list ends
                int idx;
                Item it;
                for (;;) {
                    idx = atomicAdd(p.sched, 1);
                    if (idx >= p.n_items) { idx = -1; break; }
                    it = load_item(p, idx);
                    if (it.total > 0) break;
                }
                const int sl = j % ISLOTS;
                if (j >= ISLOTS) mbar_wait<SLEEP_PRODUCER>(sh.bar(B_IEMPTY + sl), ((j / ISLOTS) - 1) & 1, abort_flag, p.status);
                item_slot[sl] = idx;
                __threadfence_block();
                mbar_arrive(sh.bar(B_IFULL + sl));
                if (idx < 0 || *abort_flag) break;
                const int brow = it.sq.start + it.n0;
                const int bb = p.cu ? 0 : it.b;
                // K and V: one buffer each, free when the item before has issued its last dQ~
                if (j >= 1) mbar_wait<SLEEP_PRODUCER>(sh.bar(B_KVFREE), (j - 1) & 1, abort_flag, p.status);
                mbar_expect_tx(sh.bar(B_KV), 2 * 32768);
                for (int x = 0; x < 2; ++x) {
                    tma_load_4d(base + SM_K + x * 16384, &maps.k, 64 * x, brow, it.hkv, bb, sh.bar(B_KV));
                    tma_load_4d(base + SM_V + x * 16384, &maps.v, 64 * x, brow, it.hkv, bb, sh.bar(B_KV));
                }
                for (int i = 0; i < it.total; ++i, ++t) {
                    const int s = t % STAGES;
                    const int g = i / it.per_head, mb = it.m_first + i % it.per_head;
                    const int h = it.hkv * p.G + it.h0 + g;
                    const int row = it.sq.start + mb * BM;
                    const int64_t wrow = static_cast<int64_t>(h) * p.rows_p + it.sq.pstart + mb * BM;
                    // Q and L: two stages, free when dK of the tile two back has read Q
                    if (t >= STAGES) mbar_wait<SLEEP_PRODUCER>(sh.bar(B_QEMPTY + s), ((t / STAGES) - 1) & 1, abort_flag, p.status);
                    mbar_expect_tx(sh.bar(B_QFULL + s), 32768 + 512);
                    for (int x = 0; x < 2; ++x) tma_load_4d(base + SM_Q + s * 32768 + x * 16384, &maps.q, 64 * x, row, h, bb, sh.bar(B_QFULL + s));
                    bulk_load(base + SM_L + s * 512, p.lse2 + wrow, 512, sh.bar(B_QFULL + s));
                    // dO: one buffer, free when dV of the tile before has read it (three GEMMs ahead of
                    // the dP^T that wants the new one); Delta rides with it but alternates between two
                    // slots, because the compute warps may still be reading the last one
                    if (t >= 1) mbar_wait<SLEEP_PRODUCER>(sh.bar(B_OEMPTY), (t - 1) & 1, abort_flag, p.status);
                    mbar_expect_tx(sh.bar(B_OFULL), 32768 + 512);
                    for (int x = 0; x < 2; ++x) tma_load_4d(base + SM_DO + x * 16384, &maps.dout, 64 * x, row, h, bb, sh.bar(B_OFULL));
                    bulk_load(base + SM_DL + s * 512, p.dpsum + wrow, 512, sh.bar(B_OFULL));
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t ID_KK = instr_desc(F16 ? 0 : 1, 128, 128, 0, 0);   // S^T, dP^T: both K-major
            constexpr uint32_t ID_KM = instr_desc(F16 ? 0 : 1, 128, 128, 0, 1);   // dV, dK: B MN-major
            constexpr uint32_t ID_MM = instr_desc(F16 ? 0 : 1, 128, 128, 1, 1);   // dQ~: both MN-major
            // K-major operand, 16 channels per step: 4 steps per 64-channel box of 16 KB;
            // MN-major operand, 16 rows per step: 2 KB on, the second 64 columns one box (16 KB) further
            uint64_t dk_kk[8], dv_kk[8], dk_mn[8];
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t kk = (ks >> 2) * 16384 + (ks & 3) * 32;
                dk_kk[ks] = smem_desc(base + SM_K + kk, 16, 1024);
                dv_kk[ks] = smem_desc(base + SM_V + kk, 16, 1024);
                dk_mn[ks] = smem_desc(base + SM_K + ks * 2048, 16384, 1024);
            }
            const uint64_t ds_kk0 = smem_desc(base + SM_DS, 16, 1024), ds_mn0 = smem_desc(base + SM_DS, 16384, 1024);
            const uint64_t o_kk0 = smem_desc(base + SM_DO, 16, 1024), o_mn0 = smem_desc(base + SM_DO, 16384, 1024);
            long long w_kv = 0, w_p = 0, w_q = 0, w_ds = 0, w_o = 0, w_dqe = 0;
            (void)w_kv; (void)w_p; (void)w_q; (void)w_ds; (void)w_o; (void)w_dqe;
            // The five GEMMs of a tile, each eight K=16 steps; `t` is the tile's number since the
            // CTA started (it picks the Q stage), `acc` whether dK / dV accumulate (not on an
            // item's first tile). The barriers they depend on are taken by the loop below.
            auto issue_s = [&](int t) {   // S^T = K Q^T -> T_S
                const uint64_t q0 = smem_desc(base + SM_Q + (t % STAGES) * 32768, 16, 1024);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ss(tmem + T_S, dk_kk[ks], q0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), ID_KK, ks > 0);
                tc_commit(sh.bar(B_S));
            };
            auto issue_dp = [&]() {       // dP^T = V dO^T -> T_DP
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ss(tmem + T_DP, dv_kk[ks], o_kk0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), ID_KK, ks > 0);
                tc_commit(sh.bar(B_DP));
            };
            auto issue_dv = [&](bool acc) {   // dV += P~^T dO: steps of 16 queries; A = 8 TMEM columns per step, at the
                                              // head of the S^T columns of the warpgroup that owns those queries
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ts(tmem + T_DV, tmem + T_S + (16 * ks / QPW) * QPW + (16 * ks % QPW) / 2, o_mn0 + ((ks * 2048) >> 4), ID_KM,
                           acc || (ks > 0));
                tc_commit(sh.bar(B_OEMPTY));
            };
            auto issue_dq_dk = [&](int t, bool acc, bool last) {
                const int s = t % STAGES;
                const uint64_t q_mn0 = smem_desc(base + SM_Q + s * 32768, 16384, 1024);
                // 8 steps of 16 keys, both operands MN-major: dQ~ = dS~ K (queries on the lanes) or
                // dQ~^T = K^T dS~^T (channels on the lanes); the same two shared tiles either way
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
#if FOLD_BWD_DRAIN_T
                    mma_ss(tmem + T_DP, ds_mn0 + ((ks * 2048) >> 4), dk_mn[ks], ID_MM, ks > 0);
#else
                    mma_ss(tmem + T_DP, dk_mn[ks], ds_mn0 + ((ks * 2048) >> 4), ID_MM, ks > 0);
#endif
                }
                tc_commit(sh.bar(B_DQF));
                if (last) tc_commit(sh.bar(B_KVFREE));   // the item's last read of K (V's was its last dP^T): the next item's may land
                // dK += dS~^T Q : 8 steps of 16 queries
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ss(tmem + T_DK, ds_kk0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), q_mn0 + ((ks * 2048) >> 4), ID_KM, acc || (ks > 0));
                tc_commit(sh.bar(B_QEMPTY + s));
            };
            int t = 0;   // tiles issued so far
            for (int j = 0;; ++j) {
                const int idx = next_item(j);
                if (idx < 0) break;
                const Item it = load_item(p, idx);
                CNT_WAIT(w_kv, sh.bar(B_KV), j & 1, abort_flag, p.status);
                // the order of a tile's GEMMs, two tiles interleaved: dP(i) | dV(i) S(i+1) | dQ(i) dK(i) dP(i+1)
                CNT_WAIT(w_q, sh.bar(B_QFULL + t % STAGES), (t / STAGES) & 1, abort_flag, p.status);
                tc_fence_after();
                issue_s(t);
                CNT_WAIT(w_o, sh.bar(B_OFULL), t & 1, abort_flag, p.status);
                if (t >= 1) CNT_WAIT(w_dqe, sh.bar(B_DQE), (t - 1) & 1, abort_flag, p.status);   // the last dQ~ has left the columns
                tc_fence_after();
                issue_dp();
                for (int i = 0; i < it.total; ++i, ++t) {
                    CNT_WAIT(w_p, sh.bar(B_P), t & 1, abort_flag, p.status);
                    // an item's first dV and dK overwrite the accumulators: the item before must have read its own out
                    if (i == 0 && j >= 1) mbar_wait<SLEEP_ISSUER>(sh.bar(B_ACCFREE), (j - 1) & 1, abort_flag, p.status);
                    tc_fence_after();
                    issue_dv(i > 0);
                    if (i + 1 < it.total) {   // over P~(i), behind dV(i)
                        CNT_WAIT(w_q, sh.bar(B_QFULL + (t + 1) % STAGES), ((t + 1) / STAGES) & 1, abort_flag, p.status);
                        tc_fence_after();
                        issue_s(t + 1);
                    }
                    CNT_WAIT(w_ds, sh.bar(B_DS), t & 1, abort_flag, p.status);
                    tc_fence_after();
                    issue_dq_dk(t, i > 0, i + 1 == it.total);
                    if (i + 1 < it.total) {
                        CNT_WAIT(w_o, sh.bar(B_OFULL), (t + 1) & 1, abort_flag, p.status);
                        CNT_WAIT(w_dqe, sh.bar(B_DQE), t & 1, abort_flag, p.status);   // dQ~(i) has left the columns
                        tc_fence_after();
                        issue_dp();
                    }
                }
                tc_commit(sh.bar(B_DONE));   // every MMA of the item has retired: dK and dV are final
                CNT_ADD(1, it.total);
            }
            CNT_ADD(0, 1);
            CNT_ADD(3, w_kv);
            CNT_ADD(13, w_p);
            CNT_ADD(14, w_q);
            CNT_ADD(15, w_ds);
            CNT_ADD(16, w_o);
            CNT_ADD(17, w_dqe);
        }
    } else if (warp < W_DRAIN) {
        // ================= compute: P~^T and dS~^T for QPW of the tile's queries; then the item's dK, dV =================
        const int wg = (warp - 2) >> 2;
        const int r = 32 * (warp & 3) + lane;   // key row = TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const float c2 = p.scale * kLog2e;
        const uint64_t c2x2 = pack2(c2, c2);
        (void)c2x2;
        const uint32_t rs = tmem + lane_addr + T_S + QPW * wg;
        const uint32_t rd = tmem + lane_addr + T_DP + QPW * wg;
        // dS~^T row r: 128 bytes = 64 queries per box, 16-byte chunk u (8 queries) at u ^ (r & 7)
        uint8_t* sds = smem + SM_DS + ((QPW * wg) / 64) * 16384 + r * 128;
        constexpr int CH0_MASK = (64 / QPW) - 1;        // warpgroups per 64-query box, minus one
        const int ch0 = (wg & CH0_MASK) * (QPW / 8);    // the warpgroup's first chunk in its box
#ifdef FOLD_BWD_COUNTERS
        long long c_ws = 0, c_exp = 0, c_wd = 0, c_ds = 0, c_epi = 0;
        const bool counting = (warp == 2 && lane == 0);
#endif
        int t = 0;
        for (int j = 0;; ++j) {
            const int idx = next_item(j);
            if (any_stops(idx < 0, 6, NCOMPUTE)) break;
            const Item it = load_item(p, idx);
            const int kj = it.n0 + r;
            for (int i = 0; i < it.total; ++i, ++t) {
                const int s = t % STAGES;
                const int mb = it.m_first + i % it.per_head;
                const int m0 = mb * BM + QPW * wg;   // the group's first query
                const uint32_t sL_addr = base + SM_L + s * 512 + 4 * QPW * wg;
                const uint32_t sDl_addr = base + SM_DL + s * 512 + 4 * QPW * wg;
                const bool need_mask = (p.causal && m0 < it.n0 + BN) || (it.n0 + BN > it.sq.len);
                float x[QPW];
                // ---- P~^T = exp2(S^T c - L), kept in registers for dS~ and written over S^T ----
                // bf16 has fp32's range, so P~ and dS~ carry the grid's exponent (it comes in with the row
                // statistic s - L); fp16 does not, and the exponent is applied to dQ's fp32 sums at the drain
                CNT_T(t_a);
                mbar_wait<SLEEP_WORKER>(sh.bar(B_QFULL + s), (t / STAGES) & 1, abort_flag, p.status);   // L (long since there)
                float lv[32];
                lds32(sL_addr, lv);   // the first 32 queries' L, in flight under the wait for S^T
                mbar_wait<SLEEP_WORKER>(sh.bar(B_S), t & 1, abort_flag, p.status);
                tc_fence_after();
                CNT_T(t_b);
#pragma unroll
                for (int c = 0; c < QPW / 32; ++c) {
                    uint32_t sv[32];
                    if (c > 0) lds32(sL_addr + 128 * c, lv);
                    tmem_ld32(rs + 32 * c, sv);
                    tmem_wait_ld();
                    uint32_t pp[16];
#pragma unroll
#if FOLD_PACKED_MATH
                    for (int q = 0; q < 32; q += 2)   // lv = s - L, from the preprocess
                        fma2(x[32 * c + q], x[32 * c + q + 1], __uint_as_float(sv[q]), __uint_as_float(sv[q + 1]), c2x2, lv[q], lv[q + 1]);
#else
                    for (int q = 0; q < 32; ++q) x[32 * c + q] = fmaf(__uint_as_float(sv[q]), c2, lv[q]);
#endif
#pragma unroll
                    for (int q = 0; q < 32; ++q) x[32 * c + q] = ex2f(x[32 * c + q]);   // 32 independent ex2 in a row
                    if (need_mask) {   // the diagonal tile and the sequence's last key block only: kept out of the common path
#pragma unroll
                        for (int q = 0; q < 32; ++q) {
                            const int qi = m0 + 32 * c + q;
                            if (kj >= it.sq.len || (p.causal && kj > qi)) x[32 * c + q] = 0.f;
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 32; q += 2)
                        pp[q >> 1] = F16 ? pack_f16x2(x[32 * c + q], x[32 * c + q + 1]) : pack_bf16x2(x[32 * c + q], x[32 * c + q + 1]);
                    tmem_st16(rs + 16 * c, pp);
                }
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(sh.bar(B_P));
                CNT_T(t_c);
                // ---- dS~^T = P~^T (dP^T - Delta) to shared, 16 queries at a time ----
                // dP^T done means dO, and Delta with it, landed (the MMA thread waited for them)
                mbar_wait<SLEEP_WORKER>(sh.bar(B_DP), t & 1, abort_flag, p.status);
                tc_fence_after();
                CNT_T(t_d);
#pragma unroll
                for (int hh = 0; hh < QPW / 16; ++hh) {
                    float dl[16];
                    uint32_t dv[16];
                    lds16(sDl_addr + 64 * hh, dl);
                    tmem_ld16(rd + 16 * hh, dv);
                    tmem_wait_ld();
                    uint32_t dd[8];
#pragma unroll
#if FOLD_PACKED_MATH
                    for (int q = 0; q < 16; q += 2)
                        submul2(dl[q], dl[q + 1], __uint_as_float(dv[q]), __uint_as_float(dv[q + 1]), dl[q], dl[q + 1], x[16 * hh + q], x[16 * hh + q + 1]);
#else
                    for (int q = 0; q < 16; ++q) dl[q] = x[16 * hh + q] * (__uint_as_float(dv[q]) - dl[q]);
#endif
#pragma unroll
                    for (int q = 0; q < 16; q += 2) dd[q >> 1] = F16 ? pack_f16x2(dl[q], dl[q + 1]) : pack_bf16x2(dl[q], dl[q + 1]);
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int cu = (ch0 + 2 * hh + u) ^ (r & 7);
                        *reinterpret_cast<uint4*>(sds + cu * 16) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
                    }
                }
                tc_fence_before();
                fence_async_smem();
                mbar_arrive(sh.bar(B_DS));
#ifdef FOLD_BWD_COUNTERS
                if (counting) {
                    const long long t_e = clock64();
                    c_ws += t_b - t_a;
                    c_exp += t_c - t_b;
                    c_wd += t_d - t_c;
                    c_ds += t_e - t_d;
                }
#endif
            }
            // ---- the item's dK and dV out of TMEM ----
            // The first half of the compute warpgroups takes dK, the second dV (with four, each takes
            // 64 of the 128 channels). Private items (the whole group, the whole query range) write
            // the 16-bit gradients; the others round their sums onto the (request, KV head)'s dK / dV
            // integer grids and add them to the accumulators, where every item of the key block meets.
            CNT_T(t_f);
            mbar_wait<SLEEP_WORKER>(sh.bar(B_DONE), j & 1, abort_flag, p.status);
            tc_fence_after();
            {
                constexpr int PARTS = NWG / 2, CW = HD / PARTS;   // channels per warpgroup
                const bool is_dv = wg >= PARTS;
                const int c0 = (wg % PARTS) * CW;
                const int* st = p.stats + (static_cast<int64_t>(it.b) * p.HKV + it.hkv) * N_STATS;
                const int s_exp = dq_scale_exp(st, root_d(HD));
                const uint32_t src = tmem + lane_addr + (is_dv ? T_DV : T_DK) + c0;
                const bool ok = it.n0 + r < it.sq.len;
                auto pk2 = [](float a, float b2) { return F16 ? pack_f16x2(a, b2) : pack_bf16x2(a, b2); };
                if (NWG == 2 && !p.fold && it.n0 + BN <= it.sq.len) {
                    // A whole key block: the 16-bit tile goes through shared memory in the swizzled layout of
                    // the loads, 64 channels (16 KB) at a time, and one thread per warpgroup stores each half
                    // with TMA: 32 KB in two instructions instead of 2048 scattered 16-byte stores. Each
                    // warpgroup stages in its own half of dS~'s buffer -- the half it alone writes in the dS~
                    // phase, free now that every MMA that read it has retired -- so dK and dV leave side by
                    // side and neither group waits for the other. (A sequence's last, partial block keeps
                    // the per-thread stores below: a tile store would write past the sequence's end in a
                    // packed tensor.)
                    const float un = F16 ? 1.f : pow2f(-s_exp);
                    const float f = is_dv ? un : p.scale * un;
                    const uint32_t buf = base + SM_DS + wg * 16384;
                    const int brow = it.sq.start + it.n0, bb = p.cu ? 0 : it.b;
#pragma unroll
                    for (int box = 0; box < 2; ++box) {
#pragma unroll
                        for (int cc = 0; cc < 2; ++cc) {
                            uint32_t v[32], pk[16];
                            tmem_ld32(src + 64 * box + 32 * cc, v);
                            tmem_wait_ld();
                            if (box == 1 && cc == 1) {   // the last read of the accumulators: the next item may overwrite them
                                tc_fence_before();
                                mbar_arrive(sh.bar(B_ACCFREE));
                            }
#pragma unroll
                            for (int q = 0; q < 32; q += 2) pk[q >> 1] = pk2(__uint_as_float(v[q]) * f, __uint_as_float(v[q + 1]) * f);
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const uint32_t a = buf + r * 128 + (static_cast<uint32_t>((cc * 4 + u) ^ (r & 7)) << 4);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pk[4 * u]), "r"(pk[4 * u + 1]),
                                             "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3]) : "memory");
                            }
                        }
                        fence_async_smem();
                        if (is_dv) asm volatile("bar.sync 3, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
                        if ((warp & 3) == 2 && lane == 0) {   // warps 2 and 6: each group's first warp
                            tma_store_4d(is_dv ? &maps.dv : &maps.dk, buf, 64 * box, brow, it.hkv, bb);
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        }
                        // the half has been read out: the group may stage the next one (or, after the second, its dS~)
                        if (is_dv) asm volatile("bar.sync 3, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
                    }
                } else if (!p.fold) {
                    const float un = F16 ? 1.f : pow2f(-s_exp);
                    const float f = is_dv ? un : p.scale * un;
                    uint16_t* dst = row_ptr<uint16_t>(is_dv ? p.dv : p.dk, it.b, it.sq.start + it.n0 + (ok ? r : 0), it.hkv) + c0;
#pragma unroll
                    for (int c = 0; c < CW / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(src + 32 * c, v);
                        tmem_wait_ld();
                        if (c == CW / 32 - 1) {   // the last read of the accumulators: the next item may overwrite them
                            tc_fence_before();
                            mbar_arrive(sh.bar(B_ACCFREE));
                        }
                        if (ok) {
#pragma unroll
                            for (int q = 0; q < 32; q += 8) {
                                uint4 w;
                                w.x = pk2(__uint_as_float(v[q]) * f, __uint_as_float(v[q + 1]) * f);
                                w.y = pk2(__uint_as_float(v[q + 2]) * f, __uint_as_float(v[q + 3]) * f);
                                w.z = pk2(__uint_as_float(v[q + 4]) * f, __uint_as_float(v[q + 5]) * f);
                                w.w = pk2(__uint_as_float(v[q + 6]) * f, __uint_as_float(v[q + 7]) * f);
                                *reinterpret_cast<uint4*>(dst + 32 * c + q) = w;
                            }
                        }
                    }
                } else {
                    // dK~ and dV~ carry the dQ grid's exponent (bf16) or none (fp16); their own grids'
                    // exponents come from the same maxima, so every item of the key block agrees
                    const float rows = static_cast<float>(p.G) * static_cast<float>(it.sq.len);
                    const int e = (is_dv ? dv_scale_exp(st, rows, p.dv_bits == 32 ? DQ_BITS : DKV_BITS) : dk_scale_exp(st, rows, root_d(HD))) -
                                  (F16 ? 0 : s_exp);
                    const int64_t off = (static_cast<int64_t>(it.hkv) * p.rows_p + it.sq.pstart + it.n0 + r) * HD + c0;
                    const bool narrow = is_dv && p.dv_bits == 32;
#pragma unroll
                    for (int c = 0; c < CW / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(src + 32 * c, v);
                        tmem_wait_ld();
                        if (c == CW / 32 - 1) {
                            tc_fence_before();
                            mbar_arrive(sh.bar(B_ACCFREE));
                        }
                        if (ok) {
                            if (narrow) {
                                int* acc = static_cast<int*>(p.dv_acc) + off + 32 * c;
#pragma unroll
                                for (int q = 0; q < 32; ++q)
                                    asm volatile("red.global.add.s32 [%0], %1;" ::"l"(acc + q), "r"(__float2int_rn(scale_pow2(__uint_as_float(v[q]), e))) : "memory");
                            } else {
                                unsigned long long* acc = static_cast<unsigned long long*>(is_dv ? p.dv_acc : static_cast<void*>(p.dk_acc)) + off + 32 * c;
#pragma unroll
                                for (int q = 0; q < 32; ++q)
                                    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(acc + q),
                                                 "l"(static_cast<unsigned long long>(__float2ll_rn(scale_pow2(__uint_as_float(v[q]), e)))) : "memory");
                            }
                        }
                    }
                }
            }
#ifdef FOLD_BWD_COUNTERS
            if (counting) c_epi += clock64() - t_f;
#endif
        }
        if ((warp & 3) == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the tile stores have landed
#ifdef FOLD_BWD_COUNTERS
        if (counting) {
            CNT_ADD(5, c_ws);
            CNT_ADD(6, c_exp);
            CNT_ADD(7, c_wd);
            CNT_ADD(8, c_ds);
            CNT_ADD(4, c_epi);
        }
#endif
    } else {
        // ================= dQ drain: TMEM -> int32 grid -> shared -> TMA add into the accumulator =================
        // The tile's int32 values are staged 16 KB at a time in one of two shared buffers and one
        // thread hands each block to the TMA engine as a reduction (integer add, so the order of
        // arrival does not matter): the same bytes as 128 `red` instructions per thread, without
        // their place in the instruction queue the compute warps' ex2 and shared loads go through.
        // The next tile's dP^T cannot be issued until this tile's dQ~ has left its columns, so the
        // time from B_DQF to B_DQE is on the kernel's critical path: blocks are converted with
        // short dependency chains and stored with as few instructions as the layout allows.
        const int ln = 32 * (warp & 3) + lane;   // TMEM lane: a query (FOLD_BWD_DRAIN_T) or a channel
        float dq_mul = 1.f;   // fp16: the grid's exponent, applied here (per item)
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const uint32_t rd = tmem + lane_addr + T_DP;
        const bool leader = (warp == W_DRAIN && lane == 0);   // issues every reduction: they form its groups
        // Float -> int32, round to nearest even. Adding 1.5 * 2^23 rounds a float below 2^22 to an
        // integer in its low mantissa bits: one add and one subtract per element when every
        // element of the warp's block is in that range (the usual case: the grid leaves 2^30 to
        // a row's whole sum), which keeps the conversion off the pipe the softmax's ex2 runs on.
        // With FOLD_BWD_BIAS the subtract is left to the accumulator's starting value.
        auto to_grid = [&](uint32_t (&v)[32]) {
            constexpr float M = 12582912.f;   // 1.5 * 2^23, bits 0x4B400000
            constexpr uint32_t MB = 0x4B400000u, KEEP = FOLD_BWD_BIAS ? MB : 0u;
            float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;   // four short chains, not one of 32
#pragma unroll
            for (int q = 0; q < 32; q += 4) {
                if (F16) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[q + u] = __float_as_uint(__uint_as_float(v[q + u]) * dq_mul);
                }
                m0 = fmaxf(m0, fabsf(__uint_as_float(v[q])));
                m1 = fmaxf(m1, fabsf(__uint_as_float(v[q + 1])));
                m2 = fmaxf(m2, fabsf(__uint_as_float(v[q + 2])));
                m3 = fmaxf(m3, fabsf(__uint_as_float(v[q + 3])));
            }
            const float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            if (!__any_sync(0xffffffffu, !(mx < 4194304.f))) {
#pragma unroll
                for (int q = 0; q < 32; q += 2) {
                    uint64_t t;
                    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(t) : "l"(pack2(__uint_as_float(v[q]), __uint_as_float(v[q + 1]))), "l"(pack2(M, M)));
                    uint32_t lo, hi;
                    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(t));
                    v[q] = lo - (MB - KEEP);
                    v[q + 1] = hi - (MB - KEEP);
                }
            } else {   // rare, and kept small: the conversion instruction (same rounding; it shares a pipe with ex2)
#pragma unroll
                for (int q = 0; q < 32; ++q) v[q] = static_cast<uint32_t>(__float2int_rn(__uint_as_float(v[q]))) + KEEP;
            }
        };
#if FOLD_BWD_DRAIN_T
        // block c of a tile: channels 32c .. 32c+31 of all 128 queries, [query][32 ch] int32, 128 bytes
        // per query with its 16-byte units XOR-swizzled by the query (SWIZZLE_128B, what the tensor
        // map expects): a quarter warp's eight stores of one unit fall in eight different bank groups
        const uint32_t stg = base + SM_STG + ln * 128;
        const uint32_t sw = static_cast<uint32_t>(ln & 7);
        auto stage = [&](int buf, uint32_t (&v)[32], int c, int row0) {
            to_grid(v);
            // the buffer's last block (two blocks ago) must have been read out
            if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const uint32_t dst = stg + buf * 16384;
#pragma unroll
            for (uint32_t u = 0; u < 8; ++u)
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + ((u ^ sw) << 4)), "r"(v[4 * u]), "r"(v[4 * u + 1]),
                             "r"(v[4 * u + 2]), "r"(v[4 * u + 3]) : "memory");
            fence_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (leader) {
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&maps.dq), "r"(32 * c), "r"(row0), "r"(base + SM_STG + buf * 16384) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        };
#else
        // block c of a tile: queries 32c .. 32c+31, all 128 channels, in the accumulator's own row-major order
        const uint32_t stg = base + SM_STG + 4 * ln;
        auto stage = [&](int buf, uint32_t (&v)[32], int c, int row0) {
            to_grid(v);
            if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const uint32_t dst = stg + buf * 16384;
#pragma unroll
            for (int q = 0; q < 32; ++q)   // row q of the block: 128 channels, one per thread
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + q * 512), "r"(v[q]) : "memory");
            fence_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (leader) {
                int* gdst = p.dq_acc + (static_cast<int64_t>(row0) + 32 * c) * HD;
                asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.s32 [%0], [%1], %2;"
                             ::"l"(gdst), "r"(base + SM_STG + buf * 16384), "r"(16384) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        };
#endif
#ifdef FOLD_BWD_COUNTERS
        long long c_wq = 0, c_busy = 0, c_rel = 0;
#endif
        int t = 0;
        for (int j = 0;; ++j) {
          const int idx = next_item(j);
          if (any_stops(idx < 0, 7, 128)) break;
          const Item it = load_item(p, idx);
          if (F16) dq_mul = pow2f(dq_scale_exp(p.stats + (static_cast<int64_t>(it.b) * p.HKV + it.hkv) * N_STATS, root_d(HD)));
          for (int i = 0; i < it.total; ++i, ++t) {
            const int g = i / it.per_head, mb = it.m_first + i % it.per_head;
            const int h = it.hkv * p.G + it.h0 + g;
            // the tile's first row in the accumulator [H * padded rows][128 ch]
            const int row0 = static_cast<int>(static_cast<int64_t>(h) * p.rows_p + it.sq.pstart + mb * BM);
            CNT_T(t_a);
            mbar_wait<SLEEP_WORKER>(sh.bar(B_DQF), t & 1, abort_flag, p.status);
            tc_fence_after();
            CNT_T(t_b);
            if constexpr (NWG == 2) {
                // three of the four blocks in registers: the columns are released after the first is staged
                uint32_t v0[32], v1[32], v2[32];
                tmem_ld32(rd, v0);
                tmem_ld32(rd + 32, v1);
                tmem_ld32(rd + 64, v2);
                tmem_wait_ld();
                stage(0, v0, 0, row0);
                tmem_ld32(rd + 96, v0);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(sh.bar(B_DQE));   // the rest of the tile is in registers: the columns are free for dP^T of the next tile
#ifdef FOLD_BWD_COUNTERS
                c_rel += clock64() - t_b;
#endif
                stage(1, v1, 1, row0);
                stage(0, v2, 2, row0);
                stage(1, v0, 3, row0);
            } else {
                // 22 warps leave a thread 80 registers: two blocks in registers at a time
                uint32_t v0[32], v1[32];
                tmem_ld32(rd, v0);
                tmem_ld32(rd + 32, v1);
                tmem_wait_ld();
                stage(0, v0, 0, row0);
                tmem_ld32(rd + 64, v0);
                tmem_wait_ld();
                stage(1, v1, 1, row0);
                tmem_ld32(rd + 96, v1);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(sh.bar(B_DQE));
#ifdef FOLD_BWD_COUNTERS
                c_rel += clock64() - t_b;
#endif
                stage(0, v0, 2, row0);
                stage(1, v1, 3, row0);
            }
#ifdef FOLD_BWD_COUNTERS
            c_wq += t_b - t_a;
            c_busy += clock64() - t_b;
#endif
          }
        }
        // the engine must be done with shared memory, and the adds complete, before the CTA goes
        if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
#ifdef FOLD_BWD_COUNTERS
        if (leader) {
            CNT_ADD(10, c_wq);
            CNT_ADD(11, c_busy);
            CNT_ADD(12, c_rel);
        }
#endif
    }

    // every role has left its loop: no MMA, load or reduction of this CTA is in flight
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
    if (tid == 0) {
        CNT_ADD(2, clock64() - cta_t0);
        // the last CTA to finish puts both counters back, so the next launch (or a graph replay) starts from zero
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            p.sched[0] = 0;
            p.sched[1] = 0;
            __threadfence();
        }
    }
}

// ---- the work list ---------------------------------------------------------------------
// One entry per (request, KV head, subgroup of query heads, key block, record of query blocks):
// eight ints (key block, KV head, request, first head of the subgroup, heads, first and
// one-past-last query block, cost in tiles). Entries are grouped in sections of `sec`
// (request, KV head, subgroup) triples -- the CTAs running at any time then share few heads' Q,
// dO and dQ, which stay in L2 -- and sorted by cost, longest first, inside each section, so
// that the persistent CTAs end every section, and the launch, on short items. The last sections
// are merged into one that holds about a wave of the longest items (one per SM), so the launch's
// last long items start while there is still a wave of work behind them. Built on the
// device from cu_seqlens, in-stream: no host synchronisation, and a captured graph replays it.
constexpr int WL_BINS = 1024;
__global__ void __launch_bounds__(256) bwd_work_list_kernel(const BwdParams p, int n_trip, int nsub, int nb_max, int nrec, int sec,
                                                            int tail_trip) {
    __shared__ int hist[WL_BINS];
    __shared__ int offs[WL_BINS];
    // the last block sorts the merged tail (the last `tail_trip` triples as one section)
    const bool tail = blockIdx.x == gridDim.x - 1;
    const int body = n_trip - tail_trip;
    const int t0 = tail ? body : blockIdx.x * sec, t1 = tail ? n_trip : min(t0 + sec, body);
    const int per = nb_max * nrec;
    const int count = (t1 - t0) * per;
    int* out = const_cast<int*>(p.work) + static_cast<int64_t>(t0) * per * 8;
    for (int i = threadIdx.x; i < WL_BINS; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    auto describe = [&](int li, int (&w)[8]) {
        const int trip = t0 + li / per, rem = li % per;
        const int nb = rem / nrec, rec = rem % nrec;
        const int b = trip / (p.HKV * nsub), hkv = (trip / nsub) % p.HKV, sub = trip % nsub;
        const SeqInfo sq = seq_info(p, b);
        const int nm = (sq.len + BM - 1) / BM;
        const int m_lo = p.record > 0 ? rec * p.record : 0;
        const int m_hi = p.record > 0 ? (rec + 1) * p.record : nm;
        const int first = max(p.causal ? nb : 0, m_lo);
        const int blocks = (nb * BN < sq.len) ? max(min(nm, m_hi) - first, 0) : 0;
        w[0] = nb; w[1] = hkv; w[2] = b; w[3] = sub * p.subgroup; w[4] = p.subgroup;
        w[5] = m_lo; w[6] = m_hi; w[7] = blocks * p.subgroup;
    };
    for (int li = threadIdx.x; li < count; li += blockDim.x) {
        int w[8];
        describe(li, w);
        atomicAdd(&hist[min(w[7], WL_BINS - 1)], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int c = WL_BINS - 1; c >= 0; --c) {
            offs[c] = at;
            at += hist[c];
        }
    }
    __syncthreads();
    for (int li = threadIdx.x; li < count; li += blockDim.x) {
        int w[8];
        describe(li, w);
        const int pos = atomicAdd(&offs[min(w[7], WL_BINS - 1)], 1);   // the order among equal costs is free: no bit depends on it
        int4* o = reinterpret_cast<int4*>(out + static_cast<int64_t>(pos) * 8);
        o[0] = make_int4(w[0], w[1], w[2], w[3]);
        o[1] = make_int4(w[4], w[5], w[6], w[7]);
    }
}

}  // namespace sm100

// ---- host side -------------------------------------------------------------------
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    }
    return fn;
}

// (channel, row, head, batch) view of a (batch, row, head, channel)-strided bf16 tensor
bool make_map(CUtensorMap* m, const TensorView& t, int64_t rows, int heads, int batch, int box_rows, bool f16) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(sm100::HD), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
    const int64_t sb = t.sb ? t.sb : t.sr * rows;
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(t.sr * 2), static_cast<cuuint64_t>(t.sh * 2),
                             static_cast<cuuint64_t>(sb * 2)};
    cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// the int32 dQ accumulator [H * padded rows][128 ch] as (channel, row), boxes of 32 channels x 128 rows
bool make_acc_map(CUtensorMap* m, const BwdParams& p) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(sm100::HD), static_cast<cuuint64_t>(p.H) * static_cast<cuuint64_t>(p.rows_p)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(sm100::HD) * 4};
    cuuint32_t box[2] = {32, 128};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, p.dq_acc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool bwd_sm100_biased() { return FOLD_BWD_BIAS != 0; }

namespace {
struct ListShape {
    int nsub, nb_max, nrec;
    int64_t n_trip, n_items;
};
ListShape list_shape(int B, int H, int HKV, int S, int subgroup, int record) {
    ListShape l;
    l.nsub = (H / HKV) / subgroup;
    l.nb_max = (S + sm100::BN - 1) / sm100::BN;
    l.nrec = record > 0 ? (l.nb_max + record - 1) / record : 1;
    l.n_trip = static_cast<int64_t>(B) * HKV * l.nsub;
    l.n_items = l.n_trip * l.nb_max * l.nrec;
    return l;
}
}  // namespace

int64_t bwd_sm100_work_items(int B, int H, int HKV, int S, int subgroup, int record) {
    return list_shape(B, H, HKV, S, subgroup, record).n_items;
}

bool bwd_sm100_supported(const BwdParams& p) {
    return p.D == 128 && encode_fn() != nullptr;
}

int launch_bwd_main_sm100(const BwdParams& p, bool build_list, bool run_main, cudaStream_t st) {
    sm100::Maps maps;
    const bool varlen = p.cu != nullptr;
    const int64_t rows = varlen ? p.total : p.S;
    const int batch = varlen ? 1 : p.B;
    const bool f16 = p.f16;
    if (!make_map(&maps.q, p.q, rows, p.H, batch, sm100::BM, f16) || !make_map(&maps.dout, p.dout, rows, p.H, batch, sm100::BM, f16) ||
        !make_map(&maps.k, p.k, rows, p.HKV, batch, sm100::BN, f16) || !make_map(&maps.v, p.v, rows, p.HKV, batch, sm100::BN, f16) ||
        !make_map(&maps.dk, p.dk, rows, p.HKV, batch, sm100::BN, f16) || !make_map(&maps.dv, p.dv, rows, p.HKV, batch, sm100::BN, f16) ||
        !make_acc_map(&maps.dq, p)) {
        set_error("bwd_main_sm100: cuTensorMapEncodeTiled failed");
        return FOLD_ERR_LAUNCH;
    }
    // The work list, then one persistent CTA per SM claiming from it. Sections: as many (request,
    // KV head, subgroup) triples as keep their Q, dO (16-bit) and dQ accumulator (int32) within a
    // share of L2 that leaves room for K, V and the other sections' tails.
    const ListShape l = list_shape(p.B, p.H, p.HKV, p.S, p.subgroup, p.record);
    if (l.n_items != p.n_items || l.n_items > (1ll << 30)) {
        set_error("bwd_main_sm100: a work list of %lld items, %d laid out", static_cast<long long>(l.n_items), p.n_items);
        return FOLD_ERR_ARGUMENT;
    }
    constexpr int64_t kSectionBytes = 48ll << 20;
    const int64_t trip_bytes = static_cast<int64_t>(p.S) * sm100::HD * (2 + 2 + 4) * p.subgroup;
    const int sec = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(kSectionBytes / std::max<int64_t>(trip_bytes, 1), 64)));
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    // the merged tail: a triple holds about nb (nb + 1) / 2 blocks per head under a causal mask and its
    // longest item nb, so a wave of longest items is 2 * SMs / (nb + 1) triples; within twice the budget
    const int64_t wave = (2ll * sms[dev] + l.nb_max) / (l.nb_max + 1);
    const int tail_trip = static_cast<int>(std::min<int64_t>(l.n_trip, std::max<int64_t>(sec, std::min<int64_t>(wave, 2 * kSectionBytes / std::max<int64_t>(trip_bytes, 1)))));
    const int n_sections = static_cast<int>((l.n_trip - tail_trip + sec - 1) / sec) + 1;
    if (build_list)
        sm100::bwd_work_list_kernel<<<n_sections, 256, 0, st>>>(p, static_cast<int>(l.n_trip), l.nsub, l.nb_max, l.nrec, sec, tail_trip);
    if (!run_main) return check_launch("bwd_work_list");
    const int grid = static_cast<int>(std::min<int64_t>(std::max(sms[dev], 1), l.n_items));
    if (f16) {
        auto kern = sm100::bwd_main_sm100_kernel<true>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm100::SMEM_BYTES);
        kern<<<grid, sm100::NTHREADS, sm100::SMEM_BYTES, st>>>(p, maps);
    } else {
        auto kern = sm100::bwd_main_sm100_kernel<false>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm100::SMEM_BYTES);
        kern<<<grid, sm100::NTHREADS, sm100::SMEM_BYTES, st>>>(p, maps);
    }
    return check_launch("bwd_main_sm100");
}

}  // namespace fold

extern "C" int fold_bwd_counters(uint64_t* out24, int reset) {
#ifdef FOLD_BWD_COUNTERS
    FOLD_CHECK_ARG(out24, "fold_bwd_counters: null pointer");
    unsigned long long h[24];
    if (cudaMemcpyFromSymbol(h, fold::sm100::g_counters, sizeof(h)) != cudaSuccess) return fold::check_launch("fold_bwd_counters");
    for (int i = 0; i < 24; ++i) out24[i] = h[i];
    if (reset) {
        memset(h, 0, sizeof(h));
        if (cudaMemcpyToSymbol(fold::sm100::g_counters, h, sizeof(h)) != cudaSuccess) return fold::check_launch("fold_bwd_counters");
    }
    return FOLD_OK;
#else
    (void)out24;
    (void)reset;
    fold::set_error("fold_bwd_counters: the library was built without -DFOLD_BWD_COUNTERS");
    return FOLD_ERR_UNSUPPORTED;
#endif
}

extern "C" int fold_wait_probe(long long limit_cycles, int32_t* status, int32_t* flag_out, void* stream) {
    FOLD_CHECK_ARG(status, "fold_wait_probe: null pointer");
    FOLD_CHECK_ARG(limit_cycles > 0 && limit_cycles <= (1ll << 31), "fold_wait_probe: a limit of %lld cycles (1 .. 2^31)", limit_cycles);
    fold::sm100::wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, status, flag_out);
    return fold::check_launch("fold_wait_probe");
}
