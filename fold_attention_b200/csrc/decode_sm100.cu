// Quantised paged-KV decode on Blackwell tensor cores (tcgen05 + TMEM), head dim 128,
// pages of a multiple of 128 keys; described for an 8-bit V (two E4M3 planes). A bf16 V
// runs the same schedule with a 256-byte row per key: 16 keys per kind::f16 MMA, the
// weight as two bf16 terms (hi, lo), no second plane, 4-slot rings.
//
// The warp-level kernel in decode.cu spends 49 warp instructions per key and is
// issue-bound at about a third of HBM bandwidth. Here a tile is 128 keys, the
// cache's planes stream through a ring of shared-memory stages by bulk copy
// and TMA with nothing in the way that depends on a verdict, and every product
// is one tcgen05.mma per 32 keys:
//   L  = Ka Q^T    kind::i8      M=128 keys, N=16 (Qa rows | Qb rows), K=32   -> TMEM int32
//   O^T += Va^T W  kind::f8f6f4  M=128 channels, N=32, K=32 keys; A = E4M3 V as stored,
//                                B = the weights as four E5M2 terms per query row
// so V is never converted: the tensor core reads the cache's own bytes. A key is
// one TMEM lane, so its 8 logits sit in one thread and the verdict (live /
// refine-K / refine-V, ORed over the group) needs no shuffle. Plane A of V is read
// for every key of a tile (a dropped key meets a zero weight): at the depths this
// kernel is chosen for nearly every key is live, and a stream has no gather latency.
//
// A weight w = exp2(s - Z) >= 0 is carried as 64 w = t1 + t2/8 + t3/64 + t4/512
// with every t an E5M2 number (each term is the rounding error of the sum before
// it, times 8): 12 bits of mantissa with E5M2's 32 binades of range; the
// denominator takes the fp32 weight.
//
// Plane B of V, where a 32-key quarter of a tile holds at least DENSE_MIN keys inside
// the refine-V gate, is fetched whole for that quarter (4 KB by TMA, two tiles ahead
// of its use) and meets the same weights, masked to those keys, in a second
// accumulator:  O2^T += Vb^T W2  (scaled by 1/8 at the end).
//
// The keys that need more than that leave the tensor-core path: a key inside the
// refine-K gate (its logits need plane B of K), a key inside the refine-V gate in a
// quarter with few of them, or a key whose weight could pass 2^8 (E5M2 ends at
// 57344) gets weight zero in W and is handed, tile by tile through bit masks in
// shared memory, to the helper warps (seven for an 8-bit V, four for a 16-bit one). A helper
// recomputes the key's logits from both planes with dp4a, takes the weight in
// fp32 and adds w (Va + Vb/8) into its own fp32 accumulators; tile t always goes
// to helper t mod NHELP and keys are taken in position order, so the sums are the
// same on every run. The partial is the tensor-core sum plus the helpers' sums.
// The helper count is what a CTA of a short request waits for: there a tenth or
// more of the keys are inside the gates, the stream is done long before the
// helpers, and the other warps idle until the helpers' last key.
// So a request of up to 8192 keys streams both planes of K (a pair of ring slots a
// tile, 32 TMEM columns of logits): its refine-K keys read their second-plane
// logits from TMEM and stay on the tensor-core path. That is a second build of the
// kernel's body, chosen at the kernel's top by the request's length alone.
//
// Warps: 0 and 2 producers (two 4-slot rings: K's plane A by bulk copy; plane A of V
// by TMA with the 128-byte swizzle, with the key scales), 1 and 3 MMA issuers (logits; values. 256 TMEM
// columns), 4-7 and 8-11 one thread per key of the even and of the odd tiles, 12 and up the
// helpers, and for an 8-bit V one more warp that issues plane B's MMAs as its quarters land. A K slot is free again as soon as its logits are out, a V slot when its
// value product has retired. Every wait is bounded (about a second); on expiry
// a status word is raised, nobody waits any more, TMEM is freed and the kernel returns.
// Arithmetic contract: src/fold_attention/decode/kernel.py:774-870, 1032-1201,
// 1400-1476 (the schedule and the weight format are this kernel's own).
#include <cuda.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"
#include "fold_b200.h"

namespace fold {
namespace dsm100 {

#ifndef FOLD_DEC_RING
#define FOLD_DEC_RING 4
#endif
#ifndef FOLD_DEC_HDK
#define FOLD_DEC_HDK 4
#endif
constexpr int TK = 128;          // keys per tile
constexpr int HD = 128;
#ifndef FOLD_DEC_QD
#define FOLD_DEC_QD 32
#endif
// tiles of helper masks in flight: how far a helper may fall behind the key threads (its tiles come
// every NHELP-th, with a bursty number of keys each) before they have to wait for it
constexpr int QD = FOLD_DEC_QD;
#ifndef FOLD_DEC_HPASS
#define FOLD_DEC_HPASS 1
#endif
// requests up to this many keys stream both planes of K: their gates are the wide ones (a tenth of the keys
// inside refine-K), and the second plane's logits from the tensor core cost less than the helpers (0: never)
#ifndef FOLD_DEC_BOTHK
#define FOLD_DEC_BOTHK 8192
#endif
constexpr int BOTHK_LEN = FOLD_DEC_BOTHK;
#ifndef FOLD_DEC_NHELP
#define FOLD_DEC_NHELP 7
#endif
#ifndef FOLD_DEC_RING_K
#define FOLD_DEC_RING_K 4
#endif
constexpr int HSLOT = 528;       // a staging slot: Ka, Kb, Va, Vb rows of 128 bytes, the scale's word, the key's note
constexpr int NBQ = 8;            // tiles of quarter flags (and their barrier) in flight: more than the key threads can lead by
#ifndef FOLD_DEC_NB2
#define FOLD_DEC_NB2 3
#endif
// tiles of plane B of V (and their masked weights) in flight. A key group takes every other tile; with two
// buffers it would need its own last tile's buffer back, whose quarters are a DRAM latency away
constexpr int NB2 = FOLD_DEC_NB2;
// 1: groups of exactly eight rows take a build of their own
#ifndef FOLD_DEC_G8
#define FOLD_DEC_G8 1
#endif
#ifndef FOLD_DEC_DENSE_MIN
#define FOLD_DEC_DENSE_MIN 3
#endif
// refine-K keys in a 32-key quarter from which their threads refine them in place (33: never). Never for an
// 8-bit V: that build runs 19 warps at 96 registers, and the call's presence alone costs its loop a quarter
#ifndef FOLD_DEC_INL
#define FOLD_DEC_INL 8
#endif
#ifndef FOLD_DEC_INL_V8
#define FOLD_DEC_INL_V8 33
#endif
constexpr int DENSE_MIN = FOLD_DEC_DENSE_MIN;   // refine-V keys in a 32-key quarter from which the quarter's plane B is fetched whole
constexpr long long WAIT_CYCLES = 1ll << 31;
// -DFOLD_DEC_COUNTERS: every role adds the cycles it spends in each of its waits, and in all, to
// global counters fold_decode_counters returns (a measurement build: the waits cost two clock reads)
#ifdef FOLD_DEC_COUNTERS
__device__ unsigned long long g_dec_counters[32];
#define CW(slot, call) do { const long long cw_t = clock64(); call; cntl[slot] += clock64() - cw_t; } while (0)
#define CW_DECL long long cntl[32] = {}; const long long cw_t0 = clock64(); (void)cw_t0
#define CW_FLUSH(total_slot) do { cntl[total_slot] += clock64() - cw_t0; for (int cw_i = 0; cw_i < 32; ++cw_i) if (cntl[cw_i]) atomicAdd(&g_dec_counters[cw_i], static_cast<unsigned long long>(cntl[cw_i])); } while (0)
#define CW_ADD(slot, v) cntl[slot] += (v)
#else
#define CW(slot, call) call
#define CW_DECL
#define CW_FLUSH(total_slot)
#define CW_ADD(slot, v)
#endif
constexpr float BIG_TOP = 8.0f;  // a key whose weight could pass 2^8 is summed in fp32 by a helper
constexpr int W_BIAS = 6;        // weights are stored times 2^6: under 2^14 on the tensor-core path

// shared memory map (1024-aligned base) and barrier numbers; an 8-bit V is two E4M3 planes of
// 128 bytes per key (plane B fetched on demand), a 16-bit V one bf16 row of 256 bytes
constexpr int SM_Q = 0;                               // [16 rows][128 B] int8, SW128
constexpr int HOUT = (8 * 128 + 8) * 4;               // a helper's sums: [8 rows][128 channels], [8] floats
template <bool V8>
struct Lay {
    static constexpr int NA = V8 ? FOLD_DEC_RING_K : 4; // ring slots of K's plane A (and logit buffers in TMEM)
    static constexpr int NHELP = V8 ? FOLD_DEC_NHELP : 4;   // helper warps
    static constexpr int NTHREADS = 384 + 32 * NHELP + (V8 ? 32 : 0);   // an 8-bit V: one more warp issues plane B's MMAs
    static constexpr int NV = V8 ? FOLD_DEC_RING : 4;   // ring slots of V (plane A) and the key scales
    static constexpr int VBYTES = V8 ? 16384 : 32768; // a V slot: [128 keys][128 B], or two 64-channel boxes of that
    static constexpr int NB2E = V8 ? NB2 : 0;
    // keys whose rows a helper has in flight into its staging slots: four random 128-byte reads a key, each
    // about a microsecond away, so the depth of this queue is what the helpers' rate comes to
    static constexpr int HD_KEYS = V8 ? FOLD_DEC_HDK : 8;
    static constexpr int HPASS = V8 ? FOLD_DEC_HPASS : 4;          // keys a helper takes in one pass, when that many are in flight
    static constexpr int SM_KA = 2048;                           // NA x Ka [128 keys][128 B]
    static constexpr int SM_VA = SM_KA + NA * 16384;             // NV x V slots
    static constexpr int SM_VB = SM_VA + NV * VBYTES;            // NB2 x Vb [128 keys][128 B], fetched by quarters
    static constexpr int SM_KS = SM_VB + NB2E * 16384;           // NV x 128 bf16 scales
    static constexpr int SM_W = SM_KS + NV * 256;                // 2 x [2 units][128 keys][16 B] weights
    static constexpr int SM_W2 = SM_W + 2 * 4096;                // NB2 x the same, masked to the dense refine-V keys
    static constexpr int SM_QM = SM_W2 + NB2E * 4096;            // QD x { refine-K, refine-V, helper } x 4 mask words, the tile's first pool row
    static constexpr int SM_QF = SM_QM + QD * 64;                // NBQ x 4 quarter flags
    static constexpr int SM_EQZ = SM_QF + NBQ * 16;              // eq[8], z[8] of the row group
    static constexpr int SM_ROW = SM_EQZ + 64;                   // NV x the first pool row of the tile in the V slot (the producer's page lookup, shared)
    static constexpr int SM_HST = (SM_ROW + 8 * NV + 15) / 16 * 16;  // NHELP x HD_KEYS staging slots
    static constexpr int SM_BAR = SM_HST + NHELP * HD_KEYS * HSLOT;
    // after the last MMA the rings are dead and hold the final reduction: 256 x 16 row sums,
    // 8 x 16 partial and 16 full column sums, per-warp counters; and the helpers' sums
    static constexpr int SM_RED = SM_KA;
    static constexpr int SM_CNT = SM_KA + (256 + 8 + 1) * 16 * 4;
    static constexpr int SM_HOUT = SM_VA;
    static constexpr int SMEM_BYTES = SM_BAR + (QD > 8 ? 1024 : 512);
    static_assert(SMEM_BYTES <= 232448, "over the 227 KB a CTA may hold");
    static_assert(NA == 4, "four logit buffers of 32 TMEM columns; with both planes of K the ring is two pairs of slots");
    static_assert(NA * 16384 >= SM_CNT - SM_KA + 1024 && NV * VBYTES >= NHELP * HOUT, "the final reduction fits the dead rings");
    enum {
        B_AFULL = 0,                 // [NA] K's plane A has landed
        B_LFULL = B_AFULL + NA,      // [NA] the tile's logit MMAs retired: its logits are in TMEM slot t % NA, its K slot is free
        B_VFULL = B_LFULL + NA,      // [NV] V's plane A and the scales have landed
        B_VEMPTY = B_VFULL + NV,     // [NV] the tile's value MMAs retired: its V slot and its weight buffer are free
        B_WREADY = B_VEMPTY + NV,    // [2] 128 arrivals: the tile's weights are in shared memory
        B_QFULL = B_WREADY + 2,      // [QD] 4 arrivals: the tile's masks are written
        B_QFREE = B_QFULL + QD,      // [QD] its helper has read them
        B_BFULL = B_QFREE + QD,      // [NBQ] 4 arrivals (+ bytes): the tile's quarters of plane B have landed
        B_BFREE = B_BFULL + NBQ,     // [NB2] its plane-B MMAs retired
        B_ALLDONE = B_BFREE + NB2,   // the last value MMAs retired
        B_COUNT = B_ALLDONE + 1,
    };
};

constexpr uint32_t T_L = 0, T_ACC = 128, T_ACC2 = 160;   // TMEM columns: 4 logit buffers of 16 + 16 (plane A of K, plane B), then the accumulators

struct Params {
    const int8_t* qa; const int8_t* qb; const float* eq;
    const int8_t* ka; const int8_t* kb; const uint16_t* ek;
    const uint8_t* va; const uint8_t* vb;
    const float* vmean; const float* z; const float* cut;
    const int* page_table; const int* seq_lens; const int* order;
    float* o_part; float* den_part; int* cnt_part;
    int nbh, G, hkv, ppr, page_size, split, chunk_keys, truncate, banded;
    float rk, rv, band_e0, band_e1, rk1, rk2, rv1, rv2;
    int* status;
};

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
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
    if (mbar_try(bar, parity)) return;   // the usual case costs one instruction
    if (*abort_flag) return;
    const long long t0 = clock64();
    for (int i = 0;; ++i) {
        if (mbar_try(bar, parity)) return;
        if ((i & 63) == 63) {
            if (*abort_flag) return;
            if (clock64() - t0 > WAIT_CYCLES) break;
        }
    }
    *abort_flag = 1;
    atomicExch(status, FOLD_ERR_TIMEOUT);
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src, int bytes /* 16 or 0: zero fill */) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_f8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// four MMAs over a tile's K steps in one go: the first overwrites or accumulates as `acc0`
// says, the rest accumulate; the descriptors advance by DA, DB (16-byte units) per step
template <int DA, int DB>
__device__ __forceinline__ void mma4_i8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{ .reg .pred p0, p1; .reg .b64 a1, b1;\n"
        "setp.ne.b32 p0, %4, 0; setp.eq.b32 p1, %4, %4;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p0;\n"
        "add.u64 a1, %1, %5; add.u64 b1, %2, %6;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %3, p1;\n"
        "add.u64 a1, a1, %5; add.u64 b1, b1, %6;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %3, p1;\n"
        "add.u64 a1, a1, %5; add.u64 b1, b1, %6;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %3, p1; }"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc0), "n"(DA), "n"(DB) : "memory");
}
template <int DA, int DB>
__device__ __forceinline__ void mma4_f8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{ .reg .pred p0, p1; .reg .b64 a1, b1;\n"
        "setp.ne.b32 p0, %4, 0; setp.eq.b32 p1, %4, %4;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p0;\n"
        "add.u64 a1, %1, %5; add.u64 b1, %2, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a1, b1, %3, p1;\n"
        "add.u64 a1, a1, %5; add.u64 b1, b1, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a1, b1, %3, p1;\n"
        "add.u64 a1, a1, %5; add.u64 b1, b1, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a1, b1, %3, p1; }"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc0), "n"(DA), "n"(DB) : "memory");
}
template <int DA, int DB>
__device__ __forceinline__ void mma4_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{ .reg .pred p0, p1; .reg .b64 a1, b1;\n"
        "setp.ne.b32 p0, %4, 0; setp.eq.b32 p1, %4, %4;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n"
        "add.u64 a1, %1, %5; add.u64 b1, %2, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n"
        "add.u64 a1, a1, %5; add.u64 b1, b1, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n"
        "add.u64 a1, a1, %5; add.u64 b1, b1, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1; }"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc0), "n"(DA), "n"(DB) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two floats -> packed E5M2 pair (lo in the low byte), round to nearest, saturating
__device__ __forceinline__ uint32_t cvt_e5m2x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// an E5M2 byte is the high byte of an fp16
__device__ __forceinline__ float e5m2_to_float(uint32_t b) {
    return __half2float(__ushort_as_half(static_cast<uint16_t>((b & 0xFFu) << 8)));
}

// four E4M3 bytes -> floats
__device__ __forceinline__ void e4m3x4_to_float(uint32_t v, float (&f)[4]) {
    uint32_t lo, hi;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"(static_cast<uint16_t>(v & 0xFFFFu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"(static_cast<uint16_t>(v >> 16)));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// shared-memory matrix descriptor; layout 2 = 128-byte swizzle, 0 = none
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= static_cast<uint64_t>(layout) << 61;
    return d;
}
// instruction descriptor: c_fmt (1 f32, 2 s32), a/b formats, majors (0 K, 1 MN), N, M
__host__ __device__ constexpr uint32_t instr_desc(int c_fmt, int a_fmt, int b_fmt, int a_mn, int b_mn, int N, int M) {
    return (static_cast<uint32_t>(c_fmt) << 4) | (static_cast<uint32_t>(a_fmt) << 7) |
           (static_cast<uint32_t>(b_fmt) << 10) | (static_cast<uint32_t>(a_mn) << 15) |
           (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
           (static_cast<uint32_t>(M >> 4) << 24);
}

// GC: the group's rows when the kernel is compiled for them (8: the per-row guards fold away, and the key
// threads' instruction stream is what the tile rate comes to: -6.6 % step time on an 8-bit V at depth 16),
// 0: read from p. A build for groups of four measured no gain on a dense bf16 V, which is HBM-bound, and a
// build of the tile body without the last tile's row guards lost 1 % to its size.
// A key's part of its eight logits that comes from K's plane B: kb . qa + kb . qb / 256 per query row, as
// the helpers compute it. A call of its own, so that the registers it needs are found on the rare path
// that takes it and not in the key threads' loop.
struct Corr8 { float v[8]; };
__device__ __noinline__ Corr8 refine_k(const uint4* kbrow, const uint8_t* q, int k, int G) {
    int ca[8], cb[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) ca[g] = cb[g] = 0;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
        uint4 kb4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) kb4[j] = __ldg(kbrow + 4 * half + j);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int lu = (4 * half + j) ^ (k & 7);   // the row's 16-byte units are stored swizzled by its slot
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g < G) {
                    const int off = g * 128 + ((lu ^ g) << 4);
                    const uint4 qa4 = *reinterpret_cast<const uint4*>(q + off);
                    const uint4 qb4 = *reinterpret_cast<const uint4*>(q + 1024 + off);
                    ca[g] = __dp4a(static_cast<int>(kb4[j].x), static_cast<int>(qa4.x), ca[g]);
                    ca[g] = __dp4a(static_cast<int>(kb4[j].y), static_cast<int>(qa4.y), ca[g]);
                    ca[g] = __dp4a(static_cast<int>(kb4[j].z), static_cast<int>(qa4.z), ca[g]);
                    ca[g] = __dp4a(static_cast<int>(kb4[j].w), static_cast<int>(qa4.w), ca[g]);
                    cb[g] = __dp4a(static_cast<int>(kb4[j].x), static_cast<int>(qb4.x), cb[g]);
                    cb[g] = __dp4a(static_cast<int>(kb4[j].y), static_cast<int>(qb4.y), cb[g]);
                    cb[g] = __dp4a(static_cast<int>(kb4[j].z), static_cast<int>(qb4.z), cb[g]);
                    cb[g] = __dp4a(static_cast<int>(kb4[j].w), static_cast<int>(qb4.w), cb[g]);
                }
            }
        }
    }
    Corr8 x;
#pragma unroll
    for (int g = 0; g < 8; ++g) x.v[g] = static_cast<float>(ca[g]) + static_cast<float>(cb[g]) * (1.0f / 256.0f);
    return x;
}

// The kernel's body, built twice: for requests that stream plane A of K alone, and (BOTHK) for short
// requests, which stream both planes. Two bodies and a branch at the kernel's top, because the first
// one's loop, at the 96 registers its 19 warps leave, loses a quarter of its speed to the second's code
// when the two share a body.
template <bool TRUNC, bool V8, int GC, bool BOTHK>
__device__ __forceinline__ void decode_sm100_body(const Params& p, const CUtensorMap* vmap_p, const CUtensorMap* vbmap_p) {
    using L = Lay<V8>;
    constexpr int NA = L::NA, NHELP = L::NHELP, NV = L::NV, VBYTES = L::VBYTES, HD_KEYS = L::HD_KEYS, HPASS = L::HPASS;
    constexpr int SM_KA = L::SM_KA, SM_VA = L::SM_VA, SM_VB = L::SM_VB, SM_KS = L::SM_KS, SM_W = L::SM_W, SM_W2 = L::SM_W2,
                  SM_QM = L::SM_QM, SM_QF = L::SM_QF, SM_EQZ = L::SM_EQZ, SM_ROW = L::SM_ROW, SM_HST = L::SM_HST, SM_BAR = L::SM_BAR,
                  SM_RED = L::SM_RED, SM_CNT = L::SM_CNT, SM_HOUT = L::SM_HOUT;
    constexpr int B_AFULL = L::B_AFULL, B_LFULL = L::B_LFULL, B_VFULL = L::B_VFULL, B_VEMPTY = L::B_VEMPTY,
                  B_WREADY = L::B_WREADY, B_QFULL = L::B_QFULL, B_QFREE = L::B_QFREE, B_BFULL = L::B_BFULL,
                  B_BFREE = L::B_BFREE, B_ALLDONE = L::B_ALLDONE, B_COUNT = L::B_COUNT;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    auto bar = [&](int i) { return base + SM_BAR + 8 * i; };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 8 * B_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 8 * B_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot = blockIdx.x / p.split, sp = blockIdx.x % p.split;
    const int bh = p.order ? p.order[slot] : slot;
    const int breq = bh / p.hkv, hkv = bh % p.hkv;
    const int slen = p.seq_lens[breq];
    const int G = GC ? GC : p.G, PS = p.page_size;

    int lo, hi, tstep, n_tiles;
    if (p.chunk_keys > 0) {
        lo = sp * p.chunk_keys;
        hi = min(lo + p.chunk_keys, slen);
        tstep = TK;
        n_tiles = hi > lo ? (hi - lo + TK - 1) / TK : 0;
        if (n_tiles == 0) return;
    } else {
        lo = sp * TK;
        hi = slen;
        tstep = p.split * TK;
        const int all = (slen + TK - 1) / TK;
        n_tiles = all > sp ? (all - sp + p.split - 1) / p.split : 0;
    }
    if (base & 1023u) {
        if (tid == 0) atomicExch(p.status, FOLD_ERR_LAUNCH);
        return;
    }
    const int64_t pix = static_cast<int64_t>(bh) * p.split + sp;
    float rk = p.rk, rv = p.rv;
    if (p.banded) {
        rk = slen > static_cast<int>(p.band_e1) ? p.rk2 : (slen > static_cast<int>(p.band_e0) ? p.rk1 : p.rk);
        rv = slen > static_cast<int>(p.band_e1) ? p.rv2 : (slen > static_cast<int>(p.band_e0) ? p.rv1 : p.rv);
    }

    // both planes of K for a short request: a tile takes a pair of ring slots (plane A, plane B), its
    // logits 32 TMEM columns; the refine-K keys' second-plane part is read from there
    constexpr bool bothk = BOTHK;

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < NA; ++i) {
            mbar_init(bar(B_AFULL + i), 1);
            mbar_init(bar(B_LFULL + i), 1);
        }
        for (int i = 0; i < NV; ++i) {
            mbar_init(bar(B_VFULL + i), 1);
            mbar_init(bar(B_VEMPTY + i), 1);
        }
        for (int i = 0; i < 2; ++i) mbar_init(bar(B_WREADY + i), 128);
        for (int i = 0; i < QD; ++i) {
            mbar_init(bar(B_QFULL + i), 4);
            mbar_init(bar(B_QFREE + i), 1);
        }
        for (int i = 0; i < NBQ; ++i) mbar_init(bar(B_BFULL + i), 4);
        for (int i = 0; i < NB2; ++i) mbar_init(bar(B_BFREE + i), 1);
        mbar_init(bar(B_ALLDONE), V8 ? 2 : 1);   // the value MMA thread's commit, and the plane-B thread's
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Q planes -> shared, 16 rows of 128 bytes with the 128-byte swizzle; rows
    // 0-7 plane A of query rows 0-7, rows 8-15 plane B; rows past G are zero
    if (tid < 128) {
        const int row = tid >> 3, u = tid & 7;          // 16 rows x 8 sixteen-byte units
        const int g = row & 7;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (g < G) {
            const int8_t* src = (row < 8 ? p.qa : p.qb) + (static_cast<int64_t>(bh) * G + g) * HD + u * 16;
            val = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(smem + SM_Q + row * 128 + ((u ^ (row & 7)) << 4)) = val;
    }
    if (tid >= 128 && tid < 144) {
        const int g = tid & 7;
        const int64_t ix = static_cast<int64_t>(bh) * G + (g < G ? g : 0);
        reinterpret_cast<float*>(smem + SM_EQZ)[tid - 128] = tid < 136 ? p.eq[ix] : p.z[ix];
    }
    fence_async_smem();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;"
                     ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(tmem_slot))) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int* ptab = p.page_table + static_cast<int64_t>(breq) * p.ppr;
    // first pool row of the tile that starts at position `pos` (a tile lies inside one page)
    auto tile_row = [&](int pos) -> int64_t {
        const int pg = pos / PS;
        return (static_cast<int64_t>(__ldg(ptab + pg)) * p.hkv + hkv) * PS + (pos - pg * PS);
    };

    if (warp == 0) {
        // ================= producer: K's plane A =================
        if (lane == 0) {
            CW_DECL;
            CW_ADD(0, 1);
            for (int t = 0; t < n_tiles; ++t) {
                const int64_t r = tile_row(lo + t * tstep);
                if (bothk) {
                    // the pair was tile t-2's, free once that tile's logits are out (tile t+2, which shares
                    // the barrier, cannot have run: its K is not loaded yet)
                    const int s = 2 * (t & 1);
                    if (t >= 2) CW(12, mbar_wait(bar(B_LFULL + (t - 2) % NA), ((t - 2) / NA) & 1, abort_flag, p.status));
                    mbar_expect_tx(bar(B_AFULL + s), 32768);
                    bulk_load(base + SM_KA + s * 16384, p.ka + r * HD, 16384, bar(B_AFULL + s));
                    bulk_load(base + SM_KA + (s + 1) * 16384, p.kb + r * HD, 16384, bar(B_AFULL + s));
                } else {
                    const int s = t % NA;
                    if (t >= NA) CW(12, mbar_wait(bar(B_LFULL + s), ((t / NA) - 1) & 1, abort_flag, p.status));
                    mbar_expect_tx(bar(B_AFULL + s), 16384);
                    bulk_load(base + SM_KA + s * 16384, p.ka + r * HD, 16384, bar(B_AFULL + s));
                }
            }
            CW_FLUSH(13);
        }
    } else if (warp == 2) {
        // ================= producer: V's plane A and the key scales =================
        if (lane == 0) {
            CW_DECL;
            for (int t = 0; t < n_tiles; ++t) {
                const int s = t % NV;
                if (t >= NV) CW(14, mbar_wait(bar(B_VEMPTY + s), ((t / NV) - 1) & 1, abort_flag, p.status));
                const int64_t r = tile_row(lo + t * tstep);
                reinterpret_cast<volatile int64_t*>(smem + SM_ROW)[s] = r;   // released by the arrive below, read after the wait on it
                mbar_expect_tx(bar(B_VFULL + s), VBYTES + 256);
                bulk_load(base + SM_KS + s * 256, p.ek + r, 256, bar(B_VFULL + s));
                tma_load_2d(base + SM_VA + s * VBYTES, vmap_p, 0, static_cast<int>(r), bar(B_VFULL + s));
                if (!V8) tma_load_2d(base + SM_VA + s * VBYTES + 16384, vmap_p, 64, static_cast<int>(r), bar(B_VFULL + s));
            }
            CW_FLUSH(15);
        }
    } else if (warp == 1) {
        // ================= MMA issuer: logits =================
        if (lane == 0) {
            constexpr uint32_t ID_L = instr_desc(2, 1, 1, 0, 0, 16, 128);    // s8 x s8 -> s32
            // descriptors of slot 0; a slot or K step further is an addition
            const uint64_t dq = smem_desc(base + SM_Q, 16, 1024, 2);
            const uint64_t dka = smem_desc(base + SM_KA, 16, 1024, 2);
            CW_DECL;
            for (int t = 0; t < n_tiles; ++t) {
                const int lb = t % NA;   // the logit buffer
                // the TMEM buffer was tile t-NA's: its value MMAs retired, so its weights were done and
                // its logits read
                if (t >= NA) CW(16, mbar_wait(bar(B_VEMPTY + (t - NA) % NV), ((t - NA) / NV) & 1, abort_flag, p.status));
                if (bothk) {
                    const int s = 2 * (t & 1);
                    CW(17, mbar_wait(bar(B_AFULL + s), (t >> 1) & 1, abort_flag, p.status));
                    tc_fence_after();
                    mma4_i8<2, 2>(tmem + T_L + 32 * lb, dka + s * 1024, dq, ID_L, 0u);
                    mma4_i8<2, 2>(tmem + T_L + 32 * lb + 16, dka + (s + 1) * 1024, dq, ID_L, 0u);
                } else {
                    const int s = t % NA;
                    CW(17, mbar_wait(bar(B_AFULL + s), (t / NA) & 1, abort_flag, p.status));
                    tc_fence_after();
                    mma4_i8<2, 2>(tmem + T_L + 32 * lb, dka + s * 1024, dq, ID_L, 0u);   // 32 bytes per K step
                }
                tc_commit(bar(B_LFULL + lb));
            }
            CW_FLUSH(18);
        }
    } else if (warp == 3) {
        // ================= MMA issuer: values =================
        if (lane == 0) {
            // an 8-bit V: e4m3 x e5m2 -> f32, N = 4 terms x 8 rows; a 16-bit V: bf16 x bf16 -> f32, N = 2 terms x 8 rows;
            // both operands MN-major
            constexpr uint32_t ID_V = V8 ? instr_desc(1, 0, 1, 1, 1, 32, 128) : instr_desc(1, 1, 1, 1, 1, 16, 128);
            const uint64_t dva = smem_desc(base + SM_VA, 16384, 1024, 2);
            const uint64_t dw = smem_desc(base + SM_W, 128, 2048, 0);
            CW_DECL;
            for (int t = 0; t < n_tiles; ++t) {
                {
                    const int s = t % NV;
                    CW(20, mbar_wait(bar(B_VFULL + s), (t / NV) & 1, abort_flag, p.status));
                    CW(21, mbar_wait(bar(B_WREADY + (t & 1)), (t >> 1) & 1, abort_flag, p.status));
                    tc_fence_after();
                    if (V8) {
                        // 32 keys per K step: 4096 bytes of V, 512 bytes of weights
                        mma4_f8<256, 32>(tmem + T_ACC, dva + s * (VBYTES >> 4), dw + (t & 1) * 256, ID_V, t > 0 ? 1u : 0u);
                    } else {
                        // 16 keys per K step: 2048 bytes of V in each 64-channel box, 256 bytes of weights
                        mma4_f16<128, 16>(tmem + T_ACC, dva + s * (VBYTES >> 4), dw + (t & 1) * 256, ID_V, t > 0 ? 1u : 0u);
                        mma4_f16<128, 16>(tmem + T_ACC, dva + s * (VBYTES >> 4) + 512, dw + (t & 1) * 256 + 64, ID_V, 1u);
                    }
                    tc_commit(bar(B_VEMPTY + s));
                }
            }
            tc_commit(bar(B_ALLDONE));
            CW_FLUSH(22);
        }
    } else if (warp >= 4 && warp < 12) {
        // ================= one thread per key; two groups take the even and the odd tiles =================
        const int wg = (warp - 4) >> 2;
        const int k = (tid - 128) & 127;                 // key in the tile = TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        float eqr[8], zr[8], cutr[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const int64_t ix = static_cast<int64_t>(bh) * G + (g < G ? g : 0);
            eqr[g] = p.eq[ix];
            zr[g] = p.z[ix];
            cutr[g] = -p.cut[ix];
        }
        float rN[8], rM[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) rN[g] = rM[g] = 0.f;
        int nlive = 0, nref = 0;
        bool any_dense = false;
        uint32_t* qm = reinterpret_cast<uint32_t*>(smem + SM_QM);
        CW_DECL;
        for (int t = wg; t < n_tiles; t += 2) {
            if ((warp & 3) == 0) CW_ADD(1, 1);
            const int s = t % NV;
            const int tb = lo + t * tstep;
            const int nrow = min(TK, hi - tb);
            CW(3, mbar_wait(bar(B_VFULL + s), (t / NV) & 1, abort_flag, p.status));   // the scales ride with V
            CW(4, mbar_wait(bar(B_LFULL + t % NA), (t / NA) & 1, abort_flag, p.status));
            tc_fence_after();
            uint32_t c[16];
            tmem_ld16(tmem + lane_addr + T_L + 32 * (t % NA), c);
            tmem_wait_ld();
            tc_fence_before();
            const bool valid = k < nrow;
            const int64_t tile_row0 = reinterpret_cast<const volatile int64_t*>(smem + SM_ROW)[s];
            const float ek = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(smem + SM_KS + s * 256)[k]) * (1.0f / 256.0f);
            float s1[8];
            float top = -INFINITY;
            bool live = !TRUNC;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                s1[g] = -INFINITY;
                if (g < G && valid) {
                    const float tk = eqr[g] * ek;
                    s1[g] = fmaf(static_cast<float>(static_cast<int>(c[g]) * 256 + static_cast<int>(c[8 + g])), tk, -zr[g]);
                    if (TRUNC && s1[g] >= cutr[g]) live = true;
                    top = fmaxf(top, s1[g]);
                }
            }
            live = live && valid;
            const bool refk = live && top >= -rk;
            // A quarter (this warp's 32 keys) with enough refine-K keys refines them in place: each such
            // key's thread reads its own row of K's plane B and adds the second plane's part to its eight
            // logits (the helper's arithmetic, on lanes that would wait for the helper otherwise); the
            // key then stays on the tensor-core path. Which keys do depends on the logits alone.
            bool refined_here = false;
            if (bothk && __any_sync(0xffffffffu, refk)) {
                // the second plane's logits are in the buffer's other 16 columns: kb . qa and kb . qb per row
                tc_fence_after();
                tmem_ld16(tmem + lane_addr + T_L + 32 * (t % NA) + 16, c);
                tmem_wait_ld();
                tc_fence_before();
                if (refk) {
                    top = -INFINITY;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        if (g < G) {
                            const float x = static_cast<float>(static_cast<int>(c[g])) + static_cast<float>(static_cast<int>(c[8 + g])) * (1.0f / 256.0f);
                            s1[g] = s1[g] + x * (eqr[g] * ek);
                            top = fmaxf(top, s1[g]);
                        }
                    }
                    refined_here = true;
                }
            }
            constexpr int INL_MIN = V8 ? FOLD_DEC_INL_V8 : FOLD_DEC_INL;
            if (INL_MIN <= 32 && !bothk && nrow == TK && __popc(__ballot_sync(0xffffffffu, refk)) >= INL_MIN) {
                if (refk) {
                    const Corr8 x = refine_k(reinterpret_cast<const uint4*>(p.kb + (tile_row0 + k) * HD), smem + SM_Q, k, G);
                    top = -INFINITY;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        if (g < G) {
                            s1[g] = s1[g] + x.v[g] * (eqr[g] * ek);
                            top = fmaxf(top, s1[g]);
                        }
                    }
                    refined_here = true;
                }
                __syncwarp();
            }
            const bool needk = refk && !refined_here;   // still needs plane B of K: a helper's
            // a 16-bit V has no second plane, and bf16 weights no range to run out of
            const bool refv = V8 && live && top >= -rv;
            const bool big = V8 && live && top >= BIG_TOP;
            // a quarter with enough refine-V keys fetches its plane B whole; so does one of the last,
            // partial tile (its rows past the range lie in the tile's page; the plane-B thread clears them)
            const bool dv = refv && !needk && !big;
            const bool dense = __popc(__ballot_sync(0xffffffffu, dv)) >= DENSE_MIN;
            any_dense = any_dense || dense;
            const bool helped = needk || big || (refv && !dense);
            nlive += live ? 1 : 0;
            nref += refk ? 1 : 0;
            // a helper will want this key's second planes some tiles from now: start them towards L2
            if (needk || refv) {
                const int64_t row = tile_row0 + k;
                if (needk) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.kb + row * HD));
                if (V8 && refv && !dense) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.vb + row * HD));
            }
            const unsigned mk = __ballot_sync(0xffffffffu, refk);
            const unsigned mv = __ballot_sync(0xffffffffu, refv);
            const unsigned mh = __ballot_sync(0xffffffffu, helped);
            if (t >= 2) CW(5, mbar_wait(bar(B_VEMPTY + (t - 2) % NV), ((t - 2) / NV) & 1, abort_flag, p.status));   // the weight buffer is free
            // a row past the group and a key past the tile have s1 = -inf: weight 0 without a guard. A key's
            // eight weights all go one way: to the dropped mass, to a helper, or into W and the denominator
            float w[8];
#pragma unroll
            for (int g = 0; g < 8; ++g) w[g] = ex2f(s1[g]);
            const bool plain = live && !helped;
            if (TRUNC && !live) {
#pragma unroll
                for (int g = 0; g < 8; ++g) rM[g] += w[g];
            }
            if (plain) {
#pragma unroll
                for (int g = 0; g < 8; ++g) rN[g] += w[g];
            }
            uint32_t wb[8];
            if (V8) {
                // four E5M2 terms per weight: bytes [term][row]. The chain runs in fp16, two rows
                // at a time: an E5M2 number is the high byte of an fp16, the differences are exact
#pragma unroll
                for (int g = 0; g < 8; g += 2) {
                    __half2 r = plain ? __floats2half2_rn(w[g] * static_cast<float>(1 << W_BIAS), w[g + 1] * static_cast<float>(1 << W_BIAS))
                                      : __floats2half2_rn(0.f, 0.f);
#pragma unroll
                    for (int term = 0; term < 4; ++term) {
                        uint16_t pk;
                        asm("cvt.rn.satfinite.e5m2x2.f16x2 %0, %1;" : "=h"(pk) : "r"(*reinterpret_cast<const uint32_t*>(&r)));
                        const int word = term * 2 + (g >> 2), sh = (g & 3) * 8;   // byte term*8 + g (and g+1)
                        if (g == 0 || g == 4) wb[word] = static_cast<uint32_t>(pk) << sh; else wb[word] |= static_cast<uint32_t>(pk) << sh;
                        const uint32_t qb = __byte_perm(static_cast<uint32_t>(pk), 0u, 0x1404);
                        r = __hmul2(__hsub2(r, *reinterpret_cast<const __half2*>(&qb)), __floats2half2_rn(8.0f, 8.0f));
                    }
                }
            } else {
                // two bf16 terms per weight, w = hi + lo with lo = bf16(w - hi): unit 0 the eight
                // rows' hi, unit 1 their lo (decode/kernel.py:1181-1189)
#pragma unroll
                for (int g = 0; g < 8; g += 2) {
                    const float w0 = plain ? w[g] : 0.f, w1 = plain ? w[g + 1] : 0.f;
                    const uint32_t hi = pack_bf16x2(w0, w1);
                    const float r0 = w0 - __uint_as_float(hi << 16), r1 = w1 - __uint_as_float(hi & 0xFFFF0000u);
                    wb[g >> 1] = hi;
                    wb[4 + (g >> 1)] = pack_bf16x2(r0, r1);
                }
            }
            uint8_t* wdst = smem + SM_W + (t & 1) * 4096 + k * 16;
            *reinterpret_cast<uint4*>(wdst) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
            *reinterpret_cast<uint4*>(wdst + 2048) = make_uint4(wb[4], wb[5], wb[6], wb[7]);
            if (!valid) {
                // rows past the range hold whatever the pool holds (an E4M3 NaN times a zero
                // weight is a NaN): clear them
                uint4* vrow = reinterpret_cast<uint4*>(smem + SM_VA + s * VBYTES + k * 128);
#pragma unroll
                for (int u = 0; u < 8; ++u) vrow[u] = make_uint4(0, 0, 0, 0);
                if (!V8) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) vrow[1024 + u] = make_uint4(0, 0, 0, 0);   // the second 64-channel box
                }
            }
            fence_async_smem();
            mbar_arrive(bar(B_WREADY + (t & 1)));
            // plane B of V for this quarter, and the weights it meets. The flags and their barrier
            // have more slots than the key threads can run ahead of the plane-B thread; the data
            // buffers are three tiles deep
            if (V8) {
                const int b2 = t % NB2, bq = t % NBQ;
                // Every tile waits for the plane-B thread to be done with tile t-NB2, dense or not: that is
                // what bounds its lag (the flags' ring is deeper), and what keeps the parity test honest:
                // at its last tile, t-2, this group waited for tile t-2-NB2's buffer; the thread commits in
                // order, so the older tile t-2*NB2's phase is complete and the test cannot pass a phase early
                if (lane == 0 && t >= NB2) CW(6, mbar_wait(bar(B_BFREE + b2), ((t / NB2) - 1) & 1, abort_flag, p.status));
                __syncwarp();
                if (dense) {
                    uint8_t* w2dst = smem + SM_W2 + b2 * 4096 + k * 16;
                    *reinterpret_cast<uint4*>(w2dst) = dv ? make_uint4(wb[0], wb[1], wb[2], wb[3]) : make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(w2dst + 2048) = dv ? make_uint4(wb[4], wb[5], wb[6], wb[7]) : make_uint4(0, 0, 0, 0);
                    fence_async_smem();
                    __syncwarp();
                }
                if (lane == 0) {
                    reinterpret_cast<volatile int*>(smem + SM_QF + bq * 16)[warp & 3] = dense ? 1 : 0;
                    if (dense) {
                        mbar_expect_tx(bar(B_BFULL + bq), 4096);
                        tma_load_2d(base + SM_VB + b2 * 16384 + 4096 * (warp & 3), vbmap_p, 0,
                                    static_cast<int>(tile_row0) + 32 * (warp & 3), bar(B_BFULL + bq));
                    } else {
                        mbar_arrive(bar(B_BFULL + bq));
                    }
                }
            }
            // hand the keys that need fp32 to the tile's helper
            if (lane == 0) {
                const int q = t % QD;
                if (t >= QD) CW(7, mbar_wait(bar(B_QFREE + q), ((t / QD) - 1) & 1, abort_flag, p.status));
                qm[q * 16 + (warp & 3)] = mk;
                qm[q * 16 + 4 + (warp & 3)] = mv;
                qm[q * 16 + 8 + (warp & 3)] = mh;
                if ((warp & 3) == 0) *reinterpret_cast<int64_t*>(qm + q * 16 + 12) = tile_row0;   // the helper's page lookup, done
                mbar_arrive(bar(B_QFULL + q));
            }
            __syncwarp();
                }

        // ---- epilogue: the first group's thread k is channel k of the output ----
        if (lane == 0) CW_FLUSH(2);
        if (n_tiles > 0) CW(23, mbar_wait(bar(B_ALLDONE), 0, abort_flag, p.status));
        tc_fence_after();
        float* sRed = reinterpret_cast<float*>(smem + SM_RED);
        const int kk2 = wg * 128 + k;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            sRed[kk2 * 16 + g] = rN[g];
            sRed[kk2 * 16 + 8 + g] = rM[g];
        }
        int* sCnt = reinterpret_cast<int*>(smem + SM_CNT);   // per key warp: live, refined, any dense quarter
        {
            const int a = __reduce_add_sync(0xffffffffu, nlive), b = __reduce_add_sync(0xffffffffu, nref);
            if (lane == 0) {
                sCnt[3 * (warp - 4)] = a;
                sCnt[3 * (warp - 4) + 1] = b;
                sCnt[3 * (warp - 4) + 2] = any_dense ? 1 : 0;
            }
        }
        asm volatile("bar.sync 2, %0;" ::"n"(256 + 32 * NHELP) : "memory");   // both groups' sums, and the helpers'
        if (wg == 0) {
            // column sums in a fixed order: 8 runs of 32 entries, then the 8 partial sums
            {
                const int col = k & 15, part = k >> 4;
                float sum = 0.f;
                for (int i = 0; i < 32; ++i) sum += sRed[(part * 32 + i) * 16 + col];
                sRed[(256 + part) * 16 + col] = sum;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (k < 16) {
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) sum += sRed[(256 + i) * 16 + k];
                sRed[(256 + 8) * 16 + k] = sum;
            }
            bool use_b = false;
#pragma unroll
            for (int i = 0; i < 8; ++i) use_b = use_b || sCnt[3 * i + 2] != 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            uint32_t a0[16], a1[16], b0[16], b1[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) a0[i] = a1[i] = b0[i] = b1[i] = 0u;   // an empty range never wrote the accumulators
            if (n_tiles > 0) {
                tmem_ld16(tmem + lane_addr + T_ACC, a0);
                if (V8) tmem_ld16(tmem + lane_addr + T_ACC + 16, a1);
                if (V8 && use_b) {
                    tmem_ld16(tmem + lane_addr + T_ACC2, b0);
                    tmem_ld16(tmem + lane_addr + T_ACC2 + 16, b1);
                }
                tmem_wait_ld();
            }
            tc_fence_before();
            const float* hout = reinterpret_cast<const float*>(smem + SM_HOUT);
            const float vm = (TRUNC && p.vmean) ? p.vmean[static_cast<int64_t>(bh) * HD + k] : 0.f;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g < G) {
                    float x;
                    if (V8) {
                        x = __uint_as_float(a0[g]) + __uint_as_float(a0[8 + g]) * 0.125f +
                            __uint_as_float(a1[g]) * (1.0f / 64.0f) + __uint_as_float(a1[8 + g]) * (1.0f / 512.0f);
                        x += 0.125f * (__uint_as_float(b0[g]) + __uint_as_float(b0[8 + g]) * 0.125f +
                                       __uint_as_float(b1[g]) * (1.0f / 64.0f) + __uint_as_float(b1[8 + g]) * (1.0f / 512.0f));
                        x *= 1.0f / static_cast<float>(1 << W_BIAS);
                    } else {
                        x = __uint_as_float(a0[g]) + __uint_as_float(a0[8 + g]);   // the hi and the lo terms' products
                    }
#pragma unroll
                    for (int h = 0; h < NHELP; ++h) x += hout[h * (HOUT / 4) + g * 128 + k];
                    x += sRed[(256 + 8) * 16 + 8 + g] * vm;
                    p.o_part[(pix * G + g) * HD + k] = x;
                }
            }
            if (k < G) {
                float d = sRed[(256 + 8) * 16 + k] + sRed[(256 + 8) * 16 + 8 + k];
#pragma unroll
                for (int h = 0; h < NHELP; ++h) d += hout[h * (HOUT / 4) + 8 * 128 + k];
                p.den_part[pix * G + k] = d;
            }
            if (k == 0) {
                int a = 0, bcount = 0;
                for (int i = 0; i < 8; ++i) { a += sCnt[3 * i]; bcount += sCnt[3 * i + 1]; }
                p.cnt_part[pix * 2] = a;
                p.cnt_part[pix * 2 + 1] = bcount;
            }
        }
    } else if (V8 && warp == 12 + NHELP) {
        // ================= MMA issuer: plane B of V, tile by tile as its quarters land =================
        // A thread of its own: behind the value products in one thread, a quarter still on its way held
        // the next tile's value product back, and with it the key threads' weight buffer.
        // Lane 0 waits and issues; the whole warp clears the rows past the range in the last, partial
        // tile's buffer once they have landed (what the pool holds there may read as an E4M3 NaN, and a
        // NaN times a zero weight is a NaN): without it that tile's refine-V keys, a third of a short
        // request's last tile, would all be one helper's, after everything else is done.
        {
            constexpr uint32_t ID_V = instr_desc(1, 0, 1, 1, 1, 32, 128);
            const uint64_t dvb = smem_desc(base + SM_VB, 16384, 1024, 2);
            const uint64_t dw2 = smem_desc(base + SM_W2, 128, 2048, 0);
            bool acc2_started = false;
            const int nrow_last = n_tiles > 0 ? min(TK, hi - (lo + (n_tiles - 1) * tstep)) : TK;
            CW_DECL;
            for (int t = 0; t < n_tiles; ++t) {
                const int b2 = t % NB2;
                if (lane == 0) CW(19, mbar_wait(bar(B_BFULL + t % NBQ), (t / NBQ) & 1, abort_flag, p.status));
                __syncwarp();
                const volatile uint32_t* qfp = reinterpret_cast<const volatile uint32_t*>(smem + SM_QF + (t % NBQ) * 16);
                const uint32_t f[4] = {qfp[0], qfp[1], qfp[2], qfp[3]};
                const bool any = (f[0] | f[1] | f[2] | f[3]) != 0u;
                if (any && t == n_tiles - 1 && nrow_last < TK) {
                    uint4* vbrow = reinterpret_cast<uint4*>(smem + SM_VB + b2 * 16384);   // [128 keys][8 units], swizzled within a row
                    for (int i = nrow_last * 8 + lane; i < TK * 8; i += 32) vbrow[i] = make_uint4(0, 0, 0, 0);
                    fence_async_smem();
                    __syncwarp();
                }
                if (lane == 0) {
                    if (any) {
                        tc_fence_after();
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            if (f[ks]) {
                                mma_f8(tmem + T_ACC2, dvb + b2 * 1024 + ks * 256, dw2 + b2 * 256 + ks * 32, ID_V, acc2_started);
                                acc2_started = true;
                            }
                        }
                    }
                    tc_commit(bar(B_BFREE + b2));
                }
            }
            if (lane == 0) {
                tc_commit(bar(B_ALLDONE));
                CW_FLUSH(29);
            }
        }
    } else if (warp >= 12 && warp < 12 + NHELP) {
        // ================= helpers: the keys that need both planes or an fp32 weight =================
        // The whole warp works on one key. Its four rows (both planes of K and of V) come into a
        // staging slot with one 16-byte copy per lane, four keys ahead of their use. For the
        // logits lane l is query row l & 7 and the quarter l >> 3 of the 128 channels: it holds
        // that part of Q's two planes, multiplies it with the key's, and two shuffles sum the
        // quarters. For the value sum every lane takes the eight weights and adds them into its
        // four channels. Keys are taken in (tile, position) order whatever the timing.
        const int h = warp - 12;
        const int hg = lane & 7, part = lane >> 3;
        int qaw[8], qbw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int lu = 2 * part + (i >> 2);   // logical 16-byte unit, word i & 3 of it
            const int off = ((lu ^ hg) << 4) + 4 * (i & 3);
            qaw[i] = *reinterpret_cast<const int*>(smem + SM_Q + hg * 128 + off);
            qbw[i] = *reinterpret_cast<const int*>(smem + SM_Q + (8 + hg) * 128 + off);
        }
        const float* eqz = reinterpret_cast<const float*>(smem + SM_EQZ);
        const float eq_l = eqz[hg], z_l = eqz[8 + hg];
        float acc[8][4], hden = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) acc[g][cc] = 0.f;
        }
        const uint32_t* qm = reinterpret_cast<const uint32_t*>(smem + SM_QM);
        uint8_t* stage = smem + SM_HST + h * HD_KEYS * HSLOT;
        const uint32_t stage_a = base + SM_HST + h * HD_KEYS * HSLOT;
        // the plane this lane copies from, and its bytes per key: K's two planes, then V's two
        // planes (8-bit) or the two halves of V's bf16 row
        const uint8_t* plane_l = part == 0 ? reinterpret_cast<const uint8_t*>(p.ka)
                               : part == 1 ? reinterpret_cast<const uint8_t*>(p.kb)
                               : (V8 ? (part == 2 ? p.va : p.vb) : (part == 2 ? p.va : p.va + 128));
        const int row_bytes_l = (!V8 && part >= 2) ? 256 : HD;

        // issue side: the tile whose marked keys are being handed out
        CW_DECL;
        int it = h;                       // next tile to open
        uint32_t mK[4] = {0, 0, 0, 0}, mV[4] = {0, 0, 0, 0}, mH[4] = {0, 0, 0, 0};
        int wi = 4;                       // word of mH in hand (4: none left)
        uint32_t rem = 0u;
        int64_t row0 = 0;
        int issued = 0, taken = 0;        // keys copied for, keys summed
        bool open_tiles = n_tiles > h;

        // one more key's rows on their way, if a key is to be had without waiting (or with, when
        // `block` says nothing else is left to do); false when no key came
        auto issue_one = [&](bool block) -> bool {
            while (true) {
                while (rem == 0u && wi < 3) {
                    ++wi;
                    rem = wi == 1 ? mH[1] : (wi == 2 ? mH[2] : mH[3]);
                }
                if (rem != 0u) break;
                if (!open_tiles) return false;
#ifdef FOLD_DEC_COUNTERS
                const long long cw_o0 = clock64();
#endif
                // open the next tile's masks
                const int q = it % QD;
                if (!mbar_try(bar(B_QFULL + q), (it / QD) & 1)) {
                    if (!block) return false;
                    CW(9, mbar_wait(bar(B_QFULL + q), (it / QD) & 1, abort_flag, p.status));
                    if (*abort_flag) { open_tiles = false; return false; }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    mK[i] = qm[q * 16 + i];
                    mV[i] = qm[q * 16 + 4 + i];
                    mH[i] = qm[q * 16 + 8 + i];
                }
                row0 = *reinterpret_cast<const int64_t*>(qm + q * 16 + 12);
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_QFREE + q));
                wi = 0;
                rem = mH[0];
                it += NHELP;
                open_tiles = it < n_tiles;
#ifdef FOLD_DEC_COUNTERS
                cntl[26] += clock64() - cw_o0;
                cntl[28] += 1;
#endif
            }
#ifdef FOLD_DEC_COUNTERS
            const long long cw_k0 = clock64();
#endif
            const int b = __ffs(rem) - 1;
            rem &= rem - 1;
            const int kk = 32 * wi + b;
            const uint32_t bit = 1u << b;
            const uint32_t wK = wi == 0 ? mK[0] : (wi == 1 ? mK[1] : (wi == 2 ? mK[2] : mK[3]));
            const uint32_t wV = wi == 0 ? mV[0] : (wi == 1 ? mV[1] : (wi == 2 ? mV[2] : mV[3]));
            const bool isK = (wK & bit) != 0u, isV = (wV & bit) != 0u;
            const int64_t row = row0 + kk;
            const int slot_i = issued % HD_KEYS;
            const uint32_t dst = stage_a + slot_i * HSLOT;
            // lane l copies unit l & 7 of plane l >> 3; a plane the key does not need is zero-filled
            const int need = part == 1 ? (isK ? 16 : 0) : ((V8 && part == 3) ? (isV ? 16 : 0) : 16);
            cp_async(dst + 128 * part + 16 * hg, plane_l + row * row_bytes_l + 16 * hg, need);
            if (lane == 0) {
                const uint16_t* e = p.ek + row;
                cp_async4(dst + 512, reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(e) & ~uintptr_t(3)));
                // the key's note: swizzle of K's units, needs plane B of K, which half of the scale's word
                *reinterpret_cast<uint32_t*>(stage + slot_i * HSLOT + 516) =
                    static_cast<uint32_t>(kk & 7) | (isK ? 8u : 0u) | ((reinterpret_cast<uintptr_t>(e) & 2) ? 16u : 0u);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            ++issued;
#ifdef FOLD_DEC_COUNTERS
            cntl[27] += clock64() - cw_k0;
#endif
            return true;
        };
        auto dot8 = [&](const uint4& lo4, const uint4& hi4, const int (&qw)[8]) -> int {
            int c = __dp4a(static_cast<int>(lo4.x), qw[0], 0);
            c = __dp4a(static_cast<int>(lo4.y), qw[1], c);
            c = __dp4a(static_cast<int>(lo4.z), qw[2], c);
            c = __dp4a(static_cast<int>(lo4.w), qw[3], c);
            c = __dp4a(static_cast<int>(hi4.x), qw[4], c);
            c = __dp4a(static_cast<int>(hi4.y), qw[5], c);
            c = __dp4a(static_cast<int>(hi4.z), qw[6], c);
            c = __dp4a(static_cast<int>(hi4.w), qw[7], c);
            c += __shfl_xor_sync(0xffffffffu, c, 8);
            c += __shfl_xor_sync(0xffffffffu, c, 16);
            return c;
        };
        while (true) {
            // keep the slots full as far as keys are to be had now; wait for one only when idle
#ifdef FOLD_DEC_COUNTERS
            const long long cw_i0 = clock64();
#endif
            while (issued - taken < HD_KEYS && issue_one(false)) {}
            if (issued == taken && !issue_one(true)) break;
#ifdef FOLD_DEC_COUNTERS
            cntl[24] += clock64() - cw_i0;
            const long long cw_c0 = clock64();
#endif
            // Several keys a pass when that many are in flight: their dot products, shuffles and
            // conversions do not depend on each other, which a lone warp's in-order issue needs to
            // stay busy. The sums still take the keys in order. (Measured: a gain on a bf16 V, where a
            // tile holds about five such keys; a small loss on an 8-bit V, where most tiles hold one or
            // two, so there a pass is one key.)
            const int avail = issued - taken;
            const int take = (HPASS >= 4 && avail >= 4) ? 4 : ((HPASS >= 2 && avail >= 2) ? 2 : 1);
            {   // the younger copies may still be in flight
#ifdef FOLD_DEC_COUNTERS
                const long long cw_w = clock64();
#endif
                const int pending = avail - take;
                switch (pending < 15 ? pending : 15) {   // the instruction takes its count as an immediate
#define FOLD_WAIT_CASE(n) case n: asm volatile("cp.async.wait_group " #n ";" ::: "memory"); break;
                    FOLD_WAIT_CASE(0) FOLD_WAIT_CASE(1) FOLD_WAIT_CASE(2) FOLD_WAIT_CASE(3) FOLD_WAIT_CASE(4) FOLD_WAIT_CASE(5)
                    FOLD_WAIT_CASE(6) FOLD_WAIT_CASE(7) FOLD_WAIT_CASE(8) FOLD_WAIT_CASE(9) FOLD_WAIT_CASE(10) FOLD_WAIT_CASE(11)
                    FOLD_WAIT_CASE(12) FOLD_WAIT_CASE(13) FOLD_WAIT_CASE(14)
                    default: asm volatile("cp.async.wait_group 15;" ::: "memory"); break;
#undef FOLD_WAIT_CASE
                }
#ifdef FOLD_DEC_COUNTERS
                cntl[10] += clock64() - cw_w;
#endif
            }
            __syncwarp();
            auto consume = [&](auto n_keys) {
                constexpr int N = decltype(n_keys)::value;
                const uint8_t* sb[N];
    #pragma unroll
                for (int j = 0; j < N; ++j) sb[j] = stage + ((taken + j) % HD_KEYS) * HSLOT;
                uint32_t note[N];
                float tk[N];
                uint4 ka0[N], ka1[N];
                int u0[N], u1[N];
    #pragma unroll
                for (int j = 0; j < N; ++j) {
                    note[j] = *reinterpret_cast<const volatile uint32_t*>(sb[j] + 516);
                    const uint32_t ekw = *reinterpret_cast<const uint32_t*>(sb[j] + 512);
                    tk[j] = eq_l * (bf16_bits_to_float(static_cast<uint16_t>((note[j] & 16u) ? (ekw >> 16) : (ekw & 0xFFFFu))) * (1.0f / 256.0f));
                    // K's planes are stored with their 16-byte units swizzled by slot
                    const int sw = note[j] & 7;
                    u0[j] = ((2 * part) ^ sw) << 4;
                    u1[j] = ((2 * part + 1) ^ sw) << 4;
                    ka0[j] = *reinterpret_cast<const uint4*>(sb[j] + u0[j]);
                    ka1[j] = *reinterpret_cast<const uint4*>(sb[j] + u1[j]);
                }
                float sv[N];
    #pragma unroll
                for (int j = 0; j < N; ++j) {
                    const int c1 = dot8(ka0[j], ka1[j], qaw), c2 = dot8(ka0[j], ka1[j], qbw);
                    sv[j] = fmaf(static_cast<float>(c1 * 256 + c2), tk[j], -z_l);
                }
                uint32_t any_note = 0u;
    #pragma unroll
                for (int j = 0; j < N; ++j) any_note |= note[j];
                if ((any_note & 8u) != 0u) {   // a key without plane B of K had zeros copied: its term is 0
    #pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const uint4 kb0 = *reinterpret_cast<const uint4*>(sb[j] + 128 + u0[j]), kb1 = *reinterpret_cast<const uint4*>(sb[j] + 128 + u1[j]);
                        const int c3a = dot8(kb0, kb1, qaw), c3b = dot8(kb0, kb1, qbw);
                        if (note[j] & 8u) sv[j] = sv[j] + (static_cast<float>(c3a) + static_cast<float>(c3b) * (1.0f / 256.0f)) * tk[j];
                    }
                }
                float wl[N], fa[N][4];
    #pragma unroll
                for (int j = 0; j < N; ++j) {
                    wl[j] = hg < G ? ex2f(sv[j]) : 0.f;   // row hg's weight, in all four quarters' lanes
                    if (V8) {
                        float fb[4];
                        e4m3x4_to_float(*reinterpret_cast<const uint32_t*>(sb[j] + 256 + 4 * lane), fa[j]);
                        e4m3x4_to_float(*reinterpret_cast<const uint32_t*>(sb[j] + 384 + 4 * lane), fb);
    #pragma unroll
                        for (int cc = 0; cc < 4; ++cc) fa[j][cc] = fmaf(fb[cc], 0.125f, fa[j][cc]);
                    } else {
                        const uint2 vv = *reinterpret_cast<const uint2*>(sb[j] + 256 + 8 * lane);   // four bf16 channels
                        fa[j][0] = __uint_as_float(vv.x << 16); fa[j][1] = __uint_as_float(vv.x & 0xFFFF0000u);
                        fa[j][2] = __uint_as_float(vv.y << 16); fa[j][3] = __uint_as_float(vv.y & 0xFFFF0000u);
                    }
                }
    #pragma unroll
                for (int j = 0; j < N; ++j) hden += wl[j];
    #pragma unroll
                for (int g = 0; g < 8; ++g) {
                    float wg_[N];
    #pragma unroll
                    for (int j = 0; j < N; ++j) wg_[j] = __shfl_sync(0xffffffffu, wl[j], g);
    #pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
    #pragma unroll
                        for (int j = 0; j < N; ++j) acc[g][cc] = fmaf(wg_[j], fa[j][cc], acc[g][cc]);
                    }
                }
            };
            if (take == 4) consume(std::integral_constant<int, (HPASS >= 4 ? 4 : 1)>{});
            else if (take == 2) consume(std::integral_constant<int, (HPASS >= 2 ? 2 : 1)>{});
            else consume(std::integral_constant<int, 1>{});
            __syncwarp();   // the slots are read out before the next copies may land in them
#ifdef FOLD_DEC_COUNTERS
            cntl[25] += clock64() - cw_c0;
#endif
            taken += take;
            CW_ADD(11, take);
        }
        if (lane == 0) CW_FLUSH(8);
        // the sums go where V's ring was: wait until nothing reads or fills it any more
        if (n_tiles > 0) mbar_wait(bar(B_ALLDONE), 0, abort_flag, p.status);
        float* hout = reinterpret_cast<float*>(smem + SM_HOUT) + h * (HOUT / 4);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            *reinterpret_cast<float4*>(hout + g * 128 + 4 * lane) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
            if (lane == g) hout[8 * 128 + g] = hden;   // lane g sums row g's weights
        }
        asm volatile("bar.sync 2, %0;" ::"n"(256 + 32 * NHELP) : "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
    }
}

template <bool TRUNC, bool V8, int GC = 0>
__global__ void __launch_bounds__(Lay<V8>::NTHREADS, 1) decode_sm100_kernel(const Params p, const __grid_constant__ CUtensorMap vmap,
                                                                   const __grid_constant__ CUtensorMap vbmap) {
    const int slot = blockIdx.x / p.split;
    const int bh = p.order ? p.order[slot] : slot;
    if (BOTHK_LEN > 0 && p.seq_lens[bh / p.hkv] <= BOTHK_LEN) decode_sm100_body<TRUNC, V8, GC, true>(p, &vmap, &vbmap);
    else decode_sm100_body<TRUNC, V8, GC, false>(p, &vmap, &vbmap);
}

}  // namespace dsm100
}  // namespace fold

using namespace fold;

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

// V in the pool as rows of `row_bytes` bytes (an E4M3 plane: 128; a bf16 row: 256); a box is 128
// bytes of `box_rows` rows, swizzled on its way into shared memory. The call does not know the
// pool's size: the row count only bounds the coordinates, and every tile asked for lies inside a page.
bool make_v_map(CUtensorMap* m, const void* v, int row_bytes, int box_rows) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const bool wide = row_bytes == 256;
    cuuint64_t dims[2] = {128, 1ull << 30};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    cuuint32_t box[2] = {wide ? 64u : 128u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, wide ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(v), dims,
              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool TRUNC, bool V8, int GC>
void launch_g(const dsm100::Params& p, const CUtensorMap& vmap, const CUtensorMap& vbmap, int ctas, cudaStream_t st) {
    auto kern = dsm100::decode_sm100_kernel<TRUNC, V8, GC>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dsm100::Lay<V8>::SMEM_BYTES);
    kern<<<ctas, dsm100::Lay<V8>::NTHREADS, dsm100::Lay<V8>::SMEM_BYTES, st>>>(p, vmap, vbmap);
}

template <bool TRUNC, bool V8>
void launch(const dsm100::Params& p, const CUtensorMap& vmap, const CUtensorMap& vbmap, int ctas, cudaStream_t st) {
    if (p.G == 8 && FOLD_DEC_G8) launch_g<TRUNC, V8, 8>(p, vmap, vbmap, ctas, st);
    else launch_g<TRUNC, V8, 0>(p, vmap, vbmap, ctas, st);
}

}  // namespace

extern "C" int fold_decode_combine(const float* o_part, const float* den_part, const int32_t* cnt_part,
                                   const int32_t* seq_lens, void* out, int out_dtype, float* den, int32_t* counts,
                                   int n_groups, int group, int head_dim, int n_kv_heads, int split, int chunk_keys,
                                   float v_scale, void* stream);

extern "C" int fold_decode_sm100_supported(int group, int head_dim, int page_size, int chunk_keys, int v8) {
    (void)v8;   // both an 8-bit and a bf16 V
    return head_dim == 128 && group >= 1 && group <= 8 && page_size % 128 == 0 && chunk_keys % 128 == 0 &&
           encode_fn() != nullptr;
}

extern "C" int fold_decode_run_sm100(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                                     const int8_t* kb, const void* ek, const void* va, const void* vb,
                                     const float* vmean, const float* z, const float* cut,
                                     const int32_t* page_table, const int32_t* seq_lens,
                                     const int32_t* order, int n_groups, int group, int n_kv_heads,
                                     int head_dim, int pages_per_request, int page_size, int split,
                                     int chunk_keys, int truncate, float refine_k, float refine_v,
                                     const float* refine_bands, float v_scale, float* o_part,
                                     float* den_part, int32_t* cnt_part, void* out, int out_dtype,
                                     float* den, int32_t* counts, int32_t* status, void* stream) {
    FOLD_CHECK_ARG(qa && qb && eq && ka && kb && ek && va && z && cut && page_table && seq_lens &&
                       o_part && den_part && cnt_part && status && (!out || (den && counts)),
                   "fold_decode_run_sm100: null pointer");
    if (!fold_decode_sm100_supported(group, head_dim, page_size, chunk_keys, 1)) {
        set_error("the tcgen05 decode takes head_dim 128, groups of 1..8 rows, pages and chunks of a multiple of 128 keys");
        return FOLD_ERR_UNSUPPORTED;
    }
    FOLD_CHECK_ARG(split >= 1 && out_dtype >= 0 && out_dtype <= 2, "fold_decode_run_sm100: bad split or out_dtype");
    FOLD_CHECK_ARG(chunk_keys >= 0, "chunk %d", chunk_keys);
    FOLD_CHECK_ARG(n_groups >= 1 && n_kv_heads >= 1 && pages_per_request >= 1, "fold_decode_run_sm100: empty call");
    dsm100::Params p;
    p.qa = qa; p.qb = qb; p.eq = eq; p.ka = ka; p.kb = kb;
    p.ek = static_cast<const uint16_t*>(ek);
    p.va = static_cast<const uint8_t*>(va); p.vb = static_cast<const uint8_t*>(vb);
    p.vmean = truncate ? vmean : nullptr; p.z = z; p.cut = cut;
    p.page_table = page_table; p.seq_lens = seq_lens; p.order = order;
    p.o_part = o_part; p.den_part = den_part; p.cnt_part = cnt_part;
    p.nbh = n_groups; p.G = group; p.hkv = n_kv_heads; p.ppr = pages_per_request;
    p.page_size = page_size; p.split = split; p.chunk_keys = chunk_keys; p.truncate = truncate;
    p.rk = refine_k; p.rv = refine_v;
    p.banded = refine_bands != nullptr;
    if (refine_bands) {
        p.band_e0 = refine_bands[0]; p.band_e1 = refine_bands[1];
        p.rk1 = refine_bands[2]; p.rk2 = refine_bands[3]; p.rv1 = refine_bands[4]; p.rv2 = refine_bands[5];
    } else {
        p.band_e0 = p.band_e1 = p.rk1 = p.rk2 = p.rv1 = p.rv2 = 0.f;
    }
    p.status = status;
    const bool v8 = vb != nullptr;   // a NULL second plane: V is one bf16 row per key
    CUtensorMap vmap, vbmap;
    if (!make_v_map(&vmap, va, v8 ? 128 : 256, 128) || !make_v_map(&vbmap, v8 ? vb : va, v8 ? 128 : 256, 32)) {
        set_error("fold_decode_run_sm100: cuTensorMapEncodeTiled failed");
        return FOLD_ERR_LAUNCH;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int ctas = n_groups * split;
    if (truncate) {
        if (v8) launch<true, true>(p, vmap, vbmap, ctas, st); else launch<true, false>(p, vmap, vbmap, ctas, st);
    } else {
        if (v8) launch<false, true>(p, vmap, vbmap, ctas, st); else launch<false, false>(p, vmap, vbmap, ctas, st);
    }
    int rc = check_launch("fold_decode_run_sm100");
    if (rc) return rc;
    if (!out) return FOLD_OK;   // partials only: the caller combines
    return fold_decode_combine(o_part, den_part, cnt_part, seq_lens, out, out_dtype, den, counts, n_groups, group,
                               head_dim, n_kv_heads, split, chunk_keys, v_scale, stream);
}

// The role counters of a -DFOLD_DEC_COUNTERS build (cycles, summed over CTAs and over each role's
// counting lanes): 0 CTAs, 1 tiles; key threads (8 warps) 2 all, 3-7 waits for V and scales,
// logits, the weight buffer, a plane-B buffer, the mask ring; helpers (4 warps) 8 all, 9 waiting
// for a tile's masks, 10 waiting for rows, 11 keys; 12-13 K producer (slot free, all); 14-15 V
// producer; 16-18 logit MMA thread (TMEM slot free, K landed, all); 19-22 value MMA thread (plane B
// landed, V landed, weights ready, all); 23 key threads' wait for the last product; helpers again:
// 24 handing out keys (opening tiles' masks, starting copies), 25 waiting for rows and summing,
// 26 inside tile opens (a try_wait that sleeps until the masks are published counts here), 27 starting
// a key's copies, 28 tiles opened.
extern "C" int fold_decode_counters(uint64_t* out32, int reset) {
#ifdef FOLD_DEC_COUNTERS
    FOLD_CHECK_ARG(out32, "fold_decode_counters: null pointer");
    unsigned long long h[32];
    if (cudaMemcpyFromSymbol(h, fold::dsm100::g_dec_counters, sizeof(h)) != cudaSuccess) return fold::check_launch("fold_decode_counters");
    for (int i = 0; i < 32; ++i) out32[i] = h[i];
    if (reset) {
        memset(h, 0, sizeof(h));
        if (cudaMemcpyToSymbol(fold::dsm100::g_dec_counters, h, sizeof(h)) != cudaSuccess) return fold::check_launch("fold_decode_counters");
    }
    return FOLD_OK;
#else
    (void)out32;
    (void)reset;
    fold::set_error("fold_decode_counters: the library was built without -DFOLD_DEC_COUNTERS");
    return FOLD_ERR_UNSUPPORTED;
#endif
}
