// Attention forward on Blackwell tensor cores (tcgen05 + TMEM), head dim 128, bf16 or fp16:
// O and the log-sum-exp the backward consumes. One CTA owns 256 query rows of one
// head as two tiles of 128; a query row is one TMEM lane of its tile, so a row's
// maximum and sum need no shuffle.
//
//   S  = Q K^T   tcgen05.mma kind::f16, M=128 queries, N=128 keys, 8 steps of 16 channels,
//                both operands K-major from shared memory (TMA, 128-byte swizzle) -> TMEM fp32
//   P  = exp2(S c log2e - m)  by the row's thread, written over S in TMEM as packed 16-bit
//   O += P V     A = P from TMEM, B = V as stored (MN-major), 8 steps of 16 keys -> TMEM fp32
//
// The two tiles share each K/V stage and take turns on the tensor core: while one tile's
// rows are in their softmax, the other's scores or P V product run. A row's softmax
// reference only ever rises, and only when the row's maximum passed it by more than 2^8; O is
// rescaled in TMEM when a row's reference moved (skipped, with the wait for the tile's previous
// product, by warps in which no row's did).
//
// Warps: 0 TMA producer, 1 MMA issuer (owns all 512 TMEM columns), 4-7 and 8-11 the two
// tiles' softmax, O rescale and epilogue. Every wait is bounded (about a second); on expiry
// a status word is raised, nobody waits any more, TMEM is freed and the kernel returns.
// Replaces the third-party forward called at src/fold_attention/interface.py:42-44,
// :70-81 and kv_cache.py:252-262 (the algorithm is the usual online softmax; the
// schedule is this kernel's own).
#include <cuda.h>

#include "bwd_common.cuh"
#include "common.cuh"
#include "fold_b200.h"

namespace fold {
namespace fsm100 {

constexpr int BM = 128, BN = 128;   // a query tile, a key tile
constexpr int CTA_M = 2 * BM;       // a CTA owns two query tiles
constexpr int NTHREADS = 384;
constexpr long long WAIT_CYCLES = 1ll << 31;
constexpr float LAZY = 8.0f;        // log2 of how far a row's maximum may pass its softmax reference before the reference moves

// shared memory map (1024-aligned base)
constexpr int SM_Q = 0;                        // 2 tiles x [2 boxes of 64 channels][128 rows][128 B]
constexpr int SM_KV = 65536;                   // 2 stages x { K 32 KB, V 32 KB }
constexpr int STAGE = 65536;
constexpr int SM_BAR = SM_KV + 2 * STAGE;
constexpr int SMEM_BYTES = SM_BAR + 256 + 1024;   // + room to align the base

enum {
    B_Q = 0,
    B_KVFULL = 1,      // [2] the stage's K and V have landed
    B_KVEMPTY = 3,     // [2] both query tiles' products with the stage retired
    B_SFULL = 5,       // [2 query tiles] the tile's scores against this key tile are in TMEM
    B_PREADY = 7,      // [2 query tiles] 128 arrivals: P is in TMEM and O is rescaled
    B_ODONE = 9,       // [2 query tiles] the tile's P V product retired
    B_COUNT = 11,
};

// TMEM columns: per query tile 128 of S (P is written over its first 64 as the row's thread
// goes), then 128 of O per tile
constexpr uint32_t T_S = 0, T_O = 256;

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
// Bounded wait. `abort` (shared) is raised by whoever runs out first; once it is up
// nobody waits any more, so every role runs to its end.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
    if (mbar_try(bar, parity)) return;
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
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Two fp32 FMAs per instruction and a three-input maximum (same results as the scalar forms): the
// softmax warps are what this kernel waits for.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack2(a0, a1)), "l"(b), "l"(c));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// shared-memory matrix descriptor, 128-byte swizzle; offsets in bytes
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// instruction descriptor: 16-bit x 16-bit -> f32 (format 1 bf16, 0 fp16), M x N, operand majors (0 K, 1 MN)
__host__ __device__ constexpr uint32_t instr_desc(int fmt, int M, int N, int a_mn, int b_mn) {
    return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) | (static_cast<uint32_t>(a_mn) << 15) |
           (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
           (static_cast<uint32_t>(M >> 4) << 24);
}

struct Params {
    TensorView o;
    float* lse;
    int64_t lse_sb, lse_sh;
    const int* cu;
    int B, H, HKV, G, S, causal;
    float scale;
    int* status;
};
struct Maps {
    CUtensorMap q, k, v;   // (channel, row, head, batch), boxes (64, 128, 1, 1)
};

template <bool F16>
__global__ void __launch_bounds__(NTHREADS, 1) fwd_sm100_kernel(const Params p, const __grid_constant__ Maps maps) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    auto bar = [&](int i) { return base + SM_BAR + 8 * i; };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 8 * B_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 8 * B_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the last query rows first: under a causal mask they meet the most key tiles
    const int mb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    int start = 0, len = p.S;
    if (p.cu) {
        start = p.cu[b];
        len = p.cu[b + 1] - start;
    }
    const int m0 = mb * CTA_M;
    if (m0 >= len) return;
    const int hkv = h / p.G;
    const int bb = p.cu ? 0 : b;
    // key tiles each of the two query tiles meets (the second tile may lie past the sequence)
    int nt[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int mx = m0 + x * BM;
        const int kv_end = mx >= len ? 0 : (p.causal ? min(len, mx + BM) : len);
        nt[x] = (kv_end + BN - 1) / BN;
    }
    const int n_tiles = max(nt[0], nt[1]);

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar(B_Q), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(B_KVFULL + i), 1);
            mbar_init(bar(B_KVEMPTY + i), 1);
            mbar_init(bar(B_SFULL + i), 1);
            mbar_init(bar(B_PREADY + i), 128);
            mbar_init(bar(B_ODONE + i), 1);
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

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            mbar_expect_tx(bar(B_Q), nt[1] > 0 ? 65536 : 32768);
            for (int x = 0; x < 2; ++x) {
                if (nt[x] == 0) continue;
                for (int c = 0; c < 2; ++c)
                    tma_load_4d(base + SM_Q + x * 32768 + c * 16384, &maps.q, 64 * c, start + m0 + x * BM, h, bb, bar(B_Q));
            }
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                if (j >= 2) mbar_wait(bar(B_KVEMPTY + s), ((j >> 1) - 1) & 1, abort_flag, p.status);
                const uint32_t st = base + SM_KV + s * STAGE;
                mbar_expect_tx(bar(B_KVFULL + s), 65536);
                for (int c = 0; c < 2; ++c) {
                    tma_load_4d(st + c * 16384, &maps.k, 64 * c, start + j * BN, hkv, bb, bar(B_KVFULL + s));
                    tma_load_4d(st + 32768 + c * 16384, &maps.v, 64 * c, start + j * BN, hkv, bb, bar(B_KVFULL + s));
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t ID_S = instr_desc(F16 ? 0 : 1, 128, 128, 0, 0);    // Q (K-major) x K (K-major)
            constexpr uint32_t ID_PV = instr_desc(F16 ? 0 : 1, 128, 128, 0, 1);   // P (TMEM) x V (MN-major)
            mbar_wait(bar(B_Q), 0, abort_flag, p.status);
            auto issue_s = [&](int x, int j) {
                const int s = j & 1;
                mbar_wait(bar(B_KVFULL + s), (j >> 1) & 1, abort_flag, p.status);
                tc_fence_after();
                const uint32_t kt = base + SM_KV + s * STAGE, qt = base + SM_Q + x * 32768;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // 16 channels per step; 4 steps per 64-channel box
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    mma_ss(tmem + T_S + 128 * x, smem_desc(qt + off, 16, 1024), smem_desc(kt + off, 16, 1024), ID_S, ks > 0);
                }
                tc_commit(bar(B_SFULL + x));
            };
            for (int x = 0; x < 2; ++x)
                if (nt[x] > 0) issue_s(x, 0);
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t vt = base + SM_KV + s * STAGE + 32768;
                for (int x = 0; x < 2; ++x) {
                    if (j >= nt[x]) continue;
                    mbar_wait(bar(B_PREADY + x), j & 1, abort_flag, p.status);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)   // 16 keys per step: 8 TMEM columns of P, 2048 bytes of V per box
                        mma_ts(tmem + T_O + 128 * x, tmem + T_S + 128 * x + 8 * ks, smem_desc(vt + ks * 2048, 16384, 1024), ID_PV,
                               (j > 0) || (ks > 0));
                    tc_commit(bar(B_ODONE + x));
                    // the next scores overwrite S (and the P just consumed): the tensor pipe runs a
                    // thread's MMAs in the order it issued them
                    if (j + 1 < nt[x]) issue_s(x, j + 1);
                }
                tc_commit(bar(B_KVEMPTY + s));
            }
        }
    } else if (warp >= 4) {
        // ================= softmax: two groups, one per query tile; thread = query row = TMEM lane =================
        const int x = (warp - 4) >> 2;
        const int r = 32 * (warp & 3) + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const float c2 = p.scale * kLog2e;
        const uint64_t c2x2 = pack2(c2, c2);
        const int mx = m0 + x * BM;
        const int qi = mx + r;                 // the row's position in its sequence
        const int my_tiles = nt[x];
        float m_run = -INFINITY, l_run = 0.f;  // running maximum (log2 domain) and sum
        const uint32_t ts = tmem + lane_addr + T_S + 128 * x;
        const uint32_t to = tmem + lane_addr + T_O + 128 * x;
        for (int j = 0; j < my_tiles; ++j) {
            const int n0 = j * BN;
            const bool need_mask = (p.causal && n0 + BN > mx) || (n0 + BN > len);
            const int kmax = min(len - 1, p.causal ? qi : len - 1) - n0;   // last key column this row may see
            mbar_wait(bar(B_SFULL + x), j & 1, abort_flag, p.status);
            tc_fence_after();
            // pass 1: the row's maximum over the tile
            float mxv = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t sv[32];
                tmem_ld32(ts + 32 * c, sv);
                tmem_wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (32 * c + e > kmax) sv[e] = 0xff800000u;   // -inf
                }
#pragma unroll
                for (int e = 0; e < 32; e += 2) mxv = max3f(mxv, __uint_as_float(sv[e]), __uint_as_float(sv[e + 1]));
            }
            // The reference point only moves when the row's maximum rose by more than 2^LAZY: weights
            // up to 2^LAZY are as exact in 16 bits as weights up to 1, the final O / l cancels the
            // choice, and a row whose reference stays has alpha = 1 exactly, so its warp neither
            // waits for the previous product nor rescales O. After a sequence's first tiles that is
            // nearly every warp.
            const float m_cand = fmaxf(m_run, mxv * c2);
            const float m_new = m_cand > m_run + LAZY ? m_cand : m_run;
            // a row that sees no key yet keeps m = -inf; its weights are exp2(-inf) = 0
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = ex2f(m_run - m_use);   // 0 on the first tile that holds a key, 1 where the reference stays
            // pass 2: weights over the scores as packed bf16 (P chunk c lands on columns the row's
            // thread has already read), and their sum
            uint64_t sum2 = 0ull;   // two partial sums, added at the end of the tile
            const uint64_t nm2 = pack2(-m_use, -m_use);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t sv[32];
                tmem_ld32(ts + 32 * c, sv);
                tmem_wait_ld();
                uint32_t pp[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float x0, x1;
                    fma2(x0, x1, __uint_as_float(sv[e]), __uint_as_float(sv[e + 1]), c2x2, nm2);
                    x0 = ex2f(x0);
                    x1 = ex2f(x1);
                    if (need_mask) {
                        if (32 * c + e > kmax) x0 = 0.f;
                        if (32 * c + e + 1 > kmax) x1 = 0.f;
                    }
                    asm("add.rn.f32x2 %0, %0, %1;" : "+l"(sum2) : "l"(pack2(x0, x1)));   // even and odd columns apart
                    pp[e >> 1] = F16 ? pack_f16x2(x0, x1) : pack_bf16x2(x0, x1);
                }
                tmem_st16(ts + 16 * c, pp);
            }
            float sum_e, sum_o;
            asm("mov.b64 {%0, %1}, %2;" : "=f"(sum_e), "=f"(sum_o) : "l"(sum2));
            l_run = l_run * alpha + (sum_e + sum_o);
            m_run = m_new;
            // O was last written by key tile j-1's product: rescale it where a row's maximum rose
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                mbar_wait(bar(B_ODONE + x), (j - 1) & 1, abort_flag, p.status);
                tc_fence_after();
                {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t ov[32];
                        tmem_ld32(to + 32 * c, ov);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
                        tmem_st32(to + 32 * c, ov);
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(B_PREADY + x));
        }
        // ---- epilogue: O / l -> bf16, LSE in nats ----
        if (my_tiles > 0) {
            mbar_wait(bar(B_ODONE + x), (my_tiles - 1) & 1, abort_flag, p.status);
            tc_fence_after();
            // the warp's tcgen05.ld is collective: every lane reads, rows past the sequence store nothing
            const bool row_ok = qi < len;
            auto pk2 = [](float a, float b2) { return F16 ? pack_f16x2(a, b2) : pack_bf16x2(a, b2); };
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            uint16_t* orow = row_ptr<uint16_t>(p.o, b, start + (row_ok ? qi : 0), h);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t ov[32];
                tmem_ld32(to + 32 * c, ov);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint4 w;
                        w.x = pk2(__uint_as_float(ov[8 * u]) * inv, __uint_as_float(ov[8 * u + 1]) * inv);
                        w.y = pk2(__uint_as_float(ov[8 * u + 2]) * inv, __uint_as_float(ov[8 * u + 3]) * inv);
                        w.z = pk2(__uint_as_float(ov[8 * u + 4]) * inv, __uint_as_float(ov[8 * u + 5]) * inv);
                        w.w = pk2(__uint_as_float(ov[8 * u + 6]) * inv, __uint_as_float(ov[8 * u + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + 32 * c + 8 * u) = w;
                    }
                }
            }
            if (row_ok) {
                const float lse = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
                p.lse[static_cast<int64_t>(b) * p.lse_sb + static_cast<int64_t>(h) * p.lse_sh + start + qi] = lse;
            }
            tc_fence_before();
        }
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

}  // namespace fsm100
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

// (channel, row, head, batch) view of a (batch, row, head, channel)-strided bf16 tensor; a box is
// 64 channels of 128 rows. Rows past the tensor read as zeros.
bool make_map(CUtensorMap* m, const void* ptr, int64_t sb, int64_t sr, int64_t sh, int64_t rows, int heads, int batch, bool f16) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
    if (!sb) sb = sr * rows;
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(sr * 2), static_cast<cuuint64_t>(sh * 2), static_cast<cuuint64_t>(sb * 2)};
    cuuint32_t box[4] = {64, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int fold_fwd_sm100_supported(int head_dim, int is_f16) {
    (void)is_f16;   // bf16 and fp16
    return head_dim == 128 && encode_fn() != nullptr;
}

extern "C" int fold_fwd_run_sm100(const void* q, const void* k, const void* v, void* o, float* lse,
                                  const int64_t* strides, const int32_t* cu_seqlens, int batch, int n_heads,
                                  int n_kv_heads, int max_seqlen, int total, int head_dim, int causal, int is_f16,
                                  float softmax_scale, int32_t* status, void* stream) {
    FOLD_CHECK_ARG(q && k && v && o && lse && strides && status, "fold_fwd_run_sm100: null pointer");
    FOLD_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0, "the query heads must be a multiple of the KV heads");
    FOLD_CHECK_ARG(batch > 0 && max_seqlen > 0, "fold_fwd_run_sm100: empty call");
    if (!fold_fwd_sm100_supported(head_dim, 0)) {
        set_error("the tcgen05 forward takes head_dim 128");
        return FOLD_ERR_UNSUPPORTED;
    }
    const void* ptrs[4] = {q, k, v, o};
    for (int i = 0; i < 4; ++i)
        FOLD_CHECK_ARG(strides[3 * i] % 8 == 0 && strides[3 * i + 1] % 8 == 0 && strides[3 * i + 2] % 8 == 0 &&
                           reinterpret_cast<uintptr_t>(ptrs[i]) % 16 == 0,
                       "fold_fwd_run_sm100: rows must be 16-byte aligned");
    fsm100::Params p;
    p.o.ptr = o; p.o.sb = strides[9]; p.o.sr = strides[10]; p.o.sh = strides[11];
    p.lse = lse;
    p.cu = cu_seqlens;
    if (cu_seqlens) {
        p.lse_sb = 0;
        p.lse_sh = total;
    } else {
        p.lse_sb = static_cast<int64_t>(n_heads) * max_seqlen;
        p.lse_sh = max_seqlen;
    }
    p.B = batch; p.H = n_heads; p.HKV = n_kv_heads; p.G = n_heads / n_kv_heads;
    p.S = max_seqlen; p.causal = causal; p.scale = softmax_scale; p.status = status;
    const int64_t rows = cu_seqlens ? total : max_seqlen;
    const int mbatch = cu_seqlens ? 1 : batch;
    fsm100::Maps maps;
    const bool f16 = is_f16 != 0;
    if (!make_map(&maps.q, q, strides[0], strides[1], strides[2], rows, n_heads, mbatch, f16) ||
        !make_map(&maps.k, k, strides[3], strides[4], strides[5], rows, n_kv_heads, mbatch, f16) ||
        !make_map(&maps.v, v, strides[6], strides[7], strides[8], rows, n_kv_heads, mbatch, f16)) {
        set_error("fold_fwd_run_sm100: cuTensorMapEncodeTiled failed");
        return FOLD_ERR_LAUNCH;
    }
    dim3 grid((max_seqlen + fsm100::CTA_M - 1) / fsm100::CTA_M, n_heads, batch);
    if (f16) {
        auto kern = fsm100::fwd_sm100_kernel<true>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fsm100::SMEM_BYTES);
        kern<<<grid, fsm100::NTHREADS, fsm100::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p, maps);
    } else {
        auto kern = fsm100::fwd_sm100_kernel<false>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fsm100::SMEM_BYTES);
        kern<<<grid, fsm100::NTHREADS, fsm100::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p, maps);
    }
    return check_launch("fold_fwd_run_sm100");
}
