// The deterministic attention backward on Blackwell tensor cores: tcgen05.mma
// with TMEM accumulators, TMA-fed 128-byte-swizzled shared tiles, mbarrier
// pipelines between specialised warps. Head dim 128, bf16 or fp16, dense or packed.
//
// One CTA owns one block of 128 keys of one (request, KV head) and walks query
// blocks of 64 rows, for each of the group's G query heads in turn. Per query
// block i (buffers b = i & 1 are double-buffered in TMEM):
//     S^T  = K Q^T            SS  M=128 keys,  N=64 queries, K=128      -> R_S[b]
//     dP^T = V dO^T           SS                                          -> R_D[b]
//     P~^T = exp2(S^T c - (L - s)), dS~^T = P~^T (dP^T - Delta)   (compute warps:
//            P~^T back to TMEM as 16-bit over S^T, dS~^T to shared, swizzled)
//     dV  += P~^T dO          TS  A from TMEM, M=128 keys, N=128, K=64
//     dK  += dS~^T Q          SS  A = dS~^T (K-major), B = Q (MN-major)
//     dQ~^T = K^T dS~^T       SS  A = K^T (MN-major), B = dS~^T (MN-major) -> R_D[b]
// dK and dV stay in TMEM for the CTA's whole life, summed in one fixed order;
// dQ~ leaves the GEMM on the request's integer grid (the softmax carries the
// grid exponent s), is rounded to nearest-even int32 and added to the
// accumulator with integer atomics, which commute exactly.
//
// Warps: 0 TMA producer, 1 MMA issuer (owns the TMEM allocation), 4-7 and
// 8-11 the two compute groups (one per TMEM buffer), 12-15 the dQ drain.
// Every mbarrier wait is bounded: on expiry the kernel raises a status word,
// stops waiting everywhere, frees its TMEM and returns.
// Reference arithmetic: src/fold_attention/backward/kernel.py:1191-1330.
#include <cuda.h>

#include "bwd_common.cuh"

namespace fold {

namespace sm100 {

constexpr int BN = 128;   // keys per CTA
constexpr int BM = 64;    // queries per step
constexpr int HD = 128;   // head dim
constexpr int STAGES = 3;
constexpr int NTHREADS = 512;
constexpr long long WAIT_CYCLES = 1ll << 31;   // about a second of SM clocks

// shared memory map (bytes from a 1024-aligned base)
constexpr int SM_K = 0;                         // [2 boxes][128 keys][64 ch] bf16, SW128
constexpr int SM_V = 32768;
constexpr int SM_STAGE = 65536;                 // per stage: Q 16 KB, dO 16 KB, L 256, Delta 256
constexpr int STAGE_BYTES = 33792;
constexpr int ST_Q = 0, ST_DO = 16384, ST_L = 32768, ST_DL = 33024;
constexpr int SM_DS = SM_STAGE + STAGES * STAGE_BYTES;   // [2][128 keys][64 queries] bf16, SW128
constexpr int SM_BAR = SM_DS + 2 * 16384;
constexpr int SM_TOTAL = SM_BAR + 256;
constexpr int SMEM_BYTES = SM_TOTAL + 1024;     // slack to align the base

// barrier indices
enum {
    B_KV = 0,
    B_QFULL = 1,                 // [STAGES]
    B_QEMPTY = B_QFULL + STAGES, // [STAGES]
    B_SDP = B_QEMPTY + STAGES,   // [2]  S^T, dP^T in TMEM
    B_PDS = B_SDP + 2,           // [2]  P~^T in TMEM, dS~^T in shared
    B_DQF = B_PDS + 2,           // [2]  dQ~^T in TMEM (and the step's MMAs retired)
    B_DQE = B_DQF + 2,           // [2]  dQ~^T drained
    B_GRP = B_DQE + 2,           // [2]  the step's dQ, dV, dK MMAs have all retired
    B_COUNT = B_GRP + 2,
};

// TMEM columns
constexpr uint32_t T_RS0 = 0, T_RS1 = 64, T_RD0 = 128, T_RD1 = 192, T_DK = 256, T_DV = 384;

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
// Bounded wait. `abort` (shared) is raised by whoever runs out first; once it
// is up nobody waits any more, so every role runs to its end.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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
    CUtensorMap q, dout, k, v;   // (channel, row, head, batch), boxes (64, 64|128, 1, 1)
};

template <bool F16>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_main_sm100_kernel(const BwdParams p, const __grid_constant__ Maps maps) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    Shared sh{base};
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 8 * B_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 8 * B_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nblocks = (p.S + BN - 1) / BN;
    const int nb = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    (void)nblocks;
    const SeqInfo sq = seq_info(p, b);
    const int n0 = nb * BN;
    if (n0 >= sq.len) return;

    // query steps: all heads of the group, each from the first block that can see this key block
    const int nm = (sq.len + BM - 1) / BM;
    const int m_min = p.causal ? (n0 / BM) : 0;
    const int per_head = nm - m_min;
    const int total = per_head * p.G;

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(sh.bar(B_KV), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sh.bar(B_QFULL + s), 1);
            mbar_init(sh.bar(B_QEMPTY + s), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(sh.bar(B_SDP + i), 1);
            mbar_init(sh.bar(B_PDS + i), 128);
            mbar_init(sh.bar(B_DQF + i), 1);
            mbar_init(sh.bar(B_DQE + i), 128);
            mbar_init(sh.bar(B_GRP + i), 1);
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

    const int s_exp = dq_scale_exp(p.stats + (static_cast<int64_t>(b) * p.HKV + hkv) * N_STATS, root_d(HD));

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            const int brow = sq.start + n0;
            const int bb = p.cu ? 0 : b;
            mbar_expect_tx(sh.bar(B_KV), 2 * 32768);
            for (int x = 0; x < 2; ++x) {
                tma_load_4d(base + SM_K + x * 16384, &maps.k, 64 * x, brow, hkv, bb, sh.bar(B_KV));
                tma_load_4d(base + SM_V + x * 16384, &maps.v, 64 * x, brow, hkv, bb, sh.bar(B_KV));
            }
            for (int i = 0; i < total; ++i) {
                const int s = i % STAGES;
                const int g = i / per_head, mb = m_min + i % per_head;
                const int h = hkv * p.G + g;
                if (i >= STAGES) mbar_wait(sh.bar(B_QEMPTY + s), ((i / STAGES) - 1) & 1, abort_flag, p.status);
                const uint32_t st = base + SM_STAGE + s * STAGE_BYTES;
                mbar_expect_tx(sh.bar(B_QFULL + s), 2 * 16384 + 512);
                const int row = sq.start + mb * BM;
                for (int x = 0; x < 2; ++x) {
                    tma_load_4d(st + ST_Q + x * 8192, &maps.q, 64 * x, row, h, bb, sh.bar(B_QFULL + s));
                    tma_load_4d(st + ST_DO + x * 8192, &maps.dout, 64 * x, row, h, bb, sh.bar(B_QFULL + s));
                }
                const int64_t wrow = static_cast<int64_t>(h) * p.rows_p + sq.pstart + mb * BM;
                bulk_load(st + ST_L, p.lse2 + wrow, 256, sh.bar(B_QFULL + s));
                bulk_load(st + ST_DL, p.dpsum + wrow, 256, sh.bar(B_QFULL + s));
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t ID_S = instr_desc(F16 ? 0 : 1, 128, 64, 0, 0);    // K (K-major) x Q (K-major)
            constexpr uint32_t ID_DV = instr_desc(F16 ? 0 : 1, 128, 128, 0, 1);  // P^T (TMEM) x dO (MN-major)
            constexpr uint32_t ID_DK = instr_desc(F16 ? 0 : 1, 128, 128, 0, 1);  // dS^T (K-major) x Q (MN-major)
            constexpr uint32_t ID_DQ = instr_desc(F16 ? 0 : 1, 128, 64, 1, 1);   // K^T (MN-major) x dS^T (MN-major)
            mbar_wait(sh.bar(B_KV), 0, abort_flag, p.status);
            tc_fence_after();
            auto issue_sdp = [&](int i) {
                const int s = i % STAGES, bf = i & 1;
                mbar_wait(sh.bar(B_QFULL + s), (i / STAGES) & 1, abort_flag, p.status);
                if (i >= 2) mbar_wait(sh.bar(B_DQE + bf), ((i >> 1) - 1) & 1, abort_flag, p.status);
                tc_fence_after();
                const uint32_t st = base + SM_STAGE + s * STAGE_BYTES;
                const uint32_t rs = tmem + (bf ? T_RS1 : T_RS0), rd = tmem + (bf ? T_RD1 : T_RD0);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // 16 channels per step; 4 steps per 64-channel box
                    const uint32_t ko = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t qo = (ks >> 2) * 8192 + (ks & 3) * 32;
                    mma_ss(rs, smem_desc(base + SM_K + ko, 16, 1024), smem_desc(st + ST_Q + qo, 16, 1024), ID_S, ks > 0);
                }
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ko = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t qo = (ks >> 2) * 8192 + (ks & 3) * 32;
                    mma_ss(rd, smem_desc(base + SM_V + ko, 16, 1024), smem_desc(st + ST_DO + qo, 16, 1024), ID_S, ks > 0);
                }
                tc_commit(sh.bar(B_SDP + bf));
            };
            if (total > 0) issue_sdp(0);
            for (int i = 0; i < total; ++i) {
                const int s = i % STAGES, bf = i & 1;
                if (i + 1 < total) issue_sdp(i + 1);
                mbar_wait(sh.bar(B_PDS + bf), (i >> 1) & 1, abort_flag, p.status);
                tc_fence_after();
                const uint32_t st = base + SM_STAGE + s * STAGE_BYTES;
                const uint32_t ds = base + SM_DS + bf * 16384;
                const uint32_t rs = tmem + (bf ? T_RS1 : T_RS0), rd = tmem + (bf ? T_RD1 : T_RD0);
                // dQ~^T = K^T dS~^T first: 8 steps of 16 keys. Its drain then runs under
                // dV and dK, so the buffer is free again when the next S^T/dP^T need it.
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ss(rd, smem_desc(base + SM_K + ks * 2048, 16384, 1024), smem_desc(ds + ks * 2048, 16384, 1024), ID_DQ, ks > 0);
                tc_commit(sh.bar(B_DQF + bf));
                // dV += P~^T dO : 4 steps of 16 queries; A = 8 TMEM columns per step
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_ts(tmem + T_DV, rs + 8 * ks, smem_desc(st + ST_DO + ks * 2048, 8192, 1024), ID_DV, (i > 0) || (ks > 0));
                // dK += dS~^T Q
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_ss(tmem + T_DK, smem_desc(ds + ks * 32, 16, 1024), smem_desc(st + ST_Q + ks * 2048, 8192, 1024), ID_DK, (i > 0) || (ks > 0));
                tc_commit(sh.bar(B_QEMPTY + s));   // the stage's Q, dO are free once these retire
                tc_commit(sh.bar(B_GRP + bf));
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ================= compute: P~^T and dS~^T for buffer bf =================
        const int bf = (warp >= 8) ? 1 : 0;
        const int r = 32 * (warp & 3) + lane;   // key row = TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const float c2 = p.scale * kLog2e;
        // bf16 has fp32's range, so P~ and dS~ carry the grid's exponent; fp16 does not, and the
        // exponent is applied to dQ's fp32 sums at the drain instead
        const float s_bias = F16 ? 0.f : static_cast<float>(s_exp);
        const int kj = n0 + r;
        for (int i = bf; i < total; i += 2) {
            const int s = i % STAGES;
            const int mb = m_min + i % per_head;
            const int m0 = mb * BM;
            mbar_wait(sh.bar(B_SDP + bf), (i >> 1) & 1, abort_flag, p.status);
            // dS~^T buffer bf was read by step i-2's dK and dQ MMAs
            if (i >= 2) mbar_wait(sh.bar(B_GRP + bf), ((i >> 1) - 1) & 1, abort_flag, p.status);
            tc_fence_after();
            const float* sL = reinterpret_cast<const float*>(smem + SM_STAGE + s * STAGE_BYTES + ST_L);
            const float* sDl = reinterpret_cast<const float*>(smem + SM_STAGE + s * STAGE_BYTES + ST_DL);
            uint8_t* sds = smem + SM_DS + bf * 16384 + r * 128;
            const uint32_t rs = tmem + lane_addr + (bf ? T_RS1 : T_RS0);
            const uint32_t rd = tmem + lane_addr + (bf ? T_RD1 : T_RD0);
            const bool need_mask = (p.causal && m0 < n0 + BN) || (n0 + BN > sq.len);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sv[32], dv[32];
                tmem_ld32(rs + 32 * c, sv);
                tmem_ld32(rd + 32 * c, dv);
                tmem_wait_ld();
                uint32_t pp[16], dd[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float pv[2], ds[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int q = 32 * c + j + e;
                        float x = ex2f(fmaf(__uint_as_float(sv[j + e]), c2, s_bias - sL[q]));
                        if (need_mask) {
                            const int qi = m0 + q;
                            if (kj >= sq.len || (p.causal && kj > qi)) x = 0.f;
                        }
                        pv[e] = x;
                        ds[e] = x * (__uint_as_float(dv[j + e]) - sDl[q]);
                    }
                    pp[j >> 1] = F16 ? pack_f16x2(pv[0], pv[1]) : pack_bf16x2(pv[0], pv[1]);
                    dd[j >> 1] = F16 ? pack_f16x2(ds[0], ds[1]) : pack_bf16x2(ds[0], ds[1]);
                }
                tmem_st16(rs + 16 * c, pp);
                // dS~^T row r: 16-byte chunk u (8 queries) at u ^ (r & 7)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int cu = (4 * c + u) ^ (r & 7);
                    *reinterpret_cast<uint4*>(sds + cu * 16) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            fence_async_smem();
            mbar_arrive(sh.bar(B_PDS + bf));
        }
    } else if (warp >= 12) {
        // ================= dQ drain: TMEM -> int32 grid -> global atomics =================
        const int d = 32 * (warp & 3) + lane;   // channel = TMEM lane
        const float dq_mul = F16 ? pow2f(s_exp) : 1.f;
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        for (int i = 0; i < total; ++i) {
            const int bf = i & 1;
            const int g = i / per_head, mb = m_min + i % per_head;
            const int h = hkv * p.G + g;
            mbar_wait(sh.bar(B_DQF + bf), (i >> 1) & 1, abort_flag, p.status);
            tc_fence_after();
            const uint32_t rd = tmem + lane_addr + (bf ? T_RD1 : T_RD0);
            uint32_t v0[32], v1[32];
            tmem_ld32(rd, v0);
            tmem_ld32(rd + 32, v1);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(sh.bar(B_DQE + bf));
            int* acc = p.dq_acc + (static_cast<int64_t>(h) * p.rows_p + sq.pstart + mb * BM) * HD + d;
#pragma unroll
            for (int q = 0; q < 32; ++q) {
                const int a = __float2int_rn(F16 ? __uint_as_float(v0[q]) * dq_mul : __uint_as_float(v0[q]));
                if (a != 0) atomicAdd(acc + q * HD, a);
            }
#pragma unroll
            for (int q = 0; q < 32; ++q) {
                const int a = __float2int_rn(F16 ? __uint_as_float(v1[q]) * dq_mul : __uint_as_float(v1[q]));
                if (a != 0) atomicAdd(acc + (32 + q) * HD, a);
            }
        }
    }

    // ================= epilogue: dK, dV out of TMEM =================
    __syncthreads();
    if (warp >= 4 && warp < 12) {
        // every MMA has retired once the last step's group barrier completes
        const int total_steps = total;
        if (total_steps > 0) {
            const int last = total_steps - 1;
            mbar_wait(sh.bar(B_GRP + (last & 1)), (last >> 1) & 1, abort_flag, p.status);
        }
        tc_fence_after();
        const int r = 32 * (warp & 3) + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const bool is_dv = warp >= 8;
        auto pk2 = [](float a, float b2) { return F16 ? pack_f16x2(a, b2) : pack_bf16x2(a, b2); };
        const float un = F16 ? 1.f : pow2f(-s_exp);
        const float f = is_dv ? un : p.scale * un;
        const uint32_t src = tmem + lane_addr + (is_dv ? T_DV : T_DK);
        const bool ok = n0 + r < sq.len;
        uint16_t* dst = row_ptr<uint16_t>(is_dv ? p.dv : p.dk, b, sq.start + n0 + (ok ? r : 0), hkv);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(src + 32 * c, v);
            tmem_wait_ld();
            if (ok && total_steps > 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 w;
                    w.x = pk2(__uint_as_float(v[j]) * f, __uint_as_float(v[j + 1]) * f);
                    w.y = pk2(__uint_as_float(v[j + 2]) * f, __uint_as_float(v[j + 3]) * f);
                    w.z = pk2(__uint_as_float(v[j + 4]) * f, __uint_as_float(v[j + 5]) * f);
                    w.w = pk2(__uint_as_float(v[j + 6]) * f, __uint_as_float(v[j + 7]) * f);
                    *reinterpret_cast<uint4*>(dst + 32 * c + j) = w;
                }
            } else if (ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) *reinterpret_cast<uint4*>(dst + 32 * c + j) = make_uint4(0, 0, 0, 0);
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
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

}  // namespace

bool bwd_sm100_supported(const BwdParams& p) {
    return p.D == 128 && encode_fn() != nullptr;
}

int launch_bwd_main_sm100(const BwdParams& p, cudaStream_t st) {
    sm100::Maps maps;
    const bool varlen = p.cu != nullptr;
    const int64_t rows = varlen ? p.total : p.S;
    const int batch = varlen ? 1 : p.B;
    const bool f16 = p.f16;
    if (!make_map(&maps.q, p.q, rows, p.H, batch, sm100::BM, f16) || !make_map(&maps.dout, p.dout, rows, p.H, batch, sm100::BM, f16) ||
        !make_map(&maps.k, p.k, rows, p.HKV, batch, sm100::BN, f16) || !make_map(&maps.v, p.v, rows, p.HKV, batch, sm100::BN, f16)) {
        set_error("bwd_main_sm100: cuTensorMapEncodeTiled failed");
        return FOLD_ERR_LAUNCH;
    }
    dim3 grid((p.S + sm100::BN - 1) / sm100::BN, p.HKV, p.B);
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
