// The deterministic attention backward for every supported shape (head dim
// 64/96/128, bf16/fp16, causal or full, dense or packed), on warp-level
// mma.sync tensor-core instructions. The tcgen05 kernel (bwd_sm100.cu) takes
// the head-dim-128 bf16 shapes; this one is the general path and the
// in-library cross-check of that kernel.
//
// One CTA owns one block of 64 keys of one (request, KV head) and walks the
// query blocks that can see it, for each of the group's G query heads in
// turn, so dK and dV never leave its registers and are summed in one fixed
// order. dQ partials are produced on the request's integer grid (the softmax
// carries the grid's exponent: P~ = P * 2^s), rounded to nearest-even int32
// and added with integer atomics, which commute exactly.
// Reference arithmetic: src/fold_attention/backward/kernel.py:1191-1330.
#include "bwd_common.cuh"
#include "mma_utils.cuh"

namespace fold {

constexpr int BM = 64, BN = 64, NTHREADS = 256;

template <int D>
struct MmaSmem {
    static constexpr int PITCH = D * 2 + 16;   // bytes; an odd number of 16-byte units
    static constexpr int TILE = 64 * PITCH;
    static constexpr int PPITCH = 64 * 2 + 16;
    static constexpr int PTILE = 64 * PPITCH;
    static constexpr int OFF_K = 0, OFF_V = TILE, OFF_Q = 2 * TILE, OFF_DO = 3 * TILE;
    static constexpr int OFF_PT = 4 * TILE, OFF_DST = 4 * TILE + PTILE;
    static constexpr int OFF_L = 4 * TILE + 2 * PTILE, OFF_DL = OFF_L + 64 * 4;
    static constexpr int BYTES = OFF_DL + 64 * 4;
};

template <int D, bool F16, bool CAUSAL>
__global__ void __launch_bounds__(NTHREADS, 2) bwd_main_mma_kernel(const BwdParams p) {
    using L = MmaSmem<D>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const SeqInfo sq = seq_info(p, b);
    const int n0 = nb * BN;
    if (n0 >= sq.len) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int wk = warp & 3, wd = warp >> 2;
    constexpr int NTD = D / 16;       // 8-channel n-tiles per warp for dK, dV, dQ
    constexpr int DH = D / 2;         // channels per warp half

    const int s_exp = dq_scale_exp(p.stats + (static_cast<int64_t>(b) * p.HKV + hkv) * N_STATS, root_d(D));
    // bf16 has fp32's range, so the softmax carries the grid's exponent
    // (P~ = P 2^s) and dQ~ leaves the GEMM on the grid. fp16 would overflow:
    // there P stays unscaled and the partial is multiplied by 2^s (exact)
    // before it is rounded. The exponent reaches the softmax inside the row
    // statistic s - L that the preprocess leaves.
    const float dq_mul = F16 ? pow2f(s_exp) : 1.f;
    const float c2 = p.scale * kLog2e;

    uint8_t* sK = smem + L::OFF_K;
    uint8_t* sV = smem + L::OFF_V;
    uint8_t* sQ = smem + L::OFF_Q;
    uint8_t* sdO = smem + L::OFF_DO;
    uint8_t* sPT = smem + L::OFF_PT;
    uint8_t* sdST = smem + L::OFF_DST;
    float* sL = reinterpret_cast<float*>(smem + L::OFF_L);
    float* sDl = reinterpret_cast<float*>(smem + L::OFF_DL);

    const int kvalid = min(BN, sq.len - n0);
    load_tile_async<D, L::PITCH, NTHREADS>(sK, row_ptr<const uint16_t>(p.k, b, sq.start + n0, hkv), p.k.sr, BN, kvalid, tid);
    load_tile_async<D, L::PITCH, NTHREADS>(sV, row_ptr<const uint16_t>(p.v, b, sq.start + n0, hkv), p.v.sr, BN, kvalid, tid);
    cp_async_commit();

    float acc_dk[NTD][4], acc_dv[NTD][4];
#pragma unroll
    for (int i = 0; i < NTD; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_dk[i][e] = acc_dv[i][e] = 0.f;

    const int nm = (sq.len + BM - 1) / BM;
    const int m_min = CAUSAL ? nb : 0;   // BM == BN

    for (int g = 0; g < p.G; ++g) {
        const int h = hkv * p.G + g;
        const int64_t wrow = static_cast<int64_t>(h) * p.rows_p + sq.pstart;
        for (int mb = m_min; mb < nm; ++mb) {
            const int m0 = mb * BM;
            const int qvalid = min(BM, sq.len - m0);
            load_tile_async<D, L::PITCH, NTHREADS>(sQ, row_ptr<const uint16_t>(p.q, b, sq.start + m0, h), p.q.sr, BM, qvalid, tid);
            load_tile_async<D, L::PITCH, NTHREADS>(sdO, row_ptr<const uint16_t>(p.dout, b, sq.start + m0, h), p.dout.sr, BM, qvalid, tid);
            cp_async_commit();
            if (tid < 64) sL[tid] = -p.lse2[wrow + m0 + tid];   // lse2 holds s - L: the same bits as L - s, negated
            else if (tid < 128) sDl[tid - 64] = p.dpsum[wrow + m0 + tid - 64];
            cp_async_wait<0>();
            __syncthreads();

            // ---- S^T = K Q^T and dP^T = V dO^T for 16 keys x 32 queries ----
            float s[4][4], dp[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[i][e] = dp[i][e] = 0.f;
            {
                const int arow = 16 * wk + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int brow = 32 * wd + (lane & 7) + 8 * (lane >> 4);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t ak[4], av[4];
                    ldmatrix_x4(ak, smem_u32(sK + arow * L::PITCH + (2 * ks + (lane >> 4)) * 16));
                    ldmatrix_x4(av, smem_u32(sV + arow * L::PITCH + (2 * ks + (lane >> 4)) * 16));
#pragma unroll
                    for (int np = 0; np < 2; ++np) {
                        uint32_t bq[4], bo[4];
                        const int off = (brow + 16 * np) * L::PITCH + (2 * ks + ((lane >> 3) & 1)) * 16;
                        ldmatrix_x4(bq, smem_u32(sQ + off));
                        ldmatrix_x4(bo, smem_u32(sdO + off));
                        mma_16816<F16>(s[2 * np], ak, bq[0], bq[1]);
                        mma_16816<F16>(s[2 * np + 1], ak, bq[2], bq[3]);
                        mma_16816<F16>(dp[2 * np], av, bo[0], bo[1]);
                        mma_16816<F16>(dp[2 * np + 1], av, bo[2], bo[3]);
                    }
                }
            }
            // ---- P~ = exp2(S c - (L - s)), dS~ = P~ (dP - Delta) ----
            const bool need_mask = (CAUSAL && mb == nb) || (n0 + BN > sq.len);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int ql = 32 * wd + 8 * nt + 2 * tq;
                const float l0 = sL[ql], l1 = sL[ql + 1];
                const float d0 = sDl[ql], d1 = sDl[ql + 1];
                float pv[4], ds[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kl = 16 * wk + gid + 8 * (e >> 1);
                    const float le = (e & 1) ? l1 : l0, de = (e & 1) ? d1 : d0;
                    float x = ex2_approx(fmaf(s[nt][e], c2, -le));
                    if (need_mask) {
                        const int kj = n0 + kl, qi = m0 + ql + (e & 1);
                        if (kj >= sq.len || (CAUSAL && kj > qi)) x = 0.f;
                    }
                    pv[e] = x;
                    ds[e] = x * (dp[nt][e] - de);
                }
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
                    const int kl = 16 * wk + gid + 8 * hlf;
                    *reinterpret_cast<uint32_t*>(sPT + kl * L::PPITCH + ql * 2) = pack16x2<F16>(pv[2 * hlf], pv[2 * hlf + 1]);
                    *reinterpret_cast<uint32_t*>(sdST + kl * L::PPITCH + ql * 2) = pack16x2<F16>(ds[2 * hlf], ds[2 * hlf + 1]);
                }
            }
            __syncthreads();

            // ---- dV += P~^T dO, dK += dS~^T Q : 16 keys x D/2 channels ----
            {
                const int arow = 16 * wk + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
                for (int ks = 0; ks < BM / 16; ++ks) {
                    uint32_t ap[4], ad[4];
                    ldmatrix_x4(ap, smem_u32(sPT + arow * L::PPITCH + (2 * ks + (lane >> 4)) * 16));
                    ldmatrix_x4(ad, smem_u32(sdST + arow * L::PPITCH + (2 * ks + (lane >> 4)) * 16));
                    const int krow = 16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
                    for (int np = 0; np < NTD / 2; ++np) {
                        uint32_t bo[4], bq[4];
                        const int off = krow * L::PITCH + (wd * (DH / 8) + 2 * np + (lane >> 4)) * 16;
                        ldmatrix_x4_trans(bo, smem_u32(sdO + off));
                        ldmatrix_x4_trans(bq, smem_u32(sQ + off));
                        mma_16816<F16>(acc_dv[2 * np], ap, bo[0], bo[1]);
                        mma_16816<F16>(acc_dv[2 * np + 1], ap, bo[2], bo[3]);
                        mma_16816<F16>(acc_dk[2 * np], ad, bq[0], bq[1]);
                        mma_16816<F16>(acc_dk[2 * np + 1], ad, bq[2], bq[3]);
                    }
                }
            }
            // ---- dQ~ = dS~ K : 16 queries x D/2 channels, onto the grid ----
            {
                float dq[NTD][4];
#pragma unroll
                for (int i = 0; i < NTD; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) dq[i][e] = 0.f;
                const int j = lane >> 3;
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    uint32_t a[4];
                    ldmatrix_x4_trans(a, smem_u32(sdST + (16 * ks + (lane & 7) + 8 * (j >> 1)) * L::PPITCH + (2 * wk + (j & 1)) * 16));
                    const int krow = 16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
                    for (int np = 0; np < NTD / 2; ++np) {
                        uint32_t bk[4];
                        ldmatrix_x4_trans(bk, smem_u32(sK + krow * L::PITCH + (wd * (DH / 8) + 2 * np + (lane >> 4)) * 16));
                        mma_16816<F16>(dq[2 * np], a, bk[0], bk[1]);
                        mma_16816<F16>(dq[2 * np + 1], a, bk[2], bk[3]);
                    }
                }
                int* acc = p.dq_acc + (wrow + m0) * D;
#pragma unroll
                for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int ql = 16 * wk + gid + 8 * (e >> 1);
                        const int d = wd * DH + 8 * nt + 2 * tq + (e & 1);
                        const int v = __float2int_rn(dq[nt][e] * dq_mul);
                        if (v != 0) atomicAdd(acc + ql * D + d, v);
                    }
            }
            __syncthreads();
        }
    }
    cp_async_wait<0>();

    // dK = round16(dK~ c 2^-s), dV = round16(dV~ 2^-s): P~ carried 2^s through
    // the whole loop, so both leave scaled by it and are put back exactly.
    const float un = F16 ? 1.f : pow2f(-s_exp);
    const float fk = p.scale * un;
#pragma unroll
    for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
            const int kl = 16 * wk + gid + 8 * hlf;
            if (n0 + kl < sq.len) {
                const int d = wd * DH + 8 * nt + 2 * tq;
                *reinterpret_cast<uint32_t*>(row_ptr<uint16_t>(p.dk, b, sq.start + n0 + kl, hkv) + d) =
                    pack16x2<F16>(acc_dk[nt][2 * hlf] * fk, acc_dk[nt][2 * hlf + 1] * fk);
                *reinterpret_cast<uint32_t*>(row_ptr<uint16_t>(p.dv, b, sq.start + n0 + kl, hkv) + d) =
                    pack16x2<F16>(acc_dv[nt][2 * hlf] * un, acc_dv[nt][2 * hlf + 1] * un);
            }
        }
}

template <int D, bool F16, bool CAUSAL>
static int launch_one(const BwdParams& p, cudaStream_t st) {
    using L = MmaSmem<D>;
    auto kern = bwd_main_mma_kernel<D, F16, CAUSAL>;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES);
        configured = true;
    }
    dim3 grid((p.S + BN - 1) / BN, p.HKV, p.B);
    kern<<<grid, NTHREADS, L::BYTES, st>>>(p);
    return check_launch("bwd_main_mma");
}

template <int D>
static int launch_d(const BwdParams& p, cudaStream_t st) {
    if (p.f16) return p.causal ? launch_one<D, true, true>(p, st) : launch_one<D, true, false>(p, st);
    return p.causal ? launch_one<D, false, true>(p, st) : launch_one<D, false, false>(p, st);
}

int launch_bwd_main_mma(const BwdParams& p, cudaStream_t st) {
    switch (p.D) {
        case 64: return launch_d<64>(p, st);
        case 96: return launch_d<96>(p, st);
        case 128: return launch_d<128>(p, st);
    }
    set_error("head_dim %d: 64, 96 and 128 are supported", p.D);
    return FOLD_ERR_UNSUPPORTED;
}

}  // namespace fold
