// Attention forward producing O and the log-sum-exp the backward consumes.
// The reference takes both from a third-party forward
// (src/fold_attention/interface.py:42-44,70-81); this is a self-contained
// online-softmax kernel on mma.sync so the package has no such dependency.
// One CTA: 64 query rows of one head; four warps of 16 rows each.
#include "bwd_common.cuh"
#include "mma_utils.cuh"

namespace fold {

struct FwdParams {
    TensorView q, k, v, o;
    float* lse;
    int64_t lse_sb, lse_sh;
    const int* cu;
    int B, H, HKV, G, S, D, causal, f16;
    float scale;
};

template <int D, bool F16, bool CAUSAL>
__global__ void __launch_bounds__(128) fwd_mma_kernel(const FwdParams p) {
    constexpr int PITCH = D * 2 + 16, TILE = 64 * PITCH, NTO = D / 8;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = smem + TILE;
    uint8_t* sV = smem + 2 * TILE;
    const int mb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    int start = 0, len = p.S;
    if (p.cu) {
        start = p.cu[b];
        len = p.cu[b + 1] - start;
    }
    const int m0 = mb * 64;
    if (m0 >= len) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tq = lane & 3;
    const int hkv = h / p.G;
    const float c2 = p.scale * kLog2e;

    load_tile_async<D, PITCH, 128>(sQ, row_ptr<const uint16_t>(p.q, b, start + m0, h), p.q.sr, 64, min(64, len - m0), tid);
    cp_async_commit();

    float o[NTO][4];
#pragma unroll
    for (int i = 0; i < NTO; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float mx[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f};

    const int n_end = CAUSAL ? min(len, m0 + 64) : len;
    for (int n0 = 0; n0 < n_end; n0 += 64) {
        __syncthreads();  // previous tile's reads are done
        const int kvalid = min(64, len - n0);
        load_tile_async<D, PITCH, 128>(sK, row_ptr<const uint16_t>(p.k, b, start + n0, hkv), p.k.sr, 64, kvalid, tid);
        load_tile_async<D, PITCH, 128>(sV, row_ptr<const uint16_t>(p.v, b, start + n0, hkv), p.v.sr, 64, kvalid, tid);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
        const int arow = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int brow = (lane & 7) + 8 * (lane >> 4);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_u32(sQ + arow * PITCH + (2 * ks + (lane >> 4)) * 16));
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bk[4];
                ldmatrix_x4(bk, smem_u32(sK + (brow + 16 * np) * PITCH + (2 * ks + ((lane >> 3) & 1)) * 16));
                mma_16816<F16>(s[2 * np], a, bk[0], bk[1]);
                mma_16816<F16>(s[2 * np + 1], a, bk[2], bk[3]);
            }
        }
        const bool need_mask = (CAUSAL && n0 + 64 > m0) || (n0 + 64 > len);
        float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x = s[nt][e] * c2;
                if (need_mask) {
                    const int kj = n0 + 8 * nt + 2 * tq + (e & 1);
                    const int qi = m0 + 16 * warp + gid + 8 * (e >> 1);
                    if (kj >= len || (CAUSAL && kj > qi)) x = -INFINITY;
                }
                s[nt][e] = x;
                rmax[e >> 1] = fmaxf(rmax[e >> 1], x);
            }
        float corr[2], mnew[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
            rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
            mnew[r] = fmaxf(mx[r], rmax[r]);
            const float ms = mnew[r] == -INFINITY ? 0.f : mnew[r];
            corr[r] = ex2_approx(mx[r] - ms);
            mx[r] = mnew[r];
            mnew[r] = ms;
        }
        float rsum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = ex2_approx(s[nt][e] - mnew[e >> 1]);
                s[nt][e] = pv;
                rsum[e >> 1] += pv;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) ls[r] = ls[r] * corr[r] + rsum[r];
#pragma unroll
        for (int i = 0; i < NTO; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack16x2<F16>(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack16x2<F16>(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack16x2<F16>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack16x2<F16>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            const int krow = 16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
            for (int np = 0; np < NTO / 2; ++np) {
                uint32_t bv[4];
                ldmatrix_x4_trans(bv, smem_u32(sV + krow * PITCH + (2 * np + (lane >> 4)) * 16));
                mma_16816<F16>(o[2 * np], a, bv[0], bv[1]);
                mma_16816<F16>(o[2 * np + 1], a, bv[2], bv[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        ls[r] += __shfl_xor_sync(0xffffffffu, ls[r], 1);
        ls[r] += __shfl_xor_sync(0xffffffffu, ls[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = m0 + 16 * warp + gid + 8 * r;
        if (qi >= len) continue;
        const float inv = ls[r] > 0.f ? 1.f / ls[r] : 0.f;
        uint16_t* orow = row_ptr<uint16_t>(p.o, b, start + qi, h);
#pragma unroll
        for (int i = 0; i < NTO; ++i)
            *reinterpret_cast<uint32_t*>(orow + 8 * i + 2 * tq) = pack16x2<F16>(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
        if (tq == 0)
            p.lse[b * p.lse_sb + h * p.lse_sh + start + qi] =
                ls[r] > 0.f ? (mx[r] + log2f(ls[r])) * 0.6931471805599453f : -INFINITY;
    }
}

template <int D, bool F16, bool CAUSAL>
static int fwd_launch_one(const FwdParams& p, cudaStream_t st) {
    constexpr int BYTES = 3 * 64 * (D * 2 + 16);
    auto kern = fwd_mma_kernel<D, F16, CAUSAL>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BYTES);
    dim3 grid((p.S + 63) / 64, p.H, p.B);
    kern<<<grid, 128, BYTES, st>>>(p);
    return check_launch("fwd_mma");
}

template <int D>
static int fwd_launch_d(const FwdParams& p, cudaStream_t st) {
    if (p.f16) return p.causal ? fwd_launch_one<D, true, true>(p, st) : fwd_launch_one<D, true, false>(p, st);
    return p.causal ? fwd_launch_one<D, false, true>(p, st) : fwd_launch_one<D, false, false>(p, st);
}

}  // namespace fold

using namespace fold;

extern "C" int fold_fwd_run(const void* q, const void* k, const void* v, void* o, float* lse,
                            const int64_t* strides, const int32_t* cu_seqlens, int batch,
                            int n_heads, int n_kv_heads, int max_seqlen, int total, int head_dim,
                            int causal, int is_f16, float softmax_scale, void* stream) {
    FOLD_CHECK_ARG(q && k && v && o && lse && strides, "fold_fwd_run: null pointer");
    FOLD_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0, "the query heads must be a multiple of the KV heads");
    FOLD_CHECK_ARG(batch > 0 && max_seqlen > 0, "fold_fwd_run: empty call");
    FwdParams p;
    const void* ptrs[4] = {q, k, v, o};
    TensorView* views[4] = {&p.q, &p.k, &p.v, &p.o};
    for (int i = 0; i < 4; ++i) {
        views[i]->ptr = const_cast<void*>(ptrs[i]);
        views[i]->sb = strides[3 * i];
        views[i]->sr = strides[3 * i + 1];
        views[i]->sh = strides[3 * i + 2];
        FOLD_CHECK_ARG(views[i]->sr % 8 == 0 && views[i]->sh % 8 == 0 && views[i]->sb % 8 == 0 &&
                           reinterpret_cast<uintptr_t>(ptrs[i]) % 16 == 0,
                       "fold_fwd_run: rows must be 16-byte aligned");
    }
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
    p.S = max_seqlen; p.D = head_dim; p.causal = causal; p.f16 = is_f16; p.scale = softmax_scale;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (head_dim) {
        case 64: return fwd_launch_d<64>(p, st);
        case 96: return fwd_launch_d<96>(p, st);
        case 128: return fwd_launch_d<128>(p, st);
    }
    set_error("head_dim %d: 64, 96 and 128 are supported", head_dim);
    return FOLD_ERR_UNSUPPORTED;
}
