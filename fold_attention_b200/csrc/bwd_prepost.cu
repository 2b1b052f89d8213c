// The backward's memory-bound ends.
//
// Preprocess (one pass over O and dO, and over K and V once per KV head):
//   Delta_i = sum_d dO_id O_id, lse * log2(e), a zeroed dQ accumulator, and the
//   four order-free maxima the integer grid is derived from, published with
//   atomicMax on float bits: max|K|, max|V|, max ||dO_i||, max |Delta_i| per
//   (request, KV head); when dK and dV are folded across CTAs, also max |dO_id|
//   and max|Q|, which their grids need. Reference: src/fold_attention/backward/preprocess.py:176-346.
// Postprocess: dQ = round16( float(acc) * (softmax_scale * 2^-s) ); and for folded
//   dK, dV: dK = round16( float(acc) * (softmax_scale * 2^-s_dK) ), dV = round16( float(acc) * 2^-s_dV ).
//   Reference: src/fold_attention/backward/postprocess.py:125-154,256-344.
#include "bwd_common.cuh"

namespace fold {

constexpr int PRE_ROWS = 64;
constexpr int PRE_THREADS = 256;

template <bool F16>
__device__ __forceinline__ void unpack4(uint2 w, float (&x)[4]) {
    x[0] = half_bits_to_float<F16>(static_cast<uint16_t>(w.x & 0xFFFF));
    x[1] = half_bits_to_float<F16>(static_cast<uint16_t>(w.x >> 16));
    x[2] = half_bits_to_float<F16>(static_cast<uint16_t>(w.y & 0xFFFF));
    x[3] = half_bits_to_float<F16>(static_cast<uint16_t>(w.y >> 16));
}
__device__ __forceinline__ uint2 ldg8(const void* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

template <bool F16>
__global__ void __launch_bounds__(PRE_THREADS) bwd_preprocess_kernel(const BwdParams p) {
    const int mb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const SeqInfo sq = seq_info(p, b);
    const int len_r = (sq.len + ROW_PAD - 1) / ROW_PAD * ROW_PAD;
    if (mb * PRE_ROWS >= len_r) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D;
    const bool active = lane * 4 < D;
    const int hkv = h / p.G;
    const bool kv_owner = (h % p.G) == 0;
    float mx_k = 0.f, mx_v = 0.f, mx_dn = 0.f, mx_dl = 0.f, mx_doc = 0.f, mx_q = 0.f;
    const int64_t wbase = static_cast<int64_t>(h) * p.rows_p + sq.pstart;
    // Four rows per pass: all of their loads are issued before the first row's reductions, so a
    // warp keeps 8-16 requests in flight instead of 2-4 (the kernel is one pass over O, dO, K, V).
    constexpr int NW = PRE_THREADS / 32, RB = 4;
    for (int r0 = warp; r0 < PRE_ROWS; r0 += RB * NW) {
        uint2 ow[RB], gw[RB], kw[RB], vw[RB], qw[RB];
        float lraw[RB];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int i = mb * PRE_ROWS + r0 + u * NW;
            ow[u] = gw[u] = kw[u] = vw[u] = qw[u] = make_uint2(0u, 0u);
            lraw[u] = 0.f;
            if (i < sq.len) {
                if (active) {
                    ow[u] = ldg8(row_ptr<const uint16_t>(p.o, b, sq.start + i, h) + lane * 4);
                    gw[u] = ldg8(row_ptr<const uint16_t>(p.dout, b, sq.start + i, h) + lane * 4);
                    if (p.fold) qw[u] = ldg8(row_ptr<const uint16_t>(p.q, b, sq.start + i, h) + lane * 4);
                    if (kv_owner) {
                        kw[u] = ldg8(row_ptr<const uint16_t>(p.k, b, sq.start + i, hkv) + lane * 4);
                        vw[u] = ldg8(row_ptr<const uint16_t>(p.v, b, sq.start + i, hkv) + lane * 4);
                    }
                }
                lraw[u] = p.lse[b * p.lse_sb + h * p.lse_sh + sq.start + i];
            }
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int i = mb * PRE_ROWS + r0 + u * NW;
            float delta = 0.f, lse2 = INFINITY;
            if (i < sq.len) {
                float o[4], g[4];
                unpack4<F16>(ow[u], o);
                unpack4<F16>(gw[u], g);
                float d = o[0] * g[0] + o[1] * g[1] + o[2] * g[2] + o[3] * g[3];
                float n2 = g[0] * g[0] + g[1] * g[1] + g[2] * g[2] + g[3] * g[3];
                d = warp_sum(d);
                n2 = warp_sum(n2);
                delta = d;
                mx_dn = fmaxf(mx_dn, sqrtf(n2));
                mx_dl = fmaxf(mx_dl, fabsf(d));
                if (p.fold) {
                    float qq[4];
                    unpack4<F16>(qw[u], qq);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        mx_doc = fmaxf(mx_doc, fabsf(g[j]));
                        mx_q = fmaxf(mx_q, fabsf(qq[j]));
                    }
                }
                if (kv_owner && active) {
                    float kk[4], vv[4];
                    unpack4<F16>(kw[u], kk);
                    unpack4<F16>(vw[u], vv);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        mx_k = fmaxf(mx_k, fabsf(kk[j]));
                        mx_v = fmaxf(mx_v, fabsf(vv[j]));
                    }
                }
                const float l = lraw[u];
                lse2 = (l == -INFINITY) ? 0.f : l * kLog2e;
            }
            if (lane == 0) {
                p.dpsum[wbase + i] = delta;
                p.lse2[wbase + i] = lse2;
            }
            // Zero, or, when the main loop's partials each carry its rounding constant's bits, minus
            // their sum over the key blocks that reach this row's tile (int32 wraps: the total is exact)
            int init = 0;
            if (p.dq_bias) {
                const int tile = i / ROW_PAD, nkb = (sq.len + ROW_PAD - 1) / ROW_PAD;
                const unsigned n_part = static_cast<unsigned>(p.causal ? min(tile + 1, nkb) : nkb);
                init = static_cast<int>(0u - n_part * 0x4B400000u);
            }
            int4* acc = reinterpret_cast<int4*>(p.dq_acc + (wbase + i) * D);
            for (int c = lane; c < D / 4; c += 32) acc[c] = make_int4(init, init, init, init);
        }
    }
    __shared__ float s_red[6][PRE_THREADS / 32];
    mx_k = warp_max(mx_k);
    mx_v = warp_max(mx_v);
    mx_doc = warp_max(mx_doc);
    mx_q = warp_max(mx_q);
    if (lane == 0) {
        s_red[0][warp] = mx_k;
        s_red[1][warp] = mx_v;
        s_red[2][warp] = mx_dn;
        s_red[3][warp] = mx_dl;
        s_red[4][warp] = mx_doc;
        s_red[5][warp] = mx_q;
    }
    __syncthreads();
    if (threadIdx.x < (p.fold ? 6 : 4)) {
        float r = s_red[threadIdx.x][0];
        for (int w = 1; w < PRE_THREADS / 32; ++w) r = fmaxf(r, s_red[threadIdx.x][w]);
        // the max of non-negative floats is the max of their bits, and a max
        // lands the same in any order
        constexpr int slots[6] = {ST_K, ST_V, ST_DO, ST_DELTA, ST_DOC, ST_Q};
        const int slot = slots[threadIdx.x];
        if (threadIdx.x >= 2 || kv_owner)
            atomicMax(reinterpret_cast<unsigned int*>(p.stats + (static_cast<int64_t>(b) * p.HKV + hkv) * N_STATS + slot),
                      __float_as_uint(r));
    }
}

// element (row r, channel d) of a dQ accumulator tile of 128 rows
__device__ __forceinline__ int64_t dq_tile_offset(int layout, int r, int d, int D) {
    if (layout == DQ_LAYOUT_ROW_MAJOR) return static_cast<int64_t>(r) * D + d;
    // DQ_LAYOUT_SM100: 16-byte chunks of a row are interleaved over the 128
    // rows of a tile: chunk c of row r sits at (c * 128 + r) * 4 ints
    return (static_cast<int64_t>(d >> 2) * 128 + (r & 127)) * 4 + (d & 3) + static_cast<int64_t>(r >> 7) * 128 * D;
}

template <bool F16>
__global__ void __launch_bounds__(256) bwd_postprocess_dq_kernel(const BwdParams p, int layout) {
    const int h = blockIdx.y, b = blockIdx.z;
    const SeqInfo sq = seq_info(p, b);
    const int D = p.D, cpr = D / 4;  // 4-channel chunks per row
    const int rows_per_block = 256 / cpr > 0 ? 256 / cpr : 1;
    const int r0 = blockIdx.x * 64;
    if (r0 >= sq.len) return;
    const int s = dq_scale_exp(p.stats + (static_cast<int64_t>(b) * p.HKV + h / p.G) * N_STATS, root_d(D));
    const float f = __fmul_rn(p.scale, pow2f(-s));
    const int64_t wbase = (static_cast<int64_t>(h) * p.rows_p + sq.pstart) * D;
    for (int rr = threadIdx.x / cpr; rr < 64; rr += rows_per_block) {
        const int i = r0 + rr;
        const int c = threadIdx.x % cpr;
        if (i >= sq.len || threadIdx.x >= rows_per_block * cpr) continue;
        const int4 a = *reinterpret_cast<const int4*>(p.dq_acc + wbase + dq_tile_offset(layout, i, c * 4, D));
        const float x0 = __fmul_rn(static_cast<float>(a.x), f), x1 = __fmul_rn(static_cast<float>(a.y), f);
        const float x2 = __fmul_rn(static_cast<float>(a.z), f), x3 = __fmul_rn(static_cast<float>(a.w), f);
        uint2 w;
        if (F16) {
            w.x = pack_f16x2(x0, x1);
            w.y = pack_f16x2(x2, x3);
        } else {
            w.x = pack_bf16x2(x0, x1);
            w.y = pack_bf16x2(x2, x3);
        }
        *reinterpret_cast<uint2*>(row_ptr<uint16_t>(p.dq, b, sq.start + i, h) + c * 4) = w;
    }
}

// Second, tiny pass of the preprocess: once the maxima are in, the grid exponent s of each
// (request, KV head) is known, and the row statistic the main loop adds inside its exponential
// becomes s - lse * log2(e) (bf16; fp16 applies s at the dQ drain and keeps -lse * log2(e)): one
// add per row here instead of one per score there. Padded rows hold -inf: their weights are 0.
__global__ void __launch_bounds__(256) bwd_finalize_l_kernel(const BwdParams p) {
    const int h = blockIdx.y, b = blockIdx.z;
    const SeqInfo sq = seq_info(p, b);
    const int len_r = (sq.len + ROW_PAD - 1) / ROW_PAD * ROW_PAD;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= len_r) return;
    const int s = dq_scale_exp(p.stats + (static_cast<int64_t>(b) * p.HKV + h / p.G) * N_STATS, root_d(p.D));
    const float s_bias = p.f16 ? 0.f : static_cast<float>(s);
    float* l = p.lse2 + static_cast<int64_t>(h) * p.rows_p + sq.pstart + i;
    *l = s_bias - *l;
}

int launch_bwd_preprocess(const BwdParams& p, cudaStream_t st) {
    // the maxima, the status word and the work list's two counters
    cudaMemsetAsync(p.stats, 0, sizeof(int) * (N_STATS * p.B * p.HKV + 3), st);
    if (p.fold) {
        cudaMemsetAsync(p.dk_acc, 0, 8 * static_cast<size_t>(p.HKV) * p.rows_p * p.D, st);
        cudaMemsetAsync(p.dv_acc, 0, (p.dv_bits / 8) * static_cast<size_t>(p.HKV) * p.rows_p * p.D, st);
    }
    const int s_r = (p.S + ROW_PAD - 1) / ROW_PAD * ROW_PAD;
    dim3 grid(s_r / PRE_ROWS, p.H, p.B);
    if (p.f16)
        bwd_preprocess_kernel<true><<<grid, PRE_THREADS, 0, st>>>(p);
    else
        bwd_preprocess_kernel<false><<<grid, PRE_THREADS, 0, st>>>(p);
    bwd_finalize_l_kernel<<<dim3((s_r + 255) / 256, p.H, p.B), 256, 0, st>>>(p);
    return check_launch("bwd_preprocess");
}

// Folded dK and dV: the integer sums back to 16-bit. One fp32 multiply per element, as for dQ;
// an int64 sum is rounded to fp32 first (nearest even), which is all the precision the 16-bit
// result keeps.
template <bool F16>
__global__ void __launch_bounds__(256) bwd_postprocess_dkv_kernel(const BwdParams p) {
    const int hkv = blockIdx.y, b = blockIdx.z;
    const SeqInfo sq = seq_info(p, b);
    const int D = p.D, cpr = D / 4;
    const int rows_per_block = 256 / cpr > 0 ? 256 / cpr : 1;
    const int r0 = blockIdx.x * 64;
    if (r0 >= sq.len) return;
    const int* st = p.stats + (static_cast<int64_t>(b) * p.HKV + hkv) * N_STATS;
    const float rows = static_cast<float>(p.G) * static_cast<float>(sq.len);
    const int s_k = dk_scale_exp(st, rows, root_d(D));
    const int s_v = dv_scale_exp(st, rows, p.dv_bits == 32 ? DQ_BITS : DKV_BITS);
    const float f_k = __fmul_rn(p.scale, pow2f(-s_k)), f_v = pow2f(-s_v);
    const int64_t wbase = (static_cast<int64_t>(hkv) * p.rows_p + sq.pstart) * D;
    auto pack4 = [](float x0, float x1, float x2, float x3) {
        uint2 w;
        w.x = F16 ? pack_f16x2(x0, x1) : pack_bf16x2(x0, x1);
        w.y = F16 ? pack_f16x2(x2, x3) : pack_bf16x2(x2, x3);
        return w;
    };
    for (int rr = threadIdx.x / cpr; rr < 64; rr += rows_per_block) {
        const int i = r0 + rr;
        const int c = threadIdx.x % cpr;
        if (i >= sq.len || threadIdx.x >= rows_per_block * cpr) continue;
        const int64_t at = wbase + static_cast<int64_t>(i) * D + c * 4;
        const longlong2 k0 = *reinterpret_cast<const longlong2*>(p.dk_acc + at), k1 = *reinterpret_cast<const longlong2*>(p.dk_acc + at + 2);
        *reinterpret_cast<uint2*>(row_ptr<uint16_t>(p.dk, b, sq.start + i, hkv) + c * 4) =
            pack4(__fmul_rn(__ll2float_rn(k0.x), f_k), __fmul_rn(__ll2float_rn(k0.y), f_k), __fmul_rn(__ll2float_rn(k1.x), f_k),
                  __fmul_rn(__ll2float_rn(k1.y), f_k));
        float v0, v1, v2, v3;
        if (p.dv_bits == 32) {
            const int4 a = *reinterpret_cast<const int4*>(static_cast<const int*>(p.dv_acc) + at);
            v0 = static_cast<float>(a.x); v1 = static_cast<float>(a.y); v2 = static_cast<float>(a.z); v3 = static_cast<float>(a.w);
        } else {
            const long long* va = static_cast<const long long*>(p.dv_acc) + at;
            const longlong2 a0 = *reinterpret_cast<const longlong2*>(va), a1 = *reinterpret_cast<const longlong2*>(va + 2);
            v0 = __ll2float_rn(a0.x); v1 = __ll2float_rn(a0.y); v2 = __ll2float_rn(a1.x); v3 = __ll2float_rn(a1.y);
        }
        *reinterpret_cast<uint2*>(row_ptr<uint16_t>(p.dv, b, sq.start + i, hkv) + c * 4) =
            pack4(__fmul_rn(v0, f_v), __fmul_rn(v1, f_v), __fmul_rn(v2, f_v), __fmul_rn(v3, f_v));
    }
}

int launch_bwd_postprocess(const BwdParams& p, int layout, cudaStream_t st) {
    dim3 grid((p.S + 63) / 64, p.H, p.B);
    if (p.f16)
        bwd_postprocess_dq_kernel<true><<<grid, 256, 0, st>>>(p, layout);
    else
        bwd_postprocess_dq_kernel<false><<<grid, 256, 0, st>>>(p, layout);
    if (p.fold) {
        dim3 gkv((p.S + 63) / 64, p.HKV, p.B);
        if (p.f16)
            bwd_postprocess_dkv_kernel<true><<<gkv, 256, 0, st>>>(p);
        else
            bwd_postprocess_dkv_kernel<false><<<gkv, 256, 0, st>>>(p);
    }
    return check_launch("bwd_postprocess");
}

}  // namespace fold
