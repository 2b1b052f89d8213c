// Every write into the paged, quantised KV cache: a prompt's K and V, and a
// decode step's query planes and appended token.
//
// A row (one token of one head) is handled by D/16 lanes that each own one
// 16-byte unit of every stored plane, so a load is two and a store one 128-bit
// access, and K's XOR swizzle moves whole units. Each fp32 operation the cache
// format specifies is issued as its own round-to-nearest instruction (never
// contracted into an FMA), which makes the planes the bits of the reference's
// torch quantisers (src/fold_attention/decode/cache.py:72-158) whatever the
// batch a row is written with.
#include "common.cuh"
#include "fold_b200.h"

namespace fold {

constexpr int NT = 128;       // threads per CTA
constexpr int CHUNK = 256;    // tokens per reduction chunk of a prompt
constexpr float INV127 = 0.007874015718698502f;  // fp32(1)/fp32(127)

// Hadamard butterfly over a row split across `LANES` lanes of 16 elements:
// stages 1..8 inside the thread, the rest across lanes, then the 1/sqrt(D)
// scale (reference: utils.py:60-78, decode/quant.py:54-72).
template <int LANES>
__device__ __forceinline__ void rotate16(float (&x)[16], int lane, float hscale) {
#pragma unroll
    for (int h = 1; h < 16; h <<= 1) {
        float y[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if ((i & h) == 0) {
                y[i] = __fadd_rn(x[i], x[i + h]);
                y[i + h] = __fsub_rn(x[i], x[i + h]);
            }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = y[i];
    }
#pragma unroll
    for (int off = 1; off < LANES; off <<= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float o = __shfl_xor_sync(0xffffffffu, x[i], off);
            x[i] = upper ? __fsub_rn(o, x[i]) : __fadd_rn(x[i], o);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = __fmul_rn(x[i], hscale);
}

template <int LANES>
__device__ __forceinline__ float row_amax16(const float (&x)[16]) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(x[i]));
#pragma unroll
    for (int off = 1; off < LANES; off <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    return m;
}

__device__ __forceinline__ uint32_t pack4_s8(int a, int b, int c, int d) {
    return (a & 0xFF) | ((b & 0xFF) << 8) | ((c & 0xFF) << 16) | ((d & 0xFF) << 24);
}

// x = e (a + b/256): plane A from one rounded reciprocal and a multiply,
// plane B from the residual times a rounded 256/e (cache.py:72-78).
__device__ __forceinline__ void int8_planes16(const float (&x)[16], float e, uint4& wa, uint4& wb) {
    const float ie = __fdiv_rn(1.0f, e);
    const float t = __fdiv_rn(256.0f, e);
    int a[16], b[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float u = fmaxf(fminf(__fmul_rn(x[i], ie), 127.0f), -128.0f);
        float pa = rintf(u);
        float r = __fsub_rn(x[i], __fmul_rn(pa, e));
        float w = fmaxf(fminf(__fmul_rn(r, t), 127.0f), -128.0f);
        a[i] = static_cast<int>(pa);
        b[i] = static_cast<int>(rintf(w));
    }
    wa = make_uint4(pack4_s8(a[0], a[1], a[2], a[3]), pack4_s8(a[4], a[5], a[6], a[7]),
                    pack4_s8(a[8], a[9], a[10], a[11]), pack4_s8(a[12], a[13], a[14], a[15]));
    wb = make_uint4(pack4_s8(b[0], b[1], b[2], b[3]), pack4_s8(b[4], b[5], b[6], b[7]),
                    pack4_s8(b[8], b[9], b[10], b[11]), pack4_s8(b[12], b[13], b[14], b[15]));
}

// two fp32 -> packed e4m3x2 (lo in the low byte), round to nearest even, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
    // exact: e4m3 -> f16 is a hardware conversion, f16 -> f32 is exact
    uint32_t h2;
    uint16_t s = static_cast<uint16_t>(b & 0xFF);
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(s));
    return __half2float(__ushort_as_half(static_cast<uint16_t>(h2 & 0xFFFF)));
}

// V's two e4m3 planes in units of the layer scale: a = e4m3(clamp(v/e)),
// b = e4m3(clamp((v/e - a) * 8)) (cache.py:81-85).
__device__ __forceinline__ void e4m3_planes16(const float (&v)[16], float ievs, uint4& wa, uint4& wb) {
    uint32_t ca[16], cb[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        float s0 = __fmul_rn(v[i], ievs), s1 = __fmul_rn(v[i + 1], ievs);
        float c0 = fmaxf(fminf(s0, 448.f), -448.f), c1 = fmaxf(fminf(s1, 448.f), -448.f);
        uint32_t p = cvt_e4m3x2(c0, c1);
        ca[i] = p & 0xFF;
        ca[i + 1] = p >> 8;
        float r0 = __fmul_rn(__fsub_rn(s0, e4m3_to_float(ca[i])), 8.0f);
        float r1 = __fmul_rn(__fsub_rn(s1, e4m3_to_float(ca[i + 1])), 8.0f);
        r0 = fmaxf(fminf(r0, 448.f), -448.f);
        r1 = fmaxf(fminf(r1, 448.f), -448.f);
        uint32_t q = cvt_e4m3x2(r0, r1);
        cb[i] = q & 0xFF;
        cb[i + 1] = q >> 8;
    }
    auto pk = [](const uint32_t* c) { return c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24); };
    wa = make_uint4(pk(ca), pk(ca + 4), pk(ca + 8), pk(ca + 12));
    wb = make_uint4(pk(cb), pk(cb + 4), pk(cb + 8), pk(cb + 12));
}

// A rotated key's planes at pool row `prow`, swizzled by its page slot, and
// its bf16 scale (amax/127 rounded up to bf16, cache.py:97-106).
template <int D>
__device__ __forceinline__ void put_key(const float (&xk)[16], int8_t* ka, int8_t* kb,
                                        __nv_bfloat16* ek, int64_t prow, int off, int lane, bool ok) {
    constexpr int LANES = D / 16;
    constexpr int NU = LANES < 8 ? LANES : 8;
    constexpr int SH = NU == 8 ? 0 : (NU == 4 ? 1 : (NU == 2 ? 2 : 3));
    float e = __fmul_rn(fmaxf(row_amax16<LANES>(xk), 1e-30f), INV127);
    uint32_t hi = (__float_as_uint(e) + 0xFFFFu) >> 16;
    float es = __uint_as_float(hi << 16);
    uint4 wa, wb;
    int8_planes16(xk, es, wa, wb);
    if (ok) {
        int64_t addr = prow * D + ((lane ^ ((off >> SH) & (NU - 1))) * 16);
        *reinterpret_cast<uint4*>(ka + addr) = wa;
        *reinterpret_cast<uint4*>(kb + addr) = wb;
        if (lane == 0) reinterpret_cast<uint16_t*>(ek)[prow] = static_cast<uint16_t>(hi);
    }
}

template <int D, bool V8, bool F16>
__device__ __forceinline__ void put_value(const float (&xv)[16], const uint4 (&wv)[2], void* va,
                                          void* vb, int64_t prow, int lane, bool ok, float ievs) {
    if constexpr (V8) {
        uint4 wa, wb;
        e4m3_planes16(xv, ievs, wa, wb);
        if (ok) {
            int64_t addr = prow * D + lane * 16;
            *reinterpret_cast<uint4*>(static_cast<uint8_t*>(va) + addr) = wa;
            *reinterpret_cast<uint4*>(static_cast<uint8_t*>(vb) + addr) = wb;
        }
    } else {
        if (ok) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(va) + (prow * D + lane * 16) * 2);
            if constexpr (F16) {
                // the pool is bf16: an fp16 token is rounded to it once
                dst[0] = make_uint4(pack_bf16x2(xv[0], xv[1]), pack_bf16x2(xv[2], xv[3]),
                                    pack_bf16x2(xv[4], xv[5]), pack_bf16x2(xv[6], xv[7]));
                dst[1] = make_uint4(pack_bf16x2(xv[8], xv[9]), pack_bf16x2(xv[10], xv[11]),
                                    pack_bf16x2(xv[12], xv[13]), pack_bf16x2(xv[14], xv[15]));
            } else {
                dst[0] = wv[0];
                dst[1] = wv[1];
            }
        }
    }
}

// ------------------------------------------------------------ the prompt ----
// chunk table rows: (request, first token in the packed tensor, first
// position in the request, token count)

template <int D, bool F16>
__global__ void __launch_bounds__(NT) prompt_stats_kernel(const void* __restrict__ v,
                                                          const int4* __restrict__ chunks, int hkv,
                                                          float* __restrict__ vmax,
                                                          float* __restrict__ part) {
    constexpr int TPR = D / 16, RPB = NT / TPR;
    __shared__ float s_part[RPB][D];
    __shared__ float s_max[NT / 32];
    const int ch = blockIdx.x, h = blockIdx.y;
    const int slot = threadIdx.x / TPR, lane = threadIdx.x % TPR;
    const int4 c = chunks[ch];
    const int t0 = c.y, cnt = c.w;
    float vm = 0.f, vs[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) vs[i] = 0.f;
    for (int it = 0; it < CHUNK / RPB; ++it) {
        int r = it * RPB + slot;
        if (r < cnt) {
            float x[16];
            uint4 w[2];
            load16<F16>(static_cast<const uint8_t*>(v) + (static_cast<int64_t>(t0 + r) * hkv + h) * (D * 2) + lane * 32, x, w);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                vm = fmaxf(vm, fabsf(x[i]));
                vs[i] = __fadd_rn(vs[i], x[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) s_part[slot][lane * 16 + i] = vs[i];
    vm = warp_max(vm);
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = vm;
    __syncthreads();
    if (threadIdx.x < D) {
        float acc = 0.f;
#pragma unroll 1
        for (int j = 0; j < RPB; ++j) acc = __fadd_rn(acc, s_part[j][threadIdx.x]);
        part[(static_cast<int64_t>(ch) * hkv + h) * D + threadIdx.x] = acc;
    }
    if (threadIdx.x == 0) {
        float m = s_max[0];
        for (int j = 1; j < NT / 32; ++j) m = fmaxf(m, s_max[j]);
        vmax[static_cast<int64_t>(ch) * hkv + h] = m;
    }
}

// Per (request, head): its chunks' sums in order, the mean in the cache's
// units, and the layer's V scale: `vfix`, or the least power of two at or
// above amax * headroom / 448 (write.py:785-845).
template <int D>
__global__ void __launch_bounds__(NT) prompt_reduce_kernel(const int4* __restrict__ chunks,
                                                           const int* __restrict__ first, int nc,
                                                           int hkv, const float* __restrict__ vmax,
                                                           const float* __restrict__ part,
                                                           float* __restrict__ vsum,
                                                           float* __restrict__ vmean,
                                                           float* __restrict__ evs_out, float vh,
                                                           float vfix) {
    __shared__ float s_max[NT / 32];
    const int b = blockIdx.x, h = blockIdx.y;
    float vm = 0.f;
    for (int i = threadIdx.x; i < nc * hkv; i += NT) vm = fmaxf(vm, vmax[i]);
    vm = warp_max(vm);
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = vm;
    __syncthreads();
    vm = s_max[0];
    for (int j = 1; j < NT / 32; ++j) vm = fmaxf(vm, s_max[j]);
    float evs = vfix;
    if (vfix == 0.0f) {
        float t = fmaxf(__fmul_rn(__fmul_rn(vm, vh), 1.0f / 448.0f), 1e-30f);
        uint32_t bits = __float_as_uint(t);
        uint32_t e = bits & 0x7f800000u;
        if (bits & 0x7fffffu) e += 0x800000u;
        evs = __uint_as_float(e);
    }
    const int lo = first[b], hi = first[b + 1];
    if (threadIdx.x < D) {
        const int c = threadIdx.x;
        float vs = 0.f;
        int n = 0;
        for (int ch = lo; ch < hi; ++ch) {
            vs = __fadd_rn(vs, part[(static_cast<int64_t>(ch) * hkv + h) * D + c]);
            n += chunks[ch].w;
        }
        int64_t row = static_cast<int64_t>(b) * hkv + h;
        vsum[row * D + c] = vs;
        vmean[row * D + c] = __fdiv_rn(vs, __fmul_rn(static_cast<float>(n), evs));
    }
    if (threadIdx.x == 0 && b + h == 0) *evs_out = evs;
}

template <int D, bool V8, bool F16>
__global__ void __launch_bounds__(NT) prompt_write_kernel(
    const void* __restrict__ k, const void* __restrict__ v, const int4* __restrict__ chunks,
    const int* __restrict__ page_table, int ppr, int page_size, int hkv, int8_t* ka, int8_t* kb,
    void* va, void* vb, __nv_bfloat16* ek, const float* __restrict__ evs) {
    constexpr int TPR = D / 16, RPB = NT / TPR;
    const int ch = blockIdx.x / (CHUNK / RPB), it = blockIdx.x % (CHUNK / RPB);
    const int h = blockIdx.y;
    const int slot = threadIdx.x / TPR, lane = threadIdx.x % TPR;
    const int4 c = chunks[ch];
    const int r = it * RPB + slot;
    const bool ok = r < c.w;
    const int rr = ok ? r : 0;
    if (it * RPB >= c.w) return;  // whole CTA past the chunk
    const float ievs = __fdiv_rn(1.0f, *evs);
    const int64_t base = (static_cast<int64_t>(c.y + rr) * hkv + h) * (D * 2) + lane * 32;
    float xk[16], xv[16];
    uint4 wk[2], wv[2];
    load16<F16>(static_cast<const uint8_t*>(k) + base, xk, wk);
    load16<F16>(static_cast<const uint8_t*>(v) + base, xv, wv);
    const int pos = c.z + rr;
    const int pg = __ldg(page_table + static_cast<int64_t>(c.x) * ppr + pos / page_size);
    const int off = pos % page_size;
    const int64_t prow = (static_cast<int64_t>(pg) * hkv + h) * page_size + off;
    rotate16<TPR>(xk, lane, D == 64 ? 0.125f : 0.08838834764831845f);
    put_key<D>(xk, ka, kb, ek, prow, off, lane, ok);
    put_value<D, V8, F16>(xv, wv, va, vb, prow, lane, ok, ievs);
}

// --------------------------------------------------------------- the step ----
// CTAs [0, nq) quantise query rows (RPB rows each); CTAs [nq, nq + batch)
// append one request's token for all KV heads, then move its length. One CTA
// owns a request, so the length is read by every thread before one moves it
// and `lens_out` may alias `lens_in`.
template <int D, bool V8, bool F16>
__global__ void __launch_bounds__(NT) step_kernel(
    const void* __restrict__ q, int q_rows, int8_t* qa, int8_t* qb, float* eq,
    const void* __restrict__ k, const void* __restrict__ v, int batch, int hkv, int nq,
    const int* __restrict__ page_table, int ppr, int page_size, const int* lens_in, int* lens_out,
    int8_t* ka, int8_t* kb, void* va, void* vb, __nv_bfloat16* ek, float evs, float* vsum,
    float* vmean) {
    constexpr int TPR = D / 16, RPB = NT / TPR;
    constexpr float HS = D == 64 ? 0.125f : 0.08838834764831845f;
    const int slot = threadIdx.x / TPR, lane = threadIdx.x % TPR;
    if (static_cast<int>(blockIdx.x) < nq) {
        const int row = blockIdx.x * RPB + slot;
        const bool ok = row < q_rows;
        const int rr = ok ? row : 0;
        float x[16];
        uint4 w[2];
        load16<F16>(static_cast<const uint8_t*>(q) + static_cast<int64_t>(rr) * (D * 2) + lane * 32, x, w);
        const float qscale = D == 64 ? 0.18033688011112042f : 0.12751743082459868f;  // log2(e)/sqrt(D)
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = __fmul_rn(x[i], qscale);
        rotate16<TPR>(x, lane, HS);
        const float e = __fmul_rn(fmaxf(row_amax16<TPR>(x), 1e-30f), INV127);
        uint4 wa, wb;
        int8_planes16(x, e, wa, wb);
        if (ok) {
            *reinterpret_cast<uint4*>(qa + static_cast<int64_t>(row) * D + lane * 16) = wa;
            *reinterpret_cast<uint4*>(qb + static_cast<int64_t>(row) * D + lane * 16) = wb;
            if (lane == 0) eq[row] = e;
        }
        return;
    }
    const int b = blockIdx.x - nq;
    const int pos = lens_in[b];
    const int pg = __ldg(page_table + static_cast<int64_t>(b) * ppr + pos / page_size);
    const int off = pos % page_size;
    const float ievs = __fdiv_rn(1.0f, evs);
    const float n = __fmul_rn(static_cast<float>(pos + 1), evs);
    for (int h0 = 0; h0 < hkv; h0 += RPB) {
        const int h = h0 + slot;
        const bool ok = h < hkv;
        const int hh = ok ? h : 0;
        const int64_t base = (static_cast<int64_t>(b) * hkv + hh) * (D * 2) + lane * 32;
        float xk[16], xv[16];
        uint4 wk[2], wv[2];
        load16<F16>(static_cast<const uint8_t*>(k) + base, xk, wk);
        load16<F16>(static_cast<const uint8_t*>(v) + base, xv, wv);
        const int64_t prow = (static_cast<int64_t>(pg) * hkv + hh) * page_size + off;
        rotate16<TPR>(xk, lane, HS);
        put_key<D>(xk, ka, kb, ek, prow, off, lane, ok);
        put_value<D, V8, F16>(xv, wv, va, vb, prow, lane, ok, ievs);
        if (ok) {
            float* ps = vsum + (static_cast<int64_t>(b) * hkv + h) * D + lane * 16;
            float* pm = vmean + (static_cast<int64_t>(b) * hkv + h) * D + lane * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 s = *reinterpret_cast<float4*>(ps + 4 * j);
                s.x = __fadd_rn(s.x, xv[4 * j]);
                s.y = __fadd_rn(s.y, xv[4 * j + 1]);
                s.z = __fadd_rn(s.z, xv[4 * j + 2]);
                s.w = __fadd_rn(s.w, xv[4 * j + 3]);
                *reinterpret_cast<float4*>(ps + 4 * j) = s;
                float4 m = make_float4(__fdiv_rn(s.x, n), __fdiv_rn(s.y, n), __fdiv_rn(s.z, n),
                                       __fdiv_rn(s.w, n));
                *reinterpret_cast<float4*>(pm + 4 * j) = m;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) lens_out[b] = pos + 1;
}


// ------------------------------------------------------ the tail's append ----
// One CTA per (request, KV head), after the step that wrote the token: the
// token's 64-key block gains its V and its projection y = (plane A . u) ek / 256
// (the integer sum is exact in any order; the key's scale rounds it once), and
// the block's row becomes vsum / n - (ysum / n) vr^T in V's bf16. A block's
// first key restarts its sums, so a page reused from an earlier prompt carries
// nothing over. Plane A and the scale are read back from the pool, where the
// step left them (reference: src/fold_attention/decode/write.py:193-300).
template <int D, bool F16>
__global__ void __launch_bounds__(NT) tail_append_kernel(
    const void* __restrict__ v, const int8_t* __restrict__ ka, const uint16_t* __restrict__ ek,
    const int* __restrict__ page_table, int ppr, int page_size, const int* __restrict__ lens, int back,
    int hkv, const int8_t* __restrict__ tu, const float* __restrict__ tvr, float* tvsum, float* tysum,
    uint16_t* trows, int rank) {
    constexpr int NU = D / 16 < 8 ? D / 16 : 8;
    constexpr int SH = NU == 8 ? 0 : (NU == 4 ? 1 : 2);
    __shared__ int sA[D];
    __shared__ float sY[16];
    const int kr = blockIdx.x, b = kr / hkv, h = kr % hkv, tid = threadIdx.x;
    const int pos = lens[b] - back;
    if (pos < 0 || pos >= ppr * page_size) return;      // no appended token at this length: touch nothing
    const int pg = __ldg(page_table + static_cast<int64_t>(b) * ppr + pos / page_size);
    const int off = pos % page_size;
    const int64_t prow = (static_cast<int64_t>(pg) * hkv + h) * page_size + off;
    const int64_t blk = prow / 64;
    const bool first = (off % 64) == 0;
    const float nk = static_cast<float>(off % 64 + 1);
    if (tid < D) sA[tid] = ka[prow * D + ((((tid >> 4) ^ ((off >> SH) & (NU - 1))) << 4) | (tid & 15))];
    if (tid < 16) sY[tid] = 0.f;
    __syncthreads();
    if (rank > 0) {
        const int warp = tid >> 5, lane = tid & 31;
        const float ekf = __fmul_rn(bf16_bits_to_float(ek[prow]), 1.0f / 256.0f);
        for (int j = warp; j < rank; j += NT / 32) {
            const int8_t* up = tu + (static_cast<int64_t>(kr) * rank + j) * D;
            int dot = 0;
            for (int c = lane; c < D; c += 32) dot += sA[c] * static_cast<int>(up[c]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) {
                const float yj = __fmul_rn(static_cast<float>(dot), ekf);
                const float ys = __fadd_rn(first ? 0.f : tysum[blk * rank + j], yj);
                tysum[blk * rank + j] = ys;
                sY[j] = __fdiv_rn(ys, nk);
            }
        }
        __syncthreads();
    }
    if (tid < D) {
        const int64_t vi = static_cast<int64_t>(kr) * D + tid;
        const float xv = F16 ? __half2float(static_cast<const __half*>(v)[vi])
                             : __bfloat162float(static_cast<const __nv_bfloat16*>(v)[vi]);
        const float sm = __fadd_rn(first ? 0.f : tvsum[blk * D + tid], xv);
        float w = __fdiv_rn(sm, nk);
        for (int j = 0; j < rank; ++j) w = __fsub_rn(w, __fmul_rn(sY[j], tvr[vi * rank + j]));
        tvsum[blk * D + tid] = sm;
        trows[blk * D + tid] = __bfloat16_as_ushort(__float2bfloat16_rn(w));
    }
}

}  // namespace fold

using namespace fold;

// The tail's share of an append (no counterpart call in the reference, whose step
// kernel does it in place): run after fold_step_append on the same stream. The token
// sits at lens[b] - back: back = 1 when `lens` are the lengths the step already moved.
extern "C" int fold_tail_append(const void* v, int is_f16, int batch, int n_kv_heads, int head_dim,
                                const int32_t* page_table, int pages_per_request, int page_size,
                                const int32_t* lens, int back, const int8_t* ka, const void* ek,
                                const int8_t* tail_u, const float* tail_vr, float* tail_vsum,
                                float* tail_ysum, void* tail_rows, int tail_rank, void* stream) {
    FOLD_CHECK_ARG(head_dim == 64 || head_dim == 128, "head_dim %d: the cache writers take 64 or 128", head_dim);
    FOLD_CHECK_ARG(tail_rank == 0 || tail_rank == 16, "tail rank %d: 0 (block rows alone) or 16", tail_rank);
    FOLD_CHECK_ARG(v && page_table && lens && ka && ek && tail_vsum && tail_rows, "fold_tail_append: null pointer");
    FOLD_CHECK_ARG(tail_rank == 0 || (tail_u && tail_vr && tail_ysum), "fold_tail_append: rank 16 needs u, vr and ysum");
    FOLD_CHECK_ARG(page_size % 64 == 0, "page_size %d: the tail keeps one row per 64 keys of a page", page_size);
    FOLD_CHECK_ARG(back == 0 || back == 1, "back %d", back);
    if (batch <= 0) return FOLD_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t* ekp = static_cast<const uint16_t*>(ek);
    uint16_t* rows = static_cast<uint16_t*>(tail_rows);
#define FOLD_TAIL(DD, FF)                                                                             \
    tail_append_kernel<DD, FF><<<batch * n_kv_heads, NT, 0, st>>>(v, ka, ekp, page_table, pages_per_request, \
        page_size, lens, back, n_kv_heads, tail_u, tail_vr, tail_vsum, tail_ysum, rows, tail_rank)
    if (head_dim == 64) { if (is_f16) FOLD_TAIL(64, true); else FOLD_TAIL(64, false); }
    else                { if (is_f16) FOLD_TAIL(128, true); else FOLD_TAIL(128, false); }
#undef FOLD_TAIL
    return check_launch("fold_tail_append");
}

extern "C" int fold_cache_write_prompt(const void* k, const void* v, int is_f16,
                                       const int32_t* chunk_meta, int n_chunks, int batch,
                                       const int32_t* page_table, int pages_per_request,
                                       int page_size, int n_kv_heads, int head_dim, int8_t* ka,
                                       int8_t* kb, void* va, void* vb, void* ek, float* vsum,
                                       float* vmean, float* scratch, float v_headroom,
                                       float v_fixed, void* stream) {
    FOLD_CHECK_ARG(head_dim == 64 || head_dim == 128, "head_dim %d: the cache writers take 64 or 128", head_dim);
    FOLD_CHECK_ARG(k && v && chunk_meta && page_table && ka && kb && va && ek && vsum && vmean && scratch,
                   "fold_cache_write_prompt: null pointer");
    FOLD_CHECK_ARG(page_size > 0 && page_size % 8 == 0, "page_size %d is not a positive multiple of 8", page_size);
    if (n_chunks == 0) return FOLD_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int* first = chunk_meta;
    const int4* chunks = reinterpret_cast<const int4*>(chunk_meta + (batch + 1 + 3) / 4 * 4);
    float* vmax = scratch;
    float* part = scratch + static_cast<int64_t>(n_chunks) * n_kv_heads;
    float* evs = part + static_cast<int64_t>(n_chunks) * n_kv_heads * head_dim;
    const bool v8 = vb != nullptr;
    const float vfix = v8 ? v_fixed : 1.0f;
    __nv_bfloat16* ekp = static_cast<__nv_bfloat16*>(ek);
#define FOLD_PROMPT(DD, FF)                                                                          \
    do {                                                                                             \
        constexpr int RPB = NT / (DD / 16);                                                          \
        prompt_stats_kernel<DD, FF><<<dim3(n_chunks, n_kv_heads), NT, 0, st>>>(v, chunks, n_kv_heads, vmax, part); \
        prompt_reduce_kernel<DD><<<dim3(batch, n_kv_heads), NT, 0, st>>>(                             \
            chunks, first, n_chunks, n_kv_heads, vmax, part, vsum, vmean, evs, v_headroom, vfix);    \
        dim3 g(n_chunks * (CHUNK / RPB), n_kv_heads);                                                \
        if (v8)                                                                                      \
            prompt_write_kernel<DD, true, FF><<<g, NT, 0, st>>>(k, v, chunks, page_table, pages_per_request, page_size, n_kv_heads, ka, kb, va, vb, ekp, evs); \
        else                                                                                         \
            prompt_write_kernel<DD, false, FF><<<g, NT, 0, st>>>(k, v, chunks, page_table, pages_per_request, page_size, n_kv_heads, ka, kb, va, vb, ekp, evs); \
    } while (0)
    if (head_dim == 64) {
        if (is_f16) FOLD_PROMPT(64, true); else FOLD_PROMPT(64, false);
    } else {
        if (is_f16) FOLD_PROMPT(128, true); else FOLD_PROMPT(128, false);
    }
#undef FOLD_PROMPT
    return check_launch("fold_cache_write_prompt");
}

extern "C" int fold_step_append(const void* q, const void* k, const void* v, int is_f16, int batch,
                                int n_heads, int n_kv_heads, int head_dim,
                                const int32_t* page_table, int pages_per_request, int page_size,
                                const int32_t* lens_in, int32_t* lens_out, int8_t* qa, int8_t* qb,
                                float* eq, int8_t* ka, int8_t* kb, void* va, void* vb, void* ek,
                                float v_scale, float* vsum, float* vmean, void* stream) {
    FOLD_CHECK_ARG(head_dim == 64 || head_dim == 128, "head_dim %d: the cache writers take 64 or 128", head_dim);
    FOLD_CHECK_ARG((k == nullptr) == (v == nullptr), "k and v are both given or both left out");
    FOLD_CHECK_ARG(q || k, "fold_step_append: nothing to do");
    FOLD_CHECK_ARG(!q || (qa && qb && eq), "fold_step_append: null query plane");
    FOLD_CHECK_ARG(!k || (page_table && lens_in && lens_out && ka && kb && va && ek && vsum && vmean),
                   "fold_step_append: null cache pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rpb = NT / (head_dim / 16);
    const int q_rows = q ? batch * n_heads : 0;
    const int nq = (q_rows + rpb - 1) / rpb;
    const int grid = nq + (k ? batch : 0);
    if (grid == 0) return FOLD_OK;
    const bool v8 = vb != nullptr;
    __nv_bfloat16* ekp = static_cast<__nv_bfloat16*>(ek);
#define FOLD_STEP(DD, VV, FF)                                                                      \
    step_kernel<DD, VV, FF><<<grid, NT, 0, st>>>(q, q_rows, qa, qb, eq, k, v, batch, n_kv_heads, nq, \
                                                 page_table, pages_per_request, page_size, lens_in, \
                                                 lens_out, ka, kb, va, vb, ekp, v_scale, vsum, vmean)
    if (head_dim == 64) {
        if (v8) { if (is_f16) FOLD_STEP(64, true, true); else FOLD_STEP(64, true, false); }
        else    { if (is_f16) FOLD_STEP(64, false, true); else FOLD_STEP(64, false, false); }
    } else {
        if (v8) { if (is_f16) FOLD_STEP(128, true, true); else FOLD_STEP(128, true, false); }
        else    { if (is_f16) FOLD_STEP(128, false, true); else FOLD_STEP(128, false, false); }
    }
#undef FOLD_STEP
    return check_launch("fold_step_append");
}
