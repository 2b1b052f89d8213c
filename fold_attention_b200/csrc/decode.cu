// Quantised paged-KV decode: the mass reference Z, the split-KV kernel and the
// additive combine.
//
// A row group is the G <= 8 query rows that share one KV head of one request.
// One CTA owns (row group, split) and walks 64-key tiles:
//   1. plane A of K and the key scales arrive by bulk copy (a tile is
//      contiguous inside its page) into a 3-slot ring, two tiles ahead;
//   2. the coarse logit 256 c1 + c2 (int8 mma.sync against both Q planes, Q
//      fragments held in registers) gives s1 = fma(int, eq ek/256, -Z) and the
//      verdict bits live / refine-K / refine-V, ORed over the group's rows;
//   3. the live keys' V rows, the refined keys' plane-B K rows and V plane-B
//      rows are gathered with 128-bit cp.async through the page table (rows
//      not selected are zero-filled and move no bytes);
//   4. one tile later, plane B refines the logits, weights w = exp2(s - Z) are
//      final at once (Z is fixed before the loop), go to bf16 (value and
//      rounding error as two terms) and meet V in a bf16 mma.sync; a cut key
//      adds its weight to the row's dropped mass instead.
// Partials (numerator, denominator + dropped mass, counts) are plain sums the
// combine adds in slot order.
// Reference: src/fold_attention/decode/kernel.py:95-1488, combine.py:10-162,
// reference.py:120-406 (the arithmetic; the schedule here is B200's own).
#include "common.cuh"
#include "fold_b200.h"
#include "mma_utils.cuh"

namespace fold {

constexpr int BNK = 64;          // keys per tile
constexpr int DEC_THREADS = 128;
constexpr int RING = 3;
constexpr long long WAIT_CYCLES = 1ll << 31;   // about a second of SM clocks
constexpr float E4W = 18446744073709551616.0f;   // 2^64 on the weights of an 8-bit V
constexpr float E4O = 72057594037927936.0f;      // 2^56 on its accumulator

struct DecodeParams {
    const int8_t* qa; const int8_t* qb; const float* eq;     // (NBH, G, D), (NBH, G)
    const int8_t* ka; const int8_t* kb; const uint16_t* ek;  // pool planes, bf16 scales
    const uint8_t* va; const uint8_t* vb;                    // bf16 or e4m3 (+ plane B)
    const float* vmean;                                      // (NBH, D) or null
    const float* z; const float* cut;                        // (NBH, G): reference, depth below it
    const int* page_table; const int* seq_lens; const int* order;
    float* o_part; float* den_part; int* cnt_part;
    int nbh, G, hkv, ppr, page_size, split, chunk_keys, truncate, banded;
    float rk, rv, band_e0, band_e1, rk1, rk2, rv1, rv2;
    int* status;
    // the tail (bf16 V, truncating): one bf16 row per 64 pool rows, each row group's int8
    // projection (16, D) and map back (D, 16); all null without a tail, u and vr null at rank 0
    const uint16_t* tail_rows; const int8_t* tail_u; const float* tail_vr;
    // levels and layouts beyond the single-level step (all neutral by default):
    const int* req_map;     // request -> row of page_table / seq_lens (a cascade's shared level: its prefix); null: itself
    const int* tree;        // (NBH, G) int32, bit j of a row: draft node j is visible to it; null without a draft
    int q_len;              // draft nodes: the cache's last q_len keys; 0 without a draft
    int gsub;               // row groups per KV head (a group wider than 8 rows runs as gsub groups of 8)
    int slots_total, slot_off;   // partial slot of (row group, split sp): bh * slots_total + slot_off + sp
    int row_cut;            // 1: a key enters a row only if that row keeps it (drafts, cascades); 0: if any row of the group does
    const float* sound;     // (NBH, G) or null: eq * sum_d (128 |qa_d| + |qb_d| / 2), the bound on what plane B of K can
                            // add to a row's logit per unit of the key's ek / 256; the verdict then tests s1 + bound
    int vmean_rows;         // 1: vmean is (NBH, G, D), a direction per query row
    int bh_limit;   // > 0: the partial buffers hold this many row groups; an `order` entry outside is refused
};

// ---- small PTX wrappers -----------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// A bounded wait: on expiry the status word is set and false returned, so the
// CTA can leave without hanging the device.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
    const long long t0 = clock64();
    for (int i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63 && clock64() - t0 > WAIT_CYCLES) break;
    }
    atomicExch(status, FOLD_ERR_TIMEOUT);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
// two e4m3 bytes (byte i of w0 -> low half, of w1 -> high half) as bf16x2 * 2^-120
__device__ __forceinline__ uint32_t e4m3_pair_bf16(uint32_t w0, uint32_t w1, int i) {
    const uint32_t sel = i | (i << 4) | ((4 + i) << 8) | ((4 + i) << 12);
    const uint32_t x = __byte_perm(w0, w1, sel);
    return (x & 0x80008000u) | ((x >> 4) & 0x07F007F0u);
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int D>
__device__ __forceinline__ int swz(int r) { return D >= 128 ? (r & 7) : ((r >> 1) & 3); }

// where 16-byte unit u of gathered V row r lands in shared memory: an XOR on
// the low unit bits, so a lane quad reading four rows hits distinct banks
template <int UNITS>
__device__ __forceinline__ int vswz(int u, int r) {
    constexpr int M = (UNITS < 8 ? UNITS : 8) - 1;
    return (u & ~M) | ((u ^ r) & M);
}

// ---- the split-KV kernel ------------------------------------------------------
template <int D, bool V8>
struct DecSmem {
    static constexpr int KA = BNK * D, KS = BNK * 2;
    static constexpr int SLOT = KA + KS;               // plane A tile + its scales
    static constexpr int VROW = V8 ? D : 2 * D;
    static constexpr int GKB = BNK * D, GVA = BNK * VROW, GVB = V8 ? BNK * D : 0;
    static constexpr int GTL = V8 ? 0 : 2 * D;         // the tile's tail row (its 64-key block's)
    static constexpr int OFF_TL = GKB + GVA + GVB;
    static constexpr int GBUF = GKB + GVA + GVB + GTL;
    static constexpr int OFF_RING = 0, OFF_G = RING * SLOT, OFF_LIVE = OFF_G + 2 * GBUF;
    static constexpr int OFF_BAR = OFF_LIVE + 2 * BNK * 4, OFF_RED = OFF_BAR + 64;
    static constexpr int OFF_FAIL = OFF_RED + 1024;
    static constexpr int BYTES = OFF_FAIL + 16;
};

// TR: the tail's rank (-1 none, 0 block rows alone, 16). With a tail a dropped key re-enters at
// its 64-key block's row plus the part of its V its K predicts: y = (plane A . u) ek / 256 comes
// out of the coarse logit's own matmul (u's rows are two more B operands), the dropped weights
// meet it in one bf16 mma per 8 ranks, and the epilogue maps the rank sums back through vr.
// EX: the layouts beyond the single-level step (a cascade's shared level, split row groups, a
// draft's visibility words, a row's own cut); a build of its own, so the step's builds keep
// their registers.
template <int D, bool V8, bool W2, bool TRUNC, int TR, bool EX = false>
__global__ void __launch_bounds__(DEC_THREADS) decode_kernel(const DecodeParams p) {
    static_assert(!EX || TR < 0, "the tail runs on single-level steps");
    static_assert(TR < 0 || (TRUNC && !V8), "the tail re-enters truncated mass on a bf16 V");
    static_assert(TR == -1 || TR == 0 || TR == 16, "tail ranks: none, 0, 16");
    using L = DecSmem<D, V8>;
    constexpr int NU = D / 16;          // 16-byte units per int8 row
    constexpr int KSTEPS = D / 32;      // k-steps of the int8 logit
    constexpr int NT = D / 8;           // 8-channel n-tiles of the value product
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tq = lane & 3;
    const int slot = blockIdx.x / p.split, sp = blockIdx.x % p.split;
    const int bh = p.order ? p.order[slot] : slot;
    if (p.bh_limit > 0 && (bh < 0 || bh >= p.bh_limit)) {   // would index past the partial buffers: touch nothing
        if (tid == 0) atomicExch(p.status, FOLD_ERR_ARGUMENT);
        return;
    }
    const int bhk = EX ? bh / p.gsub : bh;             // the KV head's row group in the cache's numbering
    const int breq = bhk / p.hkv, hkv = bhk % p.hkv;
    const int preq = (EX && p.req_map) ? p.req_map[breq] : breq;
    const int slen = p.seq_lens[preq];
    const int G = p.G, PS = p.page_size;

    // this split's tiles: interleaved (tile sp, sp + split, ...) or a fixed chunk
    int lo, hi, tstep, n_tiles;
    if (p.chunk_keys > 0) {
        lo = sp * p.chunk_keys;
        hi = min(lo + p.chunk_keys, slen);
        tstep = BNK;
        n_tiles = hi > lo ? (hi - lo + BNK - 1) / BNK : 0;
        if (n_tiles == 0) return;   // the combine reads only the splits a request reaches
    } else {
        lo = sp * BNK;
        hi = slen;
        tstep = p.split * BNK;
        const int all = (slen + BNK - 1) / BNK;
        n_tiles = all > sp ? (all - sp + p.split - 1) / p.split : 0;
    }
    const int64_t pix = EX ? static_cast<int64_t>(bh) * p.slots_total + p.slot_off + sp : static_cast<int64_t>(bh) * p.split + sp;

    float rk = p.rk, rv = p.rv;
    if (p.banded) {
        rk = slen > static_cast<int>(p.band_e1) ? p.rk2 : (slen > static_cast<int>(p.band_e0) ? p.rk1 : p.rk);
        rv = slen > static_cast<int>(p.band_e1) ? p.rv2 : (slen > static_cast<int>(p.band_e0) ? p.rv1 : p.rv);
    }

    uint32_t bars[RING];
#pragma unroll
    for (int i = 0; i < RING; ++i) bars[i] = smem_u32(smem + L::OFF_BAR + 8 * i);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_FAIL);
    if (tid == 0) {
        *sFail = 0;
#pragma unroll
        for (int i = 0; i < RING; ++i) mbar_init(bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int* ptab = p.page_table + static_cast<int64_t>(preq) * p.ppr;
    // pool row of position `pos` of this row group
    auto pool_row = [&](int pos) -> int64_t {
        return (static_cast<int64_t>(__ldg(ptab + pos / PS)) * p.hkv + hkv) * PS + pos % PS;
    };
    // tile t's plane A and scales into ring slot t % RING, in page segments
    auto issue_tile = [&](int t) {
        const int base = lo + t * tstep;
        const int nrow = min(BNK, hi - base);
        const int seg = min(PS, BNK);
        const int nseg = (nrow + seg - 1) / seg;
        uint8_t* dst = smem + L::OFF_RING + (t % RING) * L::SLOT;
        const uint32_t bar = bars[t % RING];
        mbar_expect_tx(bar, nseg * seg * (D + 2));
        for (int s = 0; s < nseg; ++s) {
            const int64_t r = pool_row(base + s * seg);
            bulk_g2s(smem_u32(dst + s * seg * D), p.ka + r * D, seg * D, bar);
            bulk_g2s(smem_u32(dst + L::KA + s * seg * 2), p.ek + r, seg * 2, bar);
        }
    };
    if (tid == 0) {
        for (int t = 0; t < min(2, n_tiles); ++t) issue_tile(t);
    }

    // Q fragments: B operand of m16n8k32, row g = gid, channels 32 ks + 4 tq (+16)
    uint32_t qfa[KSTEPS][2], qfb[KSTEPS][2];
    {
        const bool ok = gid < G;
        const int64_t qrow = (static_cast<int64_t>(bh) * G + (ok ? gid : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = 32 * ks + 16 * j + 4 * tq;
                qfa[ks][j] = ok ? *reinterpret_cast<const uint32_t*>(p.qa + qrow + c) : 0u;
                qfb[ks][j] = ok ? *reinterpret_cast<const uint32_t*>(p.qb + qrow + c) : 0u;
            }
    }
    // the tail's projection: rank rows gid and 8 + gid as B operands beside Q's
    uint32_t ufa[TR > 0 ? KSTEPS : 1][2], ufb[TR > 0 ? KSTEPS : 1][2];
    if constexpr (TR > 0) {
        const int8_t* up = p.tail_u + static_cast<int64_t>(bh) * TR * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = 32 * ks + 16 * j + 4 * tq;
                ufa[ks][j] = *reinterpret_cast<const uint32_t*>(up + gid * D + c);
                ufb[ks][j] = *reinterpret_cast<const uint32_t*>(up + (8 + gid) * D + c);
            }
    }
    float y_old[TR > 0 ? 8 : 1] = {}, yd[2][4] = {};
    (void)ufa; (void)ufb; (void)y_old; (void)yd;
    // the two rows this lane's logit registers belong to
    float eqr[2], zr[2], cutr[2];
    bool rowok[2];
    uint32_t treer[2] = {~0u, ~0u};
    float soundr[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int g = 2 * tq + j;
        rowok[j] = g < G;
        const int64_t ix = static_cast<int64_t>(bh) * G + (rowok[j] ? g : 0);
        eqr[j] = p.eq[ix];
        zr[j] = p.z[ix];
        cutr[j] = -p.cut[ix];
        if (EX && p.tree) treer[j] = static_cast<uint32_t>(p.tree[ix]);
        if (EX && p.sound) soundr[j] = p.sound[ix];
    }
    // a draft: the cache's last q_len keys are the draft's own nodes, and a row sees node j only
    // if bit j of its word is set (a chain's row t sees nodes 0..t)
    const int node0 = (EX && p.q_len > 0) ? slen - p.q_len : (1 << 30);
    auto sees = [&](int j, int kabs) { return !EX || kabs < node0 || ((treer[j] >> (kabs - node0)) & 1u) != 0u; };
    (void)treer; (void)node0; (void)soundr;
    int kb_old = 0;     // bit i: this lane's row i & 1 itself keeps its key i >> 1 (read under a row's own cut)

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    float rM[2] = {0.f, 0.f}, rN[2] = {0.f, 0.f};
    int nlive = 0, nref = 0;

    float s_old[4] = {0, 0, 0, 0}, tk_old[4] = {0, 0, 0, 0};
    int b_old[2] = {0, 0}, nrow_old = 0, base_old = 0;
    bool failed = false;

    for (int t = 0; t <= n_tiles; ++t) {
        float s_new[4] = {0, 0, 0, 0}, tk_new[4] = {0, 0, 0, 0};
        int b_new[2] = {0, 0}, nrow_new = 0, kb_new = 0;
        float y_new[TR > 0 ? 8 : 1] = {};
        (void)y_new;
        if (t < n_tiles) {
            const int base = lo + t * tstep;
            const int nrow = min(BNK, hi - base);
            nrow_new = nrow;
            uint8_t* sKa = smem + L::OFF_RING + (t % RING) * L::SLOT;
            const uint16_t* sKs = reinterpret_cast<const uint16_t*>(sKa + L::KA);
            if (!mbar_wait(bars[t % RING], (t / RING) & 1, p.status)) *sFail = 1;
            // ---- coarse logit: 16 keys x 8 rows, both Q planes ----
            int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
            int cy1[4] = {0, 0, 0, 0}, cy2[4] = {0, 0, 0, 0};
            (void)cy1; (void)cy2;
            const int arow = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t a[4];
                const int u = (2 * ks + (lane >> 4)) ^ swz<D>(arow);
                ldmatrix_x4(a, smem_u32(sKa + arow * D + u * 16));
                mma_s8(c1, a, qfa[ks][0], qfa[ks][1]);
                mma_s8(c2, a, qfb[ks][0], qfb[ks][1]);
                if constexpr (TR > 0) {
                    mma_s8(cy1, a, ufa[ks][0], ufa[ks][1]);
                    mma_s8(cy2, a, ufb[ks][0], ufb[ks][1]);
                }
            }
            int pk = TRUNC ? 0 : (1 | (1 << 3));
            float dg[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int ky = 16 * warp + gid + 8 * (i >> 1);
                const float ekf = bf16_bits_to_float(sKs[ky]) * (1.0f / 256.0f);
                const float tk = eqr[i & 1] * ekf;
                tk_new[i] = tk;
                if constexpr (TR > 0) {
                    // key (i >> 1)'s projection on ranks 2 tq + (i & 1) and 8 + that: the exact
                    // integer, rounded once by the key's scale; rows past the tile hold nothing
                    y_new[i] = ky < nrow ? static_cast<float>(cy1[i]) * ekf : 0.f;
                    y_new[4 + i] = ky < nrow ? static_cast<float>(cy2[i]) * ekf : 0.f;
                }
                float s1 = -INFINITY;
                if (rowok[i & 1] && ky < nrow && sees(i & 1, base + ky)) {
                    s1 = fmaf(static_cast<float>(c1[i] * 256 + c2[i]), tk, -zr[i & 1]);
                    // (a sound cut adds what plane B of K could still add to this row's logit)
                    const float s1c = (EX && p.sound) ? fmaf(soundr[i & 1], ekf, s1) : s1;
                    if (TRUNC && s1c >= cutr[i & 1]) {
                        pk |= 1 << (3 * (i >> 1));
                        kb_new |= 1 << i;
                    }
                    dg[i >> 1] = fmaxf(dg[i >> 1], s1);
                }
                s_new[i] = s1;
            }
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                if (dg[hf] >= -rk) pk |= 2 << (3 * hf);
                if (V8 && dg[hf] >= -rv) pk |= 4 << (3 * hf);
            }
            pk |= __shfl_xor_sync(0xffffffffu, pk, 1);
            pk |= __shfl_xor_sync(0xffffffffu, pk, 2);
            int b0 = pk & 7, b1 = (pk >> 3) & 7;
            // a key no row keeps is neither gathered nor refined
            b0 = (b0 & 1) ? b0 : 0;
            b1 = (b1 & 1) ? b1 : 0;
            if (16 * warp + gid >= nrow) b0 = 0;
            if (16 * warp + gid + 8 >= nrow) b1 = 0;
            b_new[0] = b0;
            b_new[1] = b1;
            int* sLive = reinterpret_cast<int*>(smem + L::OFF_LIVE) + (t & 1) * BNK;
            if (tq == 0) {
                sLive[16 * warp + gid] = b0;
                sLive[16 * warp + gid + 8] = b1;
            }
            {   // counts are data, not schedule: live keys and refined keys
                const unsigned m0 = __ballot_sync(0xffffffffu, tq == 0 && (b0 & 1));
                const unsigned m1 = __ballot_sync(0xffffffffu, tq == 0 && (b1 & 1));
                const unsigned r0 = __ballot_sync(0xffffffffu, tq == 0 && (b0 & 2));
                const unsigned r1 = __ballot_sync(0xffffffffu, tq == 0 && (b1 & 2));
                nlive += __popc(m0) + __popc(m1);
                nref += __popc(r0) + __popc(r1);
            }
            __syncthreads();
            // a wait that ran out ends the CTA for every thread alike
            if (*sFail) { failed = true; }
            if (failed) break;
            // every warp has read this ring slot's predecessor: refill it
            if (tid == 0 && t + 2 < n_tiles) issue_tile(t + 2);
            // ---- gathers for tile t: two threads per key row ----
            {
                uint8_t* g = smem + L::OFF_G + (t & 1) * L::GBUF;
                const int r = tid >> 1, half = tid & 1;
                const int bits = sLive[r];
                const int pos = base + (r < nrow ? r : 0);
                const int64_t prow = pool_row(pos);
                // K plane B: stored swizzled by slot, copied unit for unit
#pragma unroll
                for (int j = 0; j < NU / 2; ++j) {
                    const int u = half * (NU / 2) + j;
                    cp_async16(smem_u32(g + r * D + u * 16), p.kb + prow * D + u * 16, (bits & 2) ? 16 : 0);
                }
                // V rows: unit u lands at u ^ (r & 7)
                constexpr int VU = L::VROW / 16;
#pragma unroll
                for (int j = 0; j < VU / 2; ++j) {
                    const int u = half * (VU / 2) + j;
                    const int du = vswz<VU>(u, r);
                    cp_async16(smem_u32(g + L::GKB + r * L::VROW + du * 16), p.va + prow * L::VROW + u * 16,
                               (bits & 1) ? 16 : 0);
                }
                if (V8) {
#pragma unroll
                    for (int j = 0; j < NU / 2; ++j) {
                        const int u = half * (NU / 2) + j;
                        const int du = vswz<NU>(u, r);
                        cp_async16(smem_u32(g + L::GKB + L::GVA + r * D + du * 16), p.vb + prow * D + u * 16,
                                   (bits & 4) ? 16 : 0);
                    }
                }
                if constexpr (TR >= 0) {
                    // the tile's block row: a tile is one 64-key block of a page
                    if (tid < 2 * D / 16) {
                        const int64_t blk = pool_row(base) / BNK;
                        cp_async16(smem_u32(g + L::OFF_TL + tid * 16),
                                   reinterpret_cast<const uint8_t*>(p.tail_rows) + blk * (2 * D) + tid * 16, 16);
                    }
                }
            }
        }
        cp_async_commit();
        if (t >= 1) {
            // ---- tile t-1: refine, weights, value product ----
            cp_async_wait<1>();
            __syncthreads();
            uint8_t* g = smem + L::OFF_G + ((t - 1) & 1) * L::GBUF;
            const uint8_t* sKb = g;
            const uint8_t* sVa = g + L::GKB;
            const uint8_t* sVb = g + L::GKB + L::GVA;
            const unsigned any_ref = __ballot_sync(0xffffffffu, ((b_old[0] | b_old[1]) & 2) != 0);
            const unsigned any_live = __ballot_sync(0xffffffffu, ((b_old[0] | b_old[1]) & 1) != 0);
            const unsigned any_rv = __ballot_sync(0xffffffffu, ((b_old[0] | b_old[1]) & 4) != 0);
            int c3a[4] = {0, 0, 0, 0}, c3b[4] = {0, 0, 0, 0};
            if (any_ref) {
                const int arow = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    uint32_t a[4];
                    const int u = (2 * ks + (lane >> 4)) ^ swz<D>(arow);
                    ldmatrix_x4(a, smem_u32(sKb + arow * D + u * 16));
                    mma_s8(c3a, a, qfa[ks][0], qfa[ks][1]);
                    mma_s8(c3b, a, qfb[ks][0], qfb[ks][1]);
                }
            }
            float w[4], fd[4] = {0.f, 0.f, 0.f, 0.f};
            (void)fd;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int ky = 16 * warp + gid + 8 * (i >> 1);
                const bool valid = rowok[i & 1] && ky < nrow_old && sees(i & 1, base_old + ky);
                // under a row's own cut a gathered key enters only the rows that keep it
                const bool live = (b_old[i >> 1] & 1) != 0 && (!EX || !p.row_cut || ((kb_old >> i) & 1) != 0);
                float s = s_old[i];
                if (b_old[i >> 1] & 2)
                    s = s + (static_cast<float>(c3a[i]) + static_cast<float>(c3b[i]) * (1.0f / 256.0f)) * tk_old[i];
                const float e = valid ? ex2_approx(s) : 0.f;
                if (TRUNC) {
                    // the gather is the group's, so a live key enters every row at
                    // its true weight; a cut key's weight joins the dropped mass
                    w[i] = live ? e : 0.f;
                    rM[i & 1] += live ? 0.f : e;
                    fd[i] = live ? 0.f : e;
                } else {
                    w[i] = e;
                }
            }
            if (any_live) {
                uint32_t a[4];
#pragma unroll
                for (int hk = 0; hk < 2; ++hk) {
                    float w0 = w[2 * hk], w1 = w[2 * hk + 1];
                    if (V8) {
                        w0 *= E4W;
                        w1 *= E4W;
                    }
                    const uint32_t ph = pack_bf16x2(w0, w1);
                    const float f0 = __uint_as_float(ph << 16), f1 = __uint_as_float(ph & 0xFFFF0000u);
                    uint32_t pl = 0;
                    if (W2) {
                        pl = pack_bf16x2(w0 - f0, w1 - f1);
                        rN[0] += w[2 * hk];
                        rN[1] += w[2 * hk + 1];
                    } else {
                        rN[0] += V8 ? f0 * (1.0f / E4W) : f0;
                        rN[1] += V8 ? f1 * (1.0f / E4W) : f1;
                    }
                    // rows of A: 0-7 the weights, 8-15 their rounding errors
                    a[2 * hk] = movmatrix_t(ph);
                    a[2 * hk + 1] = movmatrix_t(pl);
                }
                const int kb16 = 16 * warp;
                if (V8) {
                    const int wo = 4 * (gid & 3);
#pragma unroll
                    for (int m = 0; m < D / 32; ++m) {
                        const int u = 2 * m + (gid >> 2);
                        uint32_t wa[4], wb[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int r = kb16 + 2 * tq + (kk & 1) + 8 * (kk >> 1);
                            const int off = r * D + (vswz<NU>(u, r) << 4) + wo;
                            wa[kk] = *reinterpret_cast<const uint32_t*>(sVa + off);
                            if (any_rv) wb[kk] = *reinterpret_cast<const uint32_t*>(sVb + off);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t b0 = e4m3_pair_bf16(wa[0], wa[1], i);
                            uint32_t b1 = e4m3_pair_bf16(wa[2], wa[3], i);
                            if (any_rv) {
                                // V~ = Va + Vb / 8 (plane B rows not gathered are zero)
                                b0 = fma_bf16x2(e4m3_pair_bf16(wb[0], wb[1], i), 0x3e003e00u, b0);
                                b1 = fma_bf16x2(e4m3_pair_bf16(wb[2], wb[3], i), 0x3e003e00u, b1);
                            }
                            mma_16816<false>(acc[4 * m + i], a, b0, b1);
                        }
                    }
                } else {
                    const int krow = kb16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
                    for (int np = 0; np < NT / 2; ++np) {
                        uint32_t bv[4];
                        const int u = 2 * np + (lane >> 4);
                        ldmatrix_x4_trans(bv, smem_u32(sVa + krow * (2 * D) + (vswz<2 * NU>(u, krow) << 4)));
                        mma_16816<false>(acc[2 * np], a, bv[0], bv[1]);
                        mma_16816<false>(acc[2 * np + 1], a, bv[2], bv[3]);
                    }
                }
            } else if (!TRUNC) {
                // unreachable: a dense tile is all live
            }
            (void)sVb;
            if constexpr (TR >= 0) {
                // this warp's 16 keys' dropped mass per row, then row gid's to the lanes that hold
                // its accumulator columns
                float t0 = fd[0] + fd[2], t1 = fd[1] + fd[3];
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    t0 += __shfl_xor_sync(0xffffffffu, t0, o);
                    t1 += __shfl_xor_sync(0xffffffffu, t1, o);
                }
                if (__ballot_sync(0xffffffffu, t0 != 0.f || t1 != 0.f)) {
                    const float v0 = __shfl_sync(0xffffffffu, t0, gid >> 1);
                    const float v1 = __shfl_sync(0xffffffffu, t1, gid >> 1);
                    const float m = (gid & 1) ? v1 : v0;
                    const uint32_t* srow = reinterpret_cast<const uint32_t*>(g + L::OFF_TL);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint32_t wv = srow[4 * nt + tq];      // channels 8 nt + 2 tq, + 1
                        acc[nt][0] = fmaf(m, __uint_as_float(wv << 16), acc[nt][0]);
                        acc[nt][1] = fmaf(m, __uint_as_float(wv & 0xFFFF0000u), acc[nt][1]);
                    }
                    if constexpr (TR > 0) {
                        uint32_t ad[4];
                        ad[0] = movmatrix_t(pack_bf16x2(fd[0], fd[1]));
                        ad[1] = 0u;
                        ad[2] = movmatrix_t(pack_bf16x2(fd[2], fd[3]));
                        ad[3] = 0u;
#pragma unroll
                        for (int n = 0; n < 2; ++n) {
                            const uint32_t y0 = movmatrix_t(pack_bf16x2(y_old[4 * n], y_old[4 * n + 1]));
                            const uint32_t y1 = movmatrix_t(pack_bf16x2(y_old[4 * n + 2], y_old[4 * n + 3]));
                            mma_16816<false>(yd[n], ad, y0, y1);
                        }
                    }
                }
            }
        }
        if constexpr (TR > 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) y_old[i] = y_new[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s_old[i] = s_new[i];
            tk_old[i] = tk_new[i];
        }
        b_old[0] = b_new[0];
        b_old[1] = b_new[1];
        nrow_old = nrow_new;
        kb_old = kb_new;
        base_old = lo + t * tstep;
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- epilogue: close the rows over lanes and warps in a fixed order ----
    float* sO = reinterpret_cast<float*>(smem + L::OFF_G);        // [4 warps][8 rows][D]
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);     // [2][4 warps][8 rows]
    int* sCnt = reinterpret_cast<int*>(smem + L::OFF_RED + 512);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        float m = rM[j], n = rN[j];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            m += __shfl_xor_sync(0xffffffffu, m, o);
            n += __shfl_xor_sync(0xffffffffu, n, o);
        }
        if (gid == 0) {
            sRed[warp * 8 + 2 * tq + j] = m;
            sRed[32 + warp * 8 + 2 * tq + j] = n;
        }
    }
    if (lane == 0) {
        sCnt[warp] = nlive;
        sCnt[4 + warp] = nref;
    }
    // channel of accumulator register (n-tile nt, column 2 tq + e)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            int ch;
            if (V8) ch = 32 * (nt >> 2) + 4 * (2 * tq + e) + (nt & 3);
            else ch = 8 * nt + 2 * tq + e;
            sO[(warp * 8 + gid) * D + ch] = acc[nt][e] + acc[nt][2 + e];
        }
    float* sY = sO + 4 * 8 * D;          // [4 warps][8 rows][16 ranks], then [8 rows][16 ranks]
    if constexpr (TR > 0) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) sY[(warp * 8 + gid) * 16 + 8 * n + 2 * tq + e] = yd[n][e];
        __syncthreads();
        sY[512 + tid] = (sY[tid] + sY[128 + tid]) + (sY[256 + tid] + sY[384 + tid]);
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += DEC_THREADS) {
        const int g = i / D, c = i % D;
        float x = 0.f, m = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) {
            x += sO[(w2 * 8 + g) * D + c];
            m += sRed[w2 * 8 + g];
        }
        if (V8) x *= E4O;
        if (TR < 0 && TRUNC && p.vmean)
            x += m * p.vmean[((EX && p.vmean_rows) ? static_cast<int64_t>(bh) * G + g : static_cast<int64_t>(preq) * p.hkv + hkv) * D + c];
        if constexpr (TR > 0) {
            const float4* vr = reinterpret_cast<const float4*>(p.tail_vr + (static_cast<int64_t>(bh) * D + c) * TR);
#pragma unroll
            for (int q4 = 0; q4 < TR / 4; ++q4) {
                const float4 r4 = __ldg(vr + q4);
                const float* yr = sY + 512 + g * 16 + 4 * q4;
                x += yr[0] * r4.x + yr[1] * r4.y + yr[2] * r4.z + yr[3] * r4.w;
            }
        }
        p.o_part[(pix * G + g) * D + c] = x;
    }
    if (tid < G) {
        float m = 0.f, n = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) {
            m += sRed[w2 * 8 + tid];
            n += sRed[32 + w2 * 8 + tid];
        }
        p.den_part[pix * G + tid] = n + m;
    }
    if (tid == 0) {
        p.cnt_part[pix * 2] = sCnt[0] + sCnt[1] + sCnt[2] + sCnt[3];
        p.cnt_part[pix * 2 + 1] = sCnt[4] + sCnt[5] + sCnt[6] + sCnt[7];
    }
}

// ---- combine: out = (sum_sp O) * e_v / sum_sp den, in slot order ----------------
template <int OUT>  // 0 fp32, 1 bf16, 2 fp16
__global__ void decode_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ den_part,
                                      const int* __restrict__ cnt_part, const int* __restrict__ seq_lens,
                                      void* out, float* den, int* counts, int G, int D, int hkv,
                                      int split, int chunk_keys, float evs) {
    const int bh = blockIdx.x;
    int ns = split;
    if (chunk_keys > 0) {
        const int slen = seq_lens[bh / hkv];
        ns = min(split, (slen + chunk_keys - 1) / chunk_keys);
    }
    for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
        const int g = i / D;
        float x = 0.f, d = 0.f;
        for (int s = 0; s < ns; ++s) {
            const int64_t pix = static_cast<int64_t>(bh) * split + s;
            x += o_part[pix * G * D + i];
            d += den_part[pix * G + g];
        }
        const float y = x * evs / d;
        const int64_t oi = static_cast<int64_t>(bh) * G * D + i;
        if (OUT == 0) static_cast<float*>(out)[oi] = y;
        else if (OUT == 1) static_cast<__nv_bfloat16*>(out)[oi] = __float2bfloat16_rn(y);
        else static_cast<__half*>(out)[oi] = __float2half_rn(y);
        if (i % D == 0) den[static_cast<int64_t>(bh) * G + g] = d;
    }
    if (threadIdx.x < 2) {
        int c = 0;
        for (int s = 0; s < ns; ++s) c += cnt_part[(static_cast<int64_t>(bh) * split + s) * 2 + threadIdx.x];
        counts[bh * 2 + threadIdx.x] = c;
    }
}

// ---- the mass reference ---------------------------------------------------------
// Z_g = M + log2( sum over the sink and the newest 63 keys (exact) + sum over
// up to 128 stratum centres (samples) + (samples' sum - their 4 largest) *
// unscored / (samples - 4) ), all on coarse (plane A) logits.
constexpr int MASS_ROWS = 192, MASS_STRATA = 128, MASS_TRIM = 4, MASS_WINDOW = 63;

template <int D>
__global__ void __launch_bounds__(DEC_THREADS) mass_z_kernel(
    const int8_t* __restrict__ qa, const int8_t* __restrict__ qb, const float* __restrict__ eq,
    const int8_t* __restrict__ ka, const uint16_t* __restrict__ ek, const int* __restrict__ page_table,
    const int* __restrict__ seq_lens, int G, int hkv, int ppr, int PS, float* __restrict__ z,
    const int* __restrict__ req_map, int gsub, const int* __restrict__ tree, int q_len) {
    __shared__ __align__(16) int8_t sQ[2][8][D];
    __shared__ float sS[MASS_ROWS][8];
    __shared__ int sKey[MASS_ROWS];
    __shared__ int sClass[MASS_ROWS];   // 0 unused, 1 exact, 2 sample
    const int bh = blockIdx.x, bhk = bh / gsub, h = bhk % hkv, tid = threadIdx.x;
    const int breq = req_map ? req_map[bhk / hkv] : bhk / hkv;   // the row of page_table / seq_lens this group reads
    const int n = seq_lens[breq];
    for (int i = tid; i < G * D / 4; i += DEC_THREADS) {
        reinterpret_cast<uint32_t*>(&sQ[0][0][0])[i] = reinterpret_cast<const uint32_t*>(qa + static_cast<int64_t>(bh) * G * D)[i];
        reinterpret_cast<uint32_t*>(&sQ[1][0][0])[i] = reinterpret_cast<const uint32_t*>(qb + static_cast<int64_t>(bh) * G * D)[i];
    }
    const int lo = n - MASS_WINDOW;
    for (int r = tid; r < MASS_ROWS; r += DEC_THREADS) {
        int key = 0, cls = 0;
        if (r == 0) {
            cls = n >= 1 ? 1 : 0;
        } else if (r <= MASS_WINDOW) {
            key = n - r;
            cls = key >= 1 ? 1 : 0;
        } else {
            const int j = r - 1 - MASS_WINDOW;
            key = static_cast<int>((static_cast<int64_t>(2 * j + 1) * n) / (2 * MASS_STRATA));
            const int prev = j > 0 ? static_cast<int>((static_cast<int64_t>(2 * j - 1) * n) / (2 * MASS_STRATA)) : -1;
            cls = (key >= 1 && key < lo && key != prev) ? 2 : 0;
        }
        sKey[r] = key;
        sClass[r] = cls;
    }
    __syncthreads();
    constexpr int NU = D / 16;
    for (int r = tid; r < MASS_ROWS; r += DEC_THREADS) {
        if (sClass[r] == 0) continue;
        const int pos = sKey[r];
        const int64_t prow = (static_cast<int64_t>(__ldg(page_table + static_cast<int64_t>(breq) * ppr + pos / PS)) * hkv + h) * PS + pos % PS;
        const int off = pos % PS;
        int c1[8], c2[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) c1[g] = c2[g] = 0;
        for (int u = 0; u < NU; ++u) {
            const uint4 kw = *reinterpret_cast<const uint4*>(ka + prow * D + ((u ^ swz<D>(off)) << 4));
            const uint32_t kk[4] = {kw.x, kw.y, kw.z, kw.w};
            for (int g = 0; g < G; ++g) {
                const uint4 a = *reinterpret_cast<const uint4*>(&sQ[0][g][u * 16]);
                const uint4 b = *reinterpret_cast<const uint4*>(&sQ[1][g][u * 16]);
                c1[g] = __dp4a(static_cast<int>(kk[0]), static_cast<int>(a.x), c1[g]);
                c1[g] = __dp4a(static_cast<int>(kk[1]), static_cast<int>(a.y), c1[g]);
                c1[g] = __dp4a(static_cast<int>(kk[2]), static_cast<int>(a.z), c1[g]);
                c1[g] = __dp4a(static_cast<int>(kk[3]), static_cast<int>(a.w), c1[g]);
                c2[g] = __dp4a(static_cast<int>(kk[0]), static_cast<int>(b.x), c2[g]);
                c2[g] = __dp4a(static_cast<int>(kk[1]), static_cast<int>(b.y), c2[g]);
                c2[g] = __dp4a(static_cast<int>(kk[2]), static_cast<int>(b.z), c2[g]);
                c2[g] = __dp4a(static_cast<int>(kk[3]), static_cast<int>(b.w), c2[g]);
            }
        }
        const float ekf = bf16_bits_to_float(ek[prow]) * (1.0f / 256.0f);
        for (int g = 0; g < G; ++g) {
            float sg = static_cast<float>(c1[g] * 256 + c2[g]) * (eq[static_cast<int64_t>(bh) * G + g] * ekf);
            // a draft node the row does not see weighs nothing (the nodes are the newest keys: all in the exact window)
            if (q_len > 0 && pos >= n - q_len && !((static_cast<uint32_t>(tree[static_cast<int64_t>(bh) * G + g]) >> (pos - (n - q_len))) & 1u))
                sg = -INFINITY;
            sS[r][g] = sg;
        }
    }
    __syncthreads();
    // one warp per query row (rows g = warp, warp + 4)
    const int warp = tid >> 5, lane = tid & 31;
    for (int g = warp; g < G; g += DEC_THREADS / 32) {
        float mx = -INFINITY;
        for (int r = lane; r < MASS_ROWS; r += 32)
            if (sClass[r]) mx = fmaxf(mx, sS[r][g]);
        mx = warp_max(mx);
        float se = 0.f, ss = 0.f;
        int ne = 0, nsamp = 0;
        float d[MASS_ROWS / 32];
#pragma unroll
        for (int k = 0; k < MASS_ROWS / 32; ++k) {
            const int r = lane + 32 * k;
            d[k] = -1.f;
            if (sClass[r] == 1) {
                se += exp2f(sS[r][g] - mx);
                ne++;
            } else if (sClass[r] == 2) {
                d[k] = exp2f(sS[r][g] - mx);
                ss += d[k];
                nsamp++;
            }
        }
        se = warp_sum(se);
        ss = warp_sum(ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ne += __shfl_xor_sync(0xffffffffu, ne, o);
            nsamp += __shfl_xor_sync(0xffffffffu, nsamp, o);
        }
        float mass = se + ss;
        const int uns = n - ne - nsamp;
        if (nsamp > MASS_TRIM && uns > 0) {
            float top = 0.f;
            for (int it = 0; it < MASS_TRIM; ++it) {
                float best = -1.f;
                int bk = -1;
#pragma unroll
                for (int k = 0; k < MASS_ROWS / 32; ++k)
                    if (d[k] > best) { best = d[k]; bk = k; }
                float wbest = warp_max(best);
                // the lowest lane holding the maximum gives it up
                const unsigned who = __ballot_sync(0xffffffffu, best == wbest);
                if (lane == __ffs(who) - 1) {
#pragma unroll
                    for (int k = 0; k < MASS_ROWS / 32; ++k)
                        if (k == bk) d[k] = -1.f;
                }
                top += wbest;
            }
            mass += (ss - top) * static_cast<float>(uns) / static_cast<float>(nsamp - MASS_TRIM);
        }
        if (lane == 0) z[static_cast<int64_t>(bh) * G + g] = mx + log2f(mass);
    }
}

}  // namespace fold

using namespace fold;

namespace {

template <int D, bool V8, bool W2, bool TRUNC, int TR = -1, bool EX = false>
int launch_decode(const DecodeParams& p, cudaStream_t st) {
    using L = DecSmem<D, V8>;
    auto kern = decode_kernel<D, V8, W2, TRUNC, TR, EX>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES);
    kern<<<p.nbh * p.split, DEC_THREADS, L::BYTES, st>>>(p);
    return check_launch("fold_decode_run");
}

template <int D>
int launch_decode_tail(const DecodeParams& p, int w2, cudaStream_t st) {
    if (p.tail_u) return w2 ? launch_decode<D, false, true, true, 16>(p, st) : launch_decode<D, false, false, true, 16>(p, st);
    return w2 ? launch_decode<D, false, true, true, 0>(p, st) : launch_decode<D, false, false, true, 0>(p, st);
}

template <int D, bool V8>
int launch_decode_ex(const DecodeParams& p, int w2, cudaStream_t st) {
    if (p.truncate) return w2 ? launch_decode<D, V8, true, true, -1, true>(p, st) : launch_decode<D, V8, false, true, -1, true>(p, st);
    return w2 ? launch_decode<D, V8, true, false, -1, true>(p, st) : launch_decode<D, V8, false, false, -1, true>(p, st);
}

template <int D, bool V8>
int launch_decode_d(const DecodeParams& p, int w2, cudaStream_t st) {
    if (p.truncate) return w2 ? launch_decode<D, V8, true, true>(p, st) : launch_decode<D, V8, false, true>(p, st);
    return w2 ? launch_decode<D, V8, true, false>(p, st) : launch_decode<D, V8, false, false>(p, st);
}

}  // namespace

extern "C" int fold_mass_z(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                           const void* ek, const int32_t* page_table, const int32_t* seq_lens,
                           int n_groups, int group, int n_kv_heads, int head_dim,
                           int pages_per_request, int page_size, float* z, void* stream) {
    FOLD_CHECK_ARG(qa && qb && eq && ka && ek && page_table && seq_lens && z, "fold_mass_z: null pointer");
    FOLD_CHECK_ARG(group >= 1 && group <= 8, "a row group of %d rows: 1..8 are supported", group);
    FOLD_CHECK_ARG(head_dim == 64 || head_dim == 128, "head_dim %d: the decode takes 64 or 128", head_dim);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t* ekp = static_cast<const uint16_t*>(ek);
    if (head_dim == 128)
        mass_z_kernel<128><<<n_groups, DEC_THREADS, 0, st>>>(qa, qb, eq, ka, ekp, page_table, seq_lens, group, n_kv_heads, pages_per_request, page_size, z, nullptr, 1, nullptr, 0);
    else
        mass_z_kernel<64><<<n_groups, DEC_THREADS, 0, st>>>(qa, qb, eq, ka, ekp, page_table, seq_lens, group, n_kv_heads, pages_per_request, page_size, z, nullptr, 1, nullptr, 0);
    return check_launch("fold_mass_z");
}

// The mass reference for the layouts fold_decode_run_ex takes: a cascade's shared level
// (`req_map`), row groups wider than 8 rows (`group_split`), a draft's rows (`tree`, `draft_len`).
extern "C" int fold_mass_z_ex(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                              const void* ek, const int32_t* page_table, const int32_t* seq_lens,
                              int n_groups, int group, int n_kv_heads, int head_dim,
                              int pages_per_request, int page_size, float* z, const int32_t* req_map,
                              int group_split, const int32_t* tree, int draft_len, void* stream) {
    FOLD_CHECK_ARG(qa && qb && eq && ka && ek && page_table && seq_lens && z, "fold_mass_z_ex: null pointer");
    FOLD_CHECK_ARG(group >= 1 && group <= 8, "a row group of %d rows: 1..8 are supported", group);
    FOLD_CHECK_ARG(head_dim == 64 || head_dim == 128, "head_dim %d: the decode takes 64 or 128", head_dim);
    FOLD_CHECK_ARG(group_split >= 1 && n_groups % group_split == 0, "group_split %d does not divide %d row groups", group_split, n_groups);
    FOLD_CHECK_ARG(draft_len >= 0 && draft_len <= 32 && (draft_len == 0) == (tree == nullptr),
                   "a draft is its node count (1..32) and its rows' visibility words");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t* ekp = static_cast<const uint16_t*>(ek);
    if (head_dim == 128)
        mass_z_kernel<128><<<n_groups, DEC_THREADS, 0, st>>>(qa, qb, eq, ka, ekp, page_table, seq_lens, group, n_kv_heads, pages_per_request, page_size, z, req_map, group_split, tree, draft_len);
    else
        mass_z_kernel<64><<<n_groups, DEC_THREADS, 0, st>>>(qa, qb, eq, ka, ekp, page_table, seq_lens, group, n_kv_heads, pages_per_request, page_size, z, req_map, group_split, tree, draft_len);
    return check_launch("fold_mass_z_ex");
}

static int decode_run(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                      const int8_t* kb, const void* ek, const void* va, const void* vb,
                      const float* vmean, const float* z, const float* cut,
                      const int32_t* page_table, const int32_t* seq_lens,
                      const int32_t* order, int n_groups, int group, int n_kv_heads,
                      int head_dim, int pages_per_request, int page_size, int split,
                      int chunk_keys, int truncate, int weight_terms, float refine_k,
                      float refine_v, const float* refine_bands, float v_scale,
                      float* o_part, float* den_part, int32_t* cnt_part, void* out,
                      int out_dtype, float* den, int32_t* counts, int32_t* status,
                      int bh_limit, void* stream, const void* tail_rows = nullptr,
                      const int8_t* tail_u = nullptr, const float* tail_vr = nullptr, int tail_rank = -1,
                      const int32_t* req_map = nullptr, int group_split = 1, const int32_t* tree = nullptr,
                      int draft_len = 0, int slots_total = 0, int slot_off = 0, int row_cut = 0,
                      const float* sound = nullptr, int vmean_per_row = 0) {
    FOLD_CHECK_ARG(!vmean_per_row || (vmean && !req_map), "a direction per query row belongs to the unique level's vmean");
    if (slots_total <= 0) slots_total = split;
    FOLD_CHECK_ARG(group_split >= 1 && n_groups % group_split == 0, "group_split %d does not divide %d row groups", group_split, n_groups);
    FOLD_CHECK_ARG(draft_len >= 0 && draft_len <= 32 && (draft_len == 0) == (tree == nullptr),
                   "a draft is its node count (1..32) and its rows' visibility words");
    FOLD_CHECK_ARG(slot_off >= 0 && slot_off + split <= slots_total, "splits %d..%d of %d partial slots", slot_off, slot_off + split, slots_total);
    FOLD_CHECK_ARG(slots_total == split || (chunk_keys == 0 && !out),
                   "a level of several writes its own slots of uncombined partials, with interleaved splits (chunk_keys 0, out NULL)");
    FOLD_CHECK_ARG(tail_rank < 0 || (!req_map && !tree && group_split == 1 && !row_cut && !sound && !vmean_per_row),
                   "the tail runs on single-level steps with the group's cut");
    if (tail_rank >= 0) {
        FOLD_CHECK_ARG(tail_rank == 0 || tail_rank == 16, "tail rank %d: 0 (block rows alone) or 16", tail_rank);
        FOLD_CHECK_ARG(tail_rows && (tail_rank == 0 ? (!tail_u && !tail_vr) : (tail_u && tail_vr)),
                       "fold_decode_run_tail: rows always, u and vr at rank 16 only");
        FOLD_CHECK_ARG(truncate && !vb, "the tail re-enters truncated mass on a bf16 V: truncate=1, no plane B of V");
        FOLD_CHECK_ARG(!vmean, "a tail replaces V's mean: pass vmean = NULL");
        FOLD_CHECK_ARG(page_size % 64 == 0, "page_size %d: the tail keeps one row per 64 keys of a page", page_size);
    }
    FOLD_CHECK_ARG(qa && qb && eq && ka && kb && ek && va && z && cut && page_table && seq_lens &&
                       o_part && den_part && cnt_part && status && (!out || (den && counts)),
                   "fold_decode_run: null pointer");
    FOLD_CHECK_ARG(group >= 1 && group <= 8, "a row group of %d rows: 1..8 are supported", group);
    FOLD_CHECK_ARG(head_dim == 64 || head_dim == 128, "head_dim %d: the decode takes 64 or 128", head_dim);
    FOLD_CHECK_ARG(page_size >= 16 && page_size % 16 == 0 && (page_size % 64 == 0 || 64 % page_size == 0),
                   "page_size %d: a multiple of 64, or 16 or 32", page_size);
    FOLD_CHECK_ARG(split >= 1, "split %d", split);
    FOLD_CHECK_ARG(chunk_keys >= 0 && chunk_keys % 64 == 0, "chunk %d is not a multiple of 64", chunk_keys);
    FOLD_CHECK_ARG(weight_terms == 1 || weight_terms == 2, "weight_terms %d", weight_terms);
    FOLD_CHECK_ARG(out_dtype >= 0 && out_dtype <= 2, "out_dtype %d", out_dtype);
    DecodeParams p;
    p.qa = qa; p.qb = qb; p.eq = eq; p.ka = ka; p.kb = kb;
    p.ek = static_cast<const uint16_t*>(ek);
    p.va = static_cast<const uint8_t*>(va); p.vb = static_cast<const uint8_t*>(vb);
    p.vmean = vmean; p.z = z; p.cut = cut;
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
    p.bh_limit = bh_limit;
    p.tail_rows = static_cast<const uint16_t*>(tail_rows); p.tail_u = tail_u; p.tail_vr = tail_vr;
    p.req_map = req_map; p.tree = tree; p.q_len = draft_len; p.gsub = group_split;
    p.slots_total = slots_total; p.slot_off = slot_off; p.row_cut = row_cut;
    p.sound = sound; p.vmean_rows = vmean_per_row;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool v8 = vb != nullptr;
    int rc;
    const bool ex = req_map || tree || group_split > 1 || slots_total != split || slot_off || row_cut || sound || vmean_per_row;
    if (tail_rank >= 0) rc = head_dim == 128 ? launch_decode_tail<128>(p, weight_terms == 2, st) : launch_decode_tail<64>(p, weight_terms == 2, st);
    else if (ex && head_dim == 128) rc = v8 ? launch_decode_ex<128, true>(p, weight_terms == 2, st) : launch_decode_ex<128, false>(p, weight_terms == 2, st);
    else if (ex) rc = v8 ? launch_decode_ex<64, true>(p, weight_terms == 2, st) : launch_decode_ex<64, false>(p, weight_terms == 2, st);
    else if (head_dim == 128) rc = v8 ? launch_decode_d<128, true>(p, weight_terms == 2, st) : launch_decode_d<128, false>(p, weight_terms == 2, st);
    else rc = v8 ? launch_decode_d<64, true>(p, weight_terms == 2, st) : launch_decode_d<64, false>(p, weight_terms == 2, st);
    if (rc) return rc;
    if (!out) return FOLD_OK;   // partials only: the caller combines
    const int threads = 256;
#define FOLD_COMBINE(OUT) decode_combine_kernel<OUT><<<n_groups, threads, 0, st>>>(o_part, den_part, cnt_part, seq_lens, out, den, counts, group, head_dim, n_kv_heads * group_split, split, chunk_keys, v_scale)
    if (out_dtype == 0) FOLD_COMBINE(0);
    else if (out_dtype == 1) FOLD_COMBINE(1);
    else FOLD_COMBINE(2);
#undef FOLD_COMBINE
    return check_launch("fold_decode_combine");
}

extern "C" int fold_decode_run(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                               const int8_t* kb, const void* ek, const void* va, const void* vb,
                               const float* vmean, const float* z, const float* cut,
                               const int32_t* page_table, const int32_t* seq_lens,
                               const int32_t* order, int n_groups, int group, int n_kv_heads,
                               int head_dim, int pages_per_request, int page_size, int split,
                               int chunk_keys, int truncate, int weight_terms, float refine_k,
                               float refine_v, const float* refine_bands, float v_scale,
                               float* o_part, float* den_part, int32_t* cnt_part, void* out,
                               int out_dtype, float* den, int32_t* counts, int32_t* status,
                               void* stream) {
    return decode_run(qa, qb, eq, ka, kb, ek, va, vb, vmean, z, cut, page_table, seq_lens, order, n_groups,
                      group, n_kv_heads, head_dim, pages_per_request, page_size, split, chunk_keys, truncate,
                      weight_terms, refine_k, refine_v, refine_bands, v_scale, o_part, den_part, cnt_part, out,
                      out_dtype, den, counts, status, /*bh_limit=*/0, stream);
}

// The same decode with a tail: dropped mass re-enters at each 64-key block's row
// (`tail_rows`, bf16, one per 64 pool rows) and, at rank 16, through each row group's
// projection `tail_u` (n_groups, 16, D) int8 and map back `tail_vr` (n_groups, D, 16).
extern "C" int fold_decode_run_tail(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                                    const int8_t* kb, const void* ek, const void* va,
                                    const void* tail_rows, const int8_t* tail_u, const float* tail_vr,
                                    int tail_rank, const float* z, const float* cut,
                                    const int32_t* page_table, const int32_t* seq_lens,
                                    const int32_t* order, int n_groups, int group, int n_kv_heads,
                                    int head_dim, int pages_per_request, int page_size, int split,
                                    int chunk_keys, int weight_terms, float refine_k,
                                    float* o_part, float* den_part, int32_t* cnt_part, void* out,
                                    int out_dtype, float* den, int32_t* counts, int32_t* status,
                                    void* stream) {
    FOLD_CHECK_ARG(tail_rank >= 0, "fold_decode_run_tail: tail rank %d", tail_rank);
    return decode_run(qa, qb, eq, ka, kb, ek, va, nullptr, nullptr, z, cut, page_table, seq_lens, order, n_groups,
                      group, n_kv_heads, head_dim, pages_per_request, page_size, split, chunk_keys, /*truncate=*/1,
                      weight_terms, refine_k, 0.f, nullptr, 1.0f, o_part, den_part, cnt_part, out,
                      out_dtype, den, counts, status, /*bh_limit=*/0, stream, tail_rows, tail_u, tail_vr, tail_rank);
}

// fold_decode_run for the layouts beyond the single-level step: a cascade's shared level reads
// another cache through `req_map` and writes its own slots of a partial buffer several levels
// share; a row group wider than 8 rows runs as `group_split` groups of 8 on one KV head; a
// draft's rows see the cache's last `draft_len` keys through `tree`; `row_cut` keeps each row's
// own cut. Warp-level kernel only.
extern "C" int fold_decode_run_ex(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                                  const int8_t* kb, const void* ek, const void* va, const void* vb,
                                  const float* vmean, const float* z, const float* cut,
                                  const int32_t* page_table, const int32_t* seq_lens,
                                  const int32_t* order, int n_groups, int group, int n_kv_heads,
                                  int head_dim, int pages_per_request, int page_size, int split,
                                  int chunk_keys, int truncate, int weight_terms, float refine_k,
                                  float refine_v, const float* refine_bands, float v_scale,
                                  float* o_part, float* den_part, int32_t* cnt_part, void* out,
                                  int out_dtype, float* den, int32_t* counts, int32_t* status,
                                  const int32_t* req_map, int group_split, const int32_t* tree,
                                  int draft_len, int slots_total, int slot_off, int row_cut,
                                  const float* sound, int vmean_per_row, void* stream) {
    return decode_run(qa, qb, eq, ka, kb, ek, va, vb, vmean, z, cut, page_table, seq_lens, order, n_groups,
                      group, n_kv_heads, head_dim, pages_per_request, page_size, split, chunk_keys, truncate,
                      weight_terms, refine_k, refine_v, refine_bands, v_scale, o_part, den_part, cnt_part, out,
                      out_dtype, den, counts, status, /*bh_limit=*/0, stream, nullptr, nullptr, nullptr, -1,
                      req_map, group_split, tree, draft_len, slots_total, slot_off, row_cut, sound, vmean_per_row);
}

// The combine alone, for decode kernels that fill the same partial buffers.
extern "C" int fold_decode_combine(const float* o_part, const float* den_part, const int32_t* cnt_part,
                                   const int32_t* seq_lens, void* out, int out_dtype, float* den, int32_t* counts,
                                   int n_groups, int group, int head_dim, int n_kv_heads, int split, int chunk_keys,
                                   float v_scale, void* stream) {
    FOLD_CHECK_ARG(o_part && den_part && cnt_part && seq_lens && out && den && counts, "fold_decode_combine: null pointer");
    FOLD_CHECK_ARG(out_dtype >= 0 && out_dtype <= 2, "out_dtype %d", out_dtype);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0)
        decode_combine_kernel<0><<<n_groups, 256, 0, st>>>(o_part, den_part, cnt_part, seq_lens, out, den, counts, group, head_dim, n_kv_heads, split, chunk_keys, v_scale);
    else if (out_dtype == 1)
        decode_combine_kernel<1><<<n_groups, 256, 0, st>>>(o_part, den_part, cnt_part, seq_lens, out, den, counts, group, head_dim, n_kv_heads, split, chunk_keys, v_scale);
    else
        decode_combine_kernel<2><<<n_groups, 256, 0, st>>>(o_part, den_part, cnt_part, seq_lens, out, den, counts, group, head_dim, n_kv_heads, split, chunk_keys, v_scale);
    return check_launch("fold_decode_combine");
}

// ---- a decode entry point that allocates nothing ------------------------------------
// Some hosts may not allocate device memory from the code that runs a decode
// step: an inference server that hands a plugin a fixed amount of memory up front
// and forbids cudaMalloc (or any allocating library call) inside its execution
// callback, or a process whose device allocator belongs to another runtime.
// For them the split partials live in this fixed array instead of in buffers
// the caller provides. The array is part of the library image: every GPU that
// loads the library holds FOLD_DECODE_STATIC_SCRATCH_BYTES of it until the
// process exits.
static __device__ __align__(256) unsigned char g_decode_scratch[FOLD_DECODE_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; the device address comes from
// the runtime, once per device, with that device current.
int static_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("fold_decode_run_static: cudaGetDevice: %s", cudaGetErrorString(e));
        return FOLD_ERR_LAUNCH;
    }
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
        if (e != cudaSuccess || !ptr) {
            set_error("fold_decode_run_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return FOLD_ERR_LAUNCH;
        }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return FOLD_OK;
}
}  // namespace

extern "C" size_t fold_decode_static_scratch_needed(int n_groups, int group, int head_dim, int split) {
    const size_t n = static_cast<size_t>(n_groups) * split;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    return up(n * group * head_dim * sizeof(float)) + up(n * group * sizeof(float)) + up(n * 2 * sizeof(int));
}

extern "C" int fold_decode_run_static(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                                      const int8_t* kb, const void* ek, const void* va, const void* vb,
                                      const float* vmean, const float* z, const float* cut,
                                      const int32_t* page_table, const int32_t* seq_lens,
                                      const int32_t* order, int n_groups, int group, int n_kv_heads,
                                      int head_dim, int pages_per_request, int page_size, int split,
                                      int chunk_keys, int truncate, int weight_terms, float refine_k,
                                      float refine_v, const float* refine_bands, float v_scale,
                                      void* out, int out_dtype, float* den, int32_t* counts,
                                      int32_t* status, void* stream) {
    FOLD_CHECK_ARG(n_groups >= 1 && group >= 1 && split >= 1 && head_dim >= 1, "fold_decode_run_static: empty call");
    // the partials stay inside the library, where the caller cannot combine them later
    FOLD_CHECK_ARG(out && den && counts, "fold_decode_run_static: out, den and counts must be given (the partials "
                                         "live in the library's own array: there is no uncombined form of this call)");
    const size_t need = fold_decode_static_scratch_needed(n_groups, group, head_dim, split);
    FOLD_CHECK_ARG(need <= FOLD_DECODE_STATIC_SCRATCH_BYTES,
                   "fold_decode_run_static: %d row groups x %d splits need %zu bytes of partials, the built-in "
                   "scratch holds %zu; lower the split or use fold_decode_run with caller-provided buffers",
                   n_groups, split, need, static_cast<size_t>(FOLD_DECODE_STATIC_SCRATCH_BYTES));
    void* base = nullptr;
    const int rc = static_scratch(&base);
    if (rc) return rc;
    const size_t n = static_cast<size_t>(n_groups) * split;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    unsigned char* p = static_cast<unsigned char*>(base);
    float* o_part = reinterpret_cast<float*>(p);
    float* den_part = reinterpret_cast<float*>(p + up(n * group * head_dim * sizeof(float)));
    int32_t* cnt_part = reinterpret_cast<int32_t*>(p + up(n * group * head_dim * sizeof(float)) + up(n * group * sizeof(float)));
    // Nothing in the partials has to start at zero: every split a request
    // reaches writes its whole slot before the combine, launched behind it on
    // the same stream, reads exactly those slots.
    // The array is laid out for n_groups row groups, so `order` (if given) must map the n_groups
    // slots onto row groups 0 .. n_groups-1. The host cannot read a device-side order without a
    // synchronisation; the kernel checks each entry instead, and a CTA handed a row group outside
    // the array raises `status` to FOLD_ERR_ARGUMENT and returns without touching memory.
    return decode_run(qa, qb, eq, ka, kb, ek, va, vb, vmean, z, cut, page_table, seq_lens, order,
                      n_groups, group, n_kv_heads, head_dim, pages_per_request, page_size, split,
                      chunk_keys, truncate, weight_terms, refine_k, refine_v, refine_bands, v_scale,
                      o_part, den_part, cnt_part, out, out_dtype, den, counts, status, /*bh_limit=*/n_groups, stream);
}
