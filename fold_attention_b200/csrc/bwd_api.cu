// C entry points of the deterministic attention backward: preprocess, main
// loop and postprocess enqueued back to back on the caller's stream.
// Stands in for src/fold_attention/backward/launch.py:75-462 (prepare_backward
// and the closure it returns).
#include "bwd_common.cuh"

using namespace fold;

namespace {

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// How a call's work is cut: `subgroup` query heads and `record` query blocks per work item
// (0, 0: the whole group and every block, which keeps a key block's dK and dV inside one CTA).
struct PlanArgs {
    int subgroup, record, fold, dv_bits;
};

bool resolve_plan(int n_heads, int n_kv_heads, int max_seqlen, int subgroup, int record, PlanArgs* out) {
    const int G = n_heads / n_kv_heads;
    if (subgroup <= 0) subgroup = G;
    if (subgroup > G || G % subgroup || record < 0) return false;
    out->subgroup = subgroup;
    out->record = record;
    out->fold = (subgroup < G || record > 0) ? 1 : 0;
    // dV's bound carries only the column mass G * S: a 30-bit grid holds it up to 16384
    // (src/fold_attention/backward/launch.py:179-182)
    out->dv_bits = static_cast<int64_t>(G) * max_seqlen <= 16384 ? 32 : 64;
    return true;
}

struct WsLayout {
    size_t dq_acc, dpsum, lse2, stats, dk_acc, dv_acc, work, total;
    int64_t rows_p, n_items;
};

WsLayout ws_layout(int B, int H, int HKV, int S, int total, int D, bool varlen, const PlanArgs& plan) {
    WsLayout w;
    w.rows_p = padded_rows(B, S, total, varlen);
    w.n_items = D == 128 ? bwd_sm100_work_items(B, H, HKV, S, plan.subgroup, plan.record) : 0;
    size_t off = 0;
    w.dq_acc = off; off = align256(off + sizeof(int) * static_cast<size_t>(H) * w.rows_p * D);
    w.dpsum = off;  off = align256(off + sizeof(float) * static_cast<size_t>(H) * w.rows_p);
    w.lse2 = off;   off = align256(off + sizeof(float) * static_cast<size_t>(H) * w.rows_p);
    // the maxima, then the status word, then the work list's two counters
    w.stats = off;  off = align256(off + sizeof(int) * (N_STATS * static_cast<size_t>(B) * HKV + 3));
    w.dk_acc = off; off = align256(off + (plan.fold ? 8 * static_cast<size_t>(HKV) * w.rows_p * D : 0));
    w.dv_acc = off; off = align256(off + (plan.fold ? (plan.dv_bits / 8) * static_cast<size_t>(HKV) * w.rows_p * D : 0));
    w.work = off;   off = align256(off + 32 * static_cast<size_t>(w.n_items));
    w.total = off;
    return w;
}

}  // namespace

extern "C" size_t fold_bwd_workspace_bytes(int batch, int n_heads, int n_kv_heads, int max_seqlen,
                                           int total, int head_dim, int varlen, int subgroup, int record) {
    PlanArgs plan;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads || !resolve_plan(n_heads, n_kv_heads, max_seqlen, subgroup, record, &plan)) return 0;
    return ws_layout(batch, n_heads, n_kv_heads, max_seqlen, total, head_dim, varlen != 0, plan).total;
}

static int bwd_run_phases(const void* q, const void* k, const void* v, const void* o,
                          const void* dout, const float* lse, void* dq, void* dk, void* dv,
                          const int64_t* strides, const int32_t* cu_seqlens, int batch,
                          int n_heads, int n_kv_heads, int max_seqlen, int total, int head_dim,
                          int causal, int is_f16, float softmax_scale, void* workspace,
                          size_t workspace_bytes, int kernel, int subgroup, int record, int phases, void* stream) {
    FOLD_CHECK_ARG(q && k && v && o && dout && lse && dq && dk && dv && strides && workspace,
                   "fold_bwd_run: null pointer");
    FOLD_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                   "the query heads must be a multiple of the KV heads");
    FOLD_CHECK_ARG(batch > 0 && max_seqlen > 0, "fold_bwd_run: empty call");
    if (head_dim != 64 && head_dim != 96 && head_dim != 128) {
        set_error("head_dim %d: 64, 96 and 128 are supported", head_dim);
        return FOLD_ERR_UNSUPPORTED;
    }
    const bool varlen = cu_seqlens != nullptr;
    PlanArgs plan;
    FOLD_CHECK_ARG(resolve_plan(n_heads, n_kv_heads, max_seqlen, subgroup, record, &plan),
                   "fold_bwd_run: a plan of %d heads and %d query blocks per work item for groups of %d heads", subgroup, record,
                   n_heads / n_kv_heads);
    const WsLayout w = ws_layout(batch, n_heads, n_kv_heads, max_seqlen, total, head_dim, varlen, plan);
    FOLD_CHECK_ARG(workspace_bytes >= w.total, "fold_bwd_run: workspace of %zu bytes, %zu needed",
                   workspace_bytes, w.total);
    FOLD_CHECK_ARG(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "fold_bwd_run: workspace must be 256-byte aligned");
    BwdParams p;
    const void* ptrs[8] = {q, k, v, o, dout, dq, dk, dv};
    TensorView* views[8] = {&p.q, &p.k, &p.v, &p.o, &p.dout, &p.dq, &p.dk, &p.dv};
    for (int i = 0; i < 8; ++i) {
        views[i]->ptr = const_cast<void*>(ptrs[i]);
        views[i]->sb = strides[3 * i];
        views[i]->sr = strides[3 * i + 1];
        views[i]->sh = strides[3 * i + 2];
        FOLD_CHECK_ARG(views[i]->sr % 8 == 0 && views[i]->sh % 8 == 0 && views[i]->sb % 8 == 0 &&
                           reinterpret_cast<uintptr_t>(ptrs[i]) % 16 == 0,
                       "fold_bwd_run: rows of tensor %d must be 16-byte aligned", i);
    }
    p.lse = lse;
    p.cu = cu_seqlens;
    if (varlen) {
        p.lse_sb = 0;
        p.lse_sh = total;
    } else {
        p.lse_sb = static_cast<int64_t>(n_heads) * max_seqlen;
        p.lse_sh = max_seqlen;
    }
    p.B = batch; p.H = n_heads; p.HKV = n_kv_heads; p.G = n_heads / n_kv_heads;
    p.S = max_seqlen; p.total = total; p.D = head_dim;
    p.causal = causal; p.f16 = is_f16; p.scale = softmax_scale;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.dq_acc = reinterpret_cast<int*>(ws + w.dq_acc);
    p.dpsum = reinterpret_cast<float*>(ws + w.dpsum);
    p.lse2 = reinterpret_cast<float*>(ws + w.lse2);
    p.stats = reinterpret_cast<int*>(ws + w.stats);
    p.status = p.stats + N_STATS * static_cast<size_t>(batch) * n_kv_heads;
    p.sched = p.status + 1;
    p.subgroup = plan.subgroup; p.record = plan.record; p.fold = plan.fold; p.dv_bits = plan.dv_bits;
    p.dk_acc = reinterpret_cast<long long*>(ws + w.dk_acc);
    p.dv_acc = ws + w.dv_acc;
    p.work = reinterpret_cast<int*>(ws + w.work);
    p.n_items = static_cast<int>(w.n_items);
    p.rows_p = w.rows_p;
    p.S_r = (max_seqlen + ROW_PAD - 1) / ROW_PAD * ROW_PAD;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool sm100 = false;
    if (kernel == FOLD_BWD_KERNEL_SM100) {
        if (!bwd_sm100_supported(p)) {
            set_error("the tcgen05 backward takes head_dim 128");
            return FOLD_ERR_UNSUPPORTED;
        }
        sm100 = true;
    } else if (kernel == FOLD_BWD_KERNEL_AUTO) {
        sm100 = bwd_sm100_supported(p);
    } else {
        FOLD_CHECK_ARG(kernel == FOLD_BWD_KERNEL_MMA, "fold_bwd_run: unknown kernel %d", kernel);
    }
    if (!sm100 && plan.fold) {
        set_error("the mma.sync main loop keeps a key block's dK and dV in one CTA: it takes whole groups and whole query ranges "
                  "(subgroup 0, record 0)");
        return FOLD_ERR_UNSUPPORTED;
    }
    p.dq_bias = (sm100 && bwd_sm100_biased()) ? 1 : 0;
    int rc = FOLD_OK;
    if (phases & FOLD_BWD_PHASE_PRE) rc = launch_bwd_preprocess(p, st);
    if (rc) return rc;
    if (sm100 && (phases & (FOLD_BWD_PHASE_LIST | FOLD_BWD_PHASE_MAIN)))
        rc = launch_bwd_main_sm100(p, (phases & FOLD_BWD_PHASE_LIST) != 0, (phases & FOLD_BWD_PHASE_MAIN) != 0, st);
    else if (phases & FOLD_BWD_PHASE_MAIN)
        rc = launch_bwd_main_mma(p, st);
    if (rc) return rc;
    if (phases & FOLD_BWD_PHASE_POST)
        rc = launch_bwd_postprocess(p, DQ_LAYOUT_ROW_MAJOR, st);
    return rc;
}

extern "C" int fold_bwd_run(const void* q, const void* k, const void* v, const void* o,
                            const void* dout, const float* lse, void* dq, void* dk, void* dv,
                            const int64_t* strides, const int32_t* cu_seqlens, int batch,
                            int n_heads, int n_kv_heads, int max_seqlen, int total, int head_dim,
                            int causal, int is_f16, float softmax_scale, void* workspace,
                            size_t workspace_bytes, int kernel, int subgroup, int record, void* stream) {
    return bwd_run_phases(q, k, v, o, dout, lse, dq, dk, dv, strides, cu_seqlens, batch, n_heads,
                          n_kv_heads, max_seqlen, total, head_dim, causal, is_f16, softmax_scale,
                          workspace, workspace_bytes, kernel, subgroup, record,
                          FOLD_BWD_PHASE_PRE | FOLD_BWD_PHASE_LIST | FOLD_BWD_PHASE_MAIN | FOLD_BWD_PHASE_POST, stream);
}

extern "C" int fold_bwd_run_phases(const void* q, const void* k, const void* v, const void* o,
                                   const void* dout, const float* lse, void* dq, void* dk, void* dv,
                                   const int64_t* strides, const int32_t* cu_seqlens, int batch,
                                   int n_heads, int n_kv_heads, int max_seqlen, int total,
                                   int head_dim, int causal, int is_f16, float softmax_scale,
                                   void* workspace, size_t workspace_bytes, int kernel, int subgroup,
                                   int record, int phases, void* stream) {
    return bwd_run_phases(q, k, v, o, dout, lse, dq, dk, dv, strides, cu_seqlens, batch, n_heads,
                          n_kv_heads, max_seqlen, total, head_dim, causal, is_f16, softmax_scale,
                          workspace, workspace_bytes, kernel, subgroup, record, phases, stream);
}

// The workspace's views, for tests that inspect the accumulators:
// out[0..3] = byte offsets of dq_acc, dpsum, lse2, stats; out[4] = padded rows per head;
// out[5] = byte offset of the status word (non-zero after a call whose device-side wait ran out);
// out[6], out[7] = byte offsets of the dK and dV accumulators (used when the plan folds);
// out[8] = dV's accumulator width in bits; out[9] = byte offset of the work list, out[10] its items.
extern "C" int fold_bwd_workspace_layout(int batch, int n_heads, int n_kv_heads, int max_seqlen,
                                         int total, int head_dim, int varlen, int subgroup, int record,
                                         int64_t* out) {
    FOLD_CHECK_ARG(out, "fold_bwd_workspace_layout: null pointer");
    PlanArgs plan;
    FOLD_CHECK_ARG(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && resolve_plan(n_heads, n_kv_heads, max_seqlen, subgroup, record, &plan),
                   "fold_bwd_workspace_layout: bad head counts or plan");
    const WsLayout w = ws_layout(batch, n_heads, n_kv_heads, max_seqlen, total, head_dim, varlen != 0, plan);
    out[0] = w.dq_acc; out[1] = w.dpsum; out[2] = w.lse2; out[3] = w.stats; out[4] = w.rows_p;
    out[5] = w.stats + sizeof(int) * N_STATS * static_cast<size_t>(batch) * n_kv_heads;
    out[6] = w.dk_acc; out[7] = w.dv_acc; out[8] = plan.fold ? plan.dv_bits : 0; out[9] = w.work; out[10] = w.n_items;
    return FOLD_OK;
}
