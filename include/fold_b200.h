/* libfold_b200 -- C ABI of the B200 (sm_100a) FoldAttention hot paths.
 *
 * Plain pointers and sizes only: every pointer is a CUDA device pointer unless
 * its comment says "host". Every entry point enqueues on `stream` (a
 * cudaStream_t passed as void*), never synchronises the host unless stated,
 * returns 0 on success and a FOLD_ERR_* code otherwise; fold_last_error()
 * then holds a message for the calling host thread. Nothing here throws.
 *
 * Each declaration cites the reference interface it stands in for, by the
 * reference's path within its project.
 */
#ifndef FOLD_B200_H
#define FOLD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FOLD_B200_ABI_VERSION 2

#define FOLD_OK 0
#define FOLD_ERR_ARGUMENT 1
#define FOLD_ERR_LAUNCH 2
#define FOLD_ERR_TIMEOUT 3
#define FOLD_ERR_UNSUPPORTED 4

/* Message of the calling thread's last failed call ("" if none). */
const char* fold_last_error(void);
int fold_abi_version(void);

/* ---- Path B: cache writes ------------------------------------------------ */

/* Quantise packed prompts into the paged cache.
 * Replaces: src/fold_attention/decode/write.py:931-1009 (write_prompt) and its
 * kernels :733-891.
 *   k, v        (total, n_kv_heads, head_dim) bf16 (is_f16=0) or fp16 (1), packed
 *   chunk_meta  int32: first[batch+1] padded to a multiple of 4 entries, then
 *               n_chunks rows (request, first token, first position, count)
 *               covering each request in 256-token chunks from its start
 *   page_table  int32 (batch, pages_per_request)
 *   ka, kb      int8 (rows, head_dim) pool planes; va/vb the V pool: bf16 va and
 *               vb == NULL, or two e4m3 planes; ek bf16 (rows,) key scales
 *   vsum, vmean fp32 (batch*n_kv_heads, head_dim)
 *   scratch     fp32, n_chunks*n_kv_heads*(head_dim+1)+1 elements; its last
 *               element receives V's scale
 *   v_fixed     a fixed power-of-two V scale, or 0 to derive it from the
 *               prompts' largest |v| times v_headroom over 448 */
int fold_cache_write_prompt(const void* k, const void* v, int is_f16, const int32_t* chunk_meta,
                            int n_chunks, int batch, const int32_t* page_table,
                            int pages_per_request, int page_size, int n_kv_heads, int head_dim,
                            int8_t* ka, int8_t* kb, void* va, void* vb, void* ek, float* vsum,
                            float* vmean, float* scratch, float v_headroom, float v_fixed,
                            void* stream);

/* One decode step's writes: query planes (q != NULL) and/or one appended
 * token per request (k, v != NULL) at position lens_in[b]; lens_out[b] =
 * lens_in[b] + 1 (lens_out may alias lens_in).
 * Replaces: src/fold_attention/decode/write.py:380-440 (step_kernel),
 * :565-673 (prepare_step) and the append half of decode/front.py:255-471.
 *   q (batch*n_heads, head_dim); k, v (batch, n_kv_heads, head_dim)
 *   qa, qb int8 (batch*n_heads, head_dim); eq fp32 (batch*n_heads,) */
int fold_step_append(const void* q, const void* k, const void* v, int is_f16, int batch,
                     int n_heads, int n_kv_heads, int head_dim, const int32_t* page_table,
                     int pages_per_request, int page_size, const int32_t* lens_in,
                     int32_t* lens_out, int8_t* qa, int8_t* qb, float* eq, int8_t* ka, int8_t* kb,
                     void* va, void* vb, void* ek, float v_scale, float* vsum, float* vmean,
                     void* stream);

/* The decode tail's share of an append: the appended token's 64-key block gains
 * its V and its projection y = (plane A . u) ek / 256, and the block's row becomes
 * vsum / n - (ysum / n) vr^T in bf16; a block's first key restarts its sums.
 * Run it after fold_step_append on the same stream (plane A and the scale are
 * read back from the pool). The token sits at lens[b] - back: back = 1 when
 * `lens` are the lengths the step already moved, 0 when they are the positions.
 * Replaces: the tail half of src/fold_attention/decode/write.py:193-300
 * (append_row), which the reference runs inside its step kernel.
 *   v (batch, n_kv_heads, head_dim) 16-bit; tail_u int8 (n_groups, 16, head_dim);
 *   tail_vr fp32 (n_groups, head_dim, 16); tail_vsum fp32 (pool_rows/64, head_dim);
 *   tail_ysum fp32 (pool_rows/64, 16); tail_rows bf16 (pool_rows/64, head_dim);
 *   tail_rank 0 (u, vr, ysum NULL) or 16; page_size a multiple of 64 */
int fold_tail_append(const void* v, int is_f16, int batch, int n_kv_heads, int head_dim,
                     const int32_t* page_table, int pages_per_request, int page_size,
                     const int32_t* lens, int back, const int8_t* ka, const void* ek,
                     const int8_t* tail_u, const float* tail_vr, float* tail_vsum,
                     float* tail_ysum, void* tail_rows, int tail_rank, void* stream);

/* ---- Path B: decode ------------------------------------------------------- */

/* The mass reference: each query row's log-sum-exp estimate Z (base 2) from
 * the sink, the newest 63 keys and up to 128 stratum centres, on coarse
 * (plane A) logits. Replaces: src/fold_attention/decode/reference.py:120-535
 * (mass_estimate, mass_z) and the mass half of decode/front.py:255-471.
 *   qa, qb int8 (n_groups, group, head_dim); eq, z fp32 (n_groups, group) */
int fold_mass_z(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                const void* ek, const int32_t* page_table, const int32_t* seq_lens, int n_groups,
                int group, int n_kv_heads, int head_dim, int pages_per_request, int page_size,
                float* z, void* stream);

/* Split-KV decode over the paged cache and its additive combine.
 * Replaces: src/fold_attention/decode/launch.py:509-1252 (_prepare, single
 * level), decode/kernel.py:95-1562 and decode/combine.py:10-162.
 *   z, cut        fp32 (n_groups, group): the reference and the depth below it
 *                 under which a key is cut (used when truncate != 0)
 *   vmean         fp32 (n_groups, head_dim) or NULL: where dropped mass re-enters
 *   order         int32 (n_groups,) grid slot -> row group, or NULL. With an
 *                 order, n_groups is the number of slots this call takes: a call
 *                 may cover a subset of the row groups (the partial buffers are
 *                 indexed by row group), e.g. the long requests on one kernel and
 *                 the short ones on the other, combined once afterwards
 *   split         CTAs per row group; chunk_keys > 0 fixes the keys per split
 *   refine_bands  host: (edge0, edge1, rk1, rk2, rv1, rv2) or NULL
 *   o_part        fp32 (n_groups*split, group, head_dim) scratch; den_part
 *                 (n_groups*split, group); cnt_part int32 (n_groups*split, 2)
 *   out           (n_groups, group, head_dim) as out_dtype: 0 fp32, 1 bf16, 2 fp16;
 *                 NULL leaves the partials uncombined (fold_decode_combine)
 *   den           fp32 (n_groups, group); counts int32 (n_groups, 2): live, refined
 *   status        int32[1]: set non-zero if a device-side wait ran out */
int fold_decode_run(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                    const int8_t* kb, const void* ek, const void* va, const void* vb,
                    const float* vmean, const float* z, const float* cut,
                    const int32_t* page_table, const int32_t* seq_lens, const int32_t* order,
                    int n_groups, int group, int n_kv_heads, int head_dim, int pages_per_request,
                    int page_size, int split, int chunk_keys, int truncate, int weight_terms,
                    float refine_k, float refine_v, const float* refine_bands /* host */,
                    float v_scale, float* o_part, float* den_part, int32_t* cnt_part, void* out,
                    int out_dtype, float* den, int32_t* counts, int32_t* status, void* stream);

/* fold_decode_run with a tail, on a bf16 V at a finite depth: a dropped key's
 * mass re-enters at its own 64-key block's row (tail_rows) and, at rank 16, at the
 * part of its V that its K predicts: y = (plane A . u) ek / 256 comes out of the
 * coarse logit's own matmul, and the epilogue maps the rows' rank sums back through
 * vr. The denominator is the whole softmax's mass, as with vmean. Always truncating,
 * no plane B of V, no vmean; page_size a multiple of 64; other arguments as
 * fold_decode_run. Replaces: the tail paths of src/fold_attention/decode/kernel.py
 * :905-1200 and decode/combine.py:38-75, fed by decode/cache.py:200-337.
 *   tail_rows bf16 (pool_rows/64, head_dim); tail_u int8 (n_groups, 16, head_dim) and
 *   tail_vr fp32 (n_groups, head_dim, 16), both NULL at tail_rank 0 */
int fold_decode_run_tail(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                         const int8_t* kb, const void* ek, const void* va, const void* tail_rows,
                         const int8_t* tail_u, const float* tail_vr, int tail_rank, const float* z,
                         const float* cut, const int32_t* page_table, const int32_t* seq_lens,
                         const int32_t* order, int n_groups, int group, int n_kv_heads, int head_dim,
                         int pages_per_request, int page_size, int split, int chunk_keys,
                         int weight_terms, float refine_k, float* o_part, float* den_part,
                         int32_t* cnt_part, void* out, int out_dtype, float* den, int32_t* counts,
                         int32_t* status, void* stream);

/* fold_decode_run and fold_mass_z for the layouts beyond the single-level step (warp-level
 * kernel only). Replaces: the draft, cascade and row-cut paths of
 * src/fold_attention/decode/launch.py:509-1252 (_prepare with draft_len / mask / shared /
 * group_cut), decode/rows.py:19-184 and the level loop of decode/combine.py.
 *   req_map      int32 (requests,) or NULL: the row of page_table / seq_lens a request reads
 *                (a cascade's shared level: the prefix the request holds; vmean is then
 *                indexed by that row and KV head)
 *   group_split  row groups per KV head: a group of 16, 24 or 32 query rows runs as 2, 3 or 4
 *                groups of 8 (qa, z, ... are then (n_groups, 8, ..) with n_groups counting them)
 *   tree         int32 (n_groups, group) or NULL: bit j of a row's word says the row sees
 *                draft node j; the nodes are the cache's last draft_len keys (1..32), which a
 *                row otherwise would all see. NULL with draft_len 0.
 *   slots_total, slot_off   the partial buffers hold slots_total slots per row group and this
 *                call's splits take slots slot_off .. slot_off + split - 1 (a cascade's levels
 *                share the buffers and one fold_decode_combine with split = slots_total adds
 *                them); a call that does not own every slot takes chunk_keys 0 and out NULL.
 *                slots_total 0 means split.
 *   row_cut      1: a key enters a row only if that row keeps it (the reference's choice for
 *                drafts and cascades); 0: if any row of its group keeps it
 *   sound        fp32 (n_groups, group) or NULL: per row eq * sum_d (128 |qa_d| + |qb_d| / 2);
 *                the verdict then tests the coarse logit plus sound * ek / 256, a bound on what
 *                K's second plane can add, so only keys the full logit would also drop are
 *                dropped (decode/kernel.py:573-612, 797-834)
 *   vmean_per_row  1: vmean is (n_groups, group, head_dim), a direction per query row */
int fold_decode_run_ex(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                       const int8_t* kb, const void* ek, const void* va, const void* vb,
                       const float* vmean, const float* z, const float* cut,
                       const int32_t* page_table, const int32_t* seq_lens, const int32_t* order,
                       int n_groups, int group, int n_kv_heads, int head_dim, int pages_per_request,
                       int page_size, int split, int chunk_keys, int truncate, int weight_terms,
                       float refine_k, float refine_v, const float* refine_bands /* host */,
                       float v_scale, float* o_part, float* den_part, int32_t* cnt_part, void* out,
                       int out_dtype, float* den, int32_t* counts, int32_t* status,
                       const int32_t* req_map, int group_split, const int32_t* tree, int draft_len,
                       int slots_total, int slot_off, int row_cut, const float* sound,
                       int vmean_per_row, void* stream);
int fold_mass_z_ex(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                   const void* ek, const int32_t* page_table, const int32_t* seq_lens, int n_groups,
                   int group, int n_kv_heads, int head_dim, int pages_per_request, int page_size,
                   float* z, const int32_t* req_map, int group_split, const int32_t* tree,
                   int draft_len, void* stream);

/* The same decode on tcgen05 tensor cores (TMEM accumulators, the E4M3 V planes
 * read by the tensor core as stored; weights carried as four E5M2 terms). K's
 * and V's first planes stream whole through shared memory; V's second plane is
 * fetched by 32-key quarters where enough keys pass the refine-V gate; the
 * remaining refined keys, and keys whose weight passes 2^8, are summed in fp32
 * by helper warps in a fixed order. A bf16 V (vb NULL) runs the same schedule
 * with two bf16 weight terms and no second plane. For head_dim 128, groups of
 * 1..8 rows, page_size and chunk_keys multiples of 128
 * (fold_decode_sm100_supported, which also wants the driver's tensor-map
 * encoder). Arguments as fold_decode_run without weight_terms; `va` and `vb`
 * 16-byte aligned. Replaces the same reference code as fold_decode_run.
 * Two things the ABI cannot check, for both decode entries: every page_table
 * entry a request's length reaches must be a page of this GPU's own pool (the
 * entries carry no pool size, so a stale index is a wild read, not a zero tile;
 * V's tensor map here spans the address space from `va`), and with chunk_keys > 0
 * the caller provides split * chunk_keys >= the longest sequence: keys past the
 * last split are not visited. The host layer (FoldKVCache) guarantees both. */
int fold_decode_sm100_supported(int group, int head_dim, int page_size, int chunk_keys, int v8);
int fold_decode_run_sm100(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                          const int8_t* kb, const void* ek, const void* va, const void* vb,
                          const float* vmean, const float* z, const float* cut,
                          const int32_t* page_table, const int32_t* seq_lens, const int32_t* order,
                          int n_groups, int group, int n_kv_heads, int head_dim,
                          int pages_per_request, int page_size, int split, int chunk_keys,
                          int truncate, float refine_k, float refine_v,
                          const float* refine_bands /* host */, float v_scale, float* o_part,
                          float* den_part, int32_t* cnt_part, void* out, int out_dtype, float* den,
                          int32_t* counts, int32_t* status, void* stream);

/* Where the tcgen05 decode kernel's roles spend their cycles: 32 counters (listed beside the
 * entry in csrc/decode_sm100.cu) that a library built with -DFOLD_DEC_COUNTERS accumulates;
 * FOLD_ERR_UNSUPPORTED from any other build. No counterpart in the reference. */
int fold_decode_counters(uint64_t* out32, int reset);

/* The combine step alone: out = (sum over splits of o_part) * v_scale / (sum of
 * den_part), in slot order. Replaces src/fold_attention/decode/combine.py:10-162. */
int fold_decode_combine(const float* o_part, const float* den_part, const int32_t* cnt_part,
                        const int32_t* seq_lens, void* out, int out_dtype, float* den,
                        int32_t* counts, int n_groups, int group, int head_dim, int n_kv_heads,
                        int split, int chunk_keys, float v_scale, void* stream);

/* fold_decode_run for callers that may not allocate device memory.
 * No counterpart in the reference (its launches allocate their partial buffers
 * with torch). Same arguments as fold_decode_run without o_part, den_part and
 * cnt_part: the split partials live in a fixed array inside the library
 * (FOLD_DECODE_STATIC_SCRATCH_BYTES per GPU, held from library load to process
 * exit). The call allocates nothing: no cudaMalloc, cudaFree or allocating
 * library routine. A call whose partials would not fit (see
 * fold_decode_static_scratch_needed) is rejected with FOLD_ERR_ARGUMENT.
 * Two differences from fold_decode_run, both because the array is laid out for
 * exactly n_groups row groups and is out of the caller's reach: `out`, `den`
 * and `counts` must be given (there is no partials-only form), and `order`
 * must be NULL or a permutation of 0 .. n_groups-1 (no subset calls). The
 * order lives on the device, so the kernel checks it: a slot mapped outside
 * 0 .. n_groups-1 touches no memory and sets *status to FOLD_ERR_ARGUMENT.
 * The first call on each device looks the array's address up (with that
 * device current); make that first call before starting any stream capture.
 * Every call on a device shares the one array and leaves the last call's
 * partials in it, so two calls that overlap on the GPU race on it -- calls on
 * different streams or from different host threads included. Keep every call
 * on a device on one stream, or order them with events. (Another process has
 * its own copy of the array.) Nothing in it needs clearing between calls. */
#define FOLD_DECODE_STATIC_SCRATCH_BYTES (4u << 20)
size_t fold_decode_static_scratch_needed(int n_groups, int group, int head_dim, int split);
int fold_decode_run_static(const int8_t* qa, const int8_t* qb, const float* eq, const int8_t* ka,
                           const int8_t* kb, const void* ek, const void* va, const void* vb,
                           const float* vmean, const float* z, const float* cut,
                           const int32_t* page_table, const int32_t* seq_lens, const int32_t* order,
                           int n_groups, int group, int n_kv_heads, int head_dim,
                           int pages_per_request, int page_size, int split, int chunk_keys,
                           int truncate, int weight_terms, float refine_k, float refine_v,
                           const float* refine_bands /* host */, float v_scale, void* out,
                           int out_dtype, float* den, int32_t* counts, int32_t* status,
                           void* stream);

/* ---- Path A: deterministic attention backward ------------------------------ */

#define FOLD_BWD_KERNEL_AUTO 0  /* tcgen05 where it applies, else mma.sync */
#define FOLD_BWD_KERNEL_MMA 1
#define FOLD_BWD_KERNEL_SM100 2

/* Tensor arguments of the training entry points are described by `strides`:
 * three int64 element strides (batch, token row, head) per tensor, channels
 * contiguous. Dense calls are (B, S, H, D); packed calls (total, H, D) with
 * batch stride 0 and cu_seqlens (batch+1) int32 on the device. lse is fp32 in
 * nats, (B, H, S) dense or (H, total) packed. */

/* How a call's work is cut for the tcgen05 main loop: `subgroup` query heads (a divisor of the
 * group; 0 = the whole group) and `record` query blocks of 128 rows (0 = every block that sees the
 * key block) per work item. With the whole group and the whole range a key block's dK and dV stay
 * inside one CTA; otherwise its work items round their sums onto the (request, KV head)'s dK / dV
 * integer grids and add them into int64 (dV: int32 while group * max_seqlen <= 16384)
 * accumulators in the workspace, which the postprocess converts. Integer adds commute, so the
 * gradients are the same bits in any execution order either way; they do depend on the plan.
 * Replaces: src/fold_attention/backward/plan.py:58-118 (Plan), launch.py:172-213. The mma.sync
 * main loop takes only (0, 0). */

/* Bytes of scratch fold_bwd_run needs (the int32 dQ accumulator, Delta, lse*log2e, the
 * per-(request, KV head) maxima, the work list and, for a folding plan, the dK / dV accumulators);
 * 0 for an impossible plan.
 * Replaces the allocations of src/fold_attention/backward/launch.py:186-216. */
size_t fold_bwd_workspace_bytes(int batch, int n_heads, int n_kv_heads, int max_seqlen, int total,
                                int head_dim, int varlen, int subgroup, int record);

/* Byte offsets of the workspace's parts, for callers that inspect the accumulators. out11: host,
 * eleven entries: [0..3] dq_acc, dpsum, lse2, stats; [4] padded rows per head; [5] the int32
 * status word (non-zero after a call in which a device-side wait ran out); [6], [7] the dK and dV
 * accumulators; [8] dV's accumulator width in bits (0: the plan does not fold); [9] the work list
 * (eight int32 per item: key block, KV head, request, first head, heads, first and one-past-last
 * query block, cost in tiles), [10] its length. */
int fold_bwd_workspace_layout(int batch, int n_heads, int n_kv_heads, int max_seqlen, int total,
                              int head_dim, int varlen, int subgroup, int record, int64_t* out11);

/* dQ, dK, dV of causal or full self-attention: preprocess, work list, main loop and
 * postprocess on `stream`, no host synchronisation.
 * Replaces: src/fold_attention/backward/launch.py:75-117 (prepare_backward) and
 * the run() closure :410-435; kernels backward/preprocess.py, kernel.py, scheduler.py,
 * postprocess.py. strides: q, k, v, o, dout, dq, dk, dv (24 entries). */
int fold_bwd_run(const void* q, const void* k, const void* v, const void* o, const void* dout,
                 const float* lse, void* dq, void* dk, void* dv, const int64_t* strides /* host */,
                 const int32_t* cu_seqlens, int batch, int n_heads, int n_kv_heads, int max_seqlen,
                 int total, int head_dim, int causal, int is_f16, float softmax_scale,
                 void* workspace, size_t workspace_bytes, int kernel, int subgroup, int record,
                 void* stream);

/* fold_bwd_run one phase at a time (a bit mask), so a caller can put events
 * between the preprocess, the main loop and the postprocess. The phases of
 * one backward must run in order on one stream with the same arguments
 * (PRE, LIST, MAIN, POST; LIST writes the tcgen05 main loop's work list into the
 * workspace, where it stays valid until the shapes or cu_seqlens change, and does
 * nothing for the other main loop).
 * No counterpart in the reference: its launch closure runs all of them. */
#define FOLD_BWD_PHASE_PRE 1
#define FOLD_BWD_PHASE_MAIN 2
#define FOLD_BWD_PHASE_POST 4
#define FOLD_BWD_PHASE_LIST 8
int fold_bwd_run_phases(const void* q, const void* k, const void* v, const void* o,
                        const void* dout, const float* lse, void* dq, void* dk, void* dv,
                        const int64_t* strides /* host */, const int32_t* cu_seqlens, int batch,
                        int n_heads, int n_kv_heads, int max_seqlen, int total, int head_dim,
                        int causal, int is_f16, float softmax_scale, void* workspace,
                        size_t workspace_bytes, int kernel, int subgroup, int record, int phases,
                        void* stream);

/* Cycle counters of the tcgen05 backward's main loop, summed over the launches since the
 * last reset: out24 (host, 24 entries) receives CTAs, tiles, CTA lifetime, prologue, epilogue,
 * the compute warps' wait for S^T / exponential phase / wait for dP^T / dS~ phase, the MMA
 * thread's cycles with nothing to issue, the drain's wait and busy cycles and its time from
 * dQ~ ready to its columns released, the MMA thread's waits for P~, Q, dS~, dO and that release
 * (then zeros). Synchronises the device. Returns FOLD_ERR_UNSUPPORTED unless the library was
 * built with -DFOLD_BWD_COUNTERS (the product build is not). No counterpart in the reference. */
int fold_bwd_counters(uint64_t* out24 /* host */, int reset);

/* The kernels' bounded wait, alone: one warp waits `limit_cycles` SM cycles (1 .. 2^31) on a
 * barrier nothing arrives at, through the same code path every role of the tcgen05 kernels
 * waits with; when the wait runs out it stores FOLD_ERR_TIMEOUT to *status and raises the
 * CTA's abort flag (copied to *flag_out if given), and the kernel returns normally. For tests of
 * the host's handling of the status word; nothing faults. No counterpart in the reference (its
 * device-side waits are unbounded). */
int fold_wait_probe(long long limit_cycles, int32_t* status, int32_t* flag_out, void* stream);

/* Attention forward: O and the log-sum-exp (nats) the backward consumes.
 * Replaces the third-party forward called at src/fold_attention/interface.py:42-44,
 * :70-81 and kv_cache.py:252-262. strides: q, k, v, o (12 entries). */
int fold_fwd_run(const void* q, const void* k, const void* v, void* o, float* lse,
                 const int64_t* strides /* host */, const int32_t* cu_seqlens, int batch,
                 int n_heads, int n_kv_heads, int max_seqlen, int total, int head_dim, int causal,
                 int is_f16, float softmax_scale, void* stream);

/* The same forward on tcgen05 tensor cores (TMA-fed Q K^T and P V with S, P and O in TMEM),
 * for head_dim 128, bf16 or fp16 (fold_fwd_sm100_supported). Arguments as fold_fwd_run, plus
 * status: int32[1], set non-zero if a device-side wait ran out. Replaces the same third-party
 * forward as fold_fwd_run. */
int fold_fwd_sm100_supported(int head_dim, int is_f16);
int fold_fwd_run_sm100(const void* q, const void* k, const void* v, void* o, float* lse,
                       const int64_t* strides /* host */, const int32_t* cu_seqlens, int batch,
                       int n_heads, int n_kv_heads, int max_seqlen, int total, int head_dim,
                       int causal, int is_f16, float softmax_scale, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FOLD_B200_H */
