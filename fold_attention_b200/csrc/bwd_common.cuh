// Shared definitions of the deterministic attention backward.
//
// One call handles B sequences ("requests"), dense (B, S, H, D) or packed
// (total, H, D) with cu_seqlens. Per-row workspaces are laid out [head][padded
// row]: a sequence's rows start on a 128-row boundary so every query tile
// belongs to one sequence.
#pragma once
#include "common.cuh"

namespace fold {

constexpr int ROW_PAD = 128;  // sequences start on this boundary in the workspaces

struct TensorView {
    void* ptr;
    int64_t sb, sr, sh;  // element strides: batch, row (token), head; channels are contiguous
};

struct BwdParams {
    TensorView q, k, v, o, dout, dq, dk, dv;
    const float* lse;      // natural log; dense (B, H, S), packed (H, total)
    int64_t lse_sb, lse_sh;
    const int* cu;         // (B + 1) int32 on the device, or null for dense
    int B, H, HKV, G, S, total, D;
    int causal, f16;
    float scale;
    // workspace
    int* dq_acc;    // int32 [H][rows_p][D], the fixed-point dQ / scale * 2^s
    float* dpsum;   // [H][rows_p]  Delta_i = sum_d dO O
    float* lse2;    // [H][rows_p]  s - lse * log2(e) (fp16: -lse * log2(e)); -inf on padded rows
    int* stats;     // [B][HKV][N_STATS] float bits of the order-free maxima
    int* status;    // one word after the stats: raised if a device-side wait ran out
    int64_t rows_p; // padded rows per head
    int dq_bias;    // the main loop adds 0x4B400000 with every partial: the accumulator starts at minus their sum
    // how the tcgen05 main loop's work is cut (the other main loop takes whole groups and ranges)
    int subgroup;   // query heads per work item; it divides G
    int record;     // query blocks per work item, 0: every block that sees the key block
    int fold;       // a key block's dK, dV are summed across work items, on integer grids
    int dv_bits;    // dV's accumulator when folding: 32 (30-bit grid) or 64 (61-bit grid)
    long long* dk_acc;   // int64 [HKV][rows_p][D], zero before the main loop (fold)
    void* dv_acc;        // int32 or int64 [HKV][rows_p][D] (fold)
    int* work;      // the work list: n_items x 8 ints, written in-stream ahead of the main loop
    int n_items;
    int* sched;     // [2]: the list's claim counter and the count of finished CTAs, zero between launches
    int S_r;        // dense: S rounded up to ROW_PAD
};

struct SeqInfo {
    int start;       // first row in the packed tensors (0 for dense)
    int len;
    int64_t pstart;  // first row in the padded workspaces
};

__device__ __forceinline__ SeqInfo seq_info(const BwdParams& p, int b) {
    SeqInfo s;
    if (p.cu) {
        s.start = p.cu[b];
        s.len = p.cu[b + 1] - s.start;
        s.pstart = (static_cast<int64_t>(s.start) + static_cast<int64_t>(b) * ROW_PAD) / ROW_PAD * ROW_PAD;
    } else {
        s.start = 0;
        s.len = p.S;
        s.pstart = static_cast<int64_t>(b) * p.S_r;
    }
    return s;
}

template <typename T>
__device__ __forceinline__ T* row_ptr(const TensorView& t, int b, int64_t row, int h) {
    return static_cast<T*>(t.ptr) + b * t.sb + row * t.sr + h * t.sh;
}

inline int64_t padded_rows(int B, int S, int total, bool varlen) {
    if (!varlen) return static_cast<int64_t>(B) * ((S + ROW_PAD - 1) / ROW_PAD * ROW_PAD);
    int64_t r = static_cast<int64_t>(total) + static_cast<int64_t>(B + 1) * ROW_PAD - 1;
    return (r + ROW_PAD - 1) / ROW_PAD * ROW_PAD;
}

// kernels
int launch_bwd_preprocess(const BwdParams& p, cudaStream_t st);
int launch_bwd_postprocess(const BwdParams& p, int layout, cudaStream_t st);
// how many work items the tcgen05 main loop's list holds for a call (0 for the other main loop)
int64_t bwd_sm100_work_items(int B, int H, int HKV, int S, int subgroup, int record);
int launch_bwd_main_mma(const BwdParams& p, cudaStream_t st);
int launch_bwd_main_sm100(const BwdParams& p, bool build_list, bool run_main, cudaStream_t st);
bool bwd_sm100_supported(const BwdParams& p);
bool bwd_sm100_biased();   // whether the tcgen05 main loop leaves its rounding constant in the partials

// dq accumulator tile layouts
enum { DQ_LAYOUT_ROW_MAJOR = 0, DQ_LAYOUT_SM100 = 1 };

}  // namespace fold
