// Warp-level tensor-core helpers (mma.sync m16n8k16, ldmatrix, cp.async) used
// by the general-shape kernels: every head dim, fp16, ragged tiles.
#pragma once
#include "common.cuh"

namespace fold {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// D (16x8 f32) += A (16x16, row) * B (16x8, col); 16-bit operands
template <bool F16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (F16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// 16-byte async copy; src_bytes = 0 zero-fills the destination
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool F16>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
    if constexpr (F16) return pack_f16x2(lo, hi);
    else return pack_bf16x2(lo, hi);
}

// Copy `rows` rows of D 16-bit channels (row stride `sr` elements) into a
// shared tile of pitch PITCH bytes; rows at or past `valid` are zero-filled.
template <int D, int PITCH, int THREADS>
__device__ __forceinline__ void load_tile_async(uint8_t* smem, const uint16_t* gbase, int64_t sr,
                                                int rows, int valid, int tid) {
    constexpr int CPR = D / 8;  // 16-byte chunks per row
    for (int i = tid; i < rows * CPR; i += THREADS) {
        const int r = i / CPR, c = i % CPR;
        const bool ok = r < valid;
        const uint16_t* src = gbase + (ok ? r : 0) * sr + c * 8;
        cp_async16(smem_u32(smem + r * PITCH + c * 16), src, ok ? 16 : 0);
    }
}

}  // namespace fold
