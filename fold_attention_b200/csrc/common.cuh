// Shared device/host helpers of libfold_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "fold_b200.h"

namespace fold {

// ---- error reporting behind the C ABI (fold_last_error) -------------------
void set_error(const char* fmt, ...);
int check_launch(const char* what);

#define FOLD_CHECK_ARG(cond, ...)        \
    do {                                 \
        if (!(cond)) {                   \
            fold::set_error(__VA_ARGS__); \
            return FOLD_ERR_ARGUMENT;    \
        }                                \
    } while (0)


constexpr float kLog2e = 1.4426950408889634f;

// ---- 16-bit loads ----------------------------------------------------------
template <bool F16>
__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    if constexpr (F16) {
        return __half2float(__ushort_as_half(h));
    } else {
        return __uint_as_float(static_cast<uint32_t>(h) << 16);
    }
}

// Sixteen 16-bit floats at a 32-byte aligned address, as fp32 and raw words.
template <bool F16>
__device__ __forceinline__ void load16(const void* p, float (&x)[16], uint4 (&w)[2]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    w[0] = __ldg(q);
    w[1] = __ldg(q + 1);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        x[2 * i] = half_bits_to_float<F16>(static_cast<uint16_t>(u[i] & 0xFFFFu));
        x[2 * i + 1] = half_bits_to_float<F16>(static_cast<uint16_t>(u[i] >> 16));
    }
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t h) {
    return __uint_as_float(static_cast<uint32_t>(h) << 16);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- the backward's integer grid (one exponent per request and KV head) ----
// stats[b, h_kv, i] are float bits, zero before the call.
enum { ST_K = 0, ST_V = 1, ST_DO = 2, ST_DELTA = 3, ST_DOC = 4, ST_Q = 5, N_STATS = 8 };
constexpr int DQ_BITS = 30;
constexpr int DKV_BITS = 61;   // dK's grid, and dV's when a group's column mass G * S can pass 16384

// 2^(bits - ceil(log2(bound * (1 + 2^-6)))), clamped to [2^-100, 2^100]; a
// zero bound takes 2^100. Every step is one rounded fp32 instruction or an
// exact bit operation, so every kernel that evaluates it gets the same scale.
__host__ __device__ __forceinline__ int pow2_scale_exp(float bound, int bits) {
#ifdef __CUDA_ARCH__
    float b = __fmul_rn(bound, 1.015625f);
    int bb = __float_as_int(b);
#else
    volatile float b = bound * 1.015625f;
    int bb;
    {
        float t = b;
        memcpy(&bb, &t, 4);
    }
#endif
    int clog = ((bb >> 23) & 0xFF) - 127 + ((bb & 0x7FFFFF) != 0 ? 1 : 0);
    int sexp = bits - clog;
    if (!(b > 0.0f)) sexp = 100;
    if (sexp > 100) sexp = 100;
    if (sexp < -100) sexp = -100;
    return sexp;
}

// sqrt(D) rounded up to a power of two
__host__ __device__ __forceinline__ float root_d(int D) {
    float c = 1.0f;
    while (c * c < static_cast<float>(D)) c *= 2.0f;
    return c;
}

#ifdef __CUDACC__
// dQ's grid exponent s for one (request, KV head): the accumulator holds
// dQ / softmax_scale * 2^s.
__device__ __forceinline__ int dq_scale_exp(const int* stats, float cd) {
    float k = __int_as_float(stats[ST_K]);
    float v = __int_as_float(stats[ST_V]);
    float dn = __int_as_float(stats[ST_DO]);
    float dl = __int_as_float(stats[ST_DELTA]);
    float s = __fadd_rn(__fmul_rn(dn, __fmul_rn(v, cd)), dl);
    return pow2_scale_exp(__fmul_rn(s, k), DQ_BITS);
}
// dK's and dV's grid exponents for one (request, KV head), used when a key block's dK / dV are
// summed across CTAs (src/fold_attention/backward/grid.py:86-100). `rows` = G * sequence length
// bounds the column mass sum_{h,i} P_hij; dV's bound is rows * max |dO_id|, dK's
// rows * (||dO||max * C_D * |V|max + |Delta|max) * |Q|max.
__device__ __forceinline__ int dv_scale_exp(const int* stats, float rows, int bits) {
    return pow2_scale_exp(__fmul_rn(rows, __int_as_float(stats[ST_DOC])), bits);
}
__device__ __forceinline__ int dk_scale_exp(const int* stats, float rows, float cd) {
    float v = __int_as_float(stats[ST_V]);
    float dn = __int_as_float(stats[ST_DO]);
    float dl = __int_as_float(stats[ST_DELTA]);
    float s = __fadd_rn(__fmul_rn(dn, __fmul_rn(v, cd)), dl);
    return pow2_scale_exp(__fmul_rn(rows, __fmul_rn(s, __int_as_float(stats[ST_Q]))), DKV_BITS);
}
__device__ __forceinline__ float pow2f(int e) { return __int_as_float((e + 127) << 23); }
#endif

}  // namespace fold
