// Shared device helpers for libtacvq (sm_100a).
//
// Floating-point orders fixed by this library (they are the orders the reference's CPU library
// calls were observed to use, so that codes agree bit for bit; see include/tacvq.h):
//   dot(x, c)      one fused-multiply-add chain, element 0 first, accumulator starts at +0
//   sqnorm(v)      products rounded to fp32 first (no fusion), then
//                    d <= 8 (or d not a multiple of 8) ... added left to right
//                    d = 16, 24 ......................... eight running lanes, lane j takes
//                                                         elements j, j+8, ...; lanes added 0..7
//                    d multiple of 32 ................... four sets of eight lanes, element i goes to
//                                                         set (i/8)%4, lane i%8; per lane the sets are
//                                                         added ((0+1)+2)+3; lanes added 0..7
//   distance       (xx + cc) - 2*dot : one add, then one fused multiply-add with the exact product -2*dot
//   argmin         ascending k, strict '<' : lowest index wins a tie
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tacvq.h"

namespace tacvq {

constexpr int kMaxWords = 256;

template <int D, typename Load>
__device__ __forceinline__ float sqnorm_ordered(Load at) {
    if constexpr (D <= 8 || (D % 8) != 0) {
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < D; ++i) {
            const float v = at(i);
            acc = __fadd_rn(acc, __fmul_rn(v, v));
        }
        return acc;
    } else if constexpr ((D % 32) != 0) {
        float lane[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = at(j);
            lane[j] = __fmul_rn(v, v);
        }
#pragma unroll
        for (int i = 8; i < D; ++i) {
            const float v = at(i);
            lane[i & 7] = __fadd_rn(lane[i & 7], __fmul_rn(v, v));
        }
        float acc = lane[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) acc = __fadd_rn(acc, lane[j]);
        return acc;
    } else {
        float set[4][8];
#pragma unroll
        for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int j = 0; j < 8; ++j) set[s][j] = 0.0f;
#pragma unroll
        for (int i = 0; i < D; ++i) {
            const float v = at(i);
            set[(i >> 3) & 3][i & 7] = __fadd_rn(set[(i >> 3) & 3][i & 7], __fmul_rn(v, v));
        }
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float lane = __fadd_rn(__fadd_rn(__fadd_rn(set[0][j], set[1][j]), set[2][j]), set[3][j]);
            acc = (j == 0) ? lane : __fadd_rn(acc, lane);
        }
        return acc;
    }
}

// Runtime-d variant of the same orders (used where d is not a template parameter).
__device__ __forceinline__ float sqnorm_ordered_rt(const float *v, int d) {
    if (d <= 8 || (d % 8) != 0) {
        float acc = 0.0f;
        for (int i = 0; i < d; ++i) acc = __fadd_rn(acc, __fmul_rn(v[i], v[i]));
        return acc;
    }
    float lane[8];
    if ((d % 32) != 0) {
        for (int j = 0; j < 8; ++j) lane[j] = __fmul_rn(v[j], v[j]);
        for (int i = 8; i < d; ++i) lane[i & 7] = __fadd_rn(lane[i & 7], __fmul_rn(v[i], v[i]));
    } else {
        for (int j = 0; j < 8; ++j) {
            float set[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int i = j; i < d; i += 8) set[(i >> 3) & 3] = __fadd_rn(set[(i >> 3) & 3], __fmul_rn(v[i], v[i]));
            lane[j] = __fadd_rn(__fadd_rn(__fadd_rn(set[0], set[1]), set[2]), set[3]);
        }
    }
    float acc = lane[0];
    for (int j = 1; j < 8; ++j) acc = __fadd_rn(acc, lane[j]);
    return acc;
}

__device__ __forceinline__ float distance_expr(float xx, float cc, float dot) {
    // (xx + cc) - 2*dot ; 2*dot is exact, so the fused form rounds once exactly like the subtraction.
    return __fmaf_rn(-2.0f, dot, __fadd_rn(xx, cc));
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ void store_as(T *p, float v);
template <>
__device__ __forceinline__ void store_as<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_as<__half>(__half *p, float v) { *p = __float2half_rn(v); }

// Arguments of one encode launch, shared by the ABI layer and the kernel dispatcher.
struct EncodeArgs {
    const void *x;
    int x_dtype;
    int64_t sxb, sxh, sxt;
    const void *tables;          // search tables: fp16 deployed words, or fp32 transformed words
    bool tables_f32;
    const float *sqnorm;         // optional caller-supplied |word|^2
    uint8_t *codes;
    void *recon;
    int recon_dtype;
    const __half *recon_tables;  // plain fp16 words the reconstruction is summed from
    int B, H, T, D, G, S, K;
    int64_t t0, T_cap;
    cudaStream_t stream;
};

// The new token of a decode step, handed to the benchmark-geometry attention when its table preparation
// also does the step's bookkeeping: rows [B][Hkv][128] of K and V to encode into the code buffers at
// `position`, and the visible range [start, end) that every sequence gets.
struct GsrqNewToken {
    const void *k_rows, *v_rows;
    int rows_f32;
    uint8_t *kcodes, *vcodes;
    int32_t *seq_start, *seq_end;
    int start, end;
    long long position, T_cap;
};

inline int launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TACVQ_OK : static_cast<int>(e);
}

}  // namespace tacvq
