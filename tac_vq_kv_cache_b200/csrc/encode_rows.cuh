// Nearest-word search of one (row, group) residual by a whole warp, shared by the row-at-a-time encode
// kernels and by the decode-step bookkeeping that is fused into the attention table preparation.
//
// Lane l scores words l, l+32, ... in ascending order (strict '<' keeps the lowest index per lane) and the
// warp takes the lexicographic minimum of (distance, index): the same first minimum as a sequential scan.
// Arithmetic per distance is the library's fixed order (common.cuh), so every caller gets the same codes.
#pragma once

#include "common.cuh"

namespace tacvq {

// lexicographic minimum of (distance, index) over the warp
__device__ __forceinline__ int warp_first_minimum(float best, int arg, int K) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
        if (ob < best || (ob == best && oa < arg)) {
            best = ob;
            arg = oa;
        }
    }
    return arg >= K ? 0 : arg;  // every distance was +inf or NaN
}

template <int DSUB>
__device__ __forceinline__ void consider_word(const float (&res)[DSUB], float xx, const float (&c)[DSUB], const float *cc_in, int k,
                                              float &best, int &arg) {
    const float cc = cc_in ? *cc_in : sqnorm_ordered<DSUB>([&](int i) { return c[i]; });
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < DSUB; ++i) dot = __fmaf_rn(res[i], c[i], dot);
    const float dist = distance_expr(xx, cc, dot);
    if (dist < best) {
        best = dist;
        arg = k;
    }
}

__device__ __forceinline__ void unpack8(const uint4 &w, float (&c)[8]) {
    const __half2 *hp = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(hp[i]);
        c[2 * i] = f.x;
        c[2 * i + 1] = f.y;
    }
}

template <int DSUB>
__device__ __forceinline__ int nearest_word_in_warp(const float (&res)[DSUB], const __half *__restrict__ words,
                                                    const float *__restrict__ sqnorm_in, int K, int lane) {
    const float xx = sqnorm_ordered<DSUB>([&](int i) { return res[i]; });
    float best = __int_as_float(0x7f800000);
    int arg = 0x7fffffff;
    const bool aligned = (reinterpret_cast<uintptr_t>(words) & 15) == 0;
    for (int k = lane; k < K; k += 32) {
        float c[DSUB];
        if constexpr (DSUB == 8) {
            if (aligned) {  // one 16-byte load per word: the same values
                unpack8(__ldg(reinterpret_cast<const uint4 *>(words + (int64_t)k * DSUB)), c);
            } else {
#pragma unroll
                for (int i = 0; i < DSUB; ++i) c[i] = __half2float(words[(int64_t)k * DSUB + i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < DSUB; ++i) c[i] = __half2float(words[(int64_t)k * DSUB + i]);
        }
        consider_word<DSUB>(res, xx, c, sqnorm_in ? sqnorm_in + k : nullptr, k, best, arg);
    }
    return warp_first_minimum(best, arg, K);
}

// The same search over 256 words of 8 channels that the caller has already fetched: w[i] is word lane + 32*i.
__device__ __forceinline__ int nearest_of_fetched_words(const float (&res)[8], const uint4 (&w)[8], int lane) {
    const float xx = sqnorm_ordered<8>([&](int i) { return res[i]; });
    float best = __int_as_float(0x7f800000);
    int arg = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float c[8];
        unpack8(w[i], c);
        consider_word<8>(res, xx, c, nullptr, lane + 32 * i, best, arg);
    }
    return warp_first_minimum(best, arg, 256);
}

}  // namespace tacvq
