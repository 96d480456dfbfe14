// Attention over stored codes - geometry-generic kernel and the log-sum-exp merge.
//
// One block serves one (batch row, KV head, sequence split).  It first builds, for each of the
// REP query heads that share the KV head, a look-up table lut[r][code][slot] = q_r[group] . word
// (slot = stage*G + group), then scans its token range one token per warp step:
//     score_r = sum_slot lut[r][kcode[slot]][slot]            (lane = slot, warp reduction)
//     online softmax (running max m_r, sum l_r)
//     acc_r  += exp(score_r - m_r) * V_row                      (lane owns D/32 channels; the V row is
//                                                               rebuilt from its codes exactly as the
//                                                               reference stores it: fp32 stage sum
//                                                               rounded once to fp16)
// and finally merges its warps' states into one partial state per split.  A second kernel merges
// the splits.  This kernel is the fallback for every geometry; the (G=16,S=2,d=8) benchmark
// geometry has a specialised kernel in attn_gsrq.cu.
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122
// (dequantised window -> repeat_kv -> softmax(q K^T) V), without the rotary step.

#include "common.cuh"

namespace tacvq {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;

template <int REP, int DPL>
__global__ void __launch_bounds__(kAttnThreads)
attn_generic_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes,
                    const uint8_t *__restrict__ vcodes, const __half *__restrict__ ktab,
                    const __half *__restrict__ vtab, const int32_t *__restrict__ seq_start,
                    const int32_t *__restrict__ seq_end, float *__restrict__ part, int B, int Hq, int Hkv, int D, int G,
                    int S, int K, int64_t T_cap, int splits) {
    extern __shared__ __align__(16) float smem[];
    const int slots = S * G;
    const int d = D / G;
    float *lut = smem;  // [REP][K][slots]

    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- look-up tables -------------------------------------------------------------------------
    for (int idx = tid; idx < slots * K; idx += kAttnThreads) {
        const int slot = idx % slots, k = idx / slots;  // slot fastest: conflict-free table writes
        const int s = slot / G, g = slot % G;
        const __half *w = ktab + ((((int64_t)h * S + s) * G + g) * K + k) * d;
        float dot[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) dot[r] = 0.0f;
        for (int i = 0; i < d; ++i) {
            const float c = __half2float(w[i]);
#pragma unroll
            for (int r = 0; r < REP; ++r)
                dot[r] = fmaf(__half2float(q[((int64_t)b * Hq + h * REP + r) * D + g * d + i]), c, dot[r]);
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) lut[((size_t)r * K + k) * slots + slot] = dot[r];
    }
    __syncthreads();

    // ---- token range of this split ---------------------------------------------------------------
    const int lo_all = seq_start ? seq_start[b] : 0;
    const int hi_all = seq_end ? seq_end[b] : (int)T_cap;
    const int n_all = hi_all > lo_all ? hi_all - lo_all : 0;
    const int per = (n_all + splits - 1) / splits;
    const int lo = lo_all + split * per;
    const int hi = min(lo + per, lo_all + n_all);

    float m[REP], l[REP], acc[REP][DPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = 0.0f;
    }
    const int c0 = lane * DPL;
    const int vg = c0 / d, vi0 = c0 % d;
    const int64_t code_row = ((int64_t)b * Hkv + h) * T_cap;

    for (int t = lo + warp; t < hi; t += kAttnWarps) {
        const uint8_t *kc = kcodes + (code_row + t) * slots;
        const uint8_t *vc = vcodes + (code_row + t) * slots;
        float sc[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) sc[r] = 0.0f;
        for (int j = lane; j < slots; j += 32) {
            const int code = kc[j];
#pragma unroll
            for (int r = 0; r < REP; ++r) sc[r] += lut[((size_t)r * K + code) * slots + j];
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], off);
        }
        float vrow[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) vrow[i] = 0.0f;
        for (int s = 0; s < S; ++s) {
            const int code = vc[s * G + vg];
            const __half *w = vtab + ((((int64_t)h * S + s) * G + vg) * K + code) * d + vi0;
#pragma unroll
            for (int i = 0; i < DPL; ++i) vrow[i] = __fadd_rn(vrow[i], __half2float(__ldg(w + i)));
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            if (sc[r] > m[r]) {
                const float scale = __expf(m[r] - sc[r]);  // exp(-inf) = 0 on the first token
                l[r] *= scale;
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[r][i] *= scale;
                m[r] = sc[r];
            }
            const float p = __expf(sc[r] - m[r]);
            l[r] += p;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[r][i] = fmaf(p, __half2float(__float2half_rn(vrow[i])), acc[r][i]);
        }
    }

    // ---- merge the warps of this block -----------------------------------------------------------
    __syncthreads();  // LUT no longer needed: reuse its storage
    float *wm = smem;                          // [warps][REP]
    float *wl = wm + kAttnWarps * REP;         // [warps][REP]
    float *wacc = wl + kAttnWarps * REP;       // [warps][REP][D]
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            wm[warp * REP + r] = m[r];
            wl[warp * REP + r] = l[r];
        }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int i = 0; i < DPL; ++i) wacc[((size_t)warp * REP + r) * D + c0 + i] = acc[r][i];
    __syncthreads();
    const int64_t rows = (int64_t)B * Hq;
    for (int idx = tid; idx < REP * (D + 2); idx += kAttnThreads) {
        const int r = idx / (D + 2), col = idx % (D + 2);
        float top = -INFINITY;
        for (int w = 0; w < kAttnWarps; ++w) top = fmaxf(top, wm[w * REP + r]);
        float sum = 0.0f;
        if (col == 0) {
            sum = top;
        } else {
            for (int w = 0; w < kAttnWarps; ++w) {
                const float mw = wm[w * REP + r];
                if (mw == -INFINITY) continue;
                const float scale = __expf(mw - top);
                sum += scale * (col == 1 ? wl[w * REP + r] : wacc[((size_t)w * REP + r) * D + (col - 2)]);
            }
        }
        const int64_t row = (int64_t)b * Hq + h * REP + r;
        part[((int64_t)split * rows + row) * (D + 2) + col] = sum;
    }
}

// Merge n_parts states laid out [n_parts][rows][2+D]; one block per row.
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float *__restrict__ states, int n_parts, int64_t rows, int D, __half *__restrict__ out,
                    float *__restrict__ merged) {
    const int64_t row = blockIdx.x;
    const int W = D + 2;
    float top = -INFINITY;
    for (int p = 0; p < n_parts; ++p) top = fmaxf(top, states[((int64_t)p * rows + row) * W]);
    float l = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
        const float *st = states + ((int64_t)p * rows + row) * W;
        if (st[0] == -INFINITY) continue;
        l += __expf(st[0] - top) * st[1];
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float a = 0.0f;
        for (int p = 0; p < n_parts; ++p) {
            const float *st = states + ((int64_t)p * rows + row) * W;
            if (st[0] == -INFINITY) continue;
            a += __expf(st[0] - top) * st[2 + i];
        }
        if (merged) merged[row * W + 2 + i] = a;
        if (out) out[row * D + i] = __float2half_rn(l > 0.0f ? a / l : 0.0f);
    }
    if (merged && threadIdx.x == 0) {
        merged[row * W] = top;
        merged[row * W + 1] = l;
    }
}

int attn_combine_dispatch(const float *states, int n_parts, __half *out, float *merged, int64_t rows, int D,
                          cudaStream_t stream) {
    if (rows == 0) return TACVQ_OK;
    attn_combine_kernel<<<(unsigned)rows, 128, 0, stream>>>(states, n_parts, rows, D, out, merged);
    return launch_status();
}

int attn_generic_splits(int B, int Hkv, int64_t T_cap, int sms) {
    const int pairs = B * Hkv;
    int splits = (2 * sms + pairs - 1) / pairs;
    const int64_t by_len = (T_cap + 255) / 256;
    if (splits > by_len) splits = (int)by_len;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    return splits;
}

size_t attn_generic_smem(int REP, int D, int G, int S, int K) {
    const size_t lut = (size_t)REP * K * S * G * sizeof(float);
    const size_t merge = ((size_t)2 * kAttnWarps * REP + (size_t)kAttnWarps * REP * D) * sizeof(float);
    return lut > merge ? lut : merge;
}

template <int REP, int DPL>
static int launch_generic(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                          const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part, int B,
                          int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream) {
    const size_t smem = attn_generic_smem(REP, D, G, S, K);
    if (smem > 227 * 1024) return TACVQ_ERR_UNSUPPORTED;
    auto kernel = attn_generic_kernel<REP, DPL>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    kernel<<<grid, kAttnThreads, smem, stream>>>(q, kcodes, vcodes, ktab, vtab, seq_start, seq_end, part, B, Hq, Hkv, D,
                                                 G, S, K, T_cap, splits);
    return launch_status();
}

template <int REP>
static int dispatch_dpl(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                        const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part, int B,
                        int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream) {
#define TACVQ_CASE(N) \
    case N: return launch_generic<REP, N>(q, kcodes, vcodes, ktab, vtab, seq_start, seq_end, part, B, Hq, Hkv, D, G, S, K, T_cap, splits, stream);
    switch (D / 32) {
        TACVQ_CASE(1)
        TACVQ_CASE(2)
        TACVQ_CASE(4)
        TACVQ_CASE(8)
        default: return TACVQ_ERR_UNSUPPORTED;
    }
#undef TACVQ_CASE
}

int attn_generic_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                          const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part, int B,
                          int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream) {
#define TACVQ_CASE(N) \
    case N: return dispatch_dpl<N>(q, kcodes, vcodes, ktab, vtab, seq_start, seq_end, part, B, Hq, Hkv, D, G, S, K, T_cap, splits, stream);
    switch (Hq / Hkv) {
        TACVQ_CASE(1)
        TACVQ_CASE(2)
        TACVQ_CASE(4)
        TACVQ_CASE(8)
        default: return TACVQ_ERR_UNSUPPORTED;
    }
#undef TACVQ_CASE
}

}  // namespace tacvq
