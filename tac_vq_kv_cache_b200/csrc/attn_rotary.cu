// Attention over stored codes of PRE-rotary keys: the rotary embedding is applied to every rebuilt
// key row on the fly.
//
// One block serves one (batch row, KV head, sequence split); a warp takes one token per step and a
// lane owns DPL = D/32 neighbouring channels of it:
//     k_row  = fp16( sum_s word_s[kcode] )                       the reference's decoded fp16 window
//     k_rot  = k_row*cos + rotate_half(k_row)*sin                fp16 products and sum, each rounded,
//                                                                as apply_rotary_pos_emb does on fp16;
//                                                                channel c pairs with c +- D/2 = lane ^ 16
//     score_r = q_r . k_rot                                      fp32, warp reduction
//     online softmax, acc_r += p_r * fp16( sum_s word_s[vcode] )
// The cos/sin pairs come from a table [T][D/2] (rope_table_kernel, positions = token index + offset),
// which is the same for every head and batch row and stays in L2.  Splits are merged by
// attn_combine_kernel like in the generic kernel.  No look-up table of scores is possible here: the
// rotation makes the effective query differ per token.
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122 including
// the rotary step (:113-118); the query arrives rotated at its own position and scaled.

#include <math.h>

#include "common.cuh"

namespace tacvq {

constexpr int kRotThreads = 256;
constexpr int kRotWarps = kRotThreads / 32;

// cos/sin of position (first + t) for frequency i.  inv_freq[i] = 1 / theta^(2i/D) is evaluated on
// the host in fp32 (a power, then a reciprocal, like transformers' MistralRotaryEmbedding with the
// default rope type) and travels as a kernel argument; angle = position * inv_freq and cos/sin are
// fp32, rounded once to fp16.
struct RopeFreqs {
    float inv[128];
};

__global__ void rope_table_kernel(__half2 *__restrict__ table, int64_t tokens, int half_dim, const RopeFreqs freqs,
                                  int64_t first) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * half_dim) return;
    const int i = (int)(idx % half_dim);
    const int64_t t = idx / half_dim;
    const float angle = (float)(first + t) * freqs.inv[i];
    float sn, cs;
    sincosf(angle, &sn, &cs);
    table[idx] = __halves2half2(__float2half_rn(cs), __float2half_rn(sn));
}

int rope_table_dispatch(__half2 *table, int64_t tokens, int D, double theta, int64_t first, cudaStream_t stream) {
    const int64_t n = tokens * (D / 2);
    if (n == 0) return TACVQ_OK;
    if (D / 2 > 128) return TACVQ_ERR_UNSUPPORTED;
    RopeFreqs freqs;
    for (int i = 0; i < 128; ++i) freqs.inv[i] = i < D / 2 ? 1.0f / powf((float)theta, (float)(2 * i) / (float)D) : 0.0f;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(table, tokens, D / 2, freqs, first);
    return launch_status();
}

template <int REP, int DPL>
__global__ void __launch_bounds__(kRotThreads)
attn_rotary_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes, const uint8_t *__restrict__ vcodes,
                   const __half *__restrict__ ktab, const __half *__restrict__ vtab, const __half2 *__restrict__ rope,
                   const int32_t *__restrict__ seq_start, const int32_t *__restrict__ seq_end, float *__restrict__ part,
                   int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits) {
    extern __shared__ __align__(16) float smem[];
    const int slots = S * G;
    const int d = D / G;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int lo_all = seq_start ? seq_start[b] : 0;
    const int hi_all = seq_end ? seq_end[b] : (int)T_cap;
    const int n_all = hi_all > lo_all ? hi_all - lo_all : 0;
    const int per = (n_all + splits - 1) / splits;
    const int lo = lo_all + split * per;
    const int hi = min(lo + per, lo_all + n_all);

    const int c0 = lane * DPL;             // first channel of this lane
    const int vg = c0 / d, vi0 = c0 % d;   // its group and offset inside the group's words
    const int f0 = c0 % (D / 2);           // its first rotary frequency
    const bool upper = c0 >= D / 2;        // rotate_half: lower half takes -partner, upper half +partner

    float qv[REP][DPL];
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int i = 0; i < DPL; ++i) qv[r][i] = __half2float(q[((int64_t)b * Hq + h * REP + r) * D + c0 + i]);

    float m[REP], l[REP], acc[REP][DPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = 0.0f;
    }
    const int64_t code_row = ((int64_t)b * Hkv + h) * T_cap;
    const int64_t word_row = (int64_t)h * S * G + vg;  // + s*G per stage, then * K + code

    for (int t = lo + warp; t < hi; t += kRotWarps) {
        const uint8_t *kc = kcodes + (code_row + t) * slots + vg;
        const uint8_t *vc = vcodes + (code_row + t) * slots + vg;
        float krow[DPL], vrow[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) krow[i] = vrow[i] = 0.0f;
        for (int s = 0; s < S; ++s) {
            const __half *kw = ktab + ((word_row + (int64_t)s * G) * K + kc[s * G]) * d + vi0;
            const __half *vw = vtab + ((word_row + (int64_t)s * G) * K + vc[s * G]) * d + vi0;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                krow[i] = __fadd_rn(krow[i], __half2float(__ldg(kw + i)));
                vrow[i] = __fadd_rn(vrow[i], __half2float(__ldg(vw + i)));
            }
        }
        float sc[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) sc[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const __half mine = __float2half_rn(krow[i]);
            const __half other = __shfl_xor_sync(0xffffffffu, mine, 16);
            const __half2 cs = rope[(int64_t)t * (D / 2) + f0 + i];
            const __half turned = upper ? other : __hneg(other);
            const __half rotated = __hadd(__hmul(mine, __low2half(cs)), __hmul(turned, __high2half(cs)));
            const float kf = __half2float(rotated);
#pragma unroll
            for (int r = 0; r < REP; ++r) sc[r] = fmaf(qv[r][i], kf, sc[r]);
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], off);
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

    // ---- merge the warps of this block (same layout of partial states as the generic kernel) --------
    float *wm = smem;                         // [warps][REP]
    float *wl = wm + kRotWarps * REP;         // [warps][REP]
    float *wacc = wl + kRotWarps * REP;       // [warps][REP][D]
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
    for (int idx = tid; idx < REP * (D + 2); idx += kRotThreads) {
        const int r = idx / (D + 2), col = idx % (D + 2);
        float top = -INFINITY;
        for (int w = 0; w < kRotWarps; ++w) top = fmaxf(top, wm[w * REP + r]);
        float sum = 0.0f;
        if (col == 0) {
            sum = top;
        } else {
            for (int w = 0; w < kRotWarps; ++w) {
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

template <int REP, int DPL>
static int launch_rotary(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                         const __half *vtab, const __half2 *rope, const int32_t *seq_start, const int32_t *seq_end,
                         float *part, int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits,
                         cudaStream_t stream) {
    const size_t smem = ((size_t)2 * kRotWarps * REP + (size_t)kRotWarps * REP * D) * sizeof(float);
    auto kernel = attn_rotary_kernel<REP, DPL>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    kernel<<<grid, kRotThreads, smem, stream>>>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv,
                                                D, G, S, K, T_cap, splits);
    return launch_status();
}

template <int REP>
static int rotary_dpl(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab, const __half *vtab,
                      const __half2 *rope, const int32_t *seq_start, const int32_t *seq_end, float *part, int B, int Hq,
                      int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream) {
#define TACVQ_CASE(N) \
    case N: return launch_rotary<REP, N>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, D, G, S, K, T_cap, splits, stream);
    switch (D / 32) {
        TACVQ_CASE(2)
        TACVQ_CASE(4)
        TACVQ_CASE(8)
        default: return TACVQ_ERR_UNSUPPORTED;
    }
#undef TACVQ_CASE
}

int attn_rotary_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                         const __half *vtab, const __half2 *rope, const int32_t *seq_start, const int32_t *seq_end,
                         float *part, int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits,
                         cudaStream_t stream) {
#define TACVQ_CASE(N) \
    case N: return rotary_dpl<N>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, D, G, S, K, T_cap, splits, stream);
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
