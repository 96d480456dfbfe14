// Attention over stored codes of PRE-rotary keys: the rotary embedding is applied to every rebuilt
// key row on the fly.
//
// One block serves one (batch row, KV head, sequence split); sixteen lanes take one token and a
// lane owns D/16 neighbouring channels of it:
//     k_row  = fp16( sum_s word_s[kcode] )                       the reference's decoded fp16 window
//     k_rot  = k_row*cos + rotate_half(k_row)*sin                fp16 products and sum, each rounded,
//                                                                as apply_rotary_pos_emb does on fp16;
//                                                                channel c pairs with c +- D/2 = lane ^ 8
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

__global__ void rope_table_kernel(__half *__restrict__ table, int64_t tokens, int half_dim, const RopeFreqs freqs,
                                  int64_t first) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * half_dim) return;
    const int i = (int)(idx % half_dim);
    const int64_t t = idx / half_dim;
    const float angle = (float)(first + t) * freqs.inv[i];
    float sn, cs;
    sincosf(angle, &sn, &cs);
    table[t * 2 * half_dim + i] = __float2half_rn(cs);             // row t: the cosines ...
    table[t * 2 * half_dim + half_dim + i] = __float2half_rn(sn);  // ... then the sines
}

int rope_table_dispatch(__half *table, int64_t tokens, int D, double theta, int64_t first, cudaStream_t stream) {
    const int64_t n = tokens * (D / 2);
    if (n == 0) return TACVQ_OK;
    if (D / 2 > 128) return TACVQ_ERR_UNSUPPORTED;
    RopeFreqs freqs;
    for (int i = 0; i < 128; ++i) freqs.inv[i] = i < D / 2 ? 1.0f / powf((float)theta, (float)(2 * i) / (float)D) : 0.0f;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(table, tokens, D / 2, freqs, first);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------------
// Sixteen lanes per token: a lane owns CPL = D/16 neighbouring channels, a warp works on two tokens at a
// time and two such pairs per trip, so that the loads of one pair overlap the arithmetic of the other.
// The rotary partner of channel c (c +- D/2) lives in lane ^ 8.
// ---------------------------------------------------------------------------------------------------

template <int N>
__device__ __forceinline__ void load_halves(const __half *src, float *out) {
    if constexpr (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(src + i));
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
            const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
            out[i] = a.x, out[i + 1] = a.y, out[i + 2] = b.x, out[i + 3] = b.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = __half2float(__ldg(src + i));
    }
}

// CPL channels of one token rebuilt from its codes: fp32 sum over stages in stage order.
// WL = channels per word piece (min(CPL, d)), CPL / WL pieces; `first_group` and `offset` locate the lane.
template <int CPL, int WL>
__device__ __forceinline__ void rebuild(const uint8_t *__restrict__ code_row, const __half *__restrict__ tab, int64_t head_words,
                                        int first_group, int offset, int G, int S, int K, int d, float (&row)[CPL]) {
#pragma unroll
    for (int i = 0; i < CPL; ++i) row[i] = 0.0f;
    for (int s = 0; s < S; ++s) {
        float piece[CPL];
#pragma unroll
        for (int w = 0; w < CPL / WL; ++w) {
            const int g = first_group + w;
            const int code = code_row[s * G + g];
            load_halves<WL>(tab + ((head_words + (int64_t)s * G + g) * K + code) * d + offset, piece + w * WL);
        }
#pragma unroll
        for (int i = 0; i < CPL; ++i) row[i] = __fadd_rn(row[i], piece[i]);
    }
}

template <int REP, int CPL, int WL>
__global__ void __launch_bounds__(kRotThreads, 2)
attn_rotary_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes, const uint8_t *__restrict__ vcodes,
                   const __half *__restrict__ ktab, const __half *__restrict__ vtab, const __half *__restrict__ rope,
                   const int32_t *__restrict__ seq_start, const int32_t *__restrict__ seq_end, float *__restrict__ part,
                   int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits) {
    extern __shared__ __align__(16) float smem[];
    constexpr int kHalfWarps = 2 * kRotWarps;
    const int slots = S * G;
    const int d = D / G;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane >> 4, l16 = lane & 15;  // which of the warp's two tokens, lane within the token

    const int lo_all = seq_start ? seq_start[b] : 0;
    const int hi_all = seq_end ? seq_end[b] : (int)T_cap;
    const int n_all = hi_all > lo_all ? hi_all - lo_all : 0;
    const int per = (n_all + splits - 1) / splits;
    const int lo = lo_all + split * per;
    const int hi = min(lo + per, lo_all + n_all);

    const int c0 = l16 * CPL;              // first channel of this lane
    const int first_group = c0 / d, offset = c0 % d;
    const int f0 = c0 % (D / 2);           // its first rotary frequency
    const bool upper = c0 >= D / 2;        // rotate_half: lower half takes -partner, upper half +partner

    float qv[REP][CPL];
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int i = 0; i < CPL; ++i) qv[r][i] = __half2float(q[((int64_t)b * Hq + h * REP + r) * D + c0 + i]);

    float m[REP], l[REP], acc[REP][CPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) acc[r][i] = 0.0f;
    }
    const int64_t code_row = ((int64_t)b * Hkv + h) * T_cap;
    const int64_t head_words = (int64_t)h * S * G;

    // a trip covers 4 * kRotWarps tokens: pair u of warp w holds tokens base + u*2*kRotWarps + 2*w + sub
    for (int base = lo; base < hi; base += 4 * kRotWarps) {
        float sc[2][REP], vrow[2][CPL];
        bool live[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int t_raw = base + u * 2 * kRotWarps + 2 * warp + sub;
            live[u] = t_raw < hi;
            const int t = live[u] ? t_raw : hi - 1;  // lanes past the end redo the last token and drop it
            float krow[CPL];
            rebuild<CPL, WL>(kcodes + (code_row + t) * slots, ktab, head_words, first_group, offset, G, S, K, d, krow);
            rebuild<CPL, WL>(vcodes + (code_row + t) * slots, vtab, head_words, first_group, offset, G, S, K, d, vrow[u]);
#pragma unroll
            for (int r = 0; r < REP; ++r) sc[u][r] = 0.0f;
#pragma unroll
            for (int i = 0; i < CPL; i += 2) {
                const __half2 mine = __floats2half2_rn(krow[i], krow[i + 1]);
                const __half2 other = __shfl_xor_sync(0xffffffffu, mine, 8);
                const __half2 cosv = *reinterpret_cast<const __half2 *>(rope + (int64_t)t * D + f0 + i);
                const __half2 sinv = *reinterpret_cast<const __half2 *>(rope + (int64_t)t * D + D / 2 + f0 + i);
                const __half2 turned = upper ? other : __hneg2(other);
                const __half2 rotated = __hadd2(__hmul2(mine, cosv), __hmul2(turned, sinv));
                const float2 kf = __half22float2(rotated);
#pragma unroll
                for (int r = 0; r < REP; ++r) sc[u][r] = fmaf(qv[r][i + 1], kf.y, fmaf(qv[r][i], kf.x, sc[u][r]));
            }
#pragma unroll
            for (int r = 0; r < REP; ++r) {
#pragma unroll
                for (int off = 8; off >= 1; off >>= 1) sc[u][r] += __shfl_xor_sync(0xffffffffu, sc[u][r], off);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!live[u]) continue;
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                if (sc[u][r] > m[r]) {
                    const float scale = __expf(m[r] - sc[u][r]);  // exp(-inf) = 0 on the first token
                    l[r] *= scale;
#pragma unroll
                    for (int i = 0; i < CPL; ++i) acc[r][i] *= scale;
                    m[r] = sc[u][r];
                }
                const float p = __expf(sc[u][r] - m[r]);
                l[r] += p;
#pragma unroll
                for (int i = 0; i < CPL; ++i) acc[r][i] = fmaf(p, __half2float(__float2half_rn(vrow[u][i])), acc[r][i]);
            }
        }
    }

    // ---- merge the half-warps of this block (same layout of partial states as the generic kernel) ----
    float *wm = smem;                          // [half-warps][REP]
    float *wl = wm + kHalfWarps * REP;         // [half-warps][REP]
    float *wacc = wl + kHalfWarps * REP;       // [half-warps][REP][D]
    const int hw = warp * 2 + sub;
    if (l16 == 0) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            wm[hw * REP + r] = m[r];
            wl[hw * REP + r] = l[r];
        }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int i = 0; i < CPL; ++i) wacc[((size_t)hw * REP + r) * D + c0 + i] = acc[r][i];
    __syncthreads();
    const int64_t rows = (int64_t)B * Hq;
    for (int idx = tid; idx < REP * (D + 2); idx += kRotThreads) {
        const int r = idx / (D + 2), col = idx % (D + 2);
        float top = -INFINITY;
        for (int w = 0; w < kHalfWarps; ++w) top = fmaxf(top, wm[w * REP + r]);
        float sum = 0.0f;
        if (col == 0) {
            sum = top;
        } else {
            for (int w = 0; w < kHalfWarps; ++w) {
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

template <int REP, int CPL, int WL>
static int launch_rotary(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                         const __half *vtab, const __half *rope, const int32_t *seq_start, const int32_t *seq_end,
                         float *part, int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits,
                         cudaStream_t stream) {
    const size_t smem = ((size_t)4 * kRotWarps * REP + (size_t)2 * kRotWarps * REP * D) * sizeof(float);
    auto kernel = attn_rotary_kernel<REP, CPL, WL>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    kernel<<<grid, kRotThreads, smem, stream>>>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv,
                                                D, G, S, K, T_cap, splits);
    return launch_status();
}

// word pieces per lane: a lane's CPL channels are either inside one word (d >= CPL) or whole words (d < CPL)
template <int REP, int CPL>
static int rotary_piece(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab, const __half *vtab,
                        const __half *rope, const int32_t *seq_start, const int32_t *seq_end, float *part, int B, int Hq,
                        int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream) {
    const int d = D / G;
#define TACVQ_CASE(N) \
    return launch_rotary<REP, CPL, N>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, D, G, S, K, T_cap, splits, stream);
    if (d >= CPL) {
        if (d % CPL != 0) return TACVQ_ERR_UNSUPPORTED;
        TACVQ_CASE(CPL)
    }
    if (CPL % d != 0) return TACVQ_ERR_UNSUPPORTED;
    if constexpr (CPL >= 8) {
        if (d == 4) { TACVQ_CASE(4) }
    }
    if constexpr (CPL >= 4) {
        if (d == 2) { TACVQ_CASE(2) }
    }
    if (d == 1) { TACVQ_CASE(1) }
    if constexpr (CPL == 16) {
        if (d == 8) { TACVQ_CASE(8) }
    }
    return TACVQ_ERR_UNSUPPORTED;
#undef TACVQ_CASE
}

template <int REP>
static int rotary_dpl(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab, const __half *vtab,
                      const __half *rope, const int32_t *seq_start, const int32_t *seq_end, float *part, int B, int Hq,
                      int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream) {
#define TACVQ_CASE(N) \
    case N: return rotary_piece<REP, N>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, D, G, S, K, T_cap, splits, stream);
    switch (D / 16) {
        TACVQ_CASE(4)
        TACVQ_CASE(8)
        TACVQ_CASE(16)
        default: return TACVQ_ERR_UNSUPPORTED;
    }
#undef TACVQ_CASE
}

// ---------------------------------------------------------------------------------------------------
// head_dim 128, groups of at least 8 channels, at most 2 stages, at most 4 query heads per KV head:
// the tables of one side fit shared memory (S x 64 KB), so a block works in two passes per chunk of
// up to 4096 tokens: pass K (key tables resident) leaves the scores in shared memory, the block takes
// their maximum and turns them into weights, pass V (value tables loaded over the key tables)
// accumulates.  Tables are stored by 16-byte piece, [stage][code][piece]: the sixteen lanes of a token
// read sixteen different pieces, which is the minimum number of shared-memory wavefronts.
// ---------------------------------------------------------------------------------------------------

#ifndef TACVQ_ROT_THREADS
#define TACVQ_ROT_THREADS 1024
#endif
constexpr int kRotBigThreads = TACVQ_ROT_THREADS;
constexpr int kRotChunk = 4096;

// ROTARY = false: the same two passes without the rotary step.  The key pass then needs no key rows at
// all: the block first fills the table area with scores, lut[stage][code][piece] = q_r . (8 channels of the
// word), r < REP, and a token's score is the sum of its S x 16 entries.
// NARROW = true: one stage of 32 groups of 4 channels.  A lane's eight channels are then two whole words of
// neighbouring groups; tables and score table are stored [code][group] (8-byte words, 16-byte scores) and the
// lane's two codes take the place of the two stage codes.
template <int REP, bool ROTARY, bool NARROW>
__global__ void __launch_bounds__(kRotBigThreads, 1)
attn_rotary_staged_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes, const uint8_t *__restrict__ vcodes,
                          const __half *__restrict__ ktab, const __half *__restrict__ vtab, const __half *__restrict__ rope,
                          const int32_t *__restrict__ seq_start, const int32_t *__restrict__ seq_end, float *__restrict__ part,
                          int B, int Hq, int Hkv, int G, int S, int64_t T_cap, int splits) {
    constexpr int D = 128, K = 256, kWarps = kRotBigThreads / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4 *tab = reinterpret_cast<uint4 *>(smem_raw);                                   // [S][256][16]
    const size_t table_bytes = NARROW ? (ROTARY ? (size_t)K * 32 * 8 : (size_t)K * 32 * 16) : (size_t)S * K * 16 * 16;
    float *score = reinterpret_cast<float *>(smem_raw + table_bytes);                   // [kRotChunk][REP]
    float *red = score + (size_t)kRotChunk * REP;                                       // [kWarps][REP], later merge scratch

    const int slots = S * G;
    const int d = D / G;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane >> 4, l16 = lane & 15;
    const int c0 = l16 * 8;
    const int group = c0 / d;
    const int f0 = c0 % (D / 2);
    const bool upper = c0 >= D / 2;

    const int lo_all = seq_start ? seq_start[b] : 0;
    const int hi_all = seq_end ? seq_end[b] : (int)T_cap;
    const int n_all = hi_all > lo_all ? hi_all - lo_all : 0;
    const int per = (n_all + splits - 1) / splits;
    const int lo = lo_all + split * per;
    const int hi = min(lo + per, lo_all + n_all);

    auto load_tables = [&](const __half *src) {
        if constexpr (NARROW) {
            uint2 *tab8 = reinterpret_cast<uint2 *>(tab);  // [256][32 groups] words of 4 channels
            for (int idx = tid; idx < K * 32; idx += kRotBigThreads) {
                const int g = idx & 31, code = idx >> 5;
                tab8[idx] = __ldg(reinterpret_cast<const uint2 *>(src + (((int64_t)h * G + g) * K + code) * 4));
            }
        } else {
            for (int idx = tid; idx < S * K * 16; idx += kRotBigThreads) {
                const int p = idx & 15, code = (idx >> 4) & 255, s = idx >> 12;
                const int g = (8 * p) / d, off = (8 * p) % d;
                tab[idx] = __ldg(reinterpret_cast<const uint4 *>(src + ((((int64_t)h * S + s) * G + g) * K + code) * d + off));
            }
        }
    };
    auto build_score_table = [&]() {  // ROTARY = false only; the query rows sit at the start of the score area
        float *q_s = score;
        for (int i = tid; i < REP * D; i += kRotBigThreads)
            q_s[i] = __half2float(q[((int64_t)b * Hq + h * REP + i / D) * D + i % D]);
        __syncthreads();
        float4 *lut = reinterpret_cast<float4 *>(tab);
        if constexpr (NARROW) {
            for (int idx = tid; idx < K * 32; idx += kRotBigThreads) {
                const int g = idx & 31, code = idx >> 5;
                const uint2 w = __ldg(reinterpret_cast<const uint2 *>(ktab + (((int64_t)h * G + g) * K + code) * 4));
                const __half2 *hp = reinterpret_cast<const __half2 *>(&w);
                float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float2 f = __half22float2(hp[i]);
#pragma unroll
                    for (int r = 0; r < REP; ++r)
                        dot[r] = fmaf(q_s[r * D + 4 * g + 2 * i + 1], f.y, fmaf(q_s[r * D + 4 * g + 2 * i], f.x, dot[r]));
                }
                lut[idx] = make_float4(dot[0], dot[1], dot[2], dot[3]);
            }
            return;
        }
        // the block size is a multiple of 16, so a thread meets the same piece p on every trip: its query
        // channels are read once
        const int p = tid & 15;
        const int g = (8 * p) / d, off = (8 * p) % d;
        float qp[REP][8];
#pragma unroll
        for (int r = 0; r < REP; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) qp[r][i] = q_s[r * D + 8 * p + i];
        for (int idx = tid; idx < S * K * 16; idx += kRotBigThreads) {
            const int code = (idx >> 4) & 255, s = idx >> 12;
            const uint4 w = __ldg(reinterpret_cast<const uint4 *>(ktab + ((((int64_t)h * S + s) * G + g) * K + code) * d + off));
            const __half2 *hp = reinterpret_cast<const __half2 *>(&w);
            float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(hp[i]);
#pragma unroll
                for (int r = 0; r < REP; ++r) dot[r] = fmaf(qp[r][2 * i + 1], f.y, fmaf(qp[r][2 * i], f.x, dot[r]));
            }
            lut[idx] = make_float4(dot[0], dot[1], dot[2], dot[3]);
        }
    };
    // This lane's eight channels of a token from the resident tables, as the fp16 row the reference
    // keeps: with at most two stages the fp32 sum of two fp16 words is exact, so its single rounding to
    // fp16 is what a packed fp16 add returns.
    // (the codes of a token are fetched one trip ahead: S <= 2 bytes per lane and side)
    auto fetch_codes = [&](const uint8_t *code_row, int (&code)[2]) {
        if constexpr (NARROW) {
            code[0] = code_row[2 * l16];
            code[1] = code_row[2 * l16 + 1];
        } else {
            code[0] = code_row[group];
            code[1] = S > 1 ? code_row[G + group] : 0;
        }
    };
    auto rebuild8 = [&](const int (&code)[2], __half2 (&row)[4]) {
        if constexpr (NARROW) {
            const uint2 *tab8 = reinterpret_cast<const uint2 *>(tab);
            const uint2 low = tab8[code[0] * 32 + 2 * l16], high = tab8[code[1] * 32 + 2 * l16 + 1];
            row[0] = *reinterpret_cast<const __half2 *>(&low.x);
            row[1] = *reinterpret_cast<const __half2 *>(&low.y);
            row[2] = *reinterpret_cast<const __half2 *>(&high.x);
            row[3] = *reinterpret_cast<const __half2 *>(&high.y);
            return;
        }
        const uint4 first = tab[code[0] * 16 + l16];
        const __half2 *h0 = reinterpret_cast<const __half2 *>(&first);
#pragma unroll
        for (int i = 0; i < 4; ++i) row[i] = h0[i];
        if (S > 1) {
            const uint4 second = tab[(K + code[1]) * 16 + l16];
            const __half2 *h1 = reinterpret_cast<const __half2 *>(&second);
#pragma unroll
            for (int i = 0; i < 4; ++i) row[i] = __hadd2(row[i], h1[i]);
        }
    };

    float qv[REP][8];
    if constexpr (ROTARY) {
#pragma unroll
        for (int r = 0; r < REP; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[r][i] = __half2float(q[((int64_t)b * Hq + h * REP + r) * D + c0 + i]);
    }
    float m[REP], l[REP], acc[REP][8];  // the sums are only live in the value pass: registers for the key pass
#pragma unroll
    for (int r = 0; r < REP; ++r) m[r] = -INFINITY;
    const int64_t code_row = ((int64_t)b * Hkv + h) * T_cap;
    const int chunk = lo;
    const int n = hi - lo;  // at most kRotChunk: the launcher picks the split count for that

    if (n > 0) {
        if constexpr (ROTARY) load_tables(ktab);
        else build_score_table();
        __syncthreads();
        // ---- pass K: scores of the chunk ------------------------------------------------------------
        int code_next[2];
        uint4 cos_next = make_uint4(0u, 0u, 0u, 0u), sin_next = cos_next;  // eight cosines and sines of this lane's frequencies
        {
            const int t = chunk + min(2 * warp + sub, n - 1);
            fetch_codes(kcodes + (code_row + t) * slots, code_next);
            if constexpr (ROTARY) {
                cos_next = __ldg(reinterpret_cast<const uint4 *>(rope + (int64_t)t * D + f0));
                sin_next = __ldg(reinterpret_cast<const uint4 *>(rope + (int64_t)t * D + D / 2 + f0));
            }
        }
        for (int base = 0; base < n; base += 2 * kWarps) {
            const int local = base + 2 * warp + sub;  // lanes past the end redo the last token and drop it
            const int code_now[2] = {code_next[0], code_next[1]};
            const uint4 cos_now = cos_next, sin_now = sin_next;
            if (base + 2 * kWarps < n) {
                const int t = chunk + min(local + 2 * kWarps, n - 1);
                fetch_codes(kcodes + (code_row + t) * slots, code_next);
                if constexpr (ROTARY) {
                    cos_next = __ldg(reinterpret_cast<const uint4 *>(rope + (int64_t)t * D + f0));
                    sin_next = __ldg(reinterpret_cast<const uint4 *>(rope + (int64_t)t * D + D / 2 + f0));
                }
            }
            float sc[REP];
            if constexpr (ROTARY) {
                __half2 krow[4];
                rebuild8(code_now, krow);
                const __half2 *cosv = reinterpret_cast<const __half2 *>(&cos_now), *sinv = reinterpret_cast<const __half2 *>(&sin_now);
#pragma unroll
                for (int r = 0; r < REP; ++r) sc[r] = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half2 other = __shfl_xor_sync(0xffffffffu, krow[i], 8);
                    const __half2 turned = upper ? other : __hneg2(other);
                    const float2 kf = __half22float2(__hadd2(__hmul2(krow[i], cosv[i]), __hmul2(turned, sinv[i])));
#pragma unroll
                    for (int r = 0; r < REP; ++r) sc[r] = fmaf(qv[r][2 * i + 1], kf.y, fmaf(qv[r][2 * i], kf.x, sc[r]));
                }
            } else {
                const float4 *lut = reinterpret_cast<const float4 *>(tab);
                float4 e;
                if constexpr (NARROW) {
                    e = lut[code_now[0] * 32 + 2 * l16];
                    const float4 e1 = lut[code_now[1] * 32 + 2 * l16 + 1];
                    e = make_float4(e.x + e1.x, e.y + e1.y, e.z + e1.z, e.w + e1.w);
                } else {
                    e = lut[code_now[0] * 16 + l16];
                    if (S > 1) {
                        const float4 e1 = lut[(K + code_now[1]) * 16 + l16];
                        e = make_float4(e.x + e1.x, e.y + e1.y, e.z + e1.z, e.w + e1.w);
                    }
                }
                const float ev[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
                for (int r = 0; r < REP; ++r) sc[r] = ev[r];
            }
            // sum over the token's 16 lanes; with 4 or 2 heads the lanes first trade heads, so that fewer
            // values travel: head (bit 3, bit 2) of the lane index ends up in the lanes with those bits
            if constexpr (REP == 4) {
                const bool b3 = (l16 & 8) != 0, b2 = (l16 & 4) != 0;
                float keep0 = b3 ? sc[2] : sc[0], keep1 = b3 ? sc[3] : sc[1];
                keep0 += __shfl_xor_sync(0xffffffffu, b3 ? sc[0] : sc[2], 8);
                keep1 += __shfl_xor_sync(0xffffffffu, b3 ? sc[1] : sc[3], 8);
                float one = (b2 ? keep1 : keep0) + __shfl_xor_sync(0xffffffffu, b2 ? keep0 : keep1, 4);
                one += __shfl_xor_sync(0xffffffffu, one, 2);
                one += __shfl_xor_sync(0xffffffffu, one, 1);
                if ((l16 & 3) == 0 && local < n) score[local * REP + (b3 ? 2 : 0) + (b2 ? 1 : 0)] = one;
            } else if constexpr (REP == 2) {
                const bool b3 = (l16 & 8) != 0;
                float one = (b3 ? sc[1] : sc[0]) + __shfl_xor_sync(0xffffffffu, b3 ? sc[0] : sc[1], 8);
                one += __shfl_xor_sync(0xffffffffu, one, 4);
                one += __shfl_xor_sync(0xffffffffu, one, 2);
                one += __shfl_xor_sync(0xffffffffu, one, 1);
                if ((l16 & 7) == 0 && local < n) score[local * REP + (b3 ? 1 : 0)] = one;
            } else {
                float one = sc[0];
#pragma unroll
                for (int off = 8; off >= 1; off >>= 1) one += __shfl_xor_sync(0xffffffffu, one, off);
                if (l16 == 0 && local < n) score[local * REP] = one;
            }
        }
        __syncthreads();
        // ---- chunk maximum, rescale of the running sums, weights -------------------------------------
        float top[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) top[r] = -INFINITY;
        for (int i = tid; i < n; i += kRotBigThreads) {
#pragma unroll
            for (int r = 0; r < REP; ++r) top[r] = fmaxf(top[r], score[i * REP + r]);
        }
#pragma unroll
        for (int r = 0; r < REP; ++r) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], off));
            if (lane == 0) red[warp * REP + r] = top[r];
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            for (int w = 0; w < kWarps; ++w) m[r] = fmaxf(m[r], red[w * REP + r]);
        }
        for (int i = tid; i < n; i += kRotBigThreads) {
#pragma unroll
            for (int r = 0; r < REP; ++r) score[i * REP + r] = __expf(score[i * REP + r] - m[r]);
        }
        load_tables(vtab);  // the key tables are no longer read: every warp passed the barrier above
        __syncthreads();
        // ---- pass V --------------------------------------------------------------------------------
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            l[r] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r][i] = 0.0f;
        }
        fetch_codes(vcodes + (code_row + chunk + min(2 * warp + sub, n - 1)) * slots, code_next);
        for (int base = 0; base < n; base += 2 * kWarps) {
            const int local = base + 2 * warp + sub;
            const int code_now[2] = {code_next[0], code_next[1]};
            if (base + 2 * kWarps < n) fetch_codes(vcodes + (code_row + chunk + min(local + 2 * kWarps, n - 1)) * slots, code_next);
            if (local >= n) continue;  // no shuffles in this pass
            __half2 vhalf[4];
            rebuild8(code_now, vhalf);
            float vrow[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(vhalf[i]);
                vrow[2 * i] = f.x, vrow[2 * i + 1] = f.y;
            }
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                const float p = score[local * REP + r];
                l[r] += p;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(p, vrow[i], acc[r][i]);
            }
        }
    }

    if (n <= 0) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            l[r] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r][i] = 0.0f;
        }
    }
    // ---- sum the half-warps (they share m), write this split's partial state ------------------------
    __syncthreads();
    float *wl = reinterpret_cast<float *>(smem_raw);       // [2*kWarps][REP]
    float *wacc = wl + 2 * kWarps * REP;                   // [2*kWarps][REP][D]
    const int hw = warp * 2 + sub;
    if (l16 == 0) {
#pragma unroll
        for (int r = 0; r < REP; ++r) wl[hw * REP + r] = l[r];
    }
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) wacc[((size_t)hw * REP + r) * D + c0 + i] = acc[r][i];
    __syncthreads();
    const int64_t rows = (int64_t)B * Hq;
    for (int idx = tid; idx < REP * (D + 2); idx += kRotBigThreads) {
        const int r = idx / (D + 2), col = idx % (D + 2);
        float sum = 0.0f;
        if (col == 0) {
            sum = m[r];
        } else {
            for (int w = 0; w < 2 * kWarps; ++w) sum += (col == 1 ? wl[w * REP + r] : wacc[((size_t)w * REP + r) * D + (col - 2)]);
        }
        const int64_t row = (int64_t)b * Hq + h * REP + r;
        part[((int64_t)split * rows + row) * (D + 2) + col] = sum;
    }
}

bool attn_rotary_staged_supported(int Hq, int Hkv, int D, int G, int S, int K) {
    const int rep = Hq / Hkv;
    const bool pieces = (D / G) >= 8 && S <= 2;   // a lane's eight channels lie inside one word
    const bool narrow = (D / G) == 4 && S == 1;   // ... or are two whole words
    return D == 128 && K == 256 && (pieces || narrow) && (rep == 1 || rep == 2 || rep == 4);
}

template <int REP>
static int launch_rotary_staged(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                                const __half *vtab, const __half *rope, const int32_t *seq_start, const int32_t *seq_end,
                                float *part, int B, int Hq, int Hkv, int G, int S, int64_t T_cap, int splits,
                                cudaStream_t stream) {
    const bool narrow = G == 32;
    const size_t tables = narrow ? (rope != nullptr ? (size_t)256 * 32 * 8 : (size_t)256 * 32 * 16) : (size_t)S * 256 * 16 * 16;
    const size_t merge = ((size_t)(kRotBigThreads / 16) * REP + (size_t)(kRotBigThreads / 16) * REP * 128) * sizeof(float);
    size_t smem = tables + ((size_t)kRotChunk * REP + (size_t)(kRotBigThreads / 32) * REP) * sizeof(float);
    if (smem < merge) smem = merge;
    auto kernel = narrow ? (rope != nullptr ? attn_rotary_staged_kernel<REP, true, true> : attn_rotary_staged_kernel<REP, false, true>)
                         : (rope != nullptr ? attn_rotary_staged_kernel<REP, true, false> : attn_rotary_staged_kernel<REP, false, false>);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    kernel<<<grid, kRotBigThreads, smem, stream>>>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, G,
                                                   S, T_cap, splits);
    return launch_status();
}

// attn_rotary_mma.cu: the same block decomposition with both contractions on the tensor cores
bool attn_rotary_mma_supported(int Hq, int Hkv, int D, int G, int S, int K);
int attn_rotary_mma_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab, const __half *vtab,
                             const __half *rope, const int32_t *seq_start, const int32_t *seq_end, float *part, int B, int Hq,
                             int Hkv, int64_t T_cap, int splits, cudaStream_t stream);

int attn_rotary_staged_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                                const __half *vtab, const __half *rope, const int32_t *seq_start, const int32_t *seq_end,
                                float *part, int B, int Hq, int Hkv, int G, int S, int64_t T_cap, int splits,
                                cudaStream_t stream) {
#ifndef TACVQ_ROTARY_SCALAR
    if (rope != nullptr && attn_rotary_mma_supported(Hq, Hkv, 128, G, S, 256) && (((uintptr_t)kcodes | (uintptr_t)vcodes | (uintptr_t)q) & 15) == 0)
        return attn_rotary_mma_dispatch(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, T_cap, splits, stream);
#endif
    switch (Hq / Hkv) {
        case 1: return launch_rotary_staged<1>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, G, S, T_cap, splits, stream);
        case 2: return launch_rotary_staged<2>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, G, S, T_cap, splits, stream);
        case 4: return launch_rotary_staged<4>(q, kcodes, vcodes, ktab, vtab, rope, seq_start, seq_end, part, B, Hq, Hkv, G, S, T_cap, splits, stream);
        default: return TACVQ_ERR_UNSUPPORTED;
    }
}

// One block per SM.  Among the split counts that leave at least 512 tokens per block, take the one whose
// last wave is fullest (ties: fewer splits), looking at two to five waves.
int attn_rotary_staged_splits(int B, int Hkv, int64_t T_cap, int sms) {
    const int pairs = B * Hkv;
    int64_t most = (T_cap + 511) / 512;
    if (most > 64) most = 64;
    if (most < 1) most = 1;
    const int least = (int)((T_cap + kRotChunk - 1) / kRotChunk);  // a block holds at most kRotChunk scores
    if (least > 64) return 0;                                      // too long for this kernel
    if (most < least) most = least;
    int best = least > 1 ? least : 1;
    double best_fill = 0.0;
    for (int splits = best; splits <= (int)most; ++splits) {
        const int64_t blocks = (int64_t)pairs * splits;
        const int64_t waves = (blocks + sms - 1) / sms;
        if (waves > 5 && best_fill > 0.0) break;
        double fill = (double)blocks / (double)(waves * sms);
        if (waves < 2) fill *= 0.9;  // a single wave cannot even out unequal rows
        if (fill > best_fill + 1e-9) best_fill = fill, best = splits;
    }
    return best;
}

// About four waves of blocks (two resident per SM), at least 256 tokens per block, at most 64 splits.
int attn_rotary_splits(int B, int Hkv, int64_t T_cap, int sms) {
    const int pairs = B * Hkv;
    int splits = (8 * sms + pairs - 1) / pairs;
    const int64_t by_len = (T_cap + 255) / 256;
    if (splits > by_len) splits = (int)by_len;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    return splits;
}

int attn_rotary_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                         const __half *vtab, const __half *rope, const int32_t *seq_start, const int32_t *seq_end,
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
