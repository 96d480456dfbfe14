// Decode-step attention over codes for full-width codebooks: G = 1 group, d = D = 128, S <= 16 stages,
// 4 query heads per KV head.  This is the reference's own residual-VQ layout (tables [H,S,256,128]) and
// the "two additive 256x128 codebooks" configuration; a token and head is only S bytes per side.
//
// With so few codes per token the value side is cheapest as a weighted histogram: instead of fetching
// S x 256 bytes of codewords per token, add the token's softmax weight to hist[stage][head][code]
// (S x 4 shared-memory atomic adds; the weights are added as 18-bit fixed point because integer adds
// are native shared-memory atomics and float adds are compare-and-swap loops) and multiply the
// histogram by the V codebook once per block:
//     acc[h][:] = sum_{s,c} hist[s][c][h] * vtab[s][c][:].
// Scores are S look-ups of a 16-byte entry (4 heads, fp32).  The per-block work that does not depend on
// the number of tokens is what bounds this kernel at decode sizes (a block reads S x 64 KB of K tables
// for its score table and S x 64 KB of V tables for the product), so:
//   - one block takes a whole (batch row, KV head) pair whenever the pairs alone fill most of the SMs,
//     and then writes the result itself (no partial states, no merge launch);
//   - the score table is built with one thread per codeword (eight 16-byte loads in flight, q read
//     as shared-memory broadcasts) instead of a warp per codeword with shuffle reductions;
//   - codes are read straight from global memory with the widest load the stage count allows, the K
//     codes twice (exact maximum first, then weights): the second read hits L2.
// Partial states (several blocks per pair) go to the [split][row][2+D] layout the generic kernel uses and
// are merged by attn_combine_kernel.
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122 (no rotary
// step).  Differences from the dense path inside the 2e-3 tolerance: the V row is the exact sum of its
// stage codewords (the reference rounds that sum to fp16 once), a score is the sum of per-stage dot
// products (the reference rounds the rebuilt key to fp16 first).

#include "common.cuh"

namespace tacvq {
namespace fullwidth {

constexpr int kThreads = 512;   // (1024 threads were measured: 14 % slower)
constexpr int kWarps = kThreads / 32;
constexpr int kDim = 128, kRep = 4, kWords = 256;
constexpr int kMaxStages = 16;
constexpr int kSegmentTokens = 8192;        // 8192 weights of at most 2^18 fit the 32-bit fixed-point bins: after that many
                                           // tokens a block folds the bins into a float histogram and clears them
constexpr float kWeightOne = 262144.0f;     // fixed-point one (2^18); the largest weight of a range is exactly 1
constexpr int kSlices = kThreads / 16;      // word slices of the histogram-times-codebook product

// S code bytes of one token as WORDS 32-bit words.  WIDE = S when one aligned load fetches them (2, 4, 8, 16),
// 0 for any other stage count (byte loads).
template <int WORDS, int WIDE>
__device__ __forceinline__ void load_codes(const uint8_t *__restrict__ p, int S, uint32_t (&w)[WORDS]) {
    if constexpr (WIDE == 2) {
        w[0] = *reinterpret_cast<const unsigned short *>(p);
    } else if constexpr (WIDE == 4) {
        w[0] = *reinterpret_cast<const uint32_t *>(p);
    } else if constexpr (WIDE == 8) {
        const uint2 v = *reinterpret_cast<const uint2 *>(p);
        w[0] = v.x; w[1] = v.y;
    } else if constexpr (WIDE == 16) {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else {
#pragma unroll
        for (int i = 0; i < WORDS; ++i) {
            w[i] = 0u;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (4 * i + j < S) w[i] |= (uint32_t)p[4 * i + j] << (8 * j);
        }
    }
}
// the next code byte of a token: the words are consumed as one shift register (no indexed access)
template <int WORDS>
__device__ __forceinline__ int next_code(uint32_t (&w)[WORDS]) {
    const int code = w[0] & 255;
#pragma unroll
    for (int i = 0; i + 1 < WORDS; ++i) w[i] = __funnelshift_r(w[i], w[i + 1], 8);
    w[WORDS - 1] >>= 8;
    return code;
}

template <int WORDS, int WIDE>
__global__ void __launch_bounds__(kThreads)
attn_fullwidth_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes,
                      const uint8_t *__restrict__ vcodes, const __half *__restrict__ ktab,
                      const __half *__restrict__ vtab, const int32_t *__restrict__ seq_start,
                      const int32_t *__restrict__ seq_end, float *__restrict__ part, __half *__restrict__ out,
                      float *__restrict__ state_out, int B, int Hkv, int S, int64_t T_cap, int splits) {
    extern __shared__ __align__(16) float smem[];
    float4 *lut = reinterpret_cast<float4 *>(smem);            // [S][256] : 4 heads
    float *hist = smem + (size_t)S * kWords * 4;                // [S][4][256] (fixed-point counts of the current segment)
    float *hist_f = hist + (size_t)S * kWords * 4;              // [S][4][256] (weights of the finished segments)
    const size_t both = max((size_t)3 * S * kWords * 4, (size_t)kWarps * kRep * kDim);  // floats
    float *q_s = smem + both;                                   // [128][4]: channel-major, one 16-byte read gives 4 heads
    float *red = q_s + kRep * kDim;                             // [warps][8] : max x4, sum x4
    __shared__ float m_s[kRep];

    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = Hkv * kRep;

    for (int i = tid; i < kRep * kDim; i += kThreads)
        q_s[(i & 127) * kRep + (i >> 7)] = __half2float(q[((size_t)b * Hq + h * kRep + (i >> 7)) * kDim + (i & 127)]);
    unsigned int *hist_u = reinterpret_cast<unsigned int *>(hist);
    for (int i = tid; i < S * kWords * 4; i += kThreads) {
        hist_u[i] = 0u;
        hist_f[i] = 0.0f;
    }
    __syncthreads();

    // ---- score table: one thread per codeword; its 256 bytes travel as 2 x 8 16-byte loads, the query
    //      comes from shared memory (every thread reads the same address: a broadcast) -----------------------
    for (int w0 = tid; w0 < S * kWords; w0 += kThreads) {
        const uint4 *row = reinterpret_cast<const uint4 *>(ktab + ((size_t)h * S * kWords + w0) * kDim);
        float dot[kRep] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
        uint4 raw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) raw[i] = __ldg(row + half * 8 + i);
#pragma unroll
        for (int i = 0; i < 8; ++i) {  // (unrolled: raw[] must stay in registers)
            const __half2 *hp = reinterpret_cast<const __half2 *>(&raw[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 c = __half22float2(hp[j]);
                const float4 qa = *reinterpret_cast<const float4 *>(q_s + (64 * half + 8 * i + 2 * j) * kRep);
                const float4 qb = *reinterpret_cast<const float4 *>(q_s + (64 * half + 8 * i + 2 * j + 1) * kRep);
                dot[0] = fmaf(qa.x, c.x, dot[0]); dot[1] = fmaf(qa.y, c.x, dot[1]);
                dot[2] = fmaf(qa.z, c.x, dot[2]); dot[3] = fmaf(qa.w, c.x, dot[3]);
                dot[0] = fmaf(qb.x, c.y, dot[0]); dot[1] = fmaf(qb.y, c.y, dot[1]);
                dot[2] = fmaf(qb.z, c.y, dot[2]); dot[3] = fmaf(qb.w, c.y, dot[3]);
            }
        }
        }
        lut[w0] = make_float4(dot[0], dot[1], dot[2], dot[3]);
    }
    __syncthreads();

    // ---- token range of this split ------------------------------------------------------------------
    const int lo_all = max(seq_start ? seq_start[b] : 0, 0);
    const int hi_all = min(seq_end ? seq_end[b] : (int)T_cap, (int)T_cap);
    const int n_all = hi_all > lo_all ? hi_all - lo_all : 0;
    const int per = (n_all + splits - 1) / splits;
    const int lo = lo_all + split * per;
    const int hi = min(lo + per, lo_all + n_all);
    const size_t row_base = ((size_t)b * Hkv + h) * (size_t)T_cap;

    constexpr int kBatch = WORDS == 1 ? 4 : WORDS == 2 ? 2 : 1;  // tokens whose code loads a thread keeps in flight together (the loop body stays small:
                               // a larger, fully unrolled body was measured to stall on instruction fetch)
    auto score = [&](uint32_t (&kc)[WORDS], float (&sc)[kRep]) {  // consumes kc
#pragma unroll
        for (int r = 0; r < kRep; ++r) sc[r] = 0.0f;
        for (int s = 0; s < S; ++s) {
            const float4 e = lut[s * kWords + next_code(kc)];
            sc[0] += e.x; sc[1] += e.y; sc[2] += e.z; sc[3] += e.w;
        }
    };

    // ---- pass 1: exact maximum of every head over the range ------------------------------------------
    float mx[kRep] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int t0 = lo + tid; t0 < hi; t0 += kBatch * kThreads) {
        uint32_t kc[kBatch][WORDS];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {  // the loads of a batch travel together; tokens past the end repeat the last one
            const int t = min(t0 + j * kThreads, hi - 1);
            load_codes<WORDS, WIDE>(kcodes + (row_base + t) * S, S, kc[j]);
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            float sc[kRep];
            score(kc[j], sc);
#pragma unroll
            for (int r = 0; r < kRep; ++r) mx[r] = fmaxf(mx[r], sc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], off));
        if (lane == 0) red[warp * 8 + r] = mx[r];
    }
    __syncthreads();
    if (tid < kRep) {
        float m = -INFINITY;
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, red[w * 8 + tid]);
        m_s[tid] = m;
    }
    __syncthreads();
    float m[kRep];
#pragma unroll
    for (int r = 0; r < kRep; ++r) m[r] = m_s[r];

    // ---- pass 2: softmax weights into the per-stage code histograms ------------------------------------
    unsigned int lsum_u[kRep] = {0u, 0u, 0u, 0u};  // per segment: at most 16 tokens of weight <= 2^18 per thread
    auto add_weights = [&](const float (&sc)[kRep], uint32_t (&vc)[WORDS]) {  // consumes vc
        unsigned int p[kRep];
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            p[r] = __float2uint_rn(__expf(sc[r] - m[r]) * kWeightOne);
            lsum_u[r] += p[r];
        }
        for (int s = 0; s < S; ++s) {
            unsigned int *bin = hist_u + (size_t)s * kRep * kWords + next_code(vc);  // [stage][head][code]: bank = code % 32
#pragma unroll
            for (int r = 0; r < kRep; ++r) atomicAdd(bin + r * kWords, p[r]);
        }
    };
    float lsum_f[kRep] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int seg = lo; seg < hi; seg += kSegmentTokens) {
        const int seg_hi = min(seg + kSegmentTokens, hi);
        for (int t0 = seg + tid; t0 < seg_hi; t0 += kBatch * kThreads) {
            uint32_t kc[kBatch][WORDS], vc[kBatch][WORDS];
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const int t = min(t0 + j * kThreads, seg_hi - 1);
                load_codes<WORDS, WIDE>(kcodes + (row_base + t) * S, S, kc[j]);
                load_codes<WORDS, WIDE>(vcodes + (row_base + t) * S, S, vc[j]);
            }
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                if (t0 + j * kThreads >= seg_hi) break;
                float sc[kRep];
                score(kc[j], sc);
                add_weights(sc, vc[j]);
            }
        }
        __syncthreads();  // the segment's weights are all in the bins: fold them into the float histogram
        for (int i = tid; i < S * kWords * 4; i += kThreads) {
            hist_f[i] += (float)hist_u[i] * (1.0f / kWeightOne);
            hist_u[i] = 0u;
        }
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            lsum_f[r] += (float)lsum_u[r] * (1.0f / kWeightOne);
            lsum_u[r] = 0u;
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
        float lsum = lsum_f[r];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
        if (lane == 0) red[warp * 8 + 4 + r] = lsum;
    }
    __syncthreads();

    // ---- acc = hist x V codebook: thread = (8-channel chunk, one of 32 slices of the code words) -------
    const int chunk = tid & 15, slice = tid >> 4;
    float acc[kRep][8];
#pragma unroll
    for (int r = 0; r < kRep; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = 0.0f;
    const int words = S * kWords;
    const uint4 *vt = reinterpret_cast<const uint4 *>(vtab + (size_t)h * words * kDim) + chunk;
#pragma unroll 4
    for (int w = slice; w < words; w += kSlices) {
        const float *cnt = hist_f + (size_t)(w >> 8) * kRep * kWords + (w & 255);
        const float4 wgt = make_float4(cnt[0], cnt[kWords], cnt[2 * kWords], cnt[3 * kWords]);
        const uint4 raw = __ldg(vt + (size_t)w * (kDim / 8));
        const __half2 *hp = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(hp[i]);
            acc[0][2 * i] = fmaf(wgt.x, v.x, acc[0][2 * i]); acc[0][2 * i + 1] = fmaf(wgt.x, v.y, acc[0][2 * i + 1]);
            acc[1][2 * i] = fmaf(wgt.y, v.x, acc[1][2 * i]); acc[1][2 * i + 1] = fmaf(wgt.y, v.y, acc[1][2 * i + 1]);
            acc[2][2 * i] = fmaf(wgt.z, v.x, acc[2][2 * i]); acc[2][2 * i + 1] = fmaf(wgt.z, v.y, acc[2][2 * i + 1]);
            acc[3][2 * i] = fmaf(wgt.w, v.x, acc[3][2 * i]); acc[3][2 * i + 1] = fmaf(wgt.w, v.y, acc[3][2 * i + 1]);
        }
    }
    // fold the slices: the two slices of a warp by shuffle, the warps through shared memory
#pragma unroll
    for (int r = 0; r < kRep; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] += __shfl_xor_sync(0xffffffffu, acc[r][i], 16);
    __syncthreads();  // histograms fully read: their storage and the score table's are free
    float *fold = smem;  // [warps][4][128]  (the launcher sizes the table area for this)
    if (lane < 16) {
#pragma unroll
        for (int r = 0; r < kRep; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) fold[(warp * kRep + r) * kDim + chunk * 8 + i] = acc[r][i];
    }
    __syncthreads();
    const int64_t rows = (int64_t)B * Hq;
    for (int o = tid; o < kRep * kDim; o += kThreads) {
        const int r = o >> 7, dim = o & 127;
        float lsum = 0.0f, asum = 0.0f;
        for (int w = 0; w < kWarps; ++w) {
            lsum += red[w * 8 + 4 + r];
            asum += fold[(w * kRep + r) * kDim + dim];
        }
        const int64_t row = (int64_t)b * Hq + h * kRep + r;
        if (splits == 1) {  // the whole pair was handled here: this is the result
            if (out) out[row * kDim + dim] = __float2half_rn(lsum > 0.0f ? asum / lsum : 0.0f);
            if (state_out) {
                float *dst = state_out + row * (kDim + 2);
                if (dim == 0) {
                    dst[0] = m[r];  // -inf for an empty range
                    dst[1] = lsum;
                }
                dst[2 + dim] = asum;
            }
        } else {
            float *dst = part + ((int64_t)split * rows + row) * (kDim + 2);
            if (dim == 0) {
                dst[0] = m[r];
                dst[1] = lsum;
            }
            dst[2 + dim] = asum;
        }
    }
}

}  // namespace fullwidth

bool attn_fullwidth_supported(int Hq, int Hkv, int D, int G, int S, int K) {
    return D == fullwidth::kDim && G == 1 && S >= 1 && S <= fullwidth::kMaxStages && K == fullwidth::kWords &&
           Hq == Hkv * fullwidth::kRep;
}

// Blocks per (batch row, KV head) pair.  Every block pays the table work (2 x S x 64 KB), so a pair is split
// only as far as idle SMs make it worthwhile.
int attn_fullwidth_splits(int B, int Hkv, int64_t T_cap, int sms) {
    const int64_t pairs = (int64_t)B * Hkv;
    int64_t splits = pairs > 0 ? sms / pairs : 1;  // 1 as soon as the pairs fill more than half of the SMs
    if (splits * 1024 > T_cap) splits = (T_cap + 1023) / 1024;
    if (splits < 1) splits = 1;
    return (int)splits;
}

int attn_fullwidth_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                            const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part,
                            __half *out, float *state_out, int B, int Hq, int Hkv, int S, int64_t T_cap, int splits,
                            cudaStream_t stream) {
    (void)Hq;
    size_t both = (size_t)3 * S * fullwidth::kWords * 4 * sizeof(float);  // score table + two histograms ...
    const size_t fold = (size_t)fullwidth::kWarps * fullwidth::kRep * fullwidth::kDim * sizeof(float);  // ... later the fold area
    if (both < fold) both = fold;
    const size_t smem = both + (fullwidth::kRep * fullwidth::kDim + fullwidth::kWarps * 8) * sizeof(float);
    auto kernel = S == 2 ? fullwidth::attn_fullwidth_kernel<1, 2> : S == 4 ? fullwidth::attn_fullwidth_kernel<1, 4>
                : S == 8 ? fullwidth::attn_fullwidth_kernel<2, 8> : S == 16 ? fullwidth::attn_fullwidth_kernel<4, 16>
                : S < 4 ? fullwidth::attn_fullwidth_kernel<1, 0> : S < 8 ? fullwidth::attn_fullwidth_kernel<2, 0>
                        : fullwidth::attn_fullwidth_kernel<4, 0>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    kernel<<<grid, fullwidth::kThreads, smem, stream>>>(q, kcodes, vcodes, ktab, vtab, seq_start, seq_end, part, out, state_out,
                                                       B, Hkv, S, T_cap, splits);
    return launch_status();
}

}  // namespace tacvq
