// Decode-step attention over codes for full-width codebooks: G = 1 group, d = D = 128, S <= 16 stages,
// 4 query heads per KV head.  This is the reference's own residual-VQ layout (tables [H,S,256,128]) and
// the "two additive 256x128 codebooks" configuration; a token and head is only S bytes per side.
//
// With so few codes per token the value side is cheapest as a weighted histogram: instead of fetching
// S x 256 bytes of codewords per token, add the token's softmax weight to hist[stage][code][head]
// (S x 4 shared-memory atomic adds; the weights are added as 18-bit fixed point because integer adds
// are native shared-memory atomics and float adds are compare-and-swap loops) and multiply the
// histogram by the V codebook once per block:
//     acc[h][:] = sum_{s,c} hist[s][c][h] * vtab[s][c][:].
// Scores are S look-ups of a 16-byte entry (4 heads, fp32).  The softmax reference of a block is the
// exact maximum of its token range, found by a first pass over the K codes (2 x S bytes per token are
// read twice; the alternative, rescaling a block-wide histogram on the fly, needs block-wide barriers).
// Partial states go to the same [split][row][2+D] layout the generic kernel uses and are merged by
// attn_combine_kernel.
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122 (no rotary
// step).  Differences from the dense path inside the 2e-3 tolerance: the V row is the exact sum of its
// stage codewords (the reference rounds that sum to fp16 once), a score is the sum of per-stage dot
// products (the reference rounds the rebuilt key to fp16 first).

#include "common.cuh"

namespace tacvq {
namespace fullwidth {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kDim = 128, kRep = 4, kWords = 256;
constexpr int kMaxStages = 16;
constexpr int kStageBytes = 16384;           // code bytes of one side staged in shared memory at a time
[[maybe_unused]] constexpr int kSplitTokens = 8192;          // a block's range: 8192 weights of at most 2^18 fit 32 bits
constexpr float kWeightOne = 262144.0f;     // fixed-point one (2^18); the largest weight of a range is exactly 1

__global__ void __launch_bounds__(kThreads)
attn_fullwidth_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes,
                      const uint8_t *__restrict__ vcodes, const __half *__restrict__ ktab,
                      const __half *__restrict__ vtab, const int32_t *__restrict__ seq_start,
                      const int32_t *__restrict__ seq_end, float *__restrict__ part, int B, int Hkv, int S,
                      int64_t T_cap, int splits) {
    extern __shared__ __align__(16) float smem[];
    float4 *lut = reinterpret_cast<float4 *>(smem);            // [S][256] : 4 heads
    float *hist = smem + (size_t)S * kWords * 4;                // [S][4][256] (fixed-point counts)
    const size_t both = max((size_t)2 * S * kWords * 4, (size_t)kWarps * kRep * kDim);
    float *q_s = smem + both;                                   // [4][128]
    float *red = q_s + kRep * kDim;                             // [warps][8] : max x4, sum x4
    unsigned char *kstage = reinterpret_cast<unsigned char *>(red + kWarps * 8);  // staged K codes (+32 B slack)
    unsigned char *vstage = kstage + kStageBytes + 32;                            // staged V codes
    __shared__ float m_s[kRep];

    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = Hkv * kRep;

    for (int i = tid; i < kRep * kDim; i += kThreads)
        q_s[i] = __half2float(q[((size_t)b * Hq + h * kRep + (i >> 7)) * kDim + (i & 127)]);
    unsigned int *hist_u = reinterpret_cast<unsigned int *>(hist);
    for (int i = tid; i < S * kWords * 4; i += kThreads) hist_u[i] = 0u;
    __syncthreads();

    // ---- score table: a warp takes 8 codewords at a time (their loads travel together), lanes split
    //      the 128 channels, partial dots are folded with shuffles ----------------------------------------
    {
        float qa[kRep][4];  // this lane's query channels 2l, 2l+1, 64+2l, 64+2l+1 of every head
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            qa[r][0] = q_s[r * kDim + 2 * lane];
            qa[r][1] = q_s[r * kDim + 2 * lane + 1];
            qa[r][2] = q_s[r * kDim + 64 + 2 * lane];
            qa[r][3] = q_s[r * kDim + 64 + 2 * lane + 1];
        }
        const __half2 *tab = reinterpret_cast<const __half2 *>(ktab + (size_t)h * S * kWords * kDim);
        for (int w0 = warp * 8; w0 < S * kWords; w0 += kWarps * 8) {
            __half2 lo2[8], hi2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                lo2[j] = tab[(size_t)(w0 + j) * (kDim / 2) + lane];
                hi2[j] = tab[(size_t)(w0 + j) * (kDim / 2) + lane + 32];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 a = __half22float2(lo2[j]), c = __half22float2(hi2[j]);
                float dot[kRep];
#pragma unroll
                for (int r = 0; r < kRep; ++r) {
                    dot[r] = fmaf(qa[r][0], a.x, fmaf(qa[r][1], a.y, fmaf(qa[r][2], c.x, qa[r][3] * c.y)));
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], off);
                }
                if (lane == 0) lut[w0 + j] = make_float4(dot[0], dot[1], dot[2], dot[3]);
            }
        }
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

    // Codes reach the lanes through shared memory: a chunk of the range is copied with coalesced 16-byte
    // asynchronous copies (all in flight at once), then read byte-wise.  [begin, end) are byte offsets
    // into the code array; the copy starts at the 16-byte boundary below `begin`.
    const size_t total_bytes = (size_t)B * Hkv * (size_t)T_cap * S;
    auto stage = [&](unsigned char *dst, const uint8_t *src, size_t begin, size_t end) -> int {
        const size_t a0 = begin & ~(size_t)15;
        const int units = (int)((end - a0 + 15) >> 4);
        for (int u = tid; u < units; u += kThreads) {
            const size_t off = a0 + (size_t)u * 16;
            if (off + 16 <= total_bytes) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + u * 16)), "l"(src + off));
            } else {
                for (int i = 0; i < 16 && off + i < total_bytes; ++i) dst[u * 16 + i] = src[off + i];
            }
        }
        return (int)(begin - a0);
    };
    auto staged = [&]() {
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
    };
    auto score = [&](const unsigned char *kc, float (&sc)[kRep]) {
#pragma unroll
        for (int r = 0; r < kRep; ++r) sc[r] = 0.0f;
        for (int s = 0; s < S; ++s) {
            const float4 e = lut[s * kWords + kc[s]];
            sc[0] += e.x; sc[1] += e.y; sc[2] += e.z; sc[3] += e.w;
        }
    };
    const int chunk_tokens = kStageBytes / S;

    // ---- pass 1: exact maximum of every head over the range ------------------------------------------
    float mx[kRep] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int c0 = lo; c0 < hi; c0 += chunk_tokens) {
        const int c1 = min(c0 + chunk_tokens, hi);
        __syncthreads();  // previous chunk fully consumed
        const int koff = stage(kstage, kcodes, (row_base + c0) * S, (row_base + c1) * S);
        staged();
        for (int t = c0 + tid; t < c1; t += kThreads) {
            float sc[kRep];
            score(kstage + koff + (size_t)(t - c0) * S, sc);
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
    unsigned int lsum_u[kRep] = {0u, 0u, 0u, 0u};  // at most 32 tokens per thread: fits
    for (int c0 = lo; c0 < hi; c0 += chunk_tokens) {
        const int c1 = min(c0 + chunk_tokens, hi);
        __syncthreads();
        const int koff = stage(kstage, kcodes, (row_base + c0) * S, (row_base + c1) * S);
        const int voff = stage(vstage, vcodes, (row_base + c0) * S, (row_base + c1) * S);
        staged();
        for (int t = c0 + tid; t < c1; t += kThreads) {
            float sc[kRep];
            score(kstage + koff + (size_t)(t - c0) * S, sc);
            unsigned int p[kRep];
#pragma unroll
            for (int r = 0; r < kRep; ++r) {
                p[r] = __float2uint_rn(__expf(sc[r] - m[r]) * kWeightOne);
                lsum_u[r] += p[r];
            }
            const unsigned char *vc = vstage + voff + (size_t)(t - c0) * S;
            for (int s = 0; s < S; ++s) {
                unsigned int *bin = hist_u + (size_t)s * kRep * kWords + vc[s];  // [stage][head][code]: bank = code % 32
#pragma unroll
                for (int r = 0; r < kRep; ++r) atomicAdd(bin + r * kWords, p[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
        float lsum = (float)lsum_u[r] * (1.0f / kWeightOne);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
        if (lane == 0) red[warp * 8 + 4 + r] = lsum;
    }
    __syncthreads();

    // ---- acc = hist x V codebook: thread = (8-channel chunk, one of 16 slices of the code words) -------
    const int chunk = tid & 15, slice = tid >> 4;
    float acc[kRep][8];
#pragma unroll
    for (int r = 0; r < kRep; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = 0.0f;
    const int words = S * kWords;
    const uint4 *vt = reinterpret_cast<const uint4 *>(vtab + (size_t)h * words * kDim) + chunk;
#pragma unroll 8
    for (int w = slice; w < words; w += 16) {
        const unsigned int *cnt = hist_u + (size_t)(w >> 8) * kRep * kWords + (w & 255);
        const float4 wgt = make_float4((float)cnt[0] * (1.0f / kWeightOne), (float)cnt[kWords] * (1.0f / kWeightOne),
                                       (float)cnt[2 * kWords] * (1.0f / kWeightOne), (float)cnt[3 * kWords] * (1.0f / kWeightOne));
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
    // fold the 16 slices: the two slices of a warp by shuffle, the 8 warps through shared memory
#pragma unroll
    for (int r = 0; r < kRep; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] += __shfl_xor_sync(0xffffffffu, acc[r][i], 16);
    __syncthreads();  // histogram fully read: its storage and the score table's are free
    float *fold = smem;  // [8 warps][4][128]  (the launcher sizes the table area for this)
    if (lane < 16) {
#pragma unroll
        for (int r = 0; r < kRep; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) fold[(warp * kRep + r) * kDim + chunk * 8 + i] = acc[r][i];
    }
    __syncthreads();
    const int64_t rows = (int64_t)B * Hq;
    for (int o = tid; o < kRep * (kDim + 2); o += kThreads) {
        const int r = o / (kDim + 2), col = o % (kDim + 2);
        float v;
        if (col == 0) {
            v = m[r];
        } else if (col == 1) {
            v = 0.0f;
            for (int w = 0; w < kWarps; ++w) v += red[w * 8 + 4 + r];
        } else {
            v = 0.0f;
            for (int w = 0; w < kWarps; ++w) v += fold[(w * kRep + r) * kDim + col - 2];
        }
        part[((int64_t)split * rows + (int64_t)b * Hq + h * kRep + r) * (kDim + 2) + col] = v;
    }
}

}  // namespace fullwidth

bool attn_fullwidth_supported(int Hq, int Hkv, int D, int G, int S, int K) {
    return D == fullwidth::kDim && G == 1 && S >= 1 && S <= fullwidth::kMaxStages && K == fullwidth::kWords &&
           Hq == Hkv * fullwidth::kRep;
}

int attn_fullwidth_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                            const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part, int B,
                            int Hq, int Hkv, int S, int64_t T_cap, int splits, cudaStream_t stream) {
    (void)Hq;
    const size_t tables = (size_t)S * fullwidth::kWords * 4 * sizeof(float);
    size_t both = 2 * tables;  // score table + histogram; later reused to fold 8 warps x 4 heads x 128 channels
    if (both < (size_t)fullwidth::kWarps * fullwidth::kRep * fullwidth::kDim * sizeof(float))
        both = (size_t)fullwidth::kWarps * fullwidth::kRep * fullwidth::kDim * sizeof(float);
    const size_t smem = both + (fullwidth::kRep * fullwidth::kDim + fullwidth::kWarps * 8) * sizeof(float) +
                        2 * (fullwidth::kStageBytes + 32);
    auto kernel = fullwidth::attn_fullwidth_kernel;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    kernel<<<grid, fullwidth::kThreads, smem, stream>>>(q, kcodes, vcodes, ktab, vtab, seq_start, seq_end, part, B, Hkv, S,
                                                       T_cap, splits);
    return launch_status();
}

}  // namespace tacvq
