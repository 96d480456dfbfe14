// Encode for 8-wide and 4-wide groups (fp16 tables): tensor cores filter, exact fp32 decides.
//
// The exact distance that decides a code costs about 16 instructions in the scalar kernel.  Here a
// warp scores 16 rows against all 256 words of a stage with 32 mma.sync.m16n8k16 instructions that
// give every dot product to within a known bound, keeps the approximate scores in registers, and
// re-evaluates in the library's exact arithmetic only the words whose approximate distance lies within
// a margin of the row's approximate minimum.  The argmin of the exact values over
// that candidate set is the argmin over all words (argument below), so the codes are bit-identical
// to the scalar kernels'.
//
// Operands.  A (16 rows x 16): columns 0..7 hold hi = fp16(r), columns 8..15 hold lo = fp16(r - hi)
// of the fp32 residual r; B (16 x 8 words): rows 0..7 and rows 8..15 both hold the fp16 word, so one
// instruction returns (hi + lo) . c accumulated in fp32.  With the m16n8k16 fragment layout that makes
// both B registers of a thread the same 32-bit word of the table.
//
// Margin.  Let e_k be the exact (library-order) distance, a_k = cc_k - 2*dot~_k + xx the approximate
// one, |a_k - e_k| <= E.  For the exact argmin k* and the approximate argmin j:
//   a_k* <= e_k* + E <= e_j + E <= a_j + 2E,
// and the same holds for every word tied with k*, so all of them pass "a_k <= a_min + 2E".
// E collects: the hi/lo split (<= 2^-22 relative per element, 2^-25 absolute where fp16 is subnormal),
// the tensor core's fp32 accumulation of 16 exact products (<= 2^-18 P, P = sum |r_i c_i|), the exact
// chain's own rounding (<= 2^-21 P) and three fp32 roundings of magnitudes <= xx + cc + 2P.  With
// P <= (xx + cc)/2 this is below 2^-17.5 (xx + cc_max); the kernel uses 2^-14 (xx + cc_max) plus
// 2^-18 sqrt(cc_max) for the subnormal term, several times the bound.  Residuals too large for fp16
// (|r| >= 2^15) make every word a candidate for that warp, which is slow and still exact.
//
// Reference statements: src/jointkv/closed_loop_vq.py:52-76 (search), :343-395 (stage recursion),
// src/jointkv/cq_tac.py:86-105.

#include "common.cuh"

#ifndef TACVQ_TC_MINBLOCKS
#define TACVQ_TC_MINBLOCKS 4  // resident blocks per SM the register budget is set for
#endif

namespace tacvq {

constexpr int kTcThreads = 128;
constexpr int kTcRows = (kTcThreads / 32) * 16;  // rows per block iteration

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1, float even, float odd) {
    // accumulator rows share their start values: columns 2q and 2q+1 of both row halves
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(even), "f"(odd));
}

__device__ __forceinline__ uint32_t pack_half2(float lo_elem, float hi_elem) {
    const __half2 v = __halves2half2(__float2half_rn(lo_elem), __float2half_rn(hi_elem));
    return *reinterpret_cast<const uint32_t *>(&v);
}

// hi/lo fp16 split of two neighbouring residual elements
__device__ __forceinline__ void split_pair(float r0, float r1, uint32_t &hi, uint32_t &lo) {
    const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
    const __half2 hv = __halves2half2(h0, h1);
    hi = *reinterpret_cast<const uint32_t *>(&hv);
    lo = pack_half2(r0 - __half2float(h0), r1 - __half2float(h1));
}

// exact distance of one row to word k, in the library's orders; keeps the lowest (distance, index)
__device__ __forceinline__ void rescore(const float (&row)[8], float xx, const float4 lo, const float4 hi, float cc, int k,
                                        float &best, int &arg) {
    float dot = __fmaf_rn(row[0], lo.x, 0.0f);
    dot = __fmaf_rn(row[1], lo.y, dot);
    dot = __fmaf_rn(row[2], lo.z, dot);
    dot = __fmaf_rn(row[3], lo.w, dot);
    dot = __fmaf_rn(row[4], hi.x, dot);
    dot = __fmaf_rn(row[5], hi.y, dot);
    dot = __fmaf_rn(row[6], hi.z, dot);
    dot = __fmaf_rn(row[7], hi.w, dot);
    const float dist = distance_expr(xx, cc, dot);
    if (dist < best || (dist == best && k < arg)) {
        best = dist;
        arg = k;
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Shared memory per stage (kTcStageBytes):
//   fragb  [8 groups][32 lanes] uint4   B operands in fragment order: lane (gid, q) finds, for the four
//                                       tiles 4m..4m+3, dims (2q, 2q+1) of word (4m+j)*8 + gid
//   seed   [8 groups][4 q][4 tiles][2]  accumulator seeds -cc/2 of words (4m+j)*8 + 2q + e
//   wordf  [256][8] fp32                the words widened once, for exact re-evaluation and the update
//   nrm    [256] fp32                   exact |word|^2 (padding words: +inf)
// and after all stages {cc_max, slack} per stage.
constexpr size_t kTcStageBytes = 4096 + 1024 + 8192 + 1024;

// DSUB = 8, or 4 run as 8 with the upper four elements of rows and words held at zero: appending zeros
// changes neither the FMA chain of a dot product nor the left-to-right sum of squares, so the codes
// are those of a 4-wide scan.
template <int DSUB, typename XT>
__global__ void __launch_bounds__(kTcThreads, TACVQ_TC_MINBLOCKS)
encode_tc8_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const __half *__restrict__ tables,
                  const float *__restrict__ sqnorm_in, uint8_t *__restrict__ codes, void *__restrict__ recon,
                  int recon_dtype, int B, int H, int T, int G, int S, int K, int64_t t0, int64_t T_cap) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *bound = reinterpret_cast<float *>(smem_raw + (size_t)S * kTcStageBytes);  // [S][2]

    const int hg = blockIdx.y;
    const int h = hg / G, g = hg % G;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, q = lane & 3;

    for (int idx = tid; idx < S * kMaxWords; idx += kTcThreads) {
        const int k = idx % kMaxWords, s = idx / kMaxWords;
        unsigned char *stage = smem_raw + (size_t)s * kTcStageBytes;
        uint32_t *fragb = reinterpret_cast<uint32_t *>(stage);
        float *seed = reinterpret_cast<float *>(stage + 4096);
        float *wordf = reinterpret_cast<float *>(stage + 4096 + 1024);
        float *nrm = reinterpret_cast<float *>(stage + 4096 + 1024 + 8192);
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        float cc = __int_as_float(0x7f800000);  // padding words can never be chosen
        if (k < K) {
            const int64_t word = (((int64_t)h * S + s) * G + g) * K + k;
            if constexpr (DSUB == 8) {
                w = *reinterpret_cast<const uint4 *>(tables + word * 8);
            } else {
                const uint2 half_word = *reinterpret_cast<const uint2 *>(tables + word * 4);
                w = make_uint4(half_word.x, half_word.y, 0u, 0u);
            }
            if (sqnorm_in != nullptr) {
                cc = sqnorm_in[word];
            } else {
                const __half *e = reinterpret_cast<const __half *>(&w);
                cc = sqnorm_ordered<DSUB>([&](int i) { return __half2float(e[i]); });
            }
        }
        const int tile = k >> 3, col = k & 7;  // word k is column col of tile `tile`
        const int m = tile >> 2, j = tile & 3;
        // as a B operand the word is read by the lanes gid = col, q = 0..3
        const uint32_t *pairs = reinterpret_cast<const uint32_t *>(&w);
#pragma unroll
        for (int qq = 0; qq < 4; ++qq) fragb[((m * 32) + col * 4 + qq) * 4 + j] = pairs[qq];
        // as an accumulator column it belongs to the lanes q = col/2, element col%2
        seed[m * 32 + (col >> 1) * 8 + j * 2 + (col & 1)] = -0.5f * cc;
        const __half2 *hp = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(hp[i]);
            wordf[k * 8 + 2 * i] = f.x;
            wordf[k * 8 + 2 * i + 1] = f.y;
        }
        nrm[k] = cc;
    }
    __syncthreads();
    if (tid < S) {
        const float *nrm = reinterpret_cast<const float *>(smem_raw + (size_t)tid * kTcStageBytes + 4096 + 1024 + 8192);
        float top = 0.0f;
        for (int k = 0; k < K; ++k) top = fmaxf(top, nrm[k]);
        bound[2 * tid] = top;
        bound[2 * tid + 1] = 3.814697265625e-06f * sqrtf(top);  // 2^-18 sqrt(cc_max)
    }
    __syncthreads();

    const uint32_t rows = (uint32_t)B * (uint32_t)T;  // the launcher keeps B*T below 2^31
    const uint32_t stride = gridDim.x * kTcRows;
    const float inf = __int_as_float(0x7f800000);

    // rows of this lane's quad in the current tile: `a` = gid, `b` = gid + 8; elements 2q, 2q+1.
    // (batch row, token) of a row is divided out once and then advanced by the tile stride.
    auto fetch = [&](bool live, uint32_t b, uint32_t t, float (&r)[2]) {
        r[0] = r[1] = 0.0f;
        if (live && 2 * q < DSUB) {
            const XT *src = x + (int64_t)b * sxb + (int64_t)h * sxh + (int64_t)t * sxt + g * DSUB + 2 * q;
            r[0] = to_float<XT>(src[0]);
            r[1] = to_float<XT>(src[1]);
        }
    };
    const uint32_t step_b = stride / (uint32_t)T, step_t = stride % (uint32_t)T;
    auto advance = [&](uint32_t &b, uint32_t &t) {
        b += step_b;
        t += step_t;
        if (t >= (uint32_t)T) {
            t -= (uint32_t)T;
            ++b;
        }
    };
    uint32_t tile = blockIdx.x * kTcRows;
    uint32_t ba = (tile + warp * 16 + gid) / (uint32_t)T, ta = (tile + warp * 16 + gid) % (uint32_t)T;
    uint32_t bb = (tile + warp * 16 + gid + 8) / (uint32_t)T, tb = (tile + warp * 16 + gid + 8) % (uint32_t)T;
    float ra[2], rb[2];
    fetch(tile + warp * 16 + gid < rows, ba, ta, ra);
    fetch(tile + warp * 16 + gid + 8 < rows, bb, tb, rb);
    for (; tile < rows; tile += stride) {
        const uint32_t row_a = tile + warp * 16 + gid, row_b = row_a + 8;
        // next tile's elements travel while this one is searched
        uint32_t nba = ba, nta = ta, nbb = bb, ntb = tb;
        advance(nba, nta);
        advance(nbb, ntb);
        float na[2] = {0.0f, 0.0f}, nb[2] = {0.0f, 0.0f};
        if (tile + stride < rows && tile + stride > tile) {
            fetch(row_a + stride < rows, nba, nta, na);
            fetch(row_b + stride < rows, nbb, ntb, nb);
        }
        const bool live_a = row_a < rows, live_b = row_b < rows;
        uint8_t *code_a = codes + (((int64_t)ba * H + h) * T_cap + t0 + ta) * ((int64_t)S * G) + g;
        uint8_t *code_b = codes + (((int64_t)bb * H + h) * T_cap + t0 + tb) * ((int64_t)S * G) + g;
        float da[2] = {0.0f, 0.0f}, db[2] = {0.0f, 0.0f};

        for (int s = 0; s < S; ++s) {
            const unsigned char *stage = smem_raw + (size_t)s * kTcStageBytes;
            const uint4 *fragb = reinterpret_cast<const uint4 *>(stage);
            const float4 *seed = reinterpret_cast<const float4 *>(stage + 4096);
            const float *wordf = reinterpret_cast<const float *>(stage + 4096 + 1024);
            const float *nrm = reinterpret_cast<const float *>(stage + 4096 + 1024 + 8192);

            // every lane of a row's quad gets the whole residual row
            float fa[8], fb[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int from = (lane & ~3) | j;
                fa[2 * j] = __shfl_sync(0xffffffffu, ra[0], from);
                fa[2 * j + 1] = __shfl_sync(0xffffffffu, ra[1], from);
                fb[2 * j] = __shfl_sync(0xffffffffu, rb[0], from);
                fb[2 * j + 1] = __shfl_sync(0xffffffffu, rb[1], from);
            }
            const float xx_a = sqnorm_ordered<8>([&](int i) { return fa[i]; });
            const float xx_b = sqnorm_ordered<8>([&](int i) { return fb[i]; });

            uint32_t a0, a1, a2, a3;
            split_pair(ra[0], ra[1], a0, a2);
            split_pair(rb[0], rb[1], a1, a3);
            const float big = fmaxf(fmaxf(fabsf(ra[0]), fabsf(ra[1])), fmaxf(fabsf(rb[0]), fabsf(rb[1])));
            const bool overflow = __any_sync(0xffffffffu, !(big < 32768.0f));

            // Approximate scores t = r.c - cc/2 (the distance is xx - 2t) of the 16 rows against all 256
            // words; -cc/2 enters as the accumulator.  Per row a thread keeps the largest score of each
            // pair of tiles (its four words there); a pair that passes the threshold is re-evaluated.
            float top_a[16], top_b[16];
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const uint4 bw = fragb[m * 32 + lane];
                const float4 s0 = seed[m * 8 + q * 2], s1 = seed[m * 8 + q * 2 + 1];
                float c0[4], c1[4], c2[4], c3[4];
                mma_f16_16816(c0, a0, a1, a2, a3, bw.x, bw.x, s0.x, s0.y);
                mma_f16_16816(c1, a0, a1, a2, a3, bw.y, bw.y, s0.z, s0.w);
                mma_f16_16816(c2, a0, a1, a2, a3, bw.z, bw.z, s1.x, s1.y);
                mma_f16_16816(c3, a0, a1, a2, a3, bw.w, bw.w, s1.z, s1.w);
                top_a[2 * m] = fmaxf(max3(c0[0], c0[1], c1[0]), c1[1]);
                top_b[2 * m] = fmaxf(max3(c0[2], c0[3], c1[2]), c1[3]);
                top_a[2 * m + 1] = fmaxf(max3(c2[0], c2[1], c3[0]), c3[1]);
                top_b[2 * m + 1] = fmaxf(max3(c2[2], c2[3], c3[2]), c3[3]);
            }
            float max_a = top_a[0], max_b = top_b[0];
#pragma unroll
            for (int p = 1; p < 15; p += 2) {
                max_a = max3(max_a, top_a[p], top_a[p + 1]);
                max_b = max3(max_b, top_b[p], top_b[p + 1]);
            }
            max_a = fmaxf(max_a, top_a[15]);
            max_b = fmaxf(max_b, top_b[15]);
            max_a = fmaxf(max_a, __shfl_xor_sync(0xffffffffu, max_a, 1));
            max_b = fmaxf(max_b, __shfl_xor_sync(0xffffffffu, max_b, 1));
            max_a = fmaxf(max_a, __shfl_xor_sync(0xffffffffu, max_a, 2));
            max_b = fmaxf(max_b, __shfl_xor_sync(0xffffffffu, max_b, 2));

            // margins in units of t (half the distance margin)
            const float cc_max = bound[2 * s], slack = bound[2 * s + 1];
            const float thr_a = overflow ? -inf : max_a - (3.0517578125e-05f * (xx_a + cc_max) + slack);
            const float thr_b = overflow ? -inf : max_b - (3.0517578125e-05f * (xx_b + cc_max) + slack);

            // Candidate pairs.  The sign of (score - threshold) is shifted into a word, pair 0 first, so
            // after 16 steps bit 15 - p is set when pair p FAILS; inverted below.
            uint32_t fail_a = 0u, fail_b = 0u;
#pragma unroll
            for (int p = 0; p < 16; ++p) {
                fail_a = __funnelshift_l(__float_as_uint(top_a[p] - thr_a), fail_a, 1);
                fail_b = __funnelshift_l(__float_as_uint(top_b[p] - thr_b), fail_b, 1);
            }
            uint32_t cand_a = ~fail_a & 0xffffu, cand_b = ~fail_b & 0xffffu;

            // Exact re-evaluation, shared by the quad: every lane holds both rows, so the four words of a
            // candidate pair (two tiles x two columns of the owning lane) go one to each lane.  Usually
            // one trip handles the single candidate of row a and of row b together.
            float best_a = inf, best_b = inf;
            int arg_a = 0x7fffffff, arg_b = 0x7fffffff;
            const int quad = lane & 28;
            while (true) {
                const uint32_t vote_a = __ballot_sync(0xffffffffu, cand_a != 0u);
                const uint32_t vote_b = __ballot_sync(0xffffffffu, cand_b != 0u);
                if ((vote_a | vote_b) == 0u) break;
                const int own_a = __ffs((vote_a >> quad) & 15u) - 1;  // lane of the quad that owns one, or -1
                const int own_b = __ffs((vote_b >> quad) & 15u) - 1;
                const int pa = __shfl_sync(0xffffffffu, __clz(cand_a) - 16, quad + (own_a & 3));
                const int pb = __shfl_sync(0xffffffffu, __clz(cand_b) - 16, quad + (own_b & 3));
                if (own_a >= 0) {
                    const int k = (2 * pa + (q >> 1)) * 8 + 2 * own_a + (q & 1);
                    const float4 *w = reinterpret_cast<const float4 *>(wordf + k * 8);
                    rescore(fa, xx_a, w[0], w[1], nrm[k], k, best_a, arg_a);
                    if (q == own_a) cand_a &= ~(0x8000u >> pa);
                }
                if (own_b >= 0) {
                    const int k = (2 * pb + (q >> 1)) * 8 + 2 * own_b + (q & 1);
                    const float4 *w = reinterpret_cast<const float4 *>(wordf + k * 8);
                    rescore(fb, xx_b, w[0], w[1], nrm[k], k, best_b, arg_b);
                    if (q == own_b) cand_b &= ~(0x8000u >> pb);
                }
            }
#pragma unroll
            for (int off = 1; off <= 2; off <<= 1) {
                const float oa = __shfl_xor_sync(0xffffffffu, best_a, off);
                const int ia = __shfl_xor_sync(0xffffffffu, arg_a, off);
                if (oa < best_a || (oa == best_a && ia < arg_a)) best_a = oa, arg_a = ia;
                const float ob = __shfl_xor_sync(0xffffffffu, best_b, off);
                const int ib = __shfl_xor_sync(0xffffffffu, arg_b, off);
                if (ob < best_b || (ob == best_b && ib < arg_b)) best_b = ob, arg_b = ib;
            }
            if (arg_a >= K) arg_a = 0;  // every distance was +inf or NaN
            if (arg_b >= K) arg_b = 0;

            const float2 sel_a = *reinterpret_cast<const float2 *>(wordf + arg_a * 8 + 2 * q);
            const float2 sel_b = *reinterpret_cast<const float2 *>(wordf + arg_b * 8 + 2 * q);
            ra[0] = __fsub_rn(ra[0], sel_a.x);
            ra[1] = __fsub_rn(ra[1], sel_a.y);
            rb[0] = __fsub_rn(rb[0], sel_b.x);
            rb[1] = __fsub_rn(rb[1], sel_b.y);
            da[0] = __fadd_rn(da[0], sel_a.x);
            da[1] = __fadd_rn(da[1], sel_a.y);
            db[0] = __fadd_rn(db[0], sel_b.x);
            db[1] = __fadd_rn(db[1], sel_b.y);
            if (q == 0) {
                if (live_a) code_a[s * G] = (uint8_t)arg_a;
                if (live_b) code_b[s * G] = (uint8_t)arg_b;
            }
        }

        if (recon != nullptr && 2 * q < DSUB) {
            if (live_a) {
                const int64_t o = (((int64_t)ba * H + h) * T + ta) * ((int64_t)G * DSUB) + g * DSUB + 2 * q;
                if (recon_dtype == TACVQ_F16) {
                    *reinterpret_cast<uint32_t *>((__half *)recon + o) = pack_half2(da[0], da[1]);
                } else {
                    *reinterpret_cast<float2 *>((float *)recon + o) = make_float2(da[0], da[1]);
                }
            }
            if (live_b) {
                const int64_t o = (((int64_t)bb * H + h) * T + tb) * ((int64_t)G * DSUB) + g * DSUB + 2 * q;
                if (recon_dtype == TACVQ_F16) {
                    *reinterpret_cast<uint32_t *>((__half *)recon + o) = pack_half2(db[0], db[1]);
                } else {
                    *reinterpret_cast<float2 *>((float *)recon + o) = make_float2(db[0], db[1]);
                }
            }
        }
        ra[0] = na[0], ra[1] = na[1], rb[0] = nb[0], rb[1] = nb[1];
        ba = nba, ta = nta, bb = nbb, tb = ntb;
    }
}

// Returns TACVQ_ERR_UNSUPPORTED when the geometry is not this kernel's, so the caller can go on to
// the scalar kernels.
int encode_tc8_launch(const EncodeArgs &a) {
    const int sub = a.D / a.G;
    if (a.tables_f32 || (sub != 8 && sub != 4) || a.K > kMaxWords) return TACVQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a.tables) & 15u) != 0) return TACVQ_ERR_UNSUPPORTED;
    if (a.recon != nullptr && (reinterpret_cast<uintptr_t>(a.recon) & 7u) != 0) return TACVQ_ERR_UNSUPPORTED;
    const size_t smem = (size_t)a.S * kTcStageBytes + (size_t)a.S * 2 * sizeof(float);
    if (smem > 200 * 1024) return TACVQ_ERR_UNSUPPORTED;
    const int64_t rows = (int64_t)a.B * a.T;
    if (rows >= (int64_t)1 << 31) return TACVQ_ERR_UNSUPPORTED;
    int64_t tiles = (rows + kTcRows - 1) / kTcRows;
    // about 16 resident blocks per SM in total; each block keeps its tables and walks over row tiles
    const int64_t want = (148 * 16 + a.H * a.G - 1) / (a.H * a.G);
    if (tiles > want) tiles = want;
    dim3 grid((unsigned)tiles, (unsigned)(a.H * a.G));
    auto launch = [&](auto kernel, auto *xp) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        kernel<<<grid, kTcThreads, smem, a.stream>>>(xp, a.sxb, a.sxh, a.sxt, (const __half *)a.tables, a.sqnorm, a.codes,
                                                     a.recon, a.recon_dtype, a.B, a.H, a.T, a.G, a.S, a.K, a.t0, a.T_cap);
        return launch_status();
    };
    if (sub == 8) {
        if (a.x_dtype == TACVQ_F16) return launch(encode_tc8_kernel<8, __half>, (const __half *)a.x);
        return launch(encode_tc8_kernel<8, float>, (const float *)a.x);
    }
    if (a.x_dtype == TACVQ_F16) return launch(encode_tc8_kernel<4, __half>, (const __half *)a.x);
    return launch(encode_tc8_kernel<4, float>, (const float *)a.x);
}

}  // namespace tacvq
