// Attention over codes of PRE-rotary keys for the benchmark geometry (head_dim 128 = 16 groups x 8,
// two residual stages, 256 words), with both contractions on the tensor cores (mma.sync).
//
// A block serves one (batch row, KV head, sequence split) of at most 4096 tokens in two passes:
//   pass K   key tables (128 KB) in shared memory.  Four lanes share a token; lane j of them rebuilds the
//            channels 16j..16j+15 and 64+16j..64+16j+15 (groups 2j, 2j+1, 2j+8, 2j+9) as fp16 (packed add
//            of the two stages = the reference's fp16 window), which are exactly the rotary partners
//            c, c+64, rotates them with the cos/sin of the token's position, and the warp multiplies
//            8 tokens x 128 channels with the 4 query heads by four m16n8k16 products: rows 0-7 of the A
//            operand carry the lower 64 channels of the 8 tokens, rows 8-15 the upper 64, and the 8 columns
//            of the B operand are (4 heads) x (lower | upper query channels); the two halves of a score
//            meet through one shuffle.  fp32 scores go to shared memory.
//   softmax  block maximum, p = exp(score - max) as fp16 [head][token] over the score area.
//   pass V   value tables loaded over the key tables (the copy overlaps the softmax step); P.V with
//            m16n8k8 products exactly as in the kernel without rotary step (attn_gsrq.cu): rows =
//            channels, columns = 4 heads x 2 visiting orders, contraction = tokens; value codes land by
//            cp.async and are handed out by ldmatrix.trans.
// Every shared-memory gather is conflict-free for arbitrary codes: a code's 32 codewords lie in one
// 512-byte row, the position of (stage, group) inside the row decides the bank, and the lanes that are
// served together read different positions (the two tokens of a quarter warp take the stages in opposite
// order in pass K; the four token pairs visit (stage, group) in four orders in pass V).
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122 including the
// rotary step (:113-118).  Differences from that dense path, inside the 2e-3 tolerance: the rotation is
// a packed multiply and a fused multiply-add per channel pair (the reference rounds both products), and
// probabilities enter the P.V product as fp16.

#include "common.cuh"

namespace tacvq {

namespace rotmma {

constexpr int kThreads = 512, kWarps = kThreads / 32;
constexpr int kDim = 128, kWords = 256, kRowBytes = 512;   // a code's 32 codewords
constexpr int kChunk = 4096;                               // tokens per block at most
constexpr int kTabBytes = kWords * kRowBytes;              // 131072
constexpr int kScoreBytes = kChunk * 4 * 4;                // fp32 [token][4 heads]
constexpr int kProbStride = kChunk * 2 + 16;               // bytes per head of the fp16 probabilities
constexpr int kVStagePerWarp = 1024;                       // one 32-token tile of value codes
constexpr int kRedFloats = kWarps * 4;
constexpr int kSmemBytes = kTabBytes + kScoreBytes + 2 * kRedFloats * 4;
static_assert(4 * kProbStride + kWarps * kVStagePerWarp <= kScoreBytes, "probabilities and code staging reuse the score area");
static_assert(kWarps * 32 * 32 * 4 <= kTabBytes, "merge scratch reuses the table area");

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&d)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t hadd2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

// position of the codeword (stage s, group g) inside a code's 512-byte row
//   key tables:   the bank (position mod 8) is s*4 + (g/2)%4: in pass K lane j reads groups 2j + {0,1,8,9}
//   value tables: the bank is s*4 + g%4 (as in attn_gsrq.cu)
__device__ __forceinline__ int key_pos(int s, int g) { return (((g >> 3) << 1) | (g & 1)) * 8 + s * 4 + ((g >> 1) & 3); }
__device__ __forceinline__ int value_pos(int s, int g) { return (g >> 2) * 8 + s * 4 + (g & 3); }

// A head's tables [stage][group][word][8] -> shared memory rows [word][position]; a warp copies, per trip,
// 4 neighbouring words of 8 positions with different banks: full 32-byte sectors in, no conflicts out.
template <bool KEYS>
__device__ __forceinline__ void copy_tables(uint32_t tab_u32, const __half *__restrict__ src, int tid) {
    for (int idx = tid; idx < kWords * 32; idx += kThreads) {
        const int pos = ((idx >> 5) & 3) * 8 + (idx & 7);
        const int word = ((idx >> 7) << 2) | ((idx >> 3) & 3);
        int s, g;
        if (KEYS) {
            s = (pos >> 2) & 1;
            g = ((pos >> 4) << 3) | ((pos & 3) << 1) | ((pos >> 3) & 1);
        } else {
            s = (pos >> 2) & 1;
            g = ((pos >> 3) << 2) | (pos & 3);
        }
        cp_async16(tab_u32 + word * kRowBytes + pos * 16, src + ((size_t)(s * 16 + g) * kWords + word) * 8);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
attn_rotary_mma_kernel(const __half *__restrict__ q, const uint8_t *__restrict__ kcodes, const uint8_t *__restrict__ vcodes,
                       const __half *__restrict__ ktab, const __half *__restrict__ vtab, const __half *__restrict__ rope,
                       const int32_t *__restrict__ seq_start, const int32_t *__restrict__ seq_end, float *__restrict__ part,
                       int B, int Hq, int Hkv, int64_t T_cap, int splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *tab_s = smem_raw;
    float *score_s = reinterpret_cast<float *>(smem_raw + kTabBytes);
    float *red_s = reinterpret_cast<float *>(smem_raw + kTabBytes + kScoreBytes);  // [2][warps][4]
    const uint32_t tab_u32 = smem_u32(tab_s), score_u32 = smem_u32(score_s);

    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rep = Hq / Hkv;  // 1, 2 or 4 query heads per KV head

    const int lo_all = seq_start ? max(seq_start[b], 0) : 0;
    const int hi_all = seq_end ? min(seq_end[b], (int)T_cap) : (int)T_cap;
    const int n_all = hi_all > lo_all ? hi_all - lo_all : 0;
    const int per = (n_all + splits - 1) / splits;
    const int chunk = lo_all + split * per;
    const int n = max(min(chunk + per, lo_all + n_all) - chunk, 0);  // at most kChunk: the launcher picks the split count
    const int64_t rows = (int64_t)B * Hq;
    const size_t code_row = ((size_t)b * Hkv + h) * (size_t)T_cap;

    if (n <= 0) {  // an empty range contributes the neutral state
        for (int idx = tid; idx < rep * (kDim + 2); idx += kThreads) {
            const int r = idx / (kDim + 2), col = idx % (kDim + 2);
            part[((int64_t)split * rows + (int64_t)b * Hq + h * rep + r) * (kDim + 2) + col] = col == 0 ? -INFINITY : 0.0f;
        }
        return;
    }

    copy_tables<true>(tab_u32, ktab + (size_t)h * 2 * 16 * kWords * 8, tid);

    // ---- pass K ------------------------------------------------------------------------------------
    const int g8 = lane >> 2, j4 = lane & 3;
    {
        // B operand: column n = g8 is (head n & 3, channel half n >> 2); this lane's 16 channels of it
        uint32_t qf[8];
        {
            const int head = g8 & 3, half = g8 >> 2;
            uint4 lo4 = make_uint4(0u, 0u, 0u, 0u), hi4 = lo4;
            if (head < rep) {
                const uint4 *src = reinterpret_cast<const uint4 *>(q + ((size_t)b * Hq + h * rep + head) * kDim + half * 64 + 16 * j4);
                lo4 = __ldg(src);
                hi4 = __ldg(src + 1);
            }
            qf[0] = lo4.x, qf[1] = lo4.y, qf[2] = lo4.z, qf[3] = lo4.w, qf[4] = hi4.x, qf[5] = hi4.y, qf[6] = hi4.z, qf[7] = hi4.w;
        }
        // gather addresses: step (ci, sf) reads group 2j + {0,1,8,9}[ci] of stage sf ^ (token parity)
        const int first_stage = g8 & 1;
        uint32_t k_off[4][2];
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
#pragma unroll
            for (int sf = 0; sf < 2; ++sf)
                k_off[ci][sf] = tab_u32 + key_pos(sf ^ first_stage, 2 * j4 + (ci & 1) + (ci >> 1) * 8) * 16;
        // a token's 32 code bytes: stage s at bytes 16s..16s+15; this lane wants bytes 2j, 2j+1 and 8+2j, 9+2j of each
        const int code_a = first_stage * 16 + 2 * j4, code_b = (first_stage ^ 1) * 16 + 2 * j4;
        const uint8_t *kc = kcodes + (code_row + chunk) * 32;
        const __half *rp = rope + (size_t)chunk * kDim + 16 * j4;

        const int trips = (n + 8 * kWarps - 1) / (8 * kWarps);
        uint32_t cn[4];
        uint4 rn[4];
        auto fetch = [&](int local) {
            const int t = min(local, n - 1);
            const uint8_t *row = kc + (size_t)t * 32;
            cn[0] = *reinterpret_cast<const unsigned short *>(row + code_a);
            cn[1] = *reinterpret_cast<const unsigned short *>(row + code_a + 8);
            cn[2] = *reinterpret_cast<const unsigned short *>(row + code_b);
            cn[3] = *reinterpret_cast<const unsigned short *>(row + code_b + 8);
            const uint4 *cs = reinterpret_cast<const uint4 *>(rp + (size_t)t * kDim);
            rn[0] = __ldg(cs), rn[1] = __ldg(cs + 1);          // cosines of frequencies 16j .. 16j+15
            rn[2] = __ldg(cs + 8), rn[3] = __ldg(cs + 9);      // sines
        };
        fetch(warp * 8 + g8);
        cp_async_wait_all();
        __syncthreads();
        for (int trip = 0; trip < trips; ++trip) {
            const int local = (trip * kWarps + warp) * 8 + g8;
            const uint32_t c0 = cn[0], c1 = cn[1], c2 = cn[2], c3 = cn[3];
            const uint32_t cosv[8] = {rn[0].x, rn[0].y, rn[0].z, rn[0].w, rn[1].x, rn[1].y, rn[1].z, rn[1].w};
            const uint32_t sinv[8] = {rn[2].x, rn[2].y, rn[2].z, rn[2].w, rn[3].x, rn[3].y, rn[3].z, rn[3].w};
            if (trip + 1 < trips) fetch(local + 8 * kWarps);
            // first stage of this lane's order, then the other; the packed fp16 sum does not depend on the order
            const uint4 a0 = lds128(k_off[0][0] + (c0 & 0xffu) * kRowBytes), a1 = lds128(k_off[1][0] + (c0 >> 8) * kRowBytes);
            const uint4 a2 = lds128(k_off[2][0] + (c1 & 0xffu) * kRowBytes), a3 = lds128(k_off[3][0] + (c1 >> 8) * kRowBytes);
            const uint4 b0 = lds128(k_off[0][1] + (c2 & 0xffu) * kRowBytes), b1 = lds128(k_off[1][1] + (c2 >> 8) * kRowBytes);
            const uint4 b2 = lds128(k_off[2][1] + (c3 & 0xffu) * kRowBytes), b3 = lds128(k_off[3][1] + (c3 >> 8) * kRowBytes);
            const uint32_t lo[8] = {hadd2(a0.x, b0.x), hadd2(a0.y, b0.y), hadd2(a0.z, b0.z), hadd2(a0.w, b0.w),
                                    hadd2(a1.x, b1.x), hadd2(a1.y, b1.y), hadd2(a1.z, b1.z), hadd2(a1.w, b1.w)};
            const uint32_t hi[8] = {hadd2(a2.x, b2.x), hadd2(a2.y, b2.y), hadd2(a2.z, b2.z), hadd2(a2.w, b2.w),
                                    hadd2(a3.x, b3.x), hadd2(a3.y, b3.y), hadd2(a3.z, b3.z), hadd2(a3.w, b3.w)};
            // k'_c = k_c cos - k_{c+64} sin ;  k'_{c+64} = k_{c+64} cos + k_c sin
            uint32_t rl[8], rh[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                rl[i] = hfma2(hi[i] ^ 0x80008000u, sinv[i], hmul2(lo[i], cosv[i]));
                rh[i] = hfma2(lo[i], sinv[i], hmul2(hi[i], cosv[i]));
            }
            float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) mma16816(d, rl[2 * ks], rh[2 * ks], rl[2 * ks + 1], rh[2 * ks + 1], qf[2 * ks], qf[2 * ks + 1]);
            // rows 0-7 x columns 0-3 hold the lower halves of the scores (lanes j < 2), rows 8-15 x columns 4-7
            // the upper halves (lanes j >= 2)
            const float up0 = __shfl_xor_sync(0xffffffffu, d[2], 2), up1 = __shfl_xor_sync(0xffffffffu, d[3], 2);
            if (j4 < 2 && local < n) *reinterpret_cast<float2 *>(score_s + (size_t)local * 4 + 2 * j4) = make_float2(d[0] + up0, d[1] + up1);
        }
    }
    __syncthreads();

    // ---- softmax over the block's tokens; value tables arrive meanwhile -------------------------------
    copy_tables<false>(tab_u32, vtab + (size_t)h * 2 * 16 * kWords * 8, tid);
    const int n_pad = (n + 31) & ~31;
    float m[4], l[4];
    {
        float4 sv[kChunk / kThreads];
        float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int k = 0; k < kChunk / kThreads; ++k) {
            const int i = tid + k * kThreads;
            if (i < n) {
                sv[k] = *reinterpret_cast<const float4 *>(score_s + (size_t)i * 4);
                top[0] = fmaxf(top[0], sv[k].x), top[1] = fmaxf(top[1], sv[k].y), top[2] = fmaxf(top[2], sv[k].z), top[3] = fmaxf(top[3], sv[k].w);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], off));
            if (lane == 0) red_s[warp * 4 + r] = top[r];
        }
        __syncthreads();  // also: every thread holds its scores, the score area may be overwritten
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            m[r] = -INFINITY;
            for (int w = 0; w < kWarps; ++w) m[r] = fmaxf(m[r], red_s[w * 4 + r]);
            l[r] = 0.0f;
        }
        __half *prob = reinterpret_cast<__half *>(score_s);
#pragma unroll
        for (int k = 0; k < kChunk / kThreads; ++k) {
            const int i = tid + k * kThreads;
            if (i < n_pad) {
                float p[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (i < n) {
                    p[0] = __expf(sv[k].x - m[0]), p[1] = __expf(sv[k].y - m[1]), p[2] = __expf(sv[k].z - m[2]), p[3] = __expf(sv[k].w - m[3]);
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    l[r] += p[r];
                    prob[(size_t)r * (kProbStride / 2) + i] = __float2half_rn(p[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) l[r] += __shfl_xor_sync(0xffffffffu, l[r], off);
            if (lane == 0) red_s[kRedFloats + warp * 4 + r] = l[r];
        }
    }

    // ---- pass V ------------------------------------------------------------------------------------
    const int r8 = lane >> 2, kq = lane & 3;
    uint32_t v_off[2][2], v_sel[2][2];
#pragma unroll
    for (int sp = 0; sp < 2; ++sp)
#pragma unroll
        for (int gsel = 0; gsel < 2; ++gsel) {
            const int s = sp ^ (kq & 1), gh = gsel ^ (kq >> 1);
            v_off[sp][gsel] = tab_u32 + value_pos(s, 2 * r8 + gh) * 16;
        }
#pragma unroll
    for (int tk = 0; tk < 2; ++tk)
#pragma unroll
        for (int gsel = 0; gsel < 2; ++gsel) v_sel[tk][gsel] = 0x4404u | ((uint32_t)(tk * 2 + (gsel ^ (kq >> 1))) << 4);  // code byte -> bits 8..15
    const int b_head = r8 & 3;                       // B-operand column n = r8: head n & 3, visiting order n >> 2
    const bool b_valid = (r8 >> 2) == (kq >> 1);
    const uint32_t vstage_u32 = score_u32 + 4 * kProbStride + warp * kVStagePerWarp;
    // landing place of this lane's (= token's) two 16-byte stage halves: odd token pairs swap the halves (stage
    // order of the value look-ups), tokens 4..7 of every eight swap them once more so that the eight rows of an
    // ldmatrix tile cover all banks
    const uint32_t v_land = vstage_u32 + lane * 32 + ((((lane >> 1) ^ (lane >> 2)) & 1) * 16);
    const uint32_t v_row0 = vstage_u32 + (8 * (lane >> 4) + (lane & 7)) * 32 + ((((lane >> 3) & 1) ^ ((lane >> 2) & 1)) * 16);
    const uint32_t p_read = score_u32 + (uint32_t)(b_head * kProbStride + kq * 4);
    const uint8_t *vc = vcodes + (code_row + chunk) * 32;

    float acc[8][4];
#pragma unroll
    for (int mm = 0; mm < 8; ++mm) acc[mm][0] = acc[mm][1] = acc[mm][2] = acc[mm][3] = 0.0f;
    const int tiles = n_pad >> 5;
    __syncthreads();  // probabilities written; nobody reads scores any more
    if (warp < tiles) {
        const uint8_t *src = vc + (size_t)min(warp * 32 + lane, n - 1) * 32;
        cp_async16(v_land, src);
        cp_async16(v_land ^ 16u, src + 16);
    }
    cp_async_wait_all();  // the value tables and the first tile of codes
    __syncthreads();
    for (int tile = warp; tile < tiles; tile += kWarps) {
        uint32_t vm_lo[4], vm_hi[4];  // tokens 0..15 and 16..31 of the tile
        ldmatrix_x4_trans(vm_lo, v_row0);
        ldmatrix_x4_trans(vm_hi, v_row0 + 512);
        __syncwarp();
        if (tile + kWarps < tiles) {
            const uint8_t *src = vc + (size_t)min((tile + kWarps) * 32 + lane, n - 1) * 32;
            cp_async16(v_land, src);
            cp_async16(v_land ^ 16u, src + 16);
        }
        const uint32_t p_tile = p_read + (uint32_t)tile * 64;
#pragma unroll 1
        for (int a = 0; a < 2; ++a) {
            const uint32_t vm[4] = {a ? vm_hi[0] : vm_lo[0], a ? vm_hi[1] : vm_lo[1], a ? vm_hi[2] : vm_lo[2], a ? vm_hi[3] : vm_lo[3]};
#pragma unroll
            for (int ksl = 0; ksl < 2; ++ksl) {
                uint32_t b0 = 0u;
                if (b_valid) b0 = lds32(p_tile + (uint32_t)(a * 2 + ksl) * 16);
                uint4 sa[2], sb[2];
#pragma unroll
                for (int tk = 0; tk < 2; ++tk) {
                    uint4 gth[2][2];
#pragma unroll
                    for (int sp = 0; sp < 2; ++sp)
#pragma unroll
                        for (int gsel = 0; gsel < 2; ++gsel) {
                            const uint32_t code256 = prmt(vm[ksl * 2 + sp], 0u, v_sel[tk][gsel]);
                            gth[sp][gsel] = lds128(v_off[sp][gsel] + code256 + code256);
                        }
                    sa[tk] = make_uint4(hadd2(gth[0][0].x, gth[1][0].x), hadd2(gth[0][0].y, gth[1][0].y),
                                        hadd2(gth[0][0].z, gth[1][0].z), hadd2(gth[0][0].w, gth[1][0].w));
                    sb[tk] = make_uint4(hadd2(gth[0][1].x, gth[1][1].x), hadd2(gth[0][1].y, gth[1][1].y),
                                        hadd2(gth[0][1].z, gth[1][1].z), hadd2(gth[0][1].w, gth[1][1].w));
                }
                const uint32_t a0[4] = {sa[0].x, sa[0].y, sa[0].z, sa[0].w}, a1[4] = {sa[1].x, sa[1].y, sa[1].z, sa[1].w};
                const uint32_t c0[4] = {sb[0].x, sb[0].y, sb[0].z, sb[0].w}, c1[4] = {sb[1].x, sb[1].y, sb[1].z, sb[1].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    mma1688(acc[2 * i], prmt(a0[i], a1[i], 0x5410u), prmt(c0[i], c1[i], 0x5410u), b0);
                    mma1688(acc[2 * i + 1], prmt(a0[i], a1[i], 0x7632u), prmt(c0[i], c1[i], 0x7632u), b0);
                }
            }
        }
        cp_async_wait_all();
        __syncwarp();  // the next tile's codes have landed and are visible to the whole warp
    }

    // ---- sum the warps, write this split's partial state ------------------------------------------------
    __syncthreads();  // the value tables are no longer read
    float *wacc = reinterpret_cast<float *>(tab_s);  // [warps][8 products x 4 registers][32 lanes]
    {
        float *base = wacc + (size_t)warp * 1024 + lane;
#pragma unroll
        for (int mm = 0; mm < 8; ++mm) {
            base[(mm * 4 + 0) * 32] = acc[mm][0];
            base[(mm * 4 + 1) * 32] = acc[mm][1];
            base[(mm * 4 + 2) * 32] = acc[mm][2];
            base[(mm * 4 + 3) * 32] = acc[mm][3];
        }
    }
    __syncthreads();
    for (int o = tid; o < 4 * kDim; o += kThreads) {
        // output o <-> (product mm, register j, lane of visiting order 0); its twin of order 1 is (mm, j^2, lane^2)
        const int mm = o >> 6, j = (o >> 4) & 3, l16 = o & 15;
        const int src_r8 = l16 >> 1, src_kq = l16 & 1;
        const int lane0 = src_r8 * 4 + src_kq;
        const int r = 2 * src_kq + (j & 1);
        if (r >= rep) continue;
        const int dim = (2 * src_r8 + (j >> 1)) * 8 + mm;
        float asum = 0.0f;
        for (int w = 0; w < kWarps; ++w) {
            const float *src = wacc + (size_t)w * 1024;
            asum += src[(mm * 4 + j) * 32 + lane0] + src[(mm * 4 + (j ^ 2)) * 32 + (lane0 ^ 2)];
        }
        float *dst = part + ((int64_t)split * rows + (int64_t)b * Hq + h * rep + r) * (kDim + 2);
        dst[2 + dim] = asum;
        if (dim == 0) {
            float lsum = 0.0f;
            for (int w = 0; w < kWarps; ++w) lsum += red_s[kRedFloats + w * 4 + r];
            dst[0] = m[r];
            dst[1] = lsum;
        }
    }
}

}  // namespace rotmma

bool attn_rotary_mma_supported(int Hq, int Hkv, int D, int G, int S, int K) {
    const int rep = Hkv > 0 ? Hq / Hkv : 0;
    return D == 128 && G == 16 && S == 2 && K == 256 && (rep == 1 || rep == 2 || rep == 4);
}

// Same grid and partial-state layout as the staged kernel: grid (splits, KV heads, batch rows), at most 4096
// tokens per block, partial states [split][B*Hq][2 + D] for attn_combine_kernel.
int attn_rotary_mma_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab, const __half *vtab,
                             const __half *rope, const int32_t *seq_start, const int32_t *seq_end, float *part, int B, int Hq,
                             int Hkv, int64_t T_cap, int splits, cudaStream_t stream) {
    static_assert(rotmma::kChunk == 4096, "the split count is chosen for 4096 tokens per block");
    cudaError_t e = cudaFuncSetAttribute(rotmma::attn_rotary_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, rotmma::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)splits, (unsigned)Hkv, (unsigned)B);
    rotmma::attn_rotary_mma_kernel<<<grid, rotmma::kThreads, rotmma::kSmemBytes, stream>>>(q, kcodes, vcodes, ktab, vtab, rope, seq_start,
                                                                                          seq_end, part, B, Hq, Hkv, T_cap, splits);
    return launch_status();
}

}  // namespace tacvq
