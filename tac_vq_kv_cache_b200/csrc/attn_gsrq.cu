// Decode-step attention over packed codes, specialised for the benchmark geometry:
// head_dim 128 = 16 groups x 8 dims, 2 residual stages (32 code bytes per token and side),
// 256 codewords, 4 query heads per KV head.
//
// Shape of the work.  Per (token, KV head) the kernel reads 64 bytes from HBM but has to perform 32
// table look-ups for the scores and 32 codeword fetches for the value row.  Shared memory moves
// 128 bytes per clock per SM, so the byte counts of those look-ups are what bounds the kernel:
//   scores  one 8-byte entry per K code: the entry holds the partial scores of all 4 query heads
//           as four 13-bit fixed-point fields, so four heads cost one load and the sums are
//           exact integer adds (two 32-bit adds add four heads).            32 x 8 B = 256 B
//   values  one 16-byte fp16 codeword per V code, fetched once and shared by the 4 heads
//           through a tensor-core product P^T.V (mma.sync m16n8k8).         32 x 16 B = 512 B
// 768 B / 128 B/clk = 6 clocks per (token, KV head) per SM is the floor of this design; everything
// else that touches the shared-memory pipe (code staging, probabilities, shuffles) is kept small:
//   K codes  two 16-byte global loads per token (lane = token), no staging
//   V codes  two 16-byte cp.async per token into a 1 KB buffer per warp, read back by two
//            ldmatrix.x4.trans, which hand every lane the codes of exactly the (token pair, group
//            pair) its A fragment covers - no byte shuffling in registers
//   softmax  the running reference is only re-derived (20 shuffles) when some lane's score exceeds
//            it by more than 8 octaves (one vote per tile); otherwise a tile costs no shuffle
//
// Conflict-free addressing for arbitrary codes.  Both tables are laid out so that the shared-memory
// bank is decided by the code SLOT (stage, group), never by the code value, and at every step the
// lanes that are served together work on different slots:
//   score table   entry(code, slot) at code*256 + slot*8; lane = token; at step i lane l handles
//                 slot i XOR perm(l), so the 16 lanes of a half warp hit 16 different bank pairs.
//   value table   entry(code, slot) at code*512 + pos(slot)*16, pos = (g/4)*8 + stage*4 + g%4; the 8
//                 lanes of a quarter warp (two group pairs x four token pairs) fetch 8 different
//                 slots: the four token pairs visit (stage, group of the pair) in four different
//                 orders.  Stage order is flipped by the cp.async that lands the codes (odd token
//                 pairs swap their stage halves), group order by the byte selector; lanes whose order
//                 swaps the two A-fragment rows are kept apart in the product by giving the 8
//                 columns of the B operand to (4 heads) x (2 visiting orders).
//
// Two launches per call, chained as programmatic dependents (each lets its successor be scheduled at
// once; the successor waits for it before touching its results):
//   prepare  one block per (batch row, KV head, stage): the score table of the pair (q . codeword for
//            4096 codewords x 4 heads straight from the fp16 K tables, quantised to 13 bits), written to
//            scratch in the order the scan's shared memory wants; its share of the V codewords in that
//            order; and, in a decode step, the codes of the pair's new K or V row and the visible ranges.  A build costs about 5 us of a 512-thread
//            block per stage (64 values per thread, quarter-rate conversions); building inside the scan
//            was measured twice and repeats that for every block that enters a pair (3.3 per pair).
//   scan     a persistent grid (one block per SM) walks the flattened (KV head, batch row, 32-token
//            tile) space; every block gets an equal share of work units.  When it enters a new (batch
//            row, KV head) pair it copies that pair's score table (64 KB, flat) and, when the head
//            changed, the head's V codewords, which the prepare grid wrote in their bank-striped
//            order (128 KB, flat).  It writes one partial
//            softmax state per pair it touches, then marks it; the block that finds every partial of a
//            pair marked merges them (log-sum-exp) and writes fp16 output and/or fp32 state.  A pair
//            that lies inside one block's share is written directly.
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122 and the
// decoded window of :53-70 (no rotary step).  Differences from that dense path, all inside the
// 2e-3 tolerance: a score is the sum of per-stage table entries (the reference rounds the rebuilt
// key to fp16 first), entries are quantised to 13 bits of the widest slot range of their head,
// probabilities enter the tensor-core product as fp16, and the two V stages are added in fp16.

#include <atomic>

#include "common.cuh"
#include "encode_rows.cuh"

namespace tacvq {

namespace gsrq {

#ifndef TACVQ_GSRQ_THREADS
#define TACVQ_GSRQ_THREADS 512
#endif
constexpr int kThreads = TACVQ_GSRQ_THREADS;
constexpr int kWarps = kThreads / 32;
constexpr int kDim = 128, kGroups = 16, kStages = 2, kSub = 8, kRep = 4, kSlots = 32, kWords = 256;
constexpr int kTile = 32;          // tokens per warp tile
constexpr int kMaxBatch = 512;
#ifndef TACVQ_ITEM_COST
#define TACVQ_ITEM_COST 48
#endif
#ifndef TACVQ_GSRQ_UNROLL_K
#define TACVQ_GSRQ_UNROLL_K 2  // 1: the two stages of the score phase as a rolled loop, 2: unrolled
#endif
#ifndef TACVQ_GSRQ_UNROLL_V
#define TACVQ_GSRQ_UNROLL_V 1  // 1: the two 16-token halves of the value phase as a rolled loop, 2: unrolled
#endif
#ifndef TACVQ_GSRQ_EARLY_K
#define TACVQ_GSRQ_EARLY_K 0  // 1: the next tile's K codes are requested before the score phase (8 more registers live)
#endif
#ifndef TACVQ_GSRQ_VPERM
#define TACVQ_GSRQ_VPERM 1  // 1: the prepare grid writes the V codewords in shared-memory order, the scan copies them flat
#endif
#ifndef TACVQ_GSRQ_LAZY_MAX
#define TACVQ_GSRQ_LAZY_MAX 1  // 0: every tile reduces its maximum over the warp (20 shuffles)
#endif
constexpr int kUnrollScore = TACVQ_GSRQ_UNROLL_K, kUnrollValue = TACVQ_GSRQ_UNROLL_V;
constexpr int kItemCost = TACVQ_ITEM_COST;         // fixed cost of starting a (row, head) pair in a block, in 32-token tiles
constexpr int kMaxScanBlocks = 256;  // persistent grid size (one block per SM) never exceeds this
constexpr int kStateWidth = kDim + 2;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleGap = 8.0f;  // log2 units a score may exceed the running reference before rescaling
constexpr int kEntryMax = 8191;      // 13-bit fields: 8 of them sum below 2^16

// shared-memory carve-up (bytes)
constexpr int kLutBytes = kWords * kSlots * 8;              // 65536
constexpr int kVtabBytes = kWords * kSlots * 16;            // 131072
constexpr int kVCodeBytes = kTile * 32;                     // one tile of V codes per warp
constexpr int kProbStride = 72;                             // bytes per head of the fp16 probabilities: 64 + 8, so the four heads' reads hit different banks
constexpr int kStagePerWarp = kVCodeBytes + 4 * kProbStride + 32;  // + fp16 probabilities [4 heads][32 tokens], 64-byte multiple
constexpr int kStageBytes = kWarps * kStagePerWarp;         // 20480 at 16 warps (also scratch of the table build)
constexpr int kPrefixBytes = (kMaxBatch + 8) * 4 + 12 * 4;
constexpr int kSmemBytes = kLutBytes + kVtabBytes + kStageBytes + kPrefixBytes;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
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
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts16(uint32_t addr, unsigned short v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
// four 8x8 b16 matrices, transposed: lane (r8 = lane/4, kq = lane%4) receives of matrix j the elements
// [row 2kq][column r8] (low half) and [row 2kq+1][column r8] (high half); lane l supplies the address of
// row l%8 of matrix l/8
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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start
// before its predecessor has finished; it must not touch the predecessor's results before this wait.
__device__ __forceinline__ void wait_for_previous_kernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {  // 2^x, ex2.approx: 2^-inf = +0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

// Tiles of batch row b and the running totals, shared by the scan and the merge kernel.
__device__ __forceinline__ int row_tokens(const int32_t *seq_start, const int32_t *seq_end, int b, int T_cap) {
    int lo = seq_start ? seq_start[b] : 0;
    int hi = seq_end ? seq_end[b] : T_cap;
    lo = max(lo, 0);
    hi = min(hi, T_cap);
    return hi > lo ? hi - lo : 0;
}

__device__ __forceinline__ long long block_first_tile(long long total, int block, int blocks) {
    return total * block / blocks;
}

// position of slot (stage s, group g) inside a code's 512-byte row of the value table
__device__ __forceinline__ int value_pos(int s, int g) { return (g >> 2) * 8 + s * 4 + (g & 3); }

__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

using NewToken = GsrqNewToken;

// ------------------------------------------------------------------------------------------------
// prepare kernel: block (pair p = h*B + b, stage) builds one stage of the pair's score table
// ------------------------------------------------------------------------------------------------
//   lut_g[p][code][slot]   8 bytes: four 13-bit fields, field r = round((q_r . word - min_slot_r) / step_stage_r)
//   scale_g[p][stage*8+r]  step_stage_r * log2 e;  [stage*8+4+r] = sum over the stage's slots of min_slot_r * log2 e
// A lane always works on group lane % 16 and on one of the two codes its warp covers per round, so the
// 16 lanes of a half warp read sixteen 4 KB-strided table rows in 32-byte sectors that the other half
// warp completes, and write 128 contiguous bytes.  Each stage has its own step, so the finer second
// stage keeps its precision.
constexpr int kPrepThreads = 512;
constexpr int kPrepWarps = kPrepThreads / 32;
constexpr int kPrepCodes = kWords / (2 * kPrepWarps);  // codes per thread

__global__ void __launch_bounds__(kPrepThreads)
attn_gsrq_prepare_kernel(const __half *__restrict__ q, const __half *__restrict__ ktab, const __half *__restrict__ vtab,
                         uint2 *__restrict__ lut_g, float *__restrict__ scale_g, uint4 *__restrict__ vperm_g, int B, int Hkv, const NewToken fresh) {
    __shared__ float red[kPrepWarps * 8 * 32];  // [warp][min x4, max x4][lane]
    __shared__ float red2[8 * 32];
    launch_dependents();  // the scan may be scheduled as soon as SMs free up; it waits for this grid itself
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pair = blockIdx.x >> 1, stage = blockIdx.x & 1;
    const int h = pair / B, b = pair % B;
    const int Hq = Hkv * kRep;
    const int g = lane & 15, half = lane >> 4;
    // A decode step's new token: this block (pair, side = stage) encodes the 16 groups of the pair's new K
    // (side 0) or V (side 1) row, a warp per group, with the arithmetic of the row-at-a-time encode kernel.
    // The words of both stages are requested at once (one memory latency instead of two); the codes are kept
    // in registers and stored after the wait below.  None of these inputs is produced by this chain.
    int fresh_code[kStages] = {0, 0};
    if (fresh.k_rows != nullptr) {
        static_assert(kPrepWarps == kGroups && kStages == 2 && kWords == 256, "a warp per group, 8 words per lane and stage");
        const __half *side_tab = stage ? vtab : ktab;
        const uint4 *words0 = reinterpret_cast<const uint4 *>(side_tab + (((size_t)h * kStages + 0) * kGroups + warp) * kWords * kSub);
        const uint4 *words1 = words0 + (size_t)kGroups * kWords;
        uint4 w0[8], w1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w0[i] = __ldg(words0 + lane + 32 * i);
#pragma unroll
        for (int i = 0; i < 8; ++i) w1[i] = __ldg(words1 + lane + 32 * i);
        const size_t at = ((size_t)b * Hkv + h) * kDim + warp * kSub;
        float res[kSub];
        if (fresh.rows_f32) {
            const float4 *src = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(stage ? fresh.v_rows : fresh.k_rows) + at);
            const float4 lo = src[0], hi = src[1];
            res[0] = lo.x, res[1] = lo.y, res[2] = lo.z, res[3] = lo.w, res[4] = hi.x, res[5] = hi.y, res[6] = hi.z, res[7] = hi.w;
        } else {
            unpack8(*reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(stage ? fresh.v_rows : fresh.k_rows) + at), res);
        }
        fresh_code[0] = nearest_of_fetched_words(res, w0, lane);
        {
            float c[kSub];
            unpack8(__ldg(words0 + fresh_code[0]), c);
#pragma unroll
            for (int i = 0; i < kSub; ++i) res[i] = __fsub_rn(res[i], c[i]);
        }
        fresh_code[1] = nearest_of_fetched_words(res, w1, lane);
    }
    // inputs of the table build (q and the K tables) are not produced by the kernels of this chain either
    const uint4 *tab = reinterpret_cast<const uint4 *>(ktab + (((size_t)h * kStages + stage) * kGroups + g) * kWords * kSub);
    uint4 raw[kPrepCodes];
#pragma unroll
    for (int c = 0; c < kPrepCodes; ++c) raw[c] = __ldg(tab + warp * 2 + half + 2 * kPrepWarps * c);
    uint4 qraw[kRep];
#pragma unroll
    for (int r = 0; r < kRep; ++r) qraw[r] = __ldg(reinterpret_cast<const uint4 *>(q + ((size_t)b * Hq + h * kRep + r) * kDim + g * kSub));
    float qv[kRep][kSub];
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
        const uint4 qr = qraw[r];
        const __half2 *hp = reinterpret_cast<const __half2 *>(&qr);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(hp[i]);
            qv[r][2 * i] = f.x;
            qv[r][2 * i + 1] = f.y;
        }
    }
    float val[kPrepCodes][kRep];
    float mn[kRep], mx[kRep];
#pragma unroll
    for (int r = 0; r < kRep; ++r) { mn[r] = INFINITY; mx[r] = -INFINITY; }
#pragma unroll
    for (int c = 0; c < kPrepCodes; ++c) {
        const __half2 *hp = reinterpret_cast<const __half2 *>(&raw[c]);
        float w[kSub];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(hp[i]);
            w[2 * i] = f.x;
            w[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < kSub; ++i) dot = fmaf(qv[r][i], w[i], dot);
            val[c][r] = dot;
            mn[r] = fminf(mn[r], dot);
            mx[r] = fmaxf(mx[r], dot);
        }
    }
    // range of every (group, head) over the 256 codes: over warps through shared memory in two levels
    // (8 x 32 threads fold the warps), then over the two lane halves and, for the common step, over the
    // 16 groups by shuffles
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
        red[(warp * 8 + r) * 32 + lane] = mn[r];       // lane-major: conflict-free writes and reads
        red[(warp * 8 + 4 + r) * 32 + lane] = mx[r];
    }
    __syncthreads();
    if (tid < 8 * 32) {
        const int v = tid >> 5;
        float t = red[v * 32 + lane];
        for (int w = 1; w < kPrepWarps; ++w) {
            const float o = red[(w * 8 + v) * 32 + lane];
            t = v < 4 ? fminf(t, o) : fmaxf(t, o);
        }
        red2[v * 32 + lane] = t;
    }
    __syncthreads();
    float inv_step[kRep], scale_step[kRep], scale_offs[kRep];
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
        mn[r] = red2[r * 32 + lane];
        mx[r] = red2[(4 + r) * 32 + lane];
        // the two lane halves hold the two codes of a round for the same group: fold them first
        mn[r] = fminf(mn[r], __shfl_xor_sync(0xffffffffu, mn[r], 16));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
        float range = mx[r] - mn[r];
        float offs = mn[r];
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) {  // over the 16 groups
            range = fmaxf(range, __shfl_xor_sync(0xffffffffu, range, off));
            offs += __shfl_xor_sync(0xffffffffu, offs, off);
        }
        const float step = range > 0.0f ? range / (float)kEntryMax : 1.0f;
        inv_step[r] = 1.0f / step;
        scale_step[r] = step * kLog2e;
        scale_offs[r] = offs * kLog2e;
    }
    uint32_t packed[kPrepCodes][2];
#pragma unroll
    for (int c = 0; c < kPrepCodes; ++c) {
        uint32_t e[kRep];
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            // round to nearest by adding 2^23 (full-rate add and mask instead of a quarter-rate conversion);
            // the argument is in [0, 8191.x]
            const float t = fmaf(val[c][r] - mn[r], inv_step[r], 8388608.0f);
            e[r] = min((uint32_t)kEntryMax, __float_as_uint(t) & 0x3fffu);
        }
        packed[c][0] = e[0] | (e[1] << 16);
        packed[c][1] = e[2] | (e[3] << 16);
    }
    // The scratch written below is read by the scan of the call before this one, which may still be
    // running when this grid starts: wait for everything before this grid, then write.
    wait_for_previous_kernel();
    if (fresh.k_rows != nullptr) {
        // the scan before this grid read the ranges and the code buffers up to its own end; both may change now
        if (lane == 0) {
            uint8_t *dst = (stage ? fresh.vcodes : fresh.kcodes) + (((size_t)b * Hkv + h) * (size_t)fresh.T_cap + (size_t)fresh.position) * kSlots;
#pragma unroll
            for (int s = 0; s < kStages; ++s) dst[s * kGroups + warp] = (uint8_t)fresh_code[s];
        }
        if (blockIdx.x == 0) {
            for (int i = tid; i < B; i += kPrepThreads) {
                fresh.seq_start[i] = fresh.start;
                fresh.seq_end[i] = fresh.end;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < kPrepCodes; ++c) {
        const int code = warp * 2 + half + 2 * kPrepWarps * c;
        lut_g[((size_t)pair * kWords + code) * kSlots + stage * kGroups + g] = make_uint2(packed[c][0], packed[c][1]);
    }
    if (tid == 0) {
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            scale_g[((size_t)pair * kStages + stage) * 8 + r] = scale_step[r];
            scale_g[((size_t)pair * kStages + stage) * 8 + 4 + r] = scale_offs[r];
        }
    }
#if TACVQ_GSRQ_VPERM
    {
        const int perm_total = Hkv * kWords * kSlots;
        const int perm_per_block = (perm_total + (int)gridDim.x - 1) / (int)gridDim.x;
        for (int local = tid; local < perm_per_block; local += kPrepThreads) {
            const int e = blockIdx.x * perm_per_block + local;
            if (e < perm_total) {
                const int hh = e >> 13, code = (e >> 5) & 255, pos = e & 31;
                const int s = (pos >> 2) & 1, gg = ((pos >> 3) << 2) | (pos & 3);
                vperm_g[e] = __ldg(reinterpret_cast<const uint4 *>(vtab + ((((size_t)hh * kStages + s) * kGroups + gg) * kWords + code) * kSub));
            }
        }
    }
#endif
}

// ------------------------------------------------------------------------------------------------
// partial states of a pair: who writes them, how they are merged
// ------------------------------------------------------------------------------------------------
// Block c owns work units [total*c/blocks, total*(c+1)/blocks); unit u therefore lies in block
// ((u+1)*blocks - 1) / total.  The blocks that scan tiles of a pair are exactly those from the owner of the
// pair's first tile unit to the owner of its last unit; block c stores its partial state at index pair + c.
__device__ __forceinline__ int block_of_unit(int unit, int total_units, int blocks) {
    return (int)(((long long)(unit + 1) * blocks - 1) / total_units);
}

// log-sum-exp merge of n_parts consecutive partial states by the whole block (4 heads x 128 channels); the
// states are fetched eight at a time in one round trip
__device__ void merge_pair_parts(const float *part, int first, int n_parts, int b, int h, int Hkv, __half *out,
                                 float *state_out) {
    const int Hq = Hkv * kRep;
    for (int o = threadIdx.x; o < kRep * kDim; o += blockDim.x) {
        const int r = o >> 7, dim = o & 127;
        float top = -INFINITY, lsum = 0.0f, asum = 0.0f;
        for (int i0 = 0; i0 < n_parts; i0 += 8) {
            float mc[8], lc[8], ac[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float *st = part + ((size_t)(first + min(i0 + i, n_parts - 1)) * kRep + r) * kStateWidth;
                mc[i] = __ldcg(st);
                lc[i] = __ldcg(st + 1);
                ac[i] = __ldcg(st + 2 + dim);
            }
            float ntop = top;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i0 + i < n_parts) ntop = fmaxf(ntop, mc[i]);
            if (ntop == -INFINITY) continue;
            const float f = __expf(top - ntop);  // 0 while nothing has been added yet
            lsum *= f;
            asum *= f;
            top = ntop;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i0 + i < n_parts && mc[i] != -INFINITY) {
                    const float sc = __expf(mc[i] - top);
                    lsum += sc * lc[i];
                    asum += sc * ac[i];
                }
            }
        }
        const size_t row = (size_t)b * Hq + h * kRep + r;
        if (out) out[row * kDim + dim] = __float2half_rn(lsum > 0.0f ? asum / lsum : 0.0f);
        if (state_out) {
            float *dst = state_out + row * kStateWidth;
            if (dim == 0) {
                dst[0] = top;
                dst[1] = lsum;
            }
            dst[2 + dim] = asum;
        }
    }
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// ------------------------------------------------------------------------------------------------
// scan kernel
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1)
attn_gsrq_scan_kernel(const uint8_t *__restrict__ kcodes, const uint8_t *__restrict__ vcodes,
                      const uint2 *__restrict__ lut_g, const float *__restrict__ scale_g,
                      const __half *__restrict__ vtab, const uint4 *__restrict__ vperm_g, const int32_t *__restrict__ seq_start,
                      const int32_t *__restrict__ seq_end, float *__restrict__ part, unsigned long long *__restrict__ marks,
                      __half *__restrict__ out, float *__restrict__ state_out, int B, int Hkv, int T_cap,
                      unsigned long long epoch) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *lut_s = smem;
    unsigned char *vtab_s = smem + kLutBytes;
    unsigned char *stage_s = vtab_s + kVtabBytes;
    int *prefix_s = reinterpret_cast<int *>(stage_s + kStageBytes);
    float *scale_s = reinterpret_cast<float *>(prefix_s + kMaxBatch + 8);  // 16-byte aligned: 12 floats

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = Hkv * kRep;

    // ---- work prefix over batch rows: a non-empty row costs its tiles plus kItemCost units (table
    //      copies, pipeline fill and drain, merge), so blocks that enter more pairs get fewer tiles ------
    auto work_prefix = [&]() {
        if (warp == 0) {
            int running = 0;
            for (int b0 = 0; b0 < B; b0 += 32) {
                const int b = b0 + lane;
                int tiles = (b < B) ? (row_tokens(seq_start, seq_end, b, T_cap) + kTile - 1) / kTile : 0;
                if (tiles > 0) tiles += kItemCost;
                int incl = tiles;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int n = __shfl_up_sync(0xffffffffu, incl, off);
                    if (lane >= off) incl += n;
                }
                if (b < B) prefix_s[b] = running + incl - tiles;
                running += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) prefix_s[B] = running;
        }
        __syncthreads();
    };
    // value codewords of a head in the bank-striped rows [word][position].  Default: a flat 128 KB copy of what the
    // prepare grid wrote in that order.  Without TACVQ_GSRQ_VPERM the block gathers them from the fp16 V tables
    // [stage][group][word][8] itself (per trip a warp copies 4 neighbouring words of 8 positions with different
    // banks: whole 32-byte sectors in, no conflicts out) and starts with the head it will most likely begin in
    // before it waits for the prepare grid; measured 6 us per step slower than the flat copy.
    auto copy_value_table = [&](int h) {
#if TACVQ_GSRQ_VPERM
        const uint4 *flat = vperm_g + (size_t)h * (kWords * kSlots);
        for (int e = tid; e < kWords * kSlots; e += kThreads) cp_async16(smem_u32(vtab_s) + e * 16, flat + e);
#else
        const __half *src = vtab + (size_t)h * (kStages * kGroups * kWords * kSub);
        const uint32_t dst = smem_u32(vtab_s);
        for (int idx = tid; idx < kWords * kSlots; idx += kThreads) {
            const int pos = ((idx >> 5) & 3) * 8 + (idx & 7);
            const int word = ((idx >> 7) << 2) | ((idx >> 3) & 3);
            const int s = (pos >> 2) & 1, g = ((pos >> 3) << 2) | (pos & 3);
            cp_async16(dst + word * (kSlots * 16) + pos * 16, src + ((size_t)(s * kGroups + g) * kWords + word) * kSub);
        }
#endif
    };

    // The score and value tables come from the prepare grid, and the visible ranges and newest code rows may be
    // written by it too (a decode step's new token): of the kernels of this chain, nothing is read before the wait.
#if TACVQ_GSRQ_VPERM
    int loaded_head = -1;
#else
    int loaded_head = min((int)(((long long)blockIdx.x * Hkv) / (long long)gridDim.x), Hkv - 1);
    copy_value_table(loaded_head);
#endif
    wait_for_previous_kernel();
    launch_dependents();  // the next kernel on the stream may take SMs as they free up; it waits for this grid itself
    work_prefix();
    const int tiles_per_head = prefix_s[B];
    const int total_tiles = tiles_per_head * Hkv;  // fits: checked by the dispatcher
    const int blocks = min((int)gridDim.x, max(total_tiles, 1));  // every working block owns at least one unit
    int cursor = 0, my_end = 0;
    if ((int)blockIdx.x < blocks) {
        cursor = (int)block_first_tile(total_tiles, blockIdx.x, blocks);
        my_end = (int)block_first_tile(total_tiles, blockIdx.x + 1, blocks);
    }

    // ---- per-lane constants ------------------------------------------------------------------
    // score side: lane = token, slot visiting order permuted by XOR so a half warp covers 16 bank pairs
    const uint32_t k_word_swap = lane & 3;
    const uint32_t k_byte_xor = (lane >> 2) & 3;
    const uint32_t k_lane_xor = (k_word_swap << 5) | (k_byte_xor << 3);
    uint32_t k_sel[4];
#pragma unroll
    for (int bi = 0; bi < 4; ++bi) k_sel[bi] = 0x4404u | (((bi ^ k_byte_xor) & 3u) << 4);
    // value side: lane = (row r8, token-pair column kq) of the A fragment; rows r8 / r8+8 carry groups
    // 2*r8 / 2*r8+1.  Static step (sp, gsel) fetches stage sp ^ (kq & 1), group 2*r8 + (gsel ^ (kq >> 1)).
    const int r8 = lane >> 2, kq = lane & 3;
    uint32_t v_off[2][2], v_sel[2][2];
#pragma unroll
    for (int sp = 0; sp < 2; ++sp)
#pragma unroll
        for (int gsel = 0; gsel < 2; ++gsel) {
            const int s = sp ^ (kq & 1), gh = gsel ^ (kq >> 1);
            v_off[sp][gsel] = smem_u32(vtab_s) + value_pos(s, 2 * r8 + gh) * 16;
        }
#pragma unroll
    for (int tk = 0; tk < 2; ++tk)
#pragma unroll
        for (int gsel = 0; gsel < 2; ++gsel)
            v_sel[tk][gsel] = 0x4404u | ((uint32_t)(tk * 2 + (gsel ^ (kq >> 1))) << 4);  // code byte -> bits 8..15
    const int x_class = kq >> 1;                 // which visiting order this lane's tokens use
    const int b_head = r8 & 3;                   // B-fragment column n = r8: head n&3, class n>>2
    const bool b_valid = (r8 >> 2) == x_class;
    const uint32_t lut_base = smem_u32(lut_s);
    const uint32_t scale_u32 = smem_u32(scale_s);
    const uint32_t vstage_u32 = smem_u32(stage_s) + warp * kStagePerWarp;
    const uint32_t pstage_u32 = vstage_u32 + kVCodeBytes;
    // landing place of this lane's (= token's) two 16-byte stage halves: odd token pairs swap the halves
    // (stage order of the value look-ups), and tokens 4..7 of every eight swap them once more so that the
    // eight 16-byte rows of an ldmatrix tile cover all 32 banks
    const uint32_t v_land = vstage_u32 + lane * 32 + ((((lane >> 1) ^ (lane >> 2)) & 1) * 16);
    // ldmatrix row addresses for tokens 0..15 of the tile (the second call adds 512 bytes): matrix j = lane / 8
    // holds tokens 8*(j/2) .. +7 of half j%2, row = lane % 8
    const uint32_t v_row0 = vstage_u32 + (8 * (lane >> 4) + (lane & 7)) * 32 + ((((lane >> 3) & 1) ^ ((lane >> 2) & 1)) * 16);
    const uint32_t p_read = pstage_u32 + (uint32_t)(b_head * kProbStride + kq * 4);  // B fragment of step ks: + ks * 16

    while (cursor < my_end) {
        // ---- which (head, batch row) does the cursor fall in ---------------------------------
        const int h = (int)(cursor / tiles_per_head);
        const int rem = cursor - h * tiles_per_head;
        int b = 0;
        {
            int lo = 0, hi = B;  // largest b with prefix[b] <= rem and a non-empty row
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (prefix_s[mid] <= rem) lo = mid; else hi = mid;
            }
            b = lo;
        }
        const int pair_first = h * tiles_per_head + prefix_s[b];
        const int pair_end = h * tiles_per_head + prefix_s[b + 1];
        const int item_end = pair_end < my_end ? pair_end : my_end;
        // work units -> tiles of the pair: the first kItemCost units of a pair carry no tile
        const int tile_lo = max(cursor - pair_first - kItemCost, 0), tile_hi = max(item_end - pair_first - kItemCost, 0);
        if (tile_hi <= tile_lo) {  // this block's share ends inside the cost zone: nothing to scan for this pair
            cursor = item_end;
            continue;
        }
        const int tok_lo_row = max(seq_start ? seq_start[b] : 0, 0);
        const int n_tokens = row_tokens(seq_start, seq_end, b, T_cap);
        const int pair = h * B + b;

        __syncthreads();  // previous item fully merged: tables and staging may be overwritten

        // ---- tables of this item: the head's V codewords when the head changed, and the pair's score table,
        //      which the prepare grid laid out for shared memory (a flat copy) ----------------------------------
        if (h != loaded_head) {
            loaded_head = h;
            copy_value_table(h);
        }
        {
            const unsigned char *l_src = reinterpret_cast<const unsigned char *>(lut_g) + (size_t)pair * kLutBytes;
            for (int j = tid; j < kLutBytes / 16; j += kThreads) cp_async16(lut_base + j * 16, l_src + (size_t)j * 16);
        }
        // the pair's steps and offset stay in shared memory (three broadcast loads per tile) rather than in
        // twelve registers of every thread: scale_s = step of stage 0 x4, step of stage 1 x4, total offset x4
        if (tid < 12) {
            const float *sg = scale_g + (size_t)pair * 16;
            scale_s[tid] = tid < 4 ? __ldg(sg + tid) : tid < 8 ? __ldg(sg + 4 + tid) : __ldg(sg + tid - 4) + __ldg(sg + tid + 4);
        }
        cp_async_wait_all();
        __syncthreads();  // tables ready

        // ---- scan this block's tiles of the pair ----------------------------------------------
        float acc[8][4];
#pragma unroll
        for (int mm = 0; mm < 8; ++mm)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mm][i] = 0.0f;
        float m_ref[kRep], l_lane[kRep];
#pragma unroll
        for (int r = 0; r < kRep; ++r) { m_ref[r] = -INFINITY; l_lane[r] = 0.0f; }

        const size_t row_base = ((size_t)b * Hkv + h) * (size_t)T_cap;

        // codes of a tile: lane = token; rows past the end of the range re-read the last valid row
        const uint8_t *k_row = kcodes + (row_base + (size_t)tok_lo_row) * 32, *v_row_g = vcodes + (row_base + (size_t)tok_lo_row) * 32;
        auto code_offset = [=](int tile) -> uint32_t {  // byte offset of this lane's 32-byte code row (T_cap <= 2^26)
            return (uint32_t)min(tile * kTile + lane, n_tokens - 1) * 32u;
        };
        uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0;
        if (tile_lo + warp < tile_hi) {
            const uint32_t off = code_offset(tile_lo + warp);
            const uint4 *kp = reinterpret_cast<const uint4 *>(k_row + off);
            k0 = ldg_stream(kp); k1 = ldg_stream(kp + 1);
            cp_async16(v_land, v_row_g + off);
            cp_async16(v_land ^ 16u, v_row_g + off + 16);
        }

        for (int tile = tile_lo + warp; tile < tile_hi; tile += kWarps) {
            const bool live = tile * kTile + lane < n_tokens;
            const bool more = tile + kWarps < tile_hi;
            __syncwarp();  // the previous tile's readers are done with the probability staging
            const uint32_t next_off = code_offset(tile + kWarps);

            // -- scores: 32 look-ups of 8 bytes, four 13-bit fields each, flushed every 8 look-ups
            //    (the two stages run as a rolled loop: half the code and half the values in flight per pass)
#if TACVQ_GSRQ_EARLY_K
            const uint4 kc0 = k0, kc1 = k1;
            if (more) {  // the next tile's K codes travel during this whole tile
                const uint4 *kp = reinterpret_cast<const uint4 *>(k_row + next_off);
                k0 = ldg_stream(kp); k1 = ldg_stream(kp + 1);
                if (tile + 3 * kWarps < tile_hi) prefetch_l2(reinterpret_cast<const unsigned char *>(kp) + (size_t)2 * kWarps * kTile * 32);  // L2 two rounds ahead
            }
#else
            const uint4 &kc0 = k0, &kc1 = k1;
#endif
            float sc[kRep];
            {
                const uint4 ofs = lds128(scale_u32 + 32);
                sc[0] = __uint_as_float(ofs.x); sc[1] = __uint_as_float(ofs.y);
                sc[2] = __uint_as_float(ofs.z); sc[3] = __uint_as_float(ofs.w);
            }
#pragma unroll kUnrollScore
            for (int st = 0; st < kStages; ++st) {  // k0 holds the codes of stage 0, k1 those of stage 1
                uint32_t kw[4] = {st ? kc1.x : kc0.x, st ? kc1.y : kc0.y, st ? kc1.z : kc0.z, st ? kc1.w : kc0.w};
                if (k_word_swap & 1) {
                    uint32_t t = kw[0]; kw[0] = kw[1]; kw[1] = t;
                    t = kw[2]; kw[2] = kw[3]; kw[3] = t;
                }
                if (k_word_swap & 2) {
                    uint32_t t = kw[0]; kw[0] = kw[2]; kw[2] = t;
                    t = kw[1]; kw[1] = kw[3]; kw[3] = t;
                }
                const uint32_t lut_st = lut_base + (uint32_t)st * (kGroups * 8);
                uint32_t isum[kRep] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int wp = 0; wp < 2; ++wp) {
                    uint32_t lo = 0u, hi = 0u;
#pragma unroll
                    for (int wj = 0; wj < 2; ++wj) {
                        const int wi = wp * 2 + wj;
#pragma unroll
                        for (int bi = 0; bi < 4; ++bi) {
                            const uint32_t code256 = prmt(kw[wi], 0u, k_sel[bi]);
                            const uint32_t addr = ((code256 | (uint32_t)(wi * 32 + bi * 8)) ^ k_lane_xor) + lut_st;
                            const uint2 e = lds64(addr);
                            lo += e.x;
                            hi += e.y;
                        }
                    }
                    isum[0] += lo & 0xffffu;
                    isum[1] += lo >> 16;
                    isum[2] += hi & 0xffffu;
                    isum[3] += hi >> 16;
                }
                const uint4 stp = lds128(scale_u32 + st * 16);
                sc[0] = fmaf((float)isum[0], __uint_as_float(stp.x), sc[0]);
                sc[1] = fmaf((float)isum[1], __uint_as_float(stp.y), sc[1]);
                sc[2] = fmaf((float)isum[2], __uint_as_float(stp.z), sc[2]);
                sc[3] = fmaf((float)isum[3], __uint_as_float(stp.w), sc[3]);
            }

#if !TACVQ_GSRQ_EARLY_K
            if (more) {  // the next tile's K codes travel during the value phase and take over the registers freed above
                const uint4 *kp = reinterpret_cast<const uint4 *>(k_row + next_off);
                k0 = ldg_stream(kp); k1 = ldg_stream(kp + 1);
                if (tile + 3 * kWarps < tile_hi) prefetch_l2(reinterpret_cast<const unsigned char *>(kp) + (size_t)2 * kWarps * kTile * 32);  // L2 two rounds ahead
            }
#endif

            // -- softmax bookkeeping (log2 domain).  The reference m_ref only has to stay within
            //    kRescaleGap of the largest score seen; it is re-derived when some live lane exceeds that.
            bool grow = false;
#pragma unroll
            for (int r = 0; r < kRep; ++r) {
                if (!live) sc[r] = -INFINITY;
                grow = grow || (sc[r] > m_ref[r] + kRescaleGap);
            }
#if TACVQ_GSRQ_LAZY_MAX
            grow = __any_sync(0xffffffffu, grow);
#else
            grow = true;
#endif
            if (grow) {  // warp-uniform; always taken by a warp's first tile (m_ref = -inf)
                float f[kRep];
#pragma unroll
                for (int r = 0; r < kRep; ++r) {
                    float t = sc[r];
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, off));
                    const float nref = fmaxf(m_ref[r], t);
                    f[r] = fast_exp2(m_ref[r] - nref);  // 0 on the first tile (m_ref = -inf)
                    m_ref[r] = nref;
                    l_lane[r] *= f[r];
                }
                // accumulator columns of this lane are heads (2kq)&3 and (2kq+1)&3
                const float f0 = (kq & 1) ? f[2] : f[0];
                const float f1 = (kq & 1) ? f[3] : f[1];
#pragma unroll
                for (int mm = 0; mm < 8; ++mm) {
                    acc[mm][0] *= f0; acc[mm][1] *= f1; acc[mm][2] *= f0; acc[mm][3] *= f1;
                }
            }
#pragma unroll
            for (int r = 0; r < kRep; ++r) {
                const float p = fast_exp2(sc[r] - m_ref[r]);
                l_lane[r] += p;
                sts16(pstage_u32 + (uint32_t)(r * kProbStride + lane * 2), __half_as_ushort(__float2half_rn(p)));
            }
            // -- value codes of this tile: landed by cp.async, handed out by ldmatrix; register j of call a holds,
            //    for the lane's token pair of 8-token step 2a + j/2, the two group codes of stage (j%2) ^ (kq&1)
            cp_async_wait_all();
            __syncwarp();  // also orders the probabilities written above before their reads below

            // -- values: per 8-token step gather this lane's two tokens (4 codewords each), add the two
            //    stages, pair the tokens into A fragments and issue 8 m16n8k8 products; 16 tokens per pass of a
            //    rolled loop
            uint32_t vm_lo[4], vm_hi[4];  // tokens 0..15 and 16..31 of the tile
            ldmatrix_x4_trans(vm_lo, v_row0);
            ldmatrix_x4_trans(vm_hi, v_row0 + 512);
            __syncwarp();  // every lane has all its codes: the buffer may take the next tile, a whole tile ahead of its use
            if (more) {
                cp_async16(v_land, v_row_g + next_off);
                cp_async16(v_land ^ 16u, v_row_g + next_off + 16);
                if (tile + 3 * kWarps < tile_hi) prefetch_l2(v_row_g + next_off + (size_t)2 * kWarps * kTile * 32);
            }
#pragma unroll kUnrollValue
            for (int a = 0; a < 2; ++a) {
                const uint32_t vm[4] = {a ? vm_hi[0] : vm_lo[0], a ? vm_hi[1] : vm_lo[1], a ? vm_hi[2] : vm_lo[2], a ? vm_hi[3] : vm_lo[3]};
#pragma unroll
                for (int ksl = 0; ksl < 2; ++ksl) {
                    uint32_t b0 = 0u;
                    if (b_valid) b0 = lds32(p_read + (uint32_t)(a * 2 + ksl) * 16);
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
        }

        // ---- merge the warps of this block into one partial state of the pair ------------------
        float l_warp[kRep];
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            float t = l_lane[r];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
            l_warp[r] = t;
        }
        __syncthreads();  // every warp is done with the tables' score part and the staging area
        static_assert(kWarps * 32 * 32 * 4 <= kLutBytes, "merge scratch must fit in the score table");
        float *wm = reinterpret_cast<float *>(stage_s);    // [warps][4]
        float *wl = wm + kWarps * kRep;                     // [warps][4]
        float *wacc = reinterpret_cast<float *>(lut_s);    // [warps][8 products x 4 registers][32 lanes]
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kRep; ++r) {
                wm[warp * kRep + r] = m_ref[r];  // reference of this warp's sums: within the rescale gap of its maximum
                wl[warp * kRep + r] = l_warp[r];
            }
        }
        {
            // accumulator register j of product mm: column 2kq + (j&1) -> head, row half j>>1; stored lane-major
            float *base = wacc + (size_t)warp * 1024 + lane;
#pragma unroll
            for (int mm = 0; mm < 8; ++mm) {
                base[(mm * 4 + 0) * 32] = acc[mm][0];
                base[(mm * 4 + 1) * 32] = acc[mm][1];
                base[(mm * 4 + 2) * 32] = acc[mm][2];
                base[(mm * 4 + 3) * 32] = acc[mm][3];
            }
        }
        // the blocks that hold a partial state of this pair (this block among them)
        const int c_lo = block_of_unit(pair_first + kItemCost, total_tiles, blocks);
        const int n_parts = block_of_unit(pair_end - 1, total_tiles, blocks) - c_lo + 1;
        __syncthreads();
        for (int o = tid; o < kRep * kDim; o += kThreads) {
            // output o <-> (product mm, register j, lane of visiting-order class 0); its class-1 twin is
            // (mm, j^2, lane^2): same head and channel (see the B-operand column assignment above)
            const int mm = o >> 6, j = (o >> 4) & 3, l16 = o & 15;
            const int src_r8 = l16 >> 1, src_kq = l16 & 1;
            const int lane0 = src_r8 * 4 + src_kq;
            const int r = 2 * src_kq + (j & 1);
            const int dim = (2 * src_r8 + (j >> 1)) * 8 + mm;  // row r8 holds group 2*r8, row r8+8 group 2*r8+1
            float top = -INFINITY;
            for (int w = 0; w < kWarps; ++w) top = fmaxf(top, wm[w * kRep + r]);
            float lsum = 0.0f, asum = 0.0f;
            for (int w = 0; w < kWarps; ++w) {
                const float mw = wm[w * kRep + r];
                if (mw == -INFINITY) continue;
                const float sc = fast_exp2(mw - top);
                lsum += sc * wl[w * kRep + r];
                const float *src = wacc + (size_t)w * 1024;
                asum += sc * (src[(mm * 4 + j) * 32 + lane0] + src[(mm * 4 + (j ^ 2)) * 32 + (lane0 ^ 2)]);
            }
            if (n_parts == 1) {  // the whole pair was scanned here: this is the result
                const size_t row = (size_t)b * Hq + h * kRep + r;
                if (out) out[row * kDim + dim] = __float2half_rn(lsum > 0.0f ? asum / lsum : 0.0f);
                if (state_out) {
                    float *dst = state_out + row * kStateWidth;
                    if (dim == 0) {
                        dst[0] = top * kLn2;  // natural-log units outside the kernel
                        dst[1] = lsum;
                    }
                    dst[2 + dim] = asum;
                }
            } else {
                float *dst = part + ((size_t)(pair + blockIdx.x) * kRep + r) * kStateWidth;
                if (dim == 0) {
                    dst[0] = top * kLn2;
                    dst[1] = lsum;
                }
                dst[2 + dim] = asum;
            }
        }
        if (n_parts > 1) {
            // Mark this partial with the call's epoch; whoever then finds every partial of the pair marked
            // merges them.  The fences order (partial, mark) and (mark, reading the other marks), so the block
            // whose mark lands last always sees all of them; two blocks may both see them and then write the same
            // result.  A merging block clears the marks, so a replayed launch (same epoch) starts clean.
            __syncthreads();
            if (tid == 0) {
                __threadfence();  // the block's partial (ordered before this by the barrier) is visible before its mark
                marks[pair + blockIdx.x] = epoch;
                __threadfence();
            }
            __syncthreads();
            const int seen = tid < n_parts ? (ld_acquire_u64(marks + pair + c_lo + tid) == epoch) : 1;
            if (__syncthreads_and(seen)) {
                __threadfence();
                merge_pair_parts(part, pair + c_lo, n_parts, b, h, Hkv, out, state_out);
                if (tid < n_parts) marks[pair + c_lo + tid] = 0ull;
            }
        }
        cursor = item_end;
    }

    // ---- rows with an empty range never enter the loop: their defined result (out 0, m -inf, l 0, acc 0) ----
    for (int pair = blockIdx.x; pair < B * Hkv; pair += gridDim.x) {
        const int h = pair / B, b = pair % B;
        if (prefix_s[b + 1] != prefix_s[b]) continue;
        for (int o = tid; o < kRep * kDim; o += kThreads) {
            const size_t row = (size_t)b * Hq + h * kRep + (o >> 7);
            if (out) out[row * kDim + (o & 127)] = __float2half_rn(0.0f);
            if (state_out) {
                state_out[row * kStateWidth + 2 + (o & 127)] = 0.0f;
                if ((o & 127) == 0) {
                    state_out[row * kStateWidth] = -INFINITY;
                    state_out[row * kStateWidth + 1] = 0.0f;
                }
            }
        }
    }
}

}  // namespace gsrq

bool attn_gsrq_supported(int Hq, int Hkv, int D, int G, int S, int K) {
    return D == gsrq::kDim && G == gsrq::kGroups && S == gsrq::kStages && K == gsrq::kWords && Hq == Hkv * gsrq::kRep;
}

// Launch `kernel` so that it may be scheduled while the previous kernel of the stream drains
// (the kernel itself waits, see wait_for_previous_kernel).
template <typename... Params, typename... Args>
static cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

static size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

struct GsrqWorkspace {  // offsets into the caller's scratch; slot index = pair + scan block
    size_t part, marks, lut, vperm, scale, total;
    GsrqWorkspace(int B, int Hkv, int sms) {
        const size_t pairs = (size_t)B * Hkv, slots = pairs + (size_t)sms;
        part = 0;  // one partial softmax state per (pair, scan block) incidence
        marks = align256(slots * gsrq::kRep * gsrq::kStateWidth * sizeof(float));
        lut = align256(marks + slots * sizeof(unsigned long long));
        vperm = lut + pairs * gsrq::kLutBytes;
        scale = vperm + (TACVQ_GSRQ_VPERM ? (size_t)Hkv * gsrq::kVtabBytes : 0);
        total = align256(scale + pairs * gsrq::kStages * 8 * sizeof(float));
    }
};

size_t attn_gsrq_workspace_bytes(int B, int Hq, int Hkv, int D, int sms) {
    (void)Hq;
    (void)D;
    return GsrqWorkspace(B, Hkv, sms).total;
}

// Calls are numbered process-wide; a partial state is valid for the call whose number marks it.  The
// counter starts at a value that uninitialised scratch is unlikely to hold (and marks are 64 bits wide).
static std::atomic<unsigned long long> g_epoch{0x9e3779b97f4a7c15ull};

int attn_gsrq_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                       const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, void *workspace,
                       __half *out, float *state_out, int B, int Hq, int Hkv, int64_t T_cap, int sms,
                       cudaStream_t stream, const GsrqNewToken *fresh) {
    (void)Hq;
    if (B > gsrq::kMaxBatch || sms > gsrq::kMaxScanBlocks) return TACVQ_ERR_UNSUPPORTED;
    if (T_cap > ((int64_t)1 << 26)) return TACVQ_ERR_UNSUPPORTED;  // byte offsets inside a row's codes are 32-bit
    if (((T_cap + gsrq::kTile - 1) / gsrq::kTile + gsrq::kItemCost) * B * Hkv > 0x7fffffffLL) return TACVQ_ERR_UNSUPPORTED;
    if ((((uintptr_t)ktab | (uintptr_t)vtab | (uintptr_t)q) & 15) != 0) return TACVQ_ERR_ALIGN;
    // first use on a device raises the scan's dynamic shared-memory limit; concurrent first calls all
    // store the same value
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(gsrq::attn_gsrq_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             gsrq::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        // both kernels ask for the largest shared-memory carve-out, so the SMs are not re-partitioned
        // between the prepare and the scan launch of every call
        e = cudaFuncSetAttribute(gsrq::attn_gsrq_scan_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gsrq::attn_gsrq_prepare_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    const GsrqWorkspace ws(B, Hkv, sms);
    unsigned char *base = (unsigned char *)workspace;
    float *part = (float *)(base + ws.part);
    unsigned long long *marks = (unsigned long long *)(base + ws.marks);
    uint2 *lut = (uint2 *)(base + ws.lut);
    float *scale = (float *)(base + ws.scale);
    const unsigned long long epoch = g_epoch.fetch_add(2, std::memory_order_relaxed);  // odd, so never 0 (= cleared)
    GsrqNewToken token = {};
    if (fresh) token = *fresh;
    cudaError_t e = launch_dependent(gsrq::attn_gsrq_prepare_kernel, dim3(2 * B * Hkv), dim3(gsrq::kPrepThreads), 0, stream, q,
                                     ktab, vtab, lut, scale, (uint4 *)(base + ws.vperm), B, Hkv, token);
    int st = e == cudaSuccess ? launch_status() : (int)e;
    if (st != TACVQ_OK) return st;
    e = launch_dependent(gsrq::attn_gsrq_scan_kernel, dim3(sms), dim3(gsrq::kThreads), gsrq::kSmemBytes, stream, kcodes, vcodes,
                         (const uint2 *)lut, (const float *)scale, vtab, (const uint4 *)(base + ws.vperm), seq_start, seq_end, part, marks, out,
                         state_out, B, Hkv, (int)T_cap, epoch);
    return e == cudaSuccess ? launch_status() : (int)e;
}

}  // namespace tacvq
