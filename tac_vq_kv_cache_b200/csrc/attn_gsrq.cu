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
//           through a tensor-core product P^T.V (mma.sync m16n8k16).        32 x 16 B = 512 B
// 768 B / 128 B/clk = 6 clocks per (token, KV head) per SM is the floor of this design.
//
// Conflict-free addressing for arbitrary codes.  Both tables are laid out so that the shared-memory
// bank is decided by the code SLOT (stage, group), never by the code value, and at every step the
// lanes that are served together work on different slots:
//   score table   entry(code, slot) at code*256 + slot*8; lane = token; at step i lane l handles
//                 slot i XOR perm(l), so the 16 lanes of a half warp hit 16 different bank pairs.
//   value table   entry(code, slot) at code*512 + pos(slot)*16; the 8 lanes of a quarter warp
//                 fetch 8 different slots.  The lanes that share an A-fragment row visit their two
//                 groups in opposite order; the product keeps them apart by giving the 8 columns
//                 of the B operand to (4 heads) x (2 visiting orders).
//
// Work split.  A persistent grid (one block per SM) walks the flattened (KV head, batch row, 32-token
// tile) space; every block gets an equal share of tiles, rebuilds the score table when it enters a new
// (batch row, KV head) pair and writes one partial softmax state per pair it touches.  A second
// kernel merges the partials of each pair (log-sum-exp) and writes fp16 output and/or fp32 state.
//
// Semantics replaced: experiments_followup_mistral/evaluate_mistral_longbench.py:112-122 and the
// decoded window of :53-70 (no rotary step).  Differences from that dense path, all inside the
// 2e-3 tolerance: a score is the sum of per-stage table entries (the reference rounds the rebuilt
// key to fp16 first), entries are quantised to 13 bits of the widest slot range of their head,
// probabilities enter the tensor-core product as fp16, and the two V stages are added in fp16.

#include <mma.h>

#include "common.cuh"

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
[[maybe_unused]] constexpr int kBulkPiece = 16384;     // bytes per bulk copy instruction
#ifndef TACVQ_FUSED_MERGE
#define TACVQ_FUSED_MERGE 0  // 1: the last scan block of a pair merges it (no merge launch); measured slower
#endif
#ifndef TACVQ_BULK_TABLES
#define TACVQ_BULK_TABLES 0  // 1: table copies as cp.async.bulk + mbarrier (measured 1 % slower than 16-byte cp.async by all threads)
#endif
#ifndef TACVQ_PDL
#define TACVQ_PDL 1  // scan and merge are launched as programmatic dependents of their predecessor
#endif
#ifndef TACVQ_ITEM_COST
#define TACVQ_ITEM_COST 32
#endif
constexpr int kItemCost = TACVQ_ITEM_COST;         // fixed cost of starting a (row, head) pair in a block, in 32-token tiles
constexpr int kMaxScanBlocks = 256;  // persistent grid size (one block per SM) never exceeds this
constexpr int kStateWidth = kDim + 2;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleGap = 8.0f;  // log2 units a tile may exceed the running reference before rescaling
constexpr int kEntryMax = 8191;      // 13-bit fields: 8 of them sum below 2^16

// shared-memory carve-up (bytes)
constexpr int kLutBytes = kWords * kSlots * 8;              // 65536
constexpr int kVtabBytes = kWords * kSlots * 16;            // 131072
constexpr int kVBlock = 144;                                // 32 words + 16 B pad: staggers the banks of odd/even tokens
constexpr int kVStage = 8 * kVBlock;                        // 1152
constexpr int kStagePerWarp = kVStage + 256;                // transposed V codes + fp16 probabilities
constexpr int kStageBytes = kWarps * kStagePerWarp;         // 20480 (also min/max scratch of the table build)
constexpr int kPrefixBytes = (kMaxBatch + 1) * 4 + 12;      // 2064
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
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts16(uint32_t addr, unsigned short v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
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
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

// ------------------------------------------------------------------------------------------------
// prepare kernel: everything that depends only on (query, tables), laid out for shared memory
// ------------------------------------------------------------------------------------------------
//   blocks [0, 2*B*Hkv)      one residual stage of the score table of pair p = h*B + b:
//                            lut_g[p][code][slot] (8 bytes: four 13-bit fields) and
//                            scale_g[p][stage] = (step_r * log2 e, offset_r * log2 e), r = 0..3;
//                            each stage has its own step, so the finer second stage keeps its precision
//   blocks [2*B*Hkv, +Hkv)   value codewords of head h in the bank-striped order the scan uses
// A lane always works on group lane % 16, so the per-group value range is a reduction over warps
// and the table is written 128 contiguous bytes at a time.

constexpr int kPrepThreads = 512;
constexpr int kPrepWarps = kPrepThreads / 32;
constexpr int kPrepCodes = kWords / (2 * kPrepWarps);  // codes per thread (a warp covers 2 codes x 16 groups per round)
constexpr int kPrepVBlocks = 8;                          // blocks that reorder one head's value table
constexpr int kPrepSlotStride = kWords * 16 + 16;      // padded so that lanes (= groups) read different banks
constexpr int kPrepSmemBytes = kGroups * kPrepSlotStride + kRep * kDim * 4 + kPrepWarps * 32 * 8 * 4;

__global__ void __launch_bounds__(kPrepThreads)
attn_gsrq_prepare_kernel(const __half *__restrict__ q, const __half *__restrict__ ktab,
                         const __half *__restrict__ vtab, uint2 *__restrict__ lut_g, uint4 *__restrict__ vperm_g,
                         float *__restrict__ scale_g, int *__restrict__ tickets, const int32_t *__restrict__ seq_start,
                         const int32_t *__restrict__ seq_end, __half *__restrict__ out, float *__restrict__ state_out,
                         int B, int Hkv, int T_cap, int chained) {
    // chained != 0: launched as a programmatic dependent of a kernel that is still writing the visible
    // ranges and the newest codes (one decode step).  Nothing here reads those (the ranges of a decode step
    // are never empty, so the empty-row case below is skipped); before it ends, every thread waits for
    // that kernel, so that the scan, which waits for this grid, also sees that kernel's results.
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pairs = B * Hkv;
    if ((int)blockIdx.x >= 2 * pairs) {
        const int h = (blockIdx.x - 2 * pairs) / kPrepVBlocks, part = (blockIdx.x - 2 * pairs) % kPrepVBlocks;
        constexpr int kPer = kWords * kSlots / kPrepVBlocks;
#pragma unroll
        for (int j = part * kPer + tid; j < (part + 1) * kPer; j += kPrepThreads) {
            const int code = j >> 5, pos = j & 31;
            const int bq = pos & 7, u = pos >> 3;
            const int s = bq >> 2, gh = (bq >> 1) & 1;
            const int g = (bq & 1) | (u << 1) | (gh << 3);
            const __half *src = vtab + ((((size_t)h * kStages + s) * kGroups + g) * kWords + code) * kSub;
            vperm_g[(size_t)h * (kWords * kSlots) + j] = __ldg(reinterpret_cast<const uint4 *>(src));
        }
        if (chained) wait_for_previous_kernel();
        return;
    }
    extern __shared__ __align__(128) unsigned char psm[];
    unsigned char *ktab_s = psm;                                                   // [group][256 words x 16 B + pad]
    float *q_s = reinterpret_cast<float *>(psm + kGroups * kPrepSlotStride);        // [4][128]
    float *red = q_s + kRep * kDim;                                                 // [warp][lane][min x4, max x4]
    const int pair = blockIdx.x >> 1, stage = blockIdx.x & 1;
    const int h = pair / B, b = pair % B;
    const int Hq = Hkv * kRep;
    if (stage == 0) {
        if (tid == 0) tickets[pair] = 0;  // the scan counts finished blocks per pair from zero
        if (!chained && row_tokens(seq_start, seq_end, b, T_cap) == 0) {
            // an empty range never reaches the scan: its result is defined here (out 0, m -inf, l 0, acc 0)
            for (int o = tid; o < kRep * kDim; o += kPrepThreads) {
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
    {   // one stage of the head's K tables is a contiguous 64 KB block [group][word]: coalesced copy, padded rows
        const unsigned char *src = reinterpret_cast<const unsigned char *>(
            ktab + ((size_t)h * kStages + stage) * kGroups * kWords * kSub);
        for (int u = tid; u < kGroups * kWords; u += kPrepThreads)
            cp_async16(smem_u32(ktab_s) + (u >> 8) * kPrepSlotStride + (u & 255) * 16, src + (size_t)u * 16);
    }
    for (int i = tid; i < kRep * kDim; i += kPrepThreads)
        q_s[i] = __half2float(q[((size_t)b * Hq + h * kRep + (i >> 7)) * kDim + (i & 127)]);
    cp_async_wait_all();
    __syncthreads();
    const int g = lane & 15, half = lane >> 4;  // lane = (group, which of the warp's two codes per round)
    float qv[kRep][kSub];
#pragma unroll
    for (int r = 0; r < kRep; ++r)
#pragma unroll
        for (int i = 0; i < kSub; ++i) qv[r][i] = q_s[r * kDim + g * kSub + i];
    const uint32_t tab_u32 = smem_u32(ktab_s) + g * kPrepSlotStride;
    float val[kPrepCodes][kRep];
    float mn[kRep], mx[kRep];
#pragma unroll
    for (int r = 0; r < kRep; ++r) { mn[r] = INFINITY; mx[r] = -INFINITY; }
#pragma unroll
    for (int c = 0; c < kPrepCodes; ++c) {
        const int code = warp * 2 + half + 2 * kPrepWarps * c;
        const uint4 raw = lds128(tab_u32 + code * 16);
        const __half2 *hp = reinterpret_cast<const __half2 *>(&raw);
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
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
        red[(warp * 8 + r) * 32 + lane] = mn[r];       // lane-major: conflict-free writes and reads
        red[(warp * 8 + 4 + r) * 32 + lane] = mx[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRep; ++r) { mn[r] = INFINITY; mx[r] = -INFINITY; }
    for (int w = 0; w < kPrepWarps; ++w) {
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            mn[r] = fminf(mn[r], red[(w * 8 + r) * 32 + lane]);
            mx[r] = fmaxf(mx[r], red[(w * 8 + 4 + r) * 32 + lane]);
        }
    }
    float inv_step[kRep];
#pragma unroll
    for (int r = 0; r < kRep; ++r) {
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
        if (tid == 0) {
            scale_g[((size_t)pair * kStages + stage) * 8 + r] = step * kLog2e;
            scale_g[((size_t)pair * kStages + stage) * 8 + 4 + r] = offs * kLog2e;
        }
    }
#pragma unroll
    for (int c = 0; c < kPrepCodes; ++c) {
        const int code = warp * 2 + half + 2 * kPrepWarps * c;
        uint32_t e[kRep];
#pragma unroll
        for (int r = 0; r < kRep; ++r)
            e[r] = min((uint32_t)kEntryMax, __float2uint_rn((val[c][r] - mn[r]) * inv_step[r]));
        uint2 packed;
        packed.x = e[0] | (e[1] << 16);
        packed.y = e[2] | (e[3] << 16);
        lut_g[((size_t)pair * kWords + code) * kSlots + stage * kGroups + g] = packed;
    }
    if (chained) wait_for_previous_kernel();
}

// Scan blocks whose share of work units [start_c, start_{c+1}) gives them at least one tile of the pair
// occupying units [pair_first, pair_end): the partial states that exist for this pair.  Index = pair + c.
__device__ int list_pair_parts(int pair_first, int pair_end, int total_units, int blocks, int pair, int *parts) {
    const int c_lo = (int)(((long long)(pair_first + 1) * blocks - 1) / total_units);
    const int c_hi = (int)(((long long)pair_end * blocks - 1) / total_units);
    int n = 0;
    long long s0 = block_first_tile(total_units, c_lo, blocks);
    for (int c = c_lo; c <= c_hi; ++c) {
        const long long s1 = block_first_tile(total_units, c + 1, blocks);
        const long long lo = s0 > pair_first ? s0 : pair_first, hi = s1 < pair_end ? s1 : pair_end;
        const long long t_lo = lo - pair_first - kItemCost, t_hi = hi - pair_first - kItemCost;
        if (hi > lo && t_hi > (t_lo > 0 ? t_lo : 0) && n < kMaxScanBlocks) parts[n++] = pair + c;
        s0 = s1;
    }
    return n;
}

// log-sum-exp merge of the listed partial states of one pair by a 512-thread block (4 heads x 128 channels)
__device__ void merge_pair_parts(const float *part, const int *parts, int n_parts, int b, int h, int Hkv,
                                 __half *out, float *state_out) {
    const int Hq = Hkv * kRep;
    for (int o = threadIdx.x; o < kRep * kDim; o += blockDim.x) {
        const int r = o >> 7, dim = o & 127;
        float top = -INFINITY;
        for (int i = 0; i < n_parts; ++i) top = fmaxf(top, __ldcg(part + ((size_t)parts[i] * kRep + r) * kStateWidth));
        float lsum = 0.0f, asum = 0.0f;
        for (int i = 0; i < n_parts; ++i) {
            const float *st = part + ((size_t)parts[i] * kRep + r) * kStateWidth;
            const float mc = __ldcg(st);
            if (mc == -INFINITY) continue;
            const float sc = __expf(mc - top);
            lsum += sc * __ldcg(st + 1);
            asum += sc * __ldcg(st + 2 + dim);
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

// ------------------------------------------------------------------------------------------------
// scan kernel
// ------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads, 1)
attn_gsrq_scan_kernel(const uint8_t *__restrict__ kcodes,
                      const uint8_t *__restrict__ vcodes, const uint2 *__restrict__ lut_g,
                      const uint4 *__restrict__ vperm_g, const float *__restrict__ scale_g,
                      const int32_t *__restrict__ seq_start, const int32_t *__restrict__ seq_end,
                      float *__restrict__ part, int *__restrict__ tickets, __half *__restrict__ out,
                      float *__restrict__ state_out, int B, int Hkv, int T_cap) {
    extern __shared__ __align__(128) unsigned char smem[];
#if TACVQ_FUSED_MERGE
    __shared__ int n_parts_s;
    __shared__ int parts_s[kMaxScanBlocks];
#endif
    unsigned char *lut_s = smem;
    unsigned char *vtab_s = smem + kLutBytes;
    unsigned char *stage_s = vtab_s + kVtabBytes;
    int *prefix_s = reinterpret_cast<int *>(stage_s + kStageBytes);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- work prefix over batch rows: a non-empty row costs its tiles plus kItemCost units (table
    //      copies, pipeline fill and drain, merge), so blocks that enter more pairs get fewer tiles ------
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
            if (b < B) prefix_s[b] = running + incl - tiles;  // 'tiles' already includes the item cost, see below
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) prefix_s[B] = running;
    }
    __syncthreads();
    const int tiles_per_head = prefix_s[B];
    const int total_tiles = tiles_per_head * Hkv;  // fits: checked by the dispatcher
    int cursor = (int)block_first_tile(total_tiles, blockIdx.x, gridDim.x);
    const int my_end = (int)block_first_tile(total_tiles, blockIdx.x + 1, gridDim.x);

    // ---- per-lane constants ------------------------------------------------------------------
    // score side: lane = token, slot visiting order permuted by XOR so a half warp covers 16 bank pairs
    const uint32_t k_word_swap = lane & 3;
    const uint32_t k_byte_xor = (lane >> 2) & 3;
    const uint32_t k_lane_xor = (k_word_swap << 5) | (k_byte_xor << 3);
    uint32_t k_sel[4];
#pragma unroll
    for (int bi = 0; bi < 4; ++bi) k_sel[bi] = 0x4404u | (((bi ^ k_byte_xor) & 3u) << 4);
    // value side: lane = (row r8, token-pair column kq) of the A fragment
    const int r8 = lane >> 2, kq = lane & 3;
    uint32_t v_sel[4], v_off[4];
#pragma unroll
    for (int st = 0; st < 4; ++st) {
        const int combo = st ^ kq;
        const int s = combo & 1, gh = combo >> 1;
        const int g = r8 + 8 * gh;
        const int bq = (g & 1) | (gh << 1) | (s << 2);
        const int pos = bq + 8 * ((g >> 1) & 3);
        v_off[st] = smem_u32(vtab_s) + pos * 16;
        v_sel[st] = 0x4404u | ((uint32_t)(s * 2 + gh) << 4);
    }
    const int x_class = kq >> 1;                 // which visiting order this lane's tokens use
    const int b_head = r8 & 3;                   // B-fragment column n = r8: head n&3, class n>>2
    const bool b_valid = (r8 >> 2) == x_class;
    const uint32_t lut_base = smem_u32(lut_s);
    const uint32_t vstage_u32 = smem_u32(stage_s) + warp * kStagePerWarp;
    const uint32_t pstage_u32 = vstage_u32 + kVStage;

    int loaded_head = -1;
#if TACVQ_BULK_TABLES
    __shared__ __align__(8) unsigned long long mbar;
    const uint32_t mbar_a = smem_u32(&mbar);
    uint32_t mbar_phase = 0;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_a));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
#endif
    wait_for_previous_kernel();  // everything above used only kernel arguments and the range arrays

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

        // ---- tables of this item: both were laid out for shared memory by the prepare kernel, so they
        //      arrive as flat copies - bulk asynchronous copies (TMA) issued by one thread and counted by an
        //      mbarrier, or, if that wait ever ran out, plain 16-byte cp.async by all threads
        const bool need_v = h != loaded_head;
        loaded_head = h;
        const unsigned char *v_src = reinterpret_cast<const unsigned char *>(vperm_g) + (size_t)h * kVtabBytes;
        const unsigned char *l_src = reinterpret_cast<const unsigned char *>(lut_g) + (size_t)pair * kLutBytes;
#if TACVQ_BULK_TABLES
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier generic accesses before async writes
            const uint32_t bytes = kLutBytes + (need_v ? kVtabBytes : 0);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar_a), "r"(bytes) : "memory");
            for (int off = 0; off < kLutBytes; off += kBulkPiece)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 lut_base + off), "l"(l_src + off), "r"(kBulkPiece), "r"(mbar_a) : "memory");
            if (need_v)
                for (int off = 0; off < kVtabBytes; off += kBulkPiece)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     smem_u32(vtab_s) + off), "l"(v_src + off), "r"(kBulkPiece), "r"(mbar_a) : "memory");
        }
#else
        if (need_v)
            for (int j = tid; j < kVtabBytes / 16; j += kThreads) cp_async16(smem_u32(vtab_s) + j * 16, v_src + (size_t)j * 16);
        for (int j = tid; j < kLutBytes / 16; j += kThreads) cp_async16(lut_base + j * 16, l_src + (size_t)j * 16);
#endif
        float step_l2[kStages][kRep], offs_l2[kRep];
#pragma unroll
        for (int r = 0; r < kRep; ++r) {
            step_l2[0][r] = __ldg(scale_g + (size_t)pair * 16 + r);
            step_l2[1][r] = __ldg(scale_g + (size_t)pair * 16 + 8 + r);
            offs_l2[r] = __ldg(scale_g + (size_t)pair * 16 + 4 + r) + __ldg(scale_g + (size_t)pair * 16 + 12 + r);
        }
#if TACVQ_BULK_TABLES
        {
            int ok = 0;
            for (int spin = 0; spin < (1 << 20) && !ok; ++spin)  // bounded wait on the copy's byte count
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.s32 %0, 1, 0, p;\n}"
                             : "=r"(ok) : "r"(mbar_a), "r"(mbar_phase) : "memory");
            mbar_phase ^= 1u;
            if (!__syncthreads_and(ok)) {  // never seen; keeps the result independent of the copy engine
                if (need_v)
                    for (int j = tid; j < kVtabBytes / 16; j += kThreads) cp_async16(smem_u32(vtab_s) + j * 16, v_src + (size_t)j * 16);
                for (int j = tid; j < kLutBytes / 16; j += kThreads) cp_async16(lut_base + j * 16, l_src + (size_t)j * 16);
                cp_async_wait_all();
                __syncthreads();
            }
        }
#else
        cp_async_wait_all();
        __syncthreads();  // tables ready
#endif

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
        auto code_offset = [=](int tile) -> size_t {  // byte offset of this lane's 32-byte code row
            const int tok = tile * kTile + lane;
            return (row_base + (size_t)(tok_lo_row + min(tok, n_tokens - 1))) * 32;
        };
        uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0, v0 = k0, v1 = k0;
        if (tile_lo + warp < tile_hi) {
            const size_t off = code_offset(tile_lo + warp);
            const uint4 *kp = reinterpret_cast<const uint4 *>(kcodes + off), *vp = reinterpret_cast<const uint4 *>(vcodes + off);
            k0 = ldg_stream(kp); k1 = ldg_stream(kp + 1);
            v0 = ldg_stream(vp); v1 = ldg_stream(vp + 1);
        }

        for (int tile = tile_lo + warp; tile < tile_hi; tile += kWarps) {
            const bool live = tile * kTile + lane < n_tokens;
            // -- value codes: byte transpose so that word r holds this token's 4 codes of groups r, r+8
            {
                const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                uint32_t tw[8];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t t0 = prmt(w[half], w[half + 2], 0x5140u), t1 = prmt(w[half], w[half + 2], 0x7362u);
                    const uint32_t t2 = prmt(w[half + 4], w[half + 6], 0x5140u), t3 = prmt(w[half + 4], w[half + 6], 0x7362u);
                    tw[half * 4 + 0] = prmt(t0, t2, 0x5410u);
                    tw[half * 4 + 1] = prmt(t0, t2, 0x7632u);
                    tw[half * 4 + 2] = prmt(t1, t3, 0x5410u);
                    tw[half * 4 + 3] = prmt(t1, t3, 0x7632u);
                }
                __syncwarp();  // previous tile's readers are done with the staging area
                const uint32_t dst = vstage_u32 + (((lane >> 3) * 2 + (lane & 1)) * kVBlock) + (((lane >> 1) & 3) * 32);
                sts128(dst, tw[0], tw[1], tw[2], tw[3]);
                sts128(dst + 16, tw[4], tw[5], tw[6], tw[7]);
            }

            // -- scores: 32 look-ups of 8 bytes, four 13-bit fields each, flushed every 8 look-ups
            uint32_t kw[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
            if (tile + kWarps < tile_hi) {  // next tile's codes travel while this tile is computed
                const size_t off = code_offset(tile + kWarps);
                const uint4 *kp = reinterpret_cast<const uint4 *>(kcodes + off), *vp = reinterpret_cast<const uint4 *>(vcodes + off);
                k0 = ldg_stream(kp); k1 = ldg_stream(kp + 1);
                v0 = ldg_stream(vp); v1 = ldg_stream(vp + 1);
                if (tile + 3 * kWarps < tile_hi) {  // and warm L2 two more rounds ahead
                    prefetch_l2(reinterpret_cast<const unsigned char *>(kp) + (size_t)2 * kWarps * kTile * 32);
                    prefetch_l2(reinterpret_cast<const unsigned char *>(vp) + (size_t)2 * kWarps * kTile * 32);
                }
            }
            if (k_word_swap & 1) {
#pragma unroll
                for (int i = 0; i < 8; i += 2) { const uint32_t t = kw[i]; kw[i] = kw[i + 1]; kw[i + 1] = t; }
            }
            if (k_word_swap & 2) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if ((i & 2) == 0) { const uint32_t t = kw[i]; kw[i] = kw[i + 2]; kw[i + 2] = t; }
                }
            }
            float sc[kRep];
#pragma unroll
            for (int r = 0; r < kRep; ++r) sc[r] = offs_l2[r];
#pragma unroll
            for (int st = 0; st < kStages; ++st) {  // words 0-3 hold stage 0, words 4-7 stage 1
                uint32_t isum[kRep] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int wp = 0; wp < 2; ++wp) {
                    uint32_t lo = 0u, hi = 0u;
#pragma unroll
                    for (int wj = 0; wj < 2; ++wj) {
                        const int wi = st * 4 + wp * 2 + wj;
#pragma unroll
                        for (int bi = 0; bi < 4; ++bi) {
                            const uint32_t code256 = prmt(kw[wi], 0u, k_sel[bi]);
                            const uint32_t addr = ((code256 | (uint32_t)(wi * 32 + bi * 8)) ^ k_lane_xor) + lut_base;
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
#pragma unroll
                for (int r = 0; r < kRep; ++r) sc[r] = fmaf((float)isum[r], step_l2[st][r], sc[r]);
            }

            // -- softmax bookkeeping (log2 domain), lazy rescale of the running reference
            float tmax[kRep];
            bool grow = false;
#pragma unroll
            for (int r = 0; r < kRep; ++r) {
                if (!live) sc[r] = -INFINITY;
                float t = sc[r];
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, off));
                tmax[r] = t;
                grow = grow || (t > m_ref[r] + kRescaleGap);
            }
            if (grow) {  // warp-uniform
                float f[kRep];
#pragma unroll
                for (int r = 0; r < kRep; ++r) {
                    const float nref = fmaxf(m_ref[r], tmax[r]);
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
                sts16(pstage_u32 + (uint32_t)(r * kTile + lane) * 2, __half_as_ushort(__float2half_rn(p)));
            }
            __syncwarp();

            // -- values: per 8-token step gather this lane's two tokens (4 codewords each), add the two
            //    stages, pair the tokens into A fragments and issue 8 m16n8k8 products
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t b0 = 0u;
                if (b_valid) b0 = lds32(pstage_u32 + (uint32_t)(b_head * kTile * 2 + (ks * 4 + kq) * 4));
                uint4 sa[2], sb[2];
#pragma unroll
                for (int tk = 0; tk < 2; ++tk) {
                    const uint32_t word = lds32(vstage_u32 + (uint32_t)((ks * 2 + tk) * kVBlock + kq * 32 + r8 * 4));
                    uint4 gth[4];
#pragma unroll
                    for (int st = 0; st < 4; ++st) {
                        const uint32_t code256 = prmt(word, 0u, v_sel[st]);
                        gth[st] = lds128(v_off[st] + code256 + code256);
                    }
                    sa[tk] = make_uint4(hadd2(gth[0].x, gth[1].x), hadd2(gth[0].y, gth[1].y), hadd2(gth[0].z, gth[1].z), hadd2(gth[0].w, gth[1].w));
                    sb[tk] = make_uint4(hadd2(gth[2].x, gth[3].x), hadd2(gth[2].y, gth[3].y), hadd2(gth[2].z, gth[3].z), hadd2(gth[2].w, gth[3].w));
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
        __syncthreads();
        for (int o = tid; o < kRep * kDim; o += kThreads) {
            // output o <-> (product mm, register j, lane of visiting-order class 0); its class-1 twin is
            // (mm, j^2, lane^2): same head and channel (see the B-operand column assignment above)
            const int mm = o >> 6, j = (o >> 4) & 3, l16 = o & 15;
            const int src_r8 = l16 >> 1, src_kq = l16 & 1;
            const int lane0 = src_r8 * 4 + src_kq;
            const int r = 2 * src_kq + (j & 1);
            const int dim = (src_r8 + 8 * (j >> 1)) * 8 + mm;
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
            float *dst = part + ((size_t)(pair + blockIdx.x) * kRep + r) * kStateWidth;
            if (dim == 0) {
                dst[0] = top * kLn2;  // natural-log units outside the kernel
                dst[1] = lsum;
            }
            dst[2 + dim] = asum;
        }

#if TACVQ_FUSED_MERGE
        // ---- the block that finishes a pair last merges the pair's partial states -----------------
        __threadfence();   // this block's partial state is visible device-wide before its ticket is drawn
        __syncthreads();
        if (tid == 0) {
            const int n = list_pair_parts(pair_first, pair_end, total_tiles, gridDim.x, pair, parts_s);
            const int drawn = atomicAdd(tickets + pair, 1);
            n_parts_s = (drawn == n - 1) ? n : 0;  // 0: another block will finish this pair
            __threadfence();
        }
        __syncthreads();
        if (n_parts_s > 0) merge_pair_parts(part, parts_s, n_parts_s, b, h, Hkv, out, state_out);
#endif
        cursor = item_end;
    }
}

// ------------------------------------------------------------------------------------------------
// merge kernel: one block per (batch row, KV head) pair merges the partial states its scan blocks wrote
// ------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(kRep * kDim)
attn_gsrq_merge_kernel(const float *__restrict__ part, const int32_t *__restrict__ seq_start,
                       const int32_t *__restrict__ seq_end, __half *__restrict__ out, float *__restrict__ state_out,
                       int B, int Hkv, int T_cap, int scan_blocks) {
    __shared__ int n_parts_s;
    __shared__ int parts_s[kMaxScanBlocks];
    const int pair = blockIdx.x, h = pair / B, b = pair % B;
    wait_for_previous_kernel();
    if (threadIdx.x == 0) {
        int before = 0, mine = 0, per_head = 0;  // work units, exactly as the scan kernel counts them
        for (int i = 0; i < B; ++i) {
            int units = (row_tokens(seq_start, seq_end, i, T_cap) + kTile - 1) / kTile;
            if (units > 0) units += kItemCost;
            if (i < b) before += units;
            if (i == b) mine = units;
            per_head += units;
        }
        const int first = h * per_head + before;
        n_parts_s = mine > 0 ? list_pair_parts(first, first + mine, per_head * Hkv, scan_blocks, pair, parts_s) : 0;
    }
    __syncthreads();
    if (n_parts_s > 0) merge_pair_parts(part, parts_s, n_parts_s, b, h, Hkv, out, state_out);
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

struct GsrqWorkspace {
    size_t part, lut, vperm, scale, tickets, total;
    GsrqWorkspace(int B, int Hkv, int sms) {
        const size_t pairs = (size_t)B * Hkv;
        part = 0;
        lut = align256((pairs + (size_t)sms) * gsrq::kRep * gsrq::kStateWidth * sizeof(float));
        vperm = lut + pairs * gsrq::kLutBytes;
        scale = vperm + (size_t)Hkv * gsrq::kVtabBytes;
        tickets = align256(scale + pairs * gsrq::kStages * 8 * sizeof(float));
        total = align256(tickets + pairs * sizeof(int));
    }
};

size_t attn_gsrq_workspace_bytes(int B, int Hq, int Hkv, int D, int sms) {
    (void)Hq;
    (void)D;
    return GsrqWorkspace(B, Hkv, sms).total;
}

int attn_gsrq_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                       const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, void *workspace,
                       __half *out, float *state_out, int B, int Hq, int Hkv, int64_t T_cap, int sms,
                       cudaStream_t stream, bool after_prologue) {
    (void)Hq;
    if (B > gsrq::kMaxBatch || sms > gsrq::kMaxScanBlocks) return TACVQ_ERR_UNSUPPORTED;
    if (((T_cap + gsrq::kTile - 1) / gsrq::kTile + gsrq::kItemCost) * B * Hkv > 0x7fffffffLL) return TACVQ_ERR_UNSUPPORTED;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gsrq::attn_gsrq_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             gsrq::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gsrq::attn_gsrq_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 gsrq::kPrepSmemBytes);
        if (e != cudaSuccess) return (int)e;
        // both kernels ask for the largest shared-memory carve-out, so the SMs are not re-partitioned
        // between the prepare and the scan launch of every step
        e = cudaFuncSetAttribute(gsrq::attn_gsrq_prepare_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gsrq::attn_gsrq_scan_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    const GsrqWorkspace ws(B, Hkv, sms);
    unsigned char *base = (unsigned char *)workspace;
    float *part = (float *)(base + ws.part);
    uint2 *lut = (uint2 *)(base + ws.lut);
    uint4 *vperm = (uint4 *)(base + ws.vperm);
    float *scale = (float *)(base + ws.scale);
    int *tickets = (int *)(base + ws.tickets);
    int st;
    if (after_prologue && TACVQ_PDL) {
        // the previous launch on this stream is the decode-step prologue, which lets this grid start at once
        cudaError_t e = launch_dependent(gsrq::attn_gsrq_prepare_kernel, dim3(2 * B * Hkv + gsrq::kPrepVBlocks * Hkv),
                                         dim3(gsrq::kPrepThreads), gsrq::kPrepSmemBytes, stream, q, ktab, vtab, lut, vperm, scale,
                                         tickets, seq_start, seq_end, out, state_out, B, Hkv, (int)T_cap, 1);
        st = e == cudaSuccess ? launch_status() : (int)e;
    } else {
        gsrq::attn_gsrq_prepare_kernel<<<2 * B * Hkv + gsrq::kPrepVBlocks * Hkv, gsrq::kPrepThreads, gsrq::kPrepSmemBytes, stream>>>(
            q, ktab, vtab, lut, vperm, scale, tickets, seq_start, seq_end, out, state_out, B, Hkv, (int)T_cap, 0);
        st = launch_status();
    }
    if (st != TACVQ_OK) return st;
#if TACVQ_PDL
    {
        cudaError_t e = launch_dependent(gsrq::attn_gsrq_scan_kernel, dim3(sms), dim3(gsrq::kThreads), gsrq::kSmemBytes, stream,
                                         kcodes, vcodes, lut, vperm, scale, seq_start, seq_end, part, tickets, out, state_out,
                                         B, Hkv, (int)T_cap);
        st = e == cudaSuccess ? launch_status() : (int)e;
    }
#else
    gsrq::attn_gsrq_scan_kernel<<<sms, gsrq::kThreads, gsrq::kSmemBytes, stream>>>(
        kcodes, vcodes, lut, vperm, scale, seq_start, seq_end, part, tickets, out, state_out, B, Hkv, (int)T_cap);
    st = launch_status();
#endif
#if !TACVQ_FUSED_MERGE
    if (st != TACVQ_OK) return st;
#if TACVQ_PDL
    {
        cudaError_t e = launch_dependent(gsrq::attn_gsrq_merge_kernel, dim3(B * Hkv), dim3(gsrq::kRep * gsrq::kDim), 0, stream,
                                         (const float *)part, seq_start, seq_end, out, state_out, B, Hkv, (int)T_cap, sms);
        st = e == cudaSuccess ? launch_status() : (int)e;
    }
#else
    gsrq::attn_gsrq_merge_kernel<<<B * Hkv, gsrq::kRep * gsrq::kDim, 0, stream>>>(part, seq_start, seq_end, out, state_out, B, Hkv,
                                                                     (int)T_cap, sms);
    st = launch_status();
#endif
#endif
    return st;
}

}  // namespace tacvq
