// Encode for wide groups (d = 32, 64, 128; fp16 tables): tensor cores filter, exact fp32 decides.
//
// Same idea as the 8-wide kernel in encode_tc.cu, shaped as a block-level GEMM.  A block owns 128
// rows of one (head, group).  Per stage it
//   1. keeps, next to the fp32 residual tile, its fp16 rounding in shared memory,
//   2. scores all 128 x 256 (row, word) pairs on the tensor cores; a score is t = r.c - |c|^2/2 and the
//      distance is |r|^2 - 2t.
//      d = 64, 128 (encode_tm_large_kernel, further down): tcgen05.mma from shared-memory panels into
//      tensor memory, where the fp32 residual tile lives too; that kernel has its own description.
//      d = 32 (encode_tc_large_kernel): mma.sync.m16n8k16 with ldmatrix fragments, accumulators seeded with
//      -|c|^2/2, each of 16 warps owning 32 rows x 64 words.  Built with TACVQ_ENCODE_TENSOR_MEMORY=1 this
//      kernel also carries d = 64, 128, with the tcgen05 product but the residual tile in shared memory.
//   3. takes the row maxima over the four word quarters and lists every pair whose score lies within
//      a margin of its row's maximum,
//   4. re-evaluates the listed pairs in the library's exact fp32 order (one d-step FMA chain each,
//      one pair per thread) and keeps the lowest (distance, index) per row with a 64-bit shared atomicMin,
//   5. subtracts the chosen words from the fp32 residual tile and refreshes the fp16 copy.
//
// Margin (see encode_tc.cu for the argument that a margin of twice the error bound keeps the exact
// argmin and everything tied with it on the list).  The fp16 rounding of the residual changes a dot
// product by at most 2^-11 sum |r_i c_i| <= 2^-11 |r| |c|; the tensor core's fp32 accumulation of the
// exact products, the exact chain's own roundings and the roundings of the distance expression add at
// most about 2^-17 (|r|^2 + |c|^2).  In units of t the kernel allows
//   1.25 * 2^-10 |r| max|c|  +  2^-14 (|r|^2 + max|c|^2)  +  2^-18 max|c|   (fp16 subnormals).
// On Gaussian data that lists about 1.07 words per row.  If the list overflows, or a residual is too
// large for fp16, the block re-evaluates every pair of that stage: slow, still exact.
//
// Reference statements: src/jointkv/closed_loop_vq.py:52-76 (search), :343-395 (stage recursion).

#include <atomic>
#include <cstring>

#include <cuda.h>  // CUtensorMap and the driver's encoder signature; the entry point is looked up at run time

#include "common.cuh"

namespace tacvq {

namespace {

constexpr int kRows = 128;     // rows per block
constexpr int kThreads = 512;  // 16 warps = 4 row blocks of 32 x 4 word quarters of 64
constexpr int kListCap = 2048;

// TM = true: the two fp16 operands are stored the way the 5th-generation tensor core reads them from
// shared memory (K-major, 128-byte rows, 128-byte swizzle: within every 1024-byte group of 8 rows the
// 16-byte piece p of row r sits at piece p ^ (r & 7); 64 elements per row, so d = 128 takes two such
// panels).  Both operands then start on 1024-byte boundaries.
template <int DSUB, bool TM>
struct TcLargeLayout {
    static constexpr int kHalfStride = DSUB + 8;  // halves: 16-byte rows that land on distinct banks for ldmatrix
    static constexpr int kResStride = DSUB + 4;   // floats
    static constexpr size_t kTab = 0;                                              // [256][kHalfStride] half
    static constexpr size_t kHi = kTab + (size_t)kMaxWords * (TM ? DSUB : kHalfStride) * 2;      // [kRows][kHalfStride] half
    static constexpr size_t kRes = kHi + (size_t)kRows * (TM ? DSUB : kHalfStride) * 2;          // [kRows][kResStride] float
    static constexpr size_t kNrm = kRes + (size_t)kRows * kResStride * 4;          // [256] float
    static constexpr size_t kSeed = kNrm + kMaxWords * 4;                          // [256] float: -|c|^2/2
    static constexpr size_t kXx = kSeed + kMaxWords * 4;                           // [kRows] float
    static constexpr size_t kRowMax = kXx + kRows * 4;                             // [4][kRows] float
    static constexpr size_t kThr = kRowMax + 4 * kRows * 4;                        // [kRows] float
    static constexpr size_t kBest = kThr + kRows * 4;                              // [kRows] u64
    static constexpr size_t kList = kBest + kRows * 8;                             // [kListCap] u16
    static constexpr size_t kMisc = kList + kListCap * 2;                          // count, big flag, cc_max, tensor-memory slot; +16: mbarrier
    static constexpr size_t kRowCnt = kMisc + 32;                                  // [kRows] int: listed words per row
    static constexpr size_t kHist = kRowCnt + kRows * 4;                           // [kRows][S] u8
    static constexpr size_t bytes(int S) { return kHist + (size_t)kRows * S + (TM ? 1024 : 0); }  // TM: room to align the base
    // half index of element e of word k / of row r
    __device__ static __forceinline__ int tab_at(int k, int e) {
        if constexpr (TM) return (e >> 6) * (kMaxWords * 64) + k * 64 + ((((e >> 3) & 7) ^ (k & 7)) << 3) + (e & 7);
        else return k * kHalfStride + e;
    }
    __device__ static __forceinline__ int hi_at(int r, int e) {
        if constexpr (TM) return (e >> 6) * (kRows * 64) + r * 64 + ((((e >> 3) & 7) ^ (r & 7)) << 3) + (e & 7);
        else return r * kHalfStride + e;
    }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void mma_acc_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 32 consecutive fp32 columns of this warp's 32 tensor-memory lanes (lane = thread)
__device__ __forceinline__ void tmem_load32(uint32_t *v, uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// Shared-memory operand descriptor of tcgen05.mma for a K-major panel with 128-byte rows and the
// 128-byte swizzle: start address / 16 in bits 0-13, leading offset (one 16-byte unit, not used by this
// layout) in bits 16-29, 1024 bytes between groups of 8 rows in bits 32-45, descriptor version 1 in
// bits 46-47, swizzle mode 2 (128 bytes) in bits 61-63.
__device__ __forceinline__ uint64_t panel_descriptor(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr & 0x3ffffu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor: fp32 accumulator (bits 4-5 = 1), fp16 A and B (bits 7-12 = 0), both K-major
// (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
constexpr uint32_t kMmaShape = (1u << 4) | ((uint32_t)(kMaxWords >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);

// monotone map float -> uint32 (total order of the values, -0 below +0)
__device__ __forceinline__ uint32_t ordered_bits(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// |v|^2 of a d-vector (d a multiple of 32) by eight neighbouring lanes, in the library's order
// (four sets of eight running sums: element i goes to set (i/8)%4, sum i%8; per sum the sets are added
// ((0+1)+2)+3; the eight sums are added 0..7).  Lane j of the group owns sum j.  All eight return the total.
template <int DSUB, typename Load>
__device__ __forceinline__ float group8_sqnorm_ordered(Load at, int lane) {
    const int j = lane & 7;
    float set[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < DSUB; i += 8) {
        const float v = at(i + j);
        set[(i >> 3) & 3] = __fadd_rn(set[(i >> 3) & 3], __fmul_rn(v, v));
    }
    const float mine = __fadd_rn(__fadd_rn(__fadd_rn(set[0], set[1]), set[2]), set[3]);
    const int first = lane & 24;
    float total = __shfl_sync(0xffffffffu, mine, first);
#pragma unroll
    for (int k = 1; k < 8; ++k) total = __fadd_rn(total, __shfl_sync(0xffffffffu, mine, first + k));
    return total;
}

// four consecutive residual elements -> fp32 tile and its fp16 rounding; returns max |element|
__device__ __forceinline__ float store_residual4(float *res_at, __half *hi_at, const float4 v) {
    *reinterpret_cast<float4 *>(res_at) = v;
    __half2 h[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
    *reinterpret_cast<uint2 *>(hi_at) = *reinterpret_cast<const uint2 *>(h);
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

template <typename XT>
__device__ __forceinline__ float4 load4(const XT *src, bool vec);
template <>
__device__ __forceinline__ float4 load4<float>(const float *src, bool vec) {
    if (vec) return *reinterpret_cast<const float4 *>(src);
    return make_float4(src[0], src[1], src[2], src[3]);
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half *src, bool vec) {
    __half2 h[2];
    if (vec) {
        *reinterpret_cast<uint2 *>(h) = *reinterpret_cast<const uint2 *>(src);
    } else {
        h[0] = __halves2half2(src[0], src[1]);
        h[1] = __halves2half2(src[2], src[3]);
    }
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    return make_float4(a.x, a.y, b.x, b.y);
}

}  // namespace

// Times a block gave up waiting for its tensor-core products (the stage then re-evaluates every pair,
// so the codes are still exact); read by tacvq_debug_tensor_memory_timeouts.  Expected to stay 0.
__device__ unsigned int g_tensor_memory_timeouts = 0;

template <int DSUB, typename XT, bool TM>
__global__ void __launch_bounds__(kThreads, 1)
encode_tc_large_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const __half *__restrict__ tables,
                       const float *__restrict__ sqnorm_in, uint8_t *__restrict__ codes, void *__restrict__ recon,
                       int recon_dtype, int B, int H, int T, int G, int S, int K, int64_t t0, int64_t T_cap, int vec_ok) {
    using L = TcLargeLayout<DSUB, TM>;
    constexpr int RS = L::kResStride;
    constexpr int kChunks = DSUB / 8;  // threads per row: each owns elements [4c, 4c+4) and [d/2 + 4c, d/2 + 4c + 4)
    constexpr int kPass = kThreads / kChunks;  // rows per pass over the tile
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    // the tensor-core operands of the TM path start on a 1024-byte boundary of the shared window
    unsigned char *smem_raw = smem_dyn;
    if constexpr (TM) smem_raw += (1024u - ((uint32_t)__cvta_generic_to_shared(smem_dyn) & 1023u)) & 1023u;
    __half *tab = reinterpret_cast<__half *>(smem_raw + L::kTab);
    __half *hi = reinterpret_cast<__half *>(smem_raw + L::kHi);
    float *res = reinterpret_cast<float *>(smem_raw + L::kRes);
    float *nrm = reinterpret_cast<float *>(smem_raw + L::kNrm);
    float *seed = reinterpret_cast<float *>(smem_raw + L::kSeed);
    float *xxs = reinterpret_cast<float *>(smem_raw + L::kXx);
    float *rowmax = reinterpret_cast<float *>(smem_raw + L::kRowMax);
    float *thr = reinterpret_cast<float *>(smem_raw + L::kThr);
    unsigned long long *best = reinterpret_cast<unsigned long long *>(smem_raw + L::kBest);
    uint16_t *list = reinterpret_cast<uint16_t *>(smem_raw + L::kList);
    int *count = reinterpret_cast<int *>(smem_raw + L::kMisc);
    int *big = count + 1;  // some residual element of the coming stage does not fit fp16
    float *cc_max = reinterpret_cast<float *>(count + 2);
    int *rowcnt = reinterpret_cast<int *>(smem_raw + L::kRowCnt);
    uint8_t *hist = smem_raw + L::kHist;

    const int hg = blockIdx.y;
    const int h = hg / G, g = hg % G;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, q = lane & 3;
    // row block (32 rows), word quarter (64 words); a warp reads the tensor-memory lanes 32 * (warp % 4)..+31
    const int wr = TM ? (warp & 3) : (warp >> 2), wq = TM ? (warp >> 2) : (warp & 3);
    const uint32_t rows = (uint32_t)B * (uint32_t)T;  // the launcher keeps B*T below 2^31
    const uint32_t tile = blockIdx.x * kRows;
    const int my_c = tid % kChunks, my_r = tid / kChunks;  // this thread's piece column and first row
    const float inf = __int_as_float(0x7f800000);

    uint8_t *code_at = nullptr;  // this row's first code byte (threads 0..kRows-1)
    if (tid < kRows && tile + tid < rows) {
        const uint32_t row = tile + tid;
        const uint32_t b = row / (uint32_t)T, t = row % (uint32_t)T;
        code_at = codes + (((int64_t)b * H + h) * T_cap + t0 + t) * ((int64_t)S * G) + g;
    }
    if (tid == 0) *big = 0;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(count + 3);
    int *tm_fail = count + 6;
    const uint32_t mbar_a = (uint32_t)__cvta_generic_to_shared(smem_raw + L::kMisc + 16);
    uint32_t tmem_base = 0;
    if constexpr (TM) {
        // 256 fp32 columns x 128 lanes of tensor memory hold the block's 128 x 256 score tile
        if (warp == 0) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(tmem_slot)), "r"((uint32_t)kMaxWords) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        if (tid == 0) {
            *tm_fail = 0;
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_a) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if constexpr (TM) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    }
#pragma unroll
    for (int r = my_r; r < kRows; r += kPass) {
        const uint32_t row = tile + r;
        float4 v0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), v1 = v0;
        if (row < rows) {
            const uint32_t b = row / (uint32_t)T, t = row % (uint32_t)T;
            const XT *src = x + (int64_t)b * sxb + (int64_t)h * sxh + (int64_t)t * sxt + (int64_t)g * DSUB + 4 * my_c;
            v0 = load4<XT>(src, vec_ok != 0);
            v1 = load4<XT>(src + DSUB / 2, vec_ok != 0);
        }
        const float top0 = store_residual4(res + r * RS + 4 * my_c, hi + L::hi_at(r, 4 * my_c), v0);
        const float top1 = store_residual4(res + r * RS + DSUB / 2 + 4 * my_c, hi + L::hi_at(r, DSUB / 2 + 4 * my_c), v1);
        if (!(fmaxf(top0, top1) < 32768.0f)) *big = 1;
    }

    for (int s = 0; s < S; ++s) {
        __syncthreads();  // residual tiles settled; the previous stage's table is no longer read
        const __half *src = tables + (((int64_t)h * S + s) * G + g) * (int64_t)K * DSUB;
        // caller-supplied word norms: fetched by the upper half of the block while the table is copied
        const int norm_k = tid - (kThreads - kMaxWords);
        float norm_v = inf;
        if (sqnorm_in != nullptr && norm_k >= 0 && norm_k < K) norm_v = sqnorm_in[(((int64_t)h * S + s) * G + g) * K + norm_k];
        if (tid == 0) {
            *count = 0;
            *cc_max = 0.0f;
        }
        for (int idx = tid; idx < kMaxWords * kChunks; idx += kThreads) {
            const int k = idx / kChunks, c = idx % kChunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (k < K) v = *reinterpret_cast<const uint4 *>(src + (int64_t)k * DSUB + c * 8);
            *reinterpret_cast<uint4 *>(tab + L::tab_at(k, c * 8)) = v;
        }
        if constexpr (TM) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads what was stored above
        __syncthreads();
        if constexpr (TM) {
            // One thread issues the whole 128 x 256 x d product (d / 16 instructions); it runs while the
            // block computes the norms below and reports to the mbarrier when the last one has finished.
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = (uint32_t)__cvta_generic_to_shared(hi), b0 = (uint32_t)__cvta_generic_to_shared(tab);
#pragma unroll
                for (int ks = 0; ks < DSUB / 16; ++ks) {
                    const uint64_t da = panel_descriptor(a0 + (ks >> 2) * (kRows * 128) + (ks & 3) * 32);
                    const uint64_t db = panel_descriptor(b0 + (ks >> 2) * (kMaxWords * 128) + (ks & 3) * 32);
                    asm volatile(
                        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                        ::"r"(tmem_base), "l"(da), "l"(db), "r"(kMmaShape), "r"(ks) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_a) : "memory");
            }
        }
        // |c|^2 per word and |r|^2 per row, eight lanes per vector (four vectors per warp and trip, placed so
        // that their loads miss each other's banks).  The largest |c|^2 is gathered with an integer atomic
        // maximum (non-negative floats order like their bit patterns).
        {
            float top = 0.0f;
            if (sqnorm_in == nullptr) {
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int k = warp * 16 + it * 4 + (lane >> 3);
                    float v = group8_sqnorm_ordered<DSUB>([&](int i) { return __half2float(tab[L::tab_at(k, i)]); }, lane);
                    if (k >= K) v = inf;  // padding words can never be chosen
                    else if (v == v) top = fmaxf(top, v);
                    if ((lane & 7) == 0) {
                        nrm[k] = v;
                        seed[k] = -0.5f * v;
                    }
                }
            } else if (norm_k >= 0) {
                nrm[norm_k] = norm_v;
                seed[norm_k] = -0.5f * norm_v;
                if (norm_k < K && norm_v == norm_v) top = norm_v;
            }
            if (sqnorm_in == nullptr || norm_k >= 0) {  // warp-uniform
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
                if (lane == 0) atomicMax(reinterpret_cast<int *>(cc_max), __float_as_int(top));
            }
        }
        // Row norms in 32 trips of 4 rows; on the tensor-memory path warp 0 takes none (its first thread is
        // busy issuing the products), the other 15 warps share them.
        for (int trip = TM ? (warp == 0 ? 32 : warp - 1) : warp; trip < 32; trip += TM ? 15 : 16) {
            const int r = (trip >> 1) * 8 + (trip & 1) + 2 * (lane >> 3);
            const float v = group8_sqnorm_ordered<DSUB>([&](int i) { return res[r * RS + i]; }, lane);
            if ((lane & 7) == 0) {
                xxs[r] = v;
                best[r] = ~0ull;
                rowcnt[r] = 0;
            }
        }
        __syncthreads();

        if constexpr (TM) {
            // ---- approximate scores from tensor memory: thread = row, 64 words of quarter wq per thread ------
            {
                int done = 0;
                for (int spin = 0; spin < (1 << 22) && !done; ++spin)  // bounded wait for the products issued above
                    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.s32 %0, 1, 0, p;\n}"
                                 : "=r"(done) : "r"(mbar_a), "r"((uint32_t)(s & 1)) : "memory");
                if (!done) {  // never seen; the stage then re-evaluates every pair, so the codes stay exact
                    *tm_fail = 1;
                    atomicAdd(&g_tensor_memory_timeouts, 1u);
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc[64];
            {
                uint32_t v[64];
                const uint32_t taddr = tmem_base + ((uint32_t)(wr * 32) << 16) + (uint32_t)(wq * 64);
                tmem_load32(v, taddr);
                tmem_load32(v + 32, taddr + 32);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                float top = -inf;
#pragma unroll
                for (int j = 0; j < 64; j += 4) {
                    const float4 sv = *reinterpret_cast<const float4 *>(seed + wq * 64 + j);
                    sc[j] = __uint_as_float(v[j]) + sv.x;
                    sc[j + 1] = __uint_as_float(v[j + 1]) + sv.y;
                    sc[j + 2] = __uint_as_float(v[j + 2]) + sv.z;
                    sc[j + 3] = __uint_as_float(v[j + 3]) + sv.w;
                    top = fmaxf(fmaxf(top, fmaxf(sc[j], sc[j + 1])), fmaxf(sc[j + 2], sc[j + 3]));
                }
                rowmax[wq * kRows + wr * 32 + lane] = top;
            }
            __syncthreads();
            if (tid < kRows) {
                const float top = fmaxf(fmaxf(rowmax[tid], rowmax[kRows + tid]), fmaxf(rowmax[2 * kRows + tid], rowmax[3 * kRows + tid]));
                const float cm = *cc_max, xx = xxs[tid];
                const float margin = 1.220703125e-03f * sqrtf(xx * cm) + 6.103515625e-05f * (xx + cm) + 3.814697265625e-06f * sqrtf(cm);
                thr[tid] = (*big != 0 || *tm_fail != 0) ? -inf : top - margin;
            }
            __syncthreads();
            if (tid == 0) *big = 0;  // read above; the update below raises it for the next stage
            // List the pairs within the margin: a thread holds one row's 64 scores, so its hits are a 64-bit mask.
            {
                const int r = wr * 32 + lane;
                const float limit = thr[r];
                uint32_t lo = 0u, hi32 = 0u;
#pragma unroll
                for (int j = 31; j >= 0; --j) {
                    lo = __funnelshift_l(__float_as_uint(sc[j] - limit), lo, 1);
                    hi32 = __funnelshift_l(__float_as_uint(sc[32 + j] - limit), hi32, 1);
                }
                unsigned long long todo = ~(((unsigned long long)hi32 << 32) | lo);  // set = not below the limit
                const int hits = __popcll(todo);
                int before = hits;  // inclusive prefix over the warp
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, before, off);
                    if (lane >= off) before += up;
                }
                int base = 0;
                if (lane == 31 && before > 0) base = atomicAdd(count, before);
                base = __shfl_sync(0xffffffffu, base, 31);
                int slot = base + before - hits;
                if (hits > 0) atomicAdd(rowcnt + r, hits);
                while (todo != 0ull) {
                    const int j = __ffsll((long long)todo) - 1;
                    todo &= todo - 1ull;
                    if (slot < kListCap) list[slot] = (uint16_t)((r << 8) | (wq * 64 + j));
                    ++slot;
                }
            }
        } else {
            // ---- approximate scores: 32 rows x 64 words per warp --------------------------------------
            float acc[2][8][4];
    #pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float2 sv = *reinterpret_cast<const float2 *>(seed + wq * 64 + n * 8 + 2 * q);
    #pragma unroll
                for (int m = 0; m < 2; ++m) {
                    acc[m][n][0] = sv.x;
                    acc[m][n][1] = sv.y;
                    acc[m][n][2] = sv.x;
                    acc[m][n][3] = sv.y;
                }
            }
            {
                // ldmatrix lane addresses: A tiles are [16 rows][16 k], B tiles [16 words][16 k] (two n-tiles)
                const int a_row = wr * 32 + (lane & 15), a_col = (lane >> 4) * 8;
                const int b_row = wq * 64 + (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
    #pragma unroll 2
                for (int ks = 0; ks < DSUB / 16; ++ks) {
                    uint32_t a[2][4];
    #pragma unroll
                    for (int m = 0; m < 2; ++m) ldmatrix_x4(a[m], hi + L::hi_at(a_row + m * 16, ks * 16 + a_col));
    #pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        uint32_t bw[4];
                        ldmatrix_x4(bw, tab + L::tab_at(b_row + np * 16, ks * 16 + b_col));
    #pragma unroll
                        for (int m = 0; m < 2; ++m) {
                            mma_acc_16816(acc[m][2 * np], a[m], bw[0], bw[1]);
                            mma_acc_16816(acc[m][2 * np + 1], a[m], bw[2], bw[3]);
                        }
                    }
                }
            }
            // row maxima over this warp's 64 words
    #pragma unroll
            for (int m = 0; m < 2; ++m) {
    #pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float top = fmaxf(acc[m][0][2 * half], acc[m][0][2 * half + 1]);
    #pragma unroll
                    for (int n = 1; n < 8; ++n) top = fmaxf(top, fmaxf(acc[m][n][2 * half], acc[m][n][2 * half + 1]));
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
                    if (q == 0) rowmax[wq * kRows + wr * 32 + m * 16 + half * 8 + gid] = top;
                }
            }
            __syncthreads();
            if (tid < kRows) {
                const float top = fmaxf(fmaxf(rowmax[tid], rowmax[kRows + tid]), fmaxf(rowmax[2 * kRows + tid], rowmax[3 * kRows + tid]));
                const float cm = *cc_max, xx = xxs[tid];
                const float margin = 1.220703125e-03f * sqrtf(xx * cm) + 6.103515625e-05f * (xx + cm) + 3.814697265625e-06f * sqrtf(cm);
                thr[tid] = (*big != 0) ? -inf : top - margin;
            }
            __syncthreads();
            if (tid == 0) *big = 0;  // read above; the update below raises it for the next stage
            // List the pairs within the margin.  Per row a thread shifts the sign of (score - limit) of its
            // 16 words into a word (first word ends at bit 15, set = below the limit); one atomic per warp
            // reserves the slots, then each thread walks its set bits.
            {
                uint32_t pass[2][2];
                int hits = 0;
    #pragma unroll
                for (int m = 0; m < 2; ++m) {
    #pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const float limit = thr[wr * 32 + m * 16 + half * 8 + gid];
                        uint32_t fail = 0u;
    #pragma unroll
                        for (int n = 0; n < 8; ++n) {
                            fail = __funnelshift_l(__float_as_uint(acc[m][n][2 * half] - limit), fail, 1);
                            fail = __funnelshift_l(__float_as_uint(acc[m][n][2 * half + 1] - limit), fail, 1);
                        }
                        pass[m][half] = ~fail & 0xffffu;
                        hits += __popc(pass[m][half]);
                    }
                }
                int before = hits;  // inclusive prefix over the warp
    #pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, before, off);
                    if (lane >= off) before += up;
                }
                int base = 0;
                if (lane == 31 && before > 0) base = atomicAdd(count, before);
                base = __shfl_sync(0xffffffffu, base, 31);
                int slot = base + before - hits;
    #pragma unroll
                for (int m = 0; m < 2; ++m) {
    #pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t todo = pass[m][half];
                        const int r = wr * 32 + m * 16 + half * 8 + gid;
                        while (todo != 0u) {
                            const int bit = 31 - __clz(todo);
                            todo &= ~(1u << bit);
                            const int pos = 15 - bit;  // n * 2 + e
                            if (slot < kListCap) list[slot] = (uint16_t)((r << 8) | (wq * 64 + (pos >> 1) * 8 + 2 * q + (pos & 1)));
                            ++slot;
                            atomicAdd(rowcnt + r, 1);
                        }
                    }
                }
            }
        }
        __syncthreads();
        // ---- exact re-evaluation ------------------------------------------------------------------
        {
            const int listed = *count;
            const bool everything = listed > kListCap;
            const int work = everything ? kRows * K : listed;
            for (int i = tid; i < work; i += kThreads) {
                int r, k;
                if (everything) {
                    r = i / K, k = i % K;
                } else {
                    const int entry = list[i];
                    r = entry >> 8, k = entry & 255;
                }
                if (k >= K) continue;
                if (!everything && rowcnt[r] == 1) {  // the only word within the margin is the argmin
                    best[r] = (unsigned long long)k;
                    continue;
                }
                const float *rv = res + r * RS;
                float dot = 0.0f;
#pragma unroll 8
                for (int i8 = 0; i8 < DSUB; i8 += 8) {
                    const uint4 cw = *reinterpret_cast<const uint4 *>(tab + L::tab_at(k, i8));
                    const __half2 *c2 = reinterpret_cast<const __half2 *>(&cw);
                    const float4 r0 = *reinterpret_cast<const float4 *>(rv + i8);
                    const float4 r1 = *reinterpret_cast<const float4 *>(rv + i8 + 4);
                    float2 c;
                    c = __half22float2(c2[0]);
                    dot = __fmaf_rn(r0.x, c.x, dot);
                    dot = __fmaf_rn(r0.y, c.y, dot);
                    c = __half22float2(c2[1]);
                    dot = __fmaf_rn(r0.z, c.x, dot);
                    dot = __fmaf_rn(r0.w, c.y, dot);
                    c = __half22float2(c2[2]);
                    dot = __fmaf_rn(r1.x, c.x, dot);
                    dot = __fmaf_rn(r1.y, c.y, dot);
                    c = __half22float2(c2[3]);
                    dot = __fmaf_rn(r1.z, c.x, dot);
                    dot = __fmaf_rn(r1.w, c.y, dot);
                }
                const float dist = distance_expr(xxs[r], nrm[k], dot);
                if (dist == dist) {  // a NaN distance never wins, as in a strict '<' scan
                    const unsigned long long key = ((unsigned long long)ordered_bits(dist) << 32) | (unsigned)k;
                    atomicMin(best + r, key);
                }
            }
        }
        __syncthreads();
        // ---- update: subtract the chosen words, refresh the fp16 copy -------------------------------
#pragma unroll
        for (int r = my_r; r < kRows; r += kPass) {
            const unsigned long long key = best[r];
            const int pick = (key == ~0ull) ? 0 : (int)(key & 0xffffffffull);
            float top = 0.0f;
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
                const int at = piece * (DSUB / 2) + 4 * my_c;
                __half2 c2[2];
                *reinterpret_cast<uint2 *>(c2) = *reinterpret_cast<const uint2 *>(tab + L::tab_at(pick, at));
                const float4 rv = *reinterpret_cast<const float4 *>(res + r * RS + at);
                const float2 w0 = __half22float2(c2[0]), w1 = __half22float2(c2[1]);
                const float4 nv = make_float4(__fsub_rn(rv.x, w0.x), __fsub_rn(rv.y, w0.y), __fsub_rn(rv.z, w1.x), __fsub_rn(rv.w, w1.y));
                top = fmaxf(top, store_residual4(res + r * RS + at, hi + L::hi_at(r, at), nv));
            }
            if (!(top < 32768.0f)) *big = 1;
        }
        if (tid < kRows) {
            const unsigned long long key = best[tid];
            const int pick = (key == ~0ull) ? 0 : (int)(key & 0xffffffffull);
            hist[tid * S + s] = (uint8_t)pick;
            if (code_at != nullptr) code_at[(int64_t)s * G] = (uint8_t)pick;
        }
    }

    if (recon != nullptr) {
        __syncthreads();
        // stage loop outermost: the gathers of a stage (this thread's rows and pieces) travel together
        constexpr int kMine = kRows / kPass;
        float4 sum[kMine][2];
#pragma unroll
        for (int i = 0; i < kMine; ++i) sum[i][0] = sum[i][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const __half *words = tables + ((int64_t)h * S * G + g) * (int64_t)K * DSUB + 4 * my_c;
        const int64_t stage_words = (int64_t)G * K * DSUB;
#pragma unroll 1
        for (int s = 0; s < S; ++s) {
            uint2 raw[kMine][2];
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
                const __half *word = words + s * stage_words + (int64_t)hist[(my_r + i * kPass) * S + s] * DSUB;
                raw[i][0] = *reinterpret_cast<const uint2 *>(word);
                raw[i][1] = *reinterpret_cast<const uint2 *>(word + DSUB / 2);
            }
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
#pragma unroll
                for (int piece = 0; piece < 2; ++piece) {
                    const __half2 *c2 = reinterpret_cast<const __half2 *>(&raw[i][piece]);
                    const float2 w0 = __half22float2(c2[0]), w1 = __half22float2(c2[1]);
                    float4 &acc = sum[i][piece];
                    acc = make_float4(__fadd_rn(acc.x, w0.x), __fadd_rn(acc.y, w0.y), __fadd_rn(acc.z, w1.x), __fadd_rn(acc.w, w1.y));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kMine; ++i) {
            const uint32_t row = tile + my_r + i * kPass;
            if (row >= rows) continue;
            const uint32_t b = row / (uint32_t)T, t = row % (uint32_t)T;
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
                const int at = piece * (DSUB / 2) + 4 * my_c;
                const int64_t o = (((int64_t)b * H + h) * T + t) * ((int64_t)G * DSUB) + (int64_t)g * DSUB + at;
                if (recon_dtype == TACVQ_F16) {
                    __half2 out[2] = {__floats2half2_rn(sum[i][piece].x, sum[i][piece].y), __floats2half2_rn(sum[i][piece].z, sum[i][piece].w)};
                    *reinterpret_cast<uint2 *>((__half *)recon + o) = *reinterpret_cast<const uint2 *>(out);
                } else {
                    *reinterpret_cast<float4 *>((float *)recon + o) = sum[i][piece];
                }
            }
        }
    }
    if constexpr (TM) {
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 0)
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kMaxWords) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// d = 64, 128 with the residual tile in tensor memory
// ------------------------------------------------------------------------------------------------
// Same search, organised around tensor memory.  Thread (row, q) = (32 * (warp % 4) + lane, warp / 4):
// a warp can reach the 32 tensor-memory lanes 32 * (warp % 4)..+31, and a lane is a row.
//   * The fp32 residual tile lives in tensor-memory columns [256, 256 + d) (the scores use [0, 256)); only
//     its fp16 rounding, the A operand of the product, is in shared memory.  Thread (row, q) owns the
//     8-element pieces q, q + 4, q + 8, ... of its row: exactly the elements of one of the four partial sums
//     the library's |r|^2 order is made of, so the residual update also yields the next stage's partial
//     sums, and a 16 KB exchange through shared memory finishes the norm.
//   * With the residual out of shared memory there is room for two table buffers: the next stage's table
//     arrives while the current stage is searched, as two cp.async.bulk.tensor (TMA) copies of a
//     [256 words x 64] box each, issued by one thread, which land in the swizzled panel order directly.
//   * A thread keeps the candidate mask of its 64 words; there is no list.  Rows with a single candidate
//     take it; otherwise every thread runs the exact chain for its own candidates, reading its row from
//     tensor memory 32 columns at a time (warp-wide loads, so the loop is warp-uniform).

template <int DSUB>
struct TmLargeLayout {
    static constexpr size_t kTabBytes = (size_t)kMaxWords * DSUB * 2;
    static constexpr size_t kTab = 0;                                   // two buffers, swizzled K-major panels
    static constexpr size_t kHi = 2 * kTabBytes;                        // [kRows][DSUB] half, swizzled K-major panels
    static constexpr size_t kExch = kHi + (size_t)kRows * DSUB * 2;     // [kRows][36] float: four partial-sum sets of 8
    static constexpr size_t kNrm = kExch + (size_t)kRows * 36 * 4;      // [256] float
    static constexpr size_t kSeed = kNrm + kMaxWords * 4;               // [256] float: -|c|^2/2
    static constexpr size_t kXx = kSeed + kMaxWords * 4;                // [kRows] float
    static constexpr size_t kRowMax = kXx + kRows * 4;                  // [4][kRows] float
    static constexpr size_t kCnt = kRowMax + 4 * kRows * 4;             // [4][kRows] int: candidates per quarter
    static constexpr size_t kBest = kCnt + 4 * kRows * 4;               // [kRows] u64
    static constexpr size_t kMisc = kBest + kRows * 8;                  // mbarrier, tensor-memory slot, flags, cc_max
    static constexpr size_t kHist = kMisc + 64;                         // [kRows][S] u8
    static constexpr size_t bytes(int S) { return kHist + (size_t)kRows * S + 1024; }  // + room to align the base
    __device__ static __forceinline__ int tab_at(int k, int e) {
        return (e >> 6) * (kMaxWords * 64) + k * 64 + ((((e >> 3) & 7) ^ (k & 7)) << 3) + (e & 7);
    }
    __device__ static __forceinline__ int hi_at(int r, int e) {
        return (e >> 6) * (kRows * 64) + r * 64 + ((((e >> 3) & 7) ^ (r & 7)) << 3) + (e & 7);
    }
};

__device__ __forceinline__ void tmem_load8(uint32_t *v, uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_store8(uint32_t taddr, const float *v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "f"(v[0]), "f"(v[1]),
                 "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                 : "memory");
}
__device__ __forceinline__ uint4 pack8_half(const float *v) {
    const __half2 h[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]), __floats2half2_rn(v[4], v[5]),
                          __floats2half2_rn(v[6], v[7])};
    return *reinterpret_cast<const uint4 *>(h);
}
__device__ __forceinline__ void unpack8_half(const uint4 raw, float *v) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <int DSUB, typename XT>
__global__ void __launch_bounds__(kThreads, 1)
encode_tm_large_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const __half *__restrict__ tables,
                       const float *__restrict__ sqnorm_in, uint8_t *__restrict__ codes, void *__restrict__ recon,
                       int recon_dtype, int B, int H, int T, int G, int S, int K, int64_t t0, int64_t T_cap, int vec_ok,
                       const __grid_constant__ CUtensorMap table_map, int use_map) {
    using L = TmLargeLayout<DSUB>;
    constexpr int kChunks = DSUB / 8;   // 16-byte pieces per row
    constexpr int kOwn = DSUB / 32;     // pieces a thread owns per row: q, q + 4, ...
    constexpr uint32_t kTmemCols = 512; // scores [0, 256), residual [256, 256 + DSUB)
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    unsigned char *smem_raw = smem_dyn + ((1024u - ((uint32_t)__cvta_generic_to_shared(smem_dyn) & 1023u)) & 1023u);
    __half *tab_buf = reinterpret_cast<__half *>(smem_raw + L::kTab);
    __half *hi = reinterpret_cast<__half *>(smem_raw + L::kHi);
    float *exch = reinterpret_cast<float *>(smem_raw + L::kExch);
    float *nrm = reinterpret_cast<float *>(smem_raw + L::kNrm);
    float *seed = reinterpret_cast<float *>(smem_raw + L::kSeed);
    float *xxs = reinterpret_cast<float *>(smem_raw + L::kXx);
    float *rowmax = reinterpret_cast<float *>(smem_raw + L::kRowMax);
    int *cnt = reinterpret_cast<int *>(smem_raw + L::kCnt);
    unsigned long long *best = reinterpret_cast<unsigned long long *>(smem_raw + L::kBest);
    const uint32_t mbar_a = (uint32_t)__cvta_generic_to_shared(smem_raw + L::kMisc);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_raw + L::kMisc + 8);
    int *big = reinterpret_cast<int *>(smem_raw + L::kMisc + 12);      // [2]: some residual element of stage parity p does not fit fp16
    int *tm_fail = reinterpret_cast<int *>(smem_raw + L::kMisc + 20);
    float *cc_max = reinterpret_cast<float *>(smem_raw + L::kMisc + 24);
    const uint32_t tma_bar = (uint32_t)__cvta_generic_to_shared(smem_raw + L::kMisc + 32);  // counts the bytes of a table copy
    uint8_t *hist = smem_raw + L::kHist;

    const int hg = blockIdx.y;
    const int h = hg / G, g = hg % G;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int row = (warp & 3) * 32 + lane, q = warp >> 2;
    const uint32_t rows = (uint32_t)B * (uint32_t)T;  // the launcher keeps B*T below 2^31
    const uint32_t tile = blockIdx.x * kRows;
    const float inf = __int_as_float(0x7f800000);

    // Table of stage s -> buffer s & 1.  Normally one thread asks the copy engine (TMA) for the table's 64-column
    // panels, which arrive in the 128-byte-swizzled order the tensor core reads and are counted by an
    // mbarrier; rows past K then hold whatever follows the group's words (never chosen: their norm is +inf).
    // Without a tensor map (use_map == 0), or if the wait for a copy ever ran out, all threads copy with cp.async.
    auto request_table = [&](int s) {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(tab_buf) + (uint32_t)(s & 1) * (uint32_t)L::kTabBytes;
        const int first_word = (((h * S + s) * G + g)) * K;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tma_bar), "r"((uint32_t)L::kTabBytes) : "memory");
#pragma unroll
        for (int panel = 0; panel < DSUB / 64; ++panel)
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst + panel * (kMaxWords * 128)), "l"(&table_map), "r"(panel * 64), "r"(first_word), "r"(tma_bar) : "memory");
    };
    auto fetch_table = [&](int s) {
        const __half *src = tables + (((int64_t)h * S + s) * G + g) * (int64_t)K * DSUB;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(tab_buf) + (uint32_t)(s & 1) * (uint32_t)L::kTabBytes;
#pragma unroll 1
        for (int idx = tid; idx < kMaxWords * kChunks; idx += kThreads) {
            const int k = idx / kChunks, c = idx % kChunks;
            const bool real = k < K;
            const __half *from = real ? src + (int64_t)k * DSUB + c * 8 : src;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (uint32_t)L::tab_at(k, c * 8) * 2), "l"(from),
                         "r"(real ? 16 : 0) : "memory");
        }
    };
    if (!use_map) fetch_table(0);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         (uint32_t)__cvta_generic_to_shared(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        big[0] = 0;
        big[1] = 0;
        *tm_fail = 0;
        *cc_max = 0.0f;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_a) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tma_bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (use_map && tid == 32) request_table(0);
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t score_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(q * 64);
    const uint32_t res_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)kMaxWords;

    uint8_t *code_at = nullptr;  // this row's first code byte (threads with q == 0)
    const bool live = tile + row < rows;
    const uint32_t rb = live ? (tile + row) / (uint32_t)T : 0u, rt = live ? (tile + row) % (uint32_t)T : 0u;
    if (q == 0 && live) code_at = codes + (((int64_t)rb * H + h) * T_cap + t0 + rt) * ((int64_t)S * G) + g;

    // ---- the block's rows: fp32 into tensor memory, fp16 rounding into shared memory, partial sums of |r|^2 ----
    {
        float part[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f}, top = 0.0f;
        float4 in[kOwn][2];  // every piece is requested before the first one is used
#pragma unroll
        for (int m = 0; m < kOwn; ++m) {
            in[m][0] = in[m][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (live) {
                const XT *src = x + (int64_t)rb * sxb + (int64_t)h * sxh + (int64_t)rt * sxt + (int64_t)g * DSUB + 8 * (q + 4 * m);
                in[m][0] = load4<XT>(src, vec_ok != 0);
                in[m][1] = load4<XT>(src + 4, vec_ok != 0);
            }
        }
#pragma unroll
        for (int m = 0; m < kOwn; ++m) {
            const int e0 = 8 * (q + 4 * m);
            const float v[8] = {in[m][0].x, in[m][0].y, in[m][0].z, in[m][0].w, in[m][1].x, in[m][1].y, in[m][1].z, in[m][1].w};
            tmem_store8(res_addr + e0, v);
            *reinterpret_cast<uint4 *>(hi + L::hi_at(row, e0)) = pack8_half(v);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                part[j] = __fadd_rn(part[j], __fmul_rn(v[j], v[j]));
                top = fmaxf(top, fabsf(v[j]));
            }
        }
        *reinterpret_cast<float4 *>(exch + row * 36 + q * 8) = make_float4(part[0], part[1], part[2], part[3]);
        *reinterpret_cast<float4 *>(exch + row * 36 + q * 8 + 4) = make_float4(part[4], part[5], part[6], part[7]);
        if (!(top < 32768.0f)) big[0] = 1;
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }

    uint64_t todo = 0ull;
    for (int s = 0; s < S; ++s) {
        const __half *tab = tab_buf + (size_t)(s & 1) * (L::kTabBytes / 2);
        // caller-supplied word norms: fetched by the upper half of the block
        const int norm_k = tid - (kThreads - kMaxWords);
        float norm_v = inf;
        if (sqnorm_in != nullptr && norm_k >= 0 && norm_k < K) norm_v = sqnorm_in[(((int64_t)h * S + s) * G + g) * K + norm_k];
        int late = 0;
        if (use_map) {
            int done = 0;
            for (int spin = 0; spin < (1 << 22) && !done; ++spin)  // bounded wait for the table's bytes
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.s32 %0, 1, 0, p;\n}"
                             : "=r"(done) : "r"(tma_bar), "r"((uint32_t)(s & 1)) : "memory");
            late = !done;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads the table and the fp16 rows
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (__syncthreads_or(late)) {  // never seen: copy the table the plain way (same bytes wherever both land)
            if (tid == 0) atomicAdd(&g_tensor_memory_timeouts, 1u);
            fetch_table(s);
            asm volatile("cp.async.wait_all;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
        }
        // table s, fp16 rows, residual and partial sums settled
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a0 = (uint32_t)__cvta_generic_to_shared(hi), b0 = (uint32_t)__cvta_generic_to_shared(tab);
#pragma unroll
            for (int ks = 0; ks < DSUB / 16; ++ks) {
                const uint64_t da = panel_descriptor(a0 + (ks >> 2) * (kRows * 128) + (ks & 3) * 32);
                const uint64_t db = panel_descriptor(b0 + (ks >> 2) * (kMaxWords * 128) + (ks & 3) * 32);
                asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                             ::"r"(tmem_base), "l"(da), "l"(db), "r"(kMmaShape), "r"(ks) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_a) : "memory");
            big[(s + 1) & 1] = 0;  // read two stages ago, raised by this stage's update
        }
        if (s + 1 < S) {  // its buffer was last read by the previous stage's update
            if (!use_map) fetch_table(s + 1);
            else if (tid == 32) request_table(s + 1);
        }
        // |c|^2 per word (eight lanes per word when the caller gave none), largest by an integer atomic maximum
        {
            float top = 0.0f;
            if (sqnorm_in == nullptr) {
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int k = warp * 16 + it * 4 + (lane >> 3);
                    float v = group8_sqnorm_ordered<DSUB>([&](int i) { return __half2float(tab[L::tab_at(k, i)]); }, lane);
                    if (k >= K) v = inf;  // padding words can never be chosen
                    else if (v == v) top = fmaxf(top, v);
                    if ((lane & 7) == 0) {
                        nrm[k] = v;
                        seed[k] = -0.5f * v;
                    }
                }
            } else if (norm_k >= 0) {
                nrm[norm_k] = norm_v;
                seed[norm_k] = -0.5f * norm_v;
                if (norm_k < K && norm_v == norm_v) top = norm_v;
            }
            if (sqnorm_in == nullptr || norm_k >= 0) {  // warp-uniform
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
                if (lane == 0) atomicMax(reinterpret_cast<int *>(cc_max), __float_as_int(top));
            }
        }
        // |r|^2 in the library's order from the four sets of partial sums: threads q == 1 (warps 4-7)
        if (q == 1) {
            const float4 *e = reinterpret_cast<const float4 *>(exch + row * 36);
            float mine[8];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const float4 s0 = e[hf], s1 = e[2 + hf], s2 = e[4 + hf], s3 = e[6 + hf];
                mine[4 * hf + 0] = __fadd_rn(__fadd_rn(__fadd_rn(s0.x, s1.x), s2.x), s3.x);
                mine[4 * hf + 1] = __fadd_rn(__fadd_rn(__fadd_rn(s0.y, s1.y), s2.y), s3.y);
                mine[4 * hf + 2] = __fadd_rn(__fadd_rn(__fadd_rn(s0.z, s1.z), s2.z), s3.z);
                mine[4 * hf + 3] = __fadd_rn(__fadd_rn(__fadd_rn(s0.w, s1.w), s2.w), s3.w);
            }
            float total = mine[0];
#pragma unroll
            for (int j = 1; j < 8; ++j) total = __fadd_rn(total, mine[j]);
            xxs[row] = total;
            best[row] = ~0ull;
        }
        __syncthreads();

        // ---- approximate scores from tensor memory: 64 words of quarter q per thread ----------------
        {
            int done = 0;
            for (int spin = 0; spin < (1 << 22) && !done; ++spin)  // bounded wait for the products issued above
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.s32 %0, 1, 0, p;\n}"
                             : "=r"(done) : "r"(mbar_a), "r"((uint32_t)(s & 1)) : "memory");
            if (!done) {  // never seen; the stage then re-evaluates every pair, so the codes stay exact
                *tm_fail = 1;
                atomicAdd(&g_tensor_memory_timeouts, 1u);
            }
            __syncwarp();
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float sc[64];
        {
            uint32_t v[64];
            tmem_load32(v, score_addr);
            tmem_load32(v + 32, score_addr + 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float top = -inf;
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
                const float4 sv = *reinterpret_cast<const float4 *>(seed + q * 64 + j);
                sc[j] = __uint_as_float(v[j]) + sv.x;
                sc[j + 1] = __uint_as_float(v[j + 1]) + sv.y;
                sc[j + 2] = __uint_as_float(v[j + 2]) + sv.z;
                sc[j + 3] = __uint_as_float(v[j + 3]) + sv.w;
                top = fmaxf(fmaxf(top, fmaxf(sc[j], sc[j + 1])), fmaxf(sc[j + 2], sc[j + 3]));
            }
            rowmax[q * kRows + row] = top;
        }
        __syncthreads();
        const bool everything = big[s & 1] != 0 || *tm_fail != 0;
        {
            const float top = fmaxf(fmaxf(rowmax[row], rowmax[kRows + row]), fmaxf(rowmax[2 * kRows + row], rowmax[3 * kRows + row]));
            const float cm = *cc_max, xx = xxs[row];
            const float margin = 1.220703125e-03f * sqrtf(xx * cm) + 6.103515625e-05f * (xx + cm) + 3.814697265625e-06f * sqrtf(cm);
            const float limit = everything ? -inf : top - margin;
            uint32_t lo = 0u, hi32 = 0u;
#pragma unroll
            for (int j = 31; j >= 0; --j) {
                lo = __funnelshift_l(__float_as_uint(sc[j] - limit), lo, 1);
                hi32 = __funnelshift_l(__float_as_uint(sc[32 + j] - limit), hi32, 1);
            }
            todo = everything ? ~0ull : ~(((uint64_t)hi32 << 32) | lo);  // set = not below the limit
            cnt[q * kRows + row] = __popcll(todo);
        }
        __syncthreads();
        if (tid == 0) *cc_max = 0.0f;  // read above; gathered again after the next stage's first barrier
        // ---- decide: a row's only candidate is its code; otherwise the exact chains of every candidate ------
        {
            const int listed = cnt[row] + cnt[kRows + row] + cnt[2 * kRows + row] + cnt[3 * kRows + row];
            if (!everything && listed == 1) {
                if (todo != 0ull) best[row] = (unsigned long long)(q * 64 + __ffsll((long long)todo) - 1);
                todo = 0ull;
            }
            const float xx = xxs[row];
            while (__any_sync(0xffffffffu, todo != 0ull)) {
                const bool active = todo != 0ull;
                int k = 0;
                if (active) {
                    k = q * 64 + __ffsll((long long)todo) - 1;
                    todo &= todo - 1ull;
                }
                const bool real = active && k < K;
                float dot = 0.0f;
#pragma unroll 1
                for (int c32 = 0; c32 < DSUB / 32; ++c32) {
                    uint32_t rv[32];
                    tmem_load32(rv, res_addr + c32 * 32);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (real) {
#pragma unroll
                        for (int i8 = 0; i8 < 4; ++i8) {
                            float c[8];
                            unpack8_half(*reinterpret_cast<const uint4 *>(tab + L::tab_at(k, c32 * 32 + i8 * 8)), c);
#pragma unroll
                            for (int j = 0; j < 8; ++j) dot = __fmaf_rn(__uint_as_float(rv[i8 * 8 + j]), c[j], dot);
                        }
                    }
                }
                if (real) {
                    const float dist = distance_expr(xx, nrm[k], dot);
                    if (dist == dist) {  // a NaN distance never wins, as in a strict '<' scan
                        const unsigned long long key = ((unsigned long long)ordered_bits(dist) << 32) | (unsigned)k;
                        atomicMin(best + row, key);
                    }
                }
            }
        }
        __syncthreads();
        // ---- update: subtract the chosen word from this thread's pieces, refresh the fp16 copy, next partial sums ----
        {
            const unsigned long long key = best[row];
            const int pick = (key == ~0ull) ? 0 : (int)(key & 0xffffffffull);
            uint32_t rv[kOwn][8];
#pragma unroll
            for (int m = 0; m < kOwn; ++m) tmem_load8(rv[m], res_addr + 8 * (q + 4 * m));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float part[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f}, top = 0.0f;
#pragma unroll
            for (int m = 0; m < kOwn; ++m) {
                const int e0 = 8 * (q + 4 * m);
                float c[8], nv[8];
                unpack8_half(*reinterpret_cast<const uint4 *>(tab + L::tab_at(pick, e0)), c);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    nv[j] = __fsub_rn(__uint_as_float(rv[m][j]), c[j]);
                    part[j] = __fadd_rn(part[j], __fmul_rn(nv[j], nv[j]));
                    top = fmaxf(top, fabsf(nv[j]));
                }
                tmem_store8(res_addr + e0, nv);
                *reinterpret_cast<uint4 *>(hi + L::hi_at(row, e0)) = pack8_half(nv);
            }
            *reinterpret_cast<float4 *>(exch + row * 36 + q * 8) = make_float4(part[0], part[1], part[2], part[3]);
            *reinterpret_cast<float4 *>(exch + row * 36 + q * 8 + 4) = make_float4(part[4], part[5], part[6], part[7]);
            if (!(top < 32768.0f)) big[(s + 1) & 1] = 1;
            if (q == 0) {
                hist[row * S + s] = (uint8_t)pick;
                if (code_at != nullptr) code_at[(int64_t)s * G] = (uint8_t)pick;
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
    }

    if (recon != nullptr) {
        __syncthreads();
        constexpr int kPass = kThreads / kChunks;
        const int my_c = tid % kChunks, my_r = tid / kChunks;
        // stage loop outermost: the gathers of a stage (this thread's rows and pieces) travel together
        constexpr int kMine = kRows / kPass;
        float4 sum[kMine][2];
#pragma unroll
        for (int i = 0; i < kMine; ++i) sum[i][0] = sum[i][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const __half *words = tables + ((int64_t)h * S * G + g) * (int64_t)K * DSUB + 4 * my_c;
        const int64_t stage_words = (int64_t)G * K * DSUB;
#pragma unroll 1
        for (int s = 0; s < S; ++s) {
            uint2 raw[kMine][2];
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
                const __half *word = words + s * stage_words + (int64_t)hist[(my_r + i * kPass) * S + s] * DSUB;
                raw[i][0] = *reinterpret_cast<const uint2 *>(word);
                raw[i][1] = *reinterpret_cast<const uint2 *>(word + DSUB / 2);
            }
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
#pragma unroll
                for (int piece = 0; piece < 2; ++piece) {
                    const __half2 *c2 = reinterpret_cast<const __half2 *>(&raw[i][piece]);
                    const float2 w0 = __half22float2(c2[0]), w1 = __half22float2(c2[1]);
                    float4 &acc = sum[i][piece];
                    acc = make_float4(__fadd_rn(acc.x, w0.x), __fadd_rn(acc.y, w0.y), __fadd_rn(acc.z, w1.x), __fadd_rn(acc.w, w1.y));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kMine; ++i) {
            const uint32_t grow = tile + my_r + i * kPass;
            if (grow >= rows) continue;
            const uint32_t b = grow / (uint32_t)T, t = grow % (uint32_t)T;
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
                const int at = piece * (DSUB / 2) + 4 * my_c;
                const int64_t o = (((int64_t)b * H + h) * T + t) * ((int64_t)G * DSUB) + (int64_t)g * DSUB + at;
                if (recon_dtype == TACVQ_F16) {
                    __half2 out[2] = {__floats2half2_rn(sum[i][piece].x, sum[i][piece].y), __floats2half2_rn(sum[i][piece].z, sum[i][piece].w)};
                    *reinterpret_cast<uint2 *>((__half *)recon + o) = *reinterpret_cast<const uint2 *>(out);
                } else {
                    *reinterpret_cast<float4 *>((float *)recon + o) = sum[i][piece];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

#ifndef TACVQ_ENCODE_TENSOR_MEMORY
#define TACVQ_ENCODE_TENSOR_MEMORY 2  // 2: residual tile in tensor memory; 1: scores only; 0: mma.sync from registers
#endif

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against the driver
typedef CUresult (*TensorMapEncoder)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                     const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncoder tensor_map_encoder() {
    static const TensorMapEncoder found = [] {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return reinterpret_cast<TensorMapEncoder>(entry);
    }();
    return found;
}

// Launches whose tables had at least 256 words but got no tensor map (no encoder in the driver, or it refused):
// added to the count that tacvq_encode_tensor_memory_timeouts reports, so a silent cp.async-only run shows up.
static std::atomic<unsigned int> g_table_map_failures{0};

// The fp16 tables as a 2-D tensor [all words][d] read in boxes of 256 words x 64 elements with the 128-byte swizzle.
// Returns 0 when no map could be made (the kernel then copies tables with cp.async).
static int make_table_map(CUtensorMap *map, const void *tables, int64_t words, int d) {
    memset(map, 0, sizeof(*map));
    const TensorMapEncoder encode = tensor_map_encoder();
    if (encode == nullptr || words < kMaxWords) return 0;
    const cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)words};
    const cuuint64_t strides[1] = {(cuuint64_t)d * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kMaxWords};
    const cuuint32_t steps[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(tables), dims, strides, box, steps,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 1 : 0;
}

template <int DSUB>
static int launch_tc_large(const EncodeArgs &a) {
    // tcgen05 panels have 64-element rows, so the tensor-memory path carries d = 64 and 128
    constexpr bool TM = TACVQ_ENCODE_TENSOR_MEMORY != 0 && DSUB >= 64;
    constexpr bool TM2 = TACVQ_ENCODE_TENSOR_MEMORY == 2 && DSUB >= 64;
    size_t smem = TcLargeLayout<DSUB, TM>::bytes(a.S);
    if constexpr (TM2) smem = TmLargeLayout<DSUB>::bytes(a.S);
    if (smem > 227 * 1024) return TACVQ_ERR_UNSUPPORTED;
    const int64_t rows = (int64_t)a.B * a.T;
    if (rows >= (int64_t)1 << 31) return TACVQ_ERR_UNSUPPORTED;
    if (a.recon != nullptr && (reinterpret_cast<uintptr_t>(a.recon) & 15u) != 0) return TACVQ_ERR_UNSUPPORTED;
    // 4-element vector loads of the states need an aligned base and strides that keep the alignment
    const size_t elem = a.x_dtype == TACVQ_F16 ? 2 : 4;
    const int vec_ok = (reinterpret_cast<uintptr_t>(a.x) % (4 * elem) == 0 && a.sxb % 4 == 0 && a.sxh % 4 == 0 && a.sxt % 4 == 0) ? 1 : 0;
    dim3 grid((unsigned)((rows + kRows - 1) / kRows), (unsigned)(a.H * a.G));
    auto launch = [&](auto kernel, auto *xp) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, kThreads, smem, a.stream>>>(xp, a.sxb, a.sxh, a.sxt, (const __half *)a.tables, a.sqnorm, a.codes,
                                                   a.recon, a.recon_dtype, a.B, a.H, a.T, a.G, a.S, a.K, a.t0, a.T_cap, vec_ok);
        return launch_status();
    };
    if constexpr (TM2) {
        CUtensorMap table_map;
        const int64_t words = (int64_t)a.H * a.S * a.G * a.K;
        const int use_map = make_table_map(&table_map, a.tables, words, DSUB);
        if (!use_map && words >= kMaxWords) g_table_map_failures.fetch_add(1u);
        auto launch_tm = [&](auto kernel, auto *xp) -> int {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            kernel<<<grid, kThreads, smem, a.stream>>>(xp, a.sxb, a.sxh, a.sxt, (const __half *)a.tables, a.sqnorm, a.codes, a.recon,
                                                       a.recon_dtype, a.B, a.H, a.T, a.G, a.S, a.K, a.t0, a.T_cap, vec_ok, table_map,
                                                       use_map);
            return launch_status();
        };
        if (a.x_dtype == TACVQ_F16) return launch_tm(encode_tm_large_kernel<DSUB, __half>, (const __half *)a.x);
        return launch_tm(encode_tm_large_kernel<DSUB, float>, (const float *)a.x);
    } else {
        if (a.x_dtype == TACVQ_F16) return launch(encode_tc_large_kernel<DSUB, __half, TM>, (const __half *)a.x);
        return launch(encode_tc_large_kernel<DSUB, float, TM>, (const float *)a.x);
    }
}

// Returns TACVQ_ERR_UNSUPPORTED when the geometry is not this kernel's, so the caller can go on to
// the scalar kernels.
int encode_tc_large_launch(const EncodeArgs &a) {
    if (a.tables_f32 || a.K > kMaxWords) return TACVQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a.tables) & 15u) != 0) return TACVQ_ERR_UNSUPPORTED;
    switch (a.D / a.G) {
        case 32: return launch_tc_large<32>(a);
        case 64: return launch_tc_large<64>(a);
        case 128: return launch_tc_large<128>(a);
        default: return TACVQ_ERR_UNSUPPORTED;
    }
}

int tensor_memory_timeouts(unsigned int *out) {
    const int st = (int)cudaMemcpyFromSymbol(out, g_tensor_memory_timeouts, sizeof(unsigned int));
    if (st == 0) *out += g_table_map_failures.load();
    return st;
}

}  // namespace tacvq
