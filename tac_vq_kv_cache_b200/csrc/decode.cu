// Decode kernels: rows from stored codes, and the matching codeword-gradient scatter.
//
// decode: out[b,h,t,g*d+i] = cast( sum_{s<S_use} tables[h,s,g,codes[b,h,t0+t,s,g],i] ), the sum taken
// in fp32 in stage order starting from zero - the only order the reference uses
// (src/jointkv/closed_loop_vq.py:332-336, 376-381, 398-403; src/jointkv/cq_tac.py:98-105;
// experiments/train_pure_uniform16_closed_loop_vq.py:395-442).  One thread produces VEC contiguous
// channels of one row; the output write is the HBM stream, table reads hit L1/L2 (a head's tables
// are at most a few hundred KB).

#include "common.cuh"

namespace tacvq {

template <int VEC>
struct HalfVec;
template <>
struct HalfVec<1> { using type = unsigned short; };
template <>
struct HalfVec<2> { using type = unsigned int; };
template <>
struct HalfVec<4> { using type = uint2; };
template <>
struct HalfVec<8> { using type = uint4; };

template <int VEC, typename OT>
__global__ void __launch_bounds__(256)
decode_kernel(const uint8_t *__restrict__ codes, const __half *__restrict__ tables, OT *__restrict__ out, int B, int H,
              int T, int D, int G, int S, int S_use, int K, int64_t t0, int64_t T_cap) {
    const int d = D / G;
    const int chunks = D / VEC;  // per row
    const int64_t total = (int64_t)B * H * T * chunks;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int chunk = (int)(idx % chunks);
        const int64_t row = idx / chunks;  // (b*H + h)*T + t
        const int t = (int)(row % T);
        const int64_t bh = row / T;
        const int h = (int)(bh % H);
        const int c0 = chunk * VEC;
        const int g = c0 / d, i0 = c0 % d;
        const uint8_t *cd = codes + ((bh * T_cap + t0 + t) * S) * G + g;
        float sum[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) sum[i] = 0.0f;
        for (int s = 0; s < S_use; ++s) {
            const int code = cd[(int64_t)s * G];
            const __half *w = tables + ((((int64_t)h * S + s) * G + g) * K + code) * d + i0;
            typename HalfVec<VEC>::type raw = __ldg(reinterpret_cast<const typename HalfVec<VEC>::type *>(w));
            const __half *hv = reinterpret_cast<const __half *>(&raw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) sum[i] = __fadd_rn(sum[i], __half2float(hv[i]));
        }
        OT *dst = out + row * D + c0;
        if constexpr (sizeof(OT) == 2) {
            typename HalfVec<VEC>::type packed;
            __half *pv = reinterpret_cast<__half *>(&packed);
#pragma unroll
            for (int i = 0; i < VEC; ++i) pv[i] = __float2half_rn(sum[i]);
            *reinterpret_cast<typename HalfVec<VEC>::type *>(dst) = packed;
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) dst[i] = sum[i];
        }
    }
}

template <typename OT>
static int launch_decode(const uint8_t *codes, const __half *tables, OT *out, int B, int H, int T, int D, int G, int S,
                         int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream) {
    const int d = D / G;
    const int vec = (d % 8 == 0) ? 8 : (d % 4 == 0) ? 4 : (d % 2 == 0) ? 2 : 1;
    const int64_t total = (int64_t)B * H * T * (D / vec);
    if (total == 0) return TACVQ_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 64) blocks = 148 * 64;
    switch (vec) {
        case 8: decode_kernel<8, OT><<<(unsigned)blocks, 256, 0, stream>>>(codes, tables, out, B, H, T, D, G, S, S_use, K, t0, T_cap); break;
        case 4: decode_kernel<4, OT><<<(unsigned)blocks, 256, 0, stream>>>(codes, tables, out, B, H, T, D, G, S, S_use, K, t0, T_cap); break;
        case 2: decode_kernel<2, OT><<<(unsigned)blocks, 256, 0, stream>>>(codes, tables, out, B, H, T, D, G, S, S_use, K, t0, T_cap); break;
        default: decode_kernel<1, OT><<<(unsigned)blocks, 256, 0, stream>>>(codes, tables, out, B, H, T, D, G, S, S_use, K, t0, T_cap); break;
    }
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// decode with the head's tables staged in shared memory by bulk asynchronous copies (TMA)
// ------------------------------------------------------------------------------------------------
// When all stages of one head's tables fit in shared memory (S*G*K*d*2 bytes <= 160 KB), a block takes
// one head, pulls its tables in with cp.async.bulk (one elected thread issues the copies, an mbarrier
// counts the bytes) and then streams rows: code bytes in, 16-byte fp16/fp32 chunks out, fully coalesced.
// The wait on the mbarrier is bounded; if it ever ran out the block would simply read the tables from
// global memory instead, so results do not depend on the copy engine.

constexpr int kStagedThreads = 1024;
constexpr int kStagedMaxBytes = 160 * 1024;
constexpr int kBulkPiece = 16 * 1024;

template <typename OT>
__global__ void __launch_bounds__(kStagedThreads)
decode_staged_kernel(const uint8_t *__restrict__ codes, const __half *__restrict__ tables, OT *__restrict__ out, int B,
                     int H, int T, int D, int G, int S, int S_use, int K, int64_t t0, int64_t T_cap) {
    extern __shared__ __align__(128) unsigned char staged[];
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int ready_s;
    const int h = blockIdx.y;
    const int d = D / G;
    const uint32_t table_bytes = (uint32_t)S * G * K * d * 2;
    const unsigned char *src = reinterpret_cast<const unsigned char *>(tables) + (size_t)h * table_bytes;
    const uint32_t mbar_a = (uint32_t)__cvta_generic_to_shared(&mbar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_a));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar_a), "r"(table_bytes) : "memory");
        for (uint32_t off = 0; off < table_bytes; off += kBulkPiece) {
            const uint32_t n = min((uint32_t)kBulkPiece, table_bytes - off);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(staged + off)),
                         "l"(src + off), "r"(n), "r"(mbar_a)
                         : "memory");
        }
        int ok = 0;
        for (int spin = 0; spin < (1 << 22) && !ok; ++spin) {  // bounded: a few milliseconds at most
            asm volatile(
                "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.s32 %0, 1, 0, p;\n}"
                : "=r"(ok)
                : "r"(mbar_a)
                : "memory");
        }
        ready_s = ok;
    }
    __syncthreads();
    const __half *tab = ready_s ? reinterpret_cast<const __half *>(staged) : tables + (size_t)h * (table_bytes / 2);

    // thread = (row lane, 8-channel chunk): chunk, group and table offset are fixed per thread; a block owns a
    // contiguous range of the head's rows and walks it with additive updates (no division in the loop)
    const int chunks = D / 8;
    const int rows_per_pass = kStagedThreads / chunks;
    const int chunk = threadIdx.x % chunks, row_lane = threadIdx.x / chunks;
    const int c0 = chunk * 8, g = c0 / d, i0 = c0 % d;
    const int rows = B * T;  // the launcher keeps this below 2^31
    const int per_block = (rows + gridDim.x - 1) / gridDim.x;
    const int r_begin = blockIdx.x * per_block, r_end = min(rows, r_begin + per_block);
    const __half *tab_g = tab + (size_t)g * K * d + i0;   // + (s*G*K + code) * d
    const int stage_stride = G * K * d;                   // halves; a head's tables are at most 160 KB
    const int slots = S * G;
    int row = r_begin + row_lane;
    int b = row / T, t = row - b * T;
    // byte offset of this thread's first code and element offset of its output chunk; both advance by a
    // constant per pass and are recomputed only when the walk enters the next batch row
    auto code_offset = [&](int bb, int tt) { return (((size_t)bb * H + h) * T_cap + t0 + tt) * slots + g; };
    auto out_offset = [&](int bb, int tt) { return (((size_t)bb * H + h) * T + tt) * (size_t)D + c0; };
    size_t code_at = code_offset(b, t), out_at = out_offset(b, t);
    // codes of the first row (at most two stages are fetched ahead; deeper stacks read the rest in the loop)
    // (groups of 4 channels: the chunk is two whole words of neighbouring groups, and the two codes fetched
    // ahead are those of the first stage)
    const bool narrow = d == 4;
    int ahead0 = 0, ahead1 = 0;
    if (row < r_end) {
        ahead0 = codes[code_at];
        if (narrow) ahead1 = codes[code_at + 1];
        else if (S_use > 1) ahead1 = codes[code_at + G];
    }
    for (; row < r_end; row += rows_per_pass) {
        const int c_first = ahead0, c_second = ahead1;
        const size_t code_now = code_at, out_now = out_at;
        t += rows_per_pass;
        if (t >= T) {
            while (t >= T) {
                t -= T;
                ++b;
            }
            code_at = code_offset(b, t);
            out_at = out_offset(b, t);
        } else {
            code_at += (size_t)rows_per_pass * slots;
            out_at += (size_t)rows_per_pass * D;
        }
        if (row + rows_per_pass < r_end) {  // the next row's codes travel while this row is rebuilt
            ahead0 = codes[code_at];
            if (narrow) ahead1 = codes[code_at + 1];
            else if (S_use > 1) ahead1 = codes[code_at + G];
        }
        OT *dst = out + out_now;
        if (narrow) {
            float sum[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
            for (int s = 0; s < S_use; ++s) {
                const int ca = s == 0 ? c_first : (int)codes[code_now + (size_t)s * G];
                const int cb = s == 0 ? c_second : (int)codes[code_now + (size_t)s * G + 1];
                const uint2 wa = *reinterpret_cast<const uint2 *>(tab_g + s * stage_stride + ca * 4);
                const uint2 wb = *reinterpret_cast<const uint2 *>(tab_g + s * stage_stride + K * 4 + cb * 4);
                const __half2 hv[4] = {*reinterpret_cast<const __half2 *>(&wa.x), *reinterpret_cast<const __half2 *>(&wa.y),
                                       *reinterpret_cast<const __half2 *>(&wb.x), *reinterpret_cast<const __half2 *>(&wb.y)};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(hv[i]);
                    sum[2 * i] = __fadd_rn(sum[2 * i], f.x);
                    sum[2 * i + 1] = __fadd_rn(sum[2 * i + 1], f.y);
                }
            }
            if constexpr (sizeof(OT) == 2) {
                uint4 packed;
                __half2 *pv = reinterpret_cast<__half2 *>(&packed);
#pragma unroll
                for (int i = 0; i < 4; ++i) pv[i] = __floats2half2_rn(sum[2 * i], sum[2 * i + 1]);
                *reinterpret_cast<uint4 *>(dst) = packed;
            } else {
                *reinterpret_cast<float4 *>(dst) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                *reinterpret_cast<float4 *>(dst + 4) = make_float4(sum[4], sum[5], sum[6], sum[7]);
            }
            continue;
        }
        if (S_use <= 2 && sizeof(OT) == 2) {
            // one or two fp16 words: their fp32 sum is exact, so its single rounding to fp16 is a packed fp16 add
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (S_use >= 1) packed = *reinterpret_cast<const uint4 *>(tab_g + c_first * d);
            if (S_use == 2) {
                const uint4 second = *reinterpret_cast<const uint4 *>(tab_g + stage_stride + c_second * d);
                __half2 *pv = reinterpret_cast<__half2 *>(&packed);
                const __half2 *sv = reinterpret_cast<const __half2 *>(&second);
#pragma unroll
                for (int i = 0; i < 4; ++i) pv[i] = __hadd2(pv[i], sv[i]);
            }
            *reinterpret_cast<uint4 *>(dst) = packed;
            continue;
        }
        float sum[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
        for (int s = 0; s < S_use; ++s) {
            const int c = s == 0 ? c_first : (s == 1 ? c_second : (int)codes[code_now + (size_t)s * G]);
            const uint4 raw = *reinterpret_cast<const uint4 *>(tab_g + s * stage_stride + c * d);
            const __half2 *hv = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(hv[i]);
                sum[2 * i] = __fadd_rn(sum[2 * i], f.x);
                sum[2 * i + 1] = __fadd_rn(sum[2 * i + 1], f.y);
            }
        }
        if constexpr (sizeof(OT) == 2) {
            uint4 packed;
            __half2 *pv = reinterpret_cast<__half2 *>(&packed);
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = __floats2half2_rn(sum[2 * i], sum[2 * i + 1]);  // one convert per pair
            *reinterpret_cast<uint4 *>(dst) = packed;
        } else {
            *reinterpret_cast<float4 *>(dst) = make_float4(sum[0], sum[1], sum[2], sum[3]);
            *reinterpret_cast<float4 *>(dst + 4) = make_float4(sum[4], sum[5], sum[6], sum[7]);
        }
    }
    if (threadIdx.x == 0 && !ready_s) {
        // the copy did not report completion in time: give it one more bounded wait so that no bulk copy
        // is still writing this block's shared memory when the block retires
        int ok = 0;
        for (int spin = 0; spin < (1 << 22) && !ok; ++spin) {
            asm volatile(
                "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.s32 %0, 1, 0, p;\n}"
                : "=r"(ok)
                : "r"(mbar_a)
                : "memory");
        }
    }
}

template <typename OT>
static int launch_decode_staged(const uint8_t *codes, const __half *tables, OT *out, int B, int H, int T, int D, int G,
                                int S, int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream) {
    const size_t bytes = (size_t)S * G * K * (D / G) * 2;
    auto kernel = decode_staged_kernel<OT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
    // whole waves of blocks (one 1024-thread block per SM), as long as a block keeps >= 512 rows to
    // amortise its table copy
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t rows = (int64_t)B * T;
    int64_t per_head = 1;
    for (int waves = 4; waves >= 1; --waves) {
        const int64_t cand = ((int64_t)waves * sms) / H;
        if (cand >= 1 && rows / cand >= 512) {
            per_head = cand;
            break;
        }
    }
    dim3 grid((unsigned)per_head, (unsigned)H);
    kernel<<<grid, kStagedThreads, bytes, stream>>>(codes, tables, out, B, H, T, D, G, S, S_use, K, t0, T_cap);
    return launch_status();
}

int decode_dispatch(const uint8_t *codes, const __half *tables, void *out, int out_dtype, int B, int H, int T, int D,
                    int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream) {
    const int d = D / G;
    const size_t head_bytes = (size_t)S * G * K * d * 2;
    const bool staged = (d % 8 == 0 || d == 4) && D % 8 == 0 && kStagedThreads % (D / 8) == 0 && (int64_t)B * T < 0x7fffffff &&
                        head_bytes <= (size_t)kStagedMaxBytes && head_bytes % 16 == 0 &&
                        ((uintptr_t)tables & 15) == 0 && ((uintptr_t)out & 15) == 0 && (int64_t)B * T >= 1024;
    if (staged) {
        if (out_dtype == TACVQ_F16)
            return launch_decode_staged<__half>(codes, tables, (__half *)out, B, H, T, D, G, S, S_use, K, t0, T_cap, stream);
        return launch_decode_staged<float>(codes, tables, (float *)out, B, H, T, D, G, S, S_use, K, t0, T_cap, stream);
    }
    if (out_dtype == TACVQ_F16)
        return launch_decode<__half>(codes, tables, (__half *)out, B, H, T, D, G, S, S_use, K, t0, T_cap, stream);
    return launch_decode<float>(codes, tables, (float *)out, B, H, T, D, G, S, S_use, K, t0, T_cap, stream);
}

// grad_tables[h,s,g,code,i] += grad_out[b,h,t,g*d+i] for s < S_use.  One thread per (row, channel);
// fp32 atomics into the (small, L2-resident) table gradient.
__global__ void __launch_bounds__(256)
codeword_grad_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ grad_out,
                     float *__restrict__ grad_tables, int B, int H, int T, int D, int G, int S, int S_use, int K,
                     int64_t t0, int64_t T_cap) {
    const int d = D / G;
    const int64_t total = (int64_t)B * H * T * D;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % D);
        const int64_t row = idx / D;
        const int t = (int)(row % T);
        const int64_t bh = row / T;
        const int h = (int)(bh % H);
        const int g = c / d, i = c % d;
        const float v = grad_out[idx];
        const uint8_t *cd = codes + ((bh * T_cap + t0 + t) * S) * G + g;
        for (int s = 0; s < S_use; ++s) {
            const int code = cd[(int64_t)s * G];
            atomicAdd(grad_tables + ((((int64_t)h * S + s) * G + g) * K + code) * d + i, v);
        }
    }
}

int codeword_grad_dispatch(const uint8_t *codes, const float *grad_out, float *grad_tables, int B, int H, int T, int D,
                           int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream) {
    const int64_t total = (int64_t)B * H * T * D;
    if (total == 0) return TACVQ_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    codeword_grad_kernel<<<(unsigned)blocks, 256, 0, stream>>>(codes, grad_out, grad_tables, B, H, T, D, G, S, S_use, K,
                                                               t0, T_cap);
    return launch_status();
}

// out[w] = |table word w|^2 in the library's order.
__global__ void __launch_bounds__(256)
table_sqnorm_kernel(const __half *__restrict__ tables, float *__restrict__ out, int64_t words, int d) {
    const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= words) return;
    float v[128];
    if (d <= 128) {
        for (int i = 0; i < d; ++i) v[i] = __half2float(tables[w * d + i]);
        out[w] = sqnorm_ordered_rt(v, d);
    }
}

// d a multiple of 32: eight neighbouring lanes per word.  Lane j owns running sum j of each of the four
// sets (element i goes to set (i/8)%4, sum i%8), adds its sets ((0+1)+2)+3, and the eight sums are added
// 0..7 - the library's order for such d.
__global__ void __launch_bounds__(256)
table_sqnorm_wide_kernel(const __half *__restrict__ tables, float *__restrict__ out, int64_t words, int d) {
    const int64_t slot = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31, j = lane & 7;
    const int64_t word = slot >> 3;
    const __half *src = tables + (word < words ? word : words - 1) * d;  // spare lanes redo the last word
    float set[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int i = 0; i < d; i += 32) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float v = __half2float(src[i + 8 * u + j]);
            set[u] = __fadd_rn(set[u], __fmul_rn(v, v));
        }
    }
    const float mine = __fadd_rn(__fadd_rn(__fadd_rn(set[0], set[1]), set[2]), set[3]);
    const int first = lane & 24;
    float total = __shfl_sync(0xffffffffu, mine, first);
#pragma unroll
    for (int k = 1; k < 8; ++k) total = __fadd_rn(total, __shfl_sync(0xffffffffu, mine, first + k));
    if (j == 0 && word < words) out[word] = total;
}

int table_sqnorm_dispatch(const __half *tables, float *out, int64_t words, int d, cudaStream_t stream) {
    if (words == 0) return TACVQ_OK;
    if (d % 32 == 0) {
        table_sqnorm_wide_kernel<<<(unsigned)((words * 8 + 255) / 256), 256, 0, stream>>>(tables, out, words, d);
        return launch_status();
    }
    table_sqnorm_kernel<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>(tables, out, words, d);
    return launch_status();
}

}  // namespace tacvq
