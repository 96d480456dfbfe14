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

int decode_dispatch(const uint8_t *codes, const __half *tables, void *out, int out_dtype, int B, int H, int T, int D,
                    int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream) {
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

int table_sqnorm_dispatch(const __half *tables, float *out, int64_t words, int d, cudaStream_t stream) {
    if (words == 0) return TACVQ_OK;
    table_sqnorm_kernel<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>(tables, out, words, d);
    return launch_status();
}

}  // namespace tacvq
