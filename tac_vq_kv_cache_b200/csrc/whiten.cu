// Whitened assignment geometry: transform rows and codewords once, before the search.
//
//   search_rows[b,h,t,g*d+i]   = sum_j W[h,g,i,j] * x[b,h,t,g*d+j]
//   search_tables[h,s,g,k,i]   = sum_j W[h,g,i,j] * tables[h,s,g,k,j]
// each as one fused-multiply-add chain over j ascending.  The encode kernels then search the
// transformed rows against the transformed words and subtract transformed words stage by stage,
// which is the reference's "transform once, subtract transformed codewords" recursion
// (src/jointkv/closed_loop_vq.py:312-320, 384-390; src/jointkv/cq_tac.py:80-85).

#include "common.cuh"

namespace tacvq {

template <typename XT>
__global__ void __launch_bounds__(256)
whiten_rows_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const float *__restrict__ whitener,
                   float *__restrict__ out, int B, int H, int T, int D, int G) {
    const int d = D / G;
    const int64_t total = (int64_t)B * H * T * D;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % D);
        const int64_t row = idx / D;
        const int t = (int)(row % T);
        const int64_t bh = row / T;
        const int h = (int)(bh % H);
        const int64_t b = bh / H;
        const int g = c / d, i = c % d;
        const XT *src = x + b * sxb + (int64_t)h * sxh + (int64_t)t * sxt + (int64_t)g * d;
        const float *w = whitener + (((int64_t)h * G + g) * d + i) * d;
        float acc = 0.0f;
        for (int j = 0; j < d; ++j) acc = __fmaf_rn(w[j], to_float<XT>(src[j]), acc);
        out[idx] = acc;
    }
}

__global__ void __launch_bounds__(256)
whiten_tables_kernel(const __half *__restrict__ tables, const float *__restrict__ whitener, float *__restrict__ out,
                     int H, int S, int G, int K, int d) {
    const int64_t total = (int64_t)H * S * G * K * d;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % d);
        const int64_t word = idx / d;  // ((h*S+s)*G+g)*K+k
        const int g = (int)((word / K) % G);
        const int h = (int)(word / ((int64_t)K * G * S));
        const float *w = whitener + (((int64_t)h * G + g) * d + i) * d;
        const __half *src = tables + word * d;
        float acc = 0.0f;
        for (int j = 0; j < d; ++j) acc = __fmaf_rn(__half2float(src[j]), w[j], acc);
        out[idx] = acc;
    }
}

int whiten_dispatch(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt, const __half *tables,
                    const float *whitener, float *search_tables, float *search_rows, int B, int H, int T, int D, int G,
                    int S, int K, cudaStream_t stream) {
    const int d = D / G;
    const int64_t tt = (int64_t)H * S * G * K * d;
    int64_t blocks = (tt + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    whiten_tables_kernel<<<(unsigned)blocks, 256, 0, stream>>>(tables, whitener, search_tables, H, S, G, K, d);
    int st = launch_status();
    if (st != TACVQ_OK) return st;
    const int64_t rt = (int64_t)B * H * T * D;
    blocks = (rt + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (x_dtype == TACVQ_F16)
        whiten_rows_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>((const __half *)x, sxb, sxh, sxt, whitener, search_rows, B, H, T, D, G);
    else
        whiten_rows_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((const float *)x, sxb, sxh, sxt, whitener, search_rows, B, H, T, D, G);
    return launch_status();
}

}  // namespace tacvq
