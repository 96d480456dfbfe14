// Whitened assignment geometry: transform rows and codewords once, before the search.
//
//   search_rows[b,h,t,g*d+i]   = sum_j W[h,g,i,j] * x[b,h,t,g*d+j]
//   search_tables[h,s,g,k,i]   = sum_j W[h,g,i,j] * tables[h,s,g,k,j]
// each as one fused-multiply-add chain over j ascending.  The encode kernels then search the
// transformed rows against the transformed words and subtract transformed words stage by stage,
// which is the reference's "transform once, subtract transformed codewords" recursion
// (src/jointkv/closed_loop_vq.py:312-320, 384-390; src/jointkv/cq_tac.py:80-85).
//
// Wide groups (d = 32, 64, 128) are a d x d product per row: a block keeps one (head, group) matrix,
// transposed, and a tile of 64 rows in shared memory; a thread owns 4 outputs of several rows and
// walks j in order, four steps per 16-byte shared-memory load.  Narrow groups (d <= 16) cost d
// multiply-adds per output and stay one thread per output.

#include "common.cuh"

namespace tacvq {

// ------------------------------------------------------------------------------------------------
// narrow groups: one thread = one output element
// ------------------------------------------------------------------------------------------------

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

// ------------------------------------------------------------------------------------------------
// wide groups: shared-memory tiles, 4 outputs x several rows per thread
// ------------------------------------------------------------------------------------------------

constexpr int kWideThreads = 256;
constexpr int kWideRows = 64;  // rows of one (head, group) per block

// Where the rows of one (head, group) live: row r of the problem -> element offsets of its d inputs and outputs.
struct StateRows {   // rows = (batch, token) of states [B,H,T,D]; outputs [B,H,T,D] contiguous
    int64_t sxb, sxt, in_base, out_base;
    int T, D;
    __device__ int64_t in(int64_t r) const { return in_base + (r / T) * sxb + (r % T) * sxt; }
    __device__ int64_t out(int64_t r) const { return out_base + ((r / T) * out_sxb + (r % T)) * D; }
    int64_t out_sxb;  // H*T: rows of the contiguous output between two batch entries
};
struct TableRows {   // rows = (stage, word) of tables [H,S,G,K,d]; outputs in the same layout
    int64_t base, stage_stride;
    int K, d;
    __device__ int64_t in(int64_t r) const { return base + (r / K) * stage_stride + (r % K) * d; }
    __device__ int64_t out(int64_t r) const { return in(r); }
};

template <int DSUB>
struct WideLayout {
    static constexpr int kWStride = DSUB + 4;  // floats; rows of the transposed matrix stay 16-byte aligned, banks staggered
    static constexpr int kOutPerRow = DSUB / 4;                       // threads that share a row
    static constexpr int kRowGroups = kWideThreads / kOutPerRow;      // rows handled side by side
    static constexpr int kRowsPerThread = kWideRows / kRowGroups;
    static constexpr size_t kBytes = ((size_t)DSUB * kWStride + (size_t)kWideRows * DSUB) * sizeof(float);
    static_assert(kWideRows % kRowGroups == 0 && kRowsPerThread >= 1, "row tile must divide among the threads");
};

template <int DSUB, typename XT, typename Rows>
__global__ void __launch_bounds__(kWideThreads)
whiten_wide_kernel(const XT *__restrict__ x, const float *__restrict__ whitener, float *__restrict__ out, Rows map_proto,
                   int64_t rows, int G, int64_t in_group_stride, int64_t out_group_stride, int64_t in_head_stride,
                   int64_t out_head_stride) {
    using L = WideLayout<DSUB>;
    extern __shared__ __align__(16) float wsm[];
    float *wt = wsm;                                  // [j][i] : W transposed
    float *xs = wsm + (size_t)DSUB * L::kWStride;     // [row][j]
    const int hg = blockIdx.y, h = hg / G, g = hg % G;
    const int tid = threadIdx.x;
    Rows map = map_proto;
    const int64_t in_off = (int64_t)h * in_head_stride + (int64_t)g * in_group_stride;
    const int64_t out_off = (int64_t)h * out_head_stride + (int64_t)g * out_group_stride;
    const float *w = whitener + (int64_t)hg * DSUB * DSUB;
    for (int e = tid; e < DSUB * DSUB; e += kWideThreads) {  // coalesced read of W[i][j], transposed store
        const int i = e / DSUB, j = e % DSUB;
        wt[j * L::kWStride + i] = w[e];
    }
    const int64_t row0 = (int64_t)blockIdx.x * kWideRows;
    for (int e = tid; e < kWideRows * DSUB; e += kWideThreads) {
        const int r = e / DSUB, j = e % DSUB;
        const int64_t row = row0 + r;
        xs[e] = row < rows ? to_float<XT>(x[in_off + map.in(row) + j]) : 0.0f;
    }
    __syncthreads();
    const int i0 = (tid % L::kOutPerRow) * 4, rg = tid / L::kOutPerRow;
    float acc[L::kRowsPerThread][4];
#pragma unroll
    for (int r = 0; r < L::kRowsPerThread; ++r)
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) acc[r][ii] = 0.0f;
#pragma unroll 2
    for (int j4 = 0; j4 < DSUB; j4 += 4) {
        float4 wv[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) wv[jj] = *reinterpret_cast<const float4 *>(wt + (j4 + jj) * L::kWStride + i0);
#pragma unroll
        for (int r = 0; r < L::kRowsPerThread; ++r) {
            const float4 xv = *reinterpret_cast<const float4 *>(xs + (rg + r * L::kRowGroups) * DSUB + j4);
            const float xj[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {  // j ascending for every output: the chain order of the scalar form
                acc[r][0] = __fmaf_rn(wv[jj].x, xj[jj], acc[r][0]);
                acc[r][1] = __fmaf_rn(wv[jj].y, xj[jj], acc[r][1]);
                acc[r][2] = __fmaf_rn(wv[jj].z, xj[jj], acc[r][2]);
                acc[r][3] = __fmaf_rn(wv[jj].w, xj[jj], acc[r][3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < L::kRowsPerThread; ++r) {
        const int64_t row = row0 + rg + r * L::kRowGroups;
        if (row < rows)
            *reinterpret_cast<float4 *>(out + out_off + map.out(row) + i0) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
}

template <int DSUB, typename XT, typename Rows>
static int launch_wide(const XT *x, const float *whitener, float *out, const Rows &map, int64_t rows, int H, int G,
                       int64_t in_group_stride, int64_t out_group_stride, int64_t in_head_stride, int64_t out_head_stride,
                       cudaStream_t stream) {
    using L = WideLayout<DSUB>;
    auto kernel = whiten_wide_kernel<DSUB, XT, Rows>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kBytes);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)((rows + kWideRows - 1) / kWideRows), (unsigned)(H * G));
    kernel<<<grid, kWideThreads, L::kBytes, stream>>>(x, whitener, out, map, rows, G, in_group_stride, out_group_stride,
                                                      in_head_stride, out_head_stride);
    return launch_status();
}

template <int DSUB>
static int whiten_wide(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt, const __half *tables,
                       const float *whitener, float *search_tables, float *search_rows, int B, int H, int T, int D, int G,
                       int S, int K, cudaStream_t stream) {
    TableRows tr{0, (int64_t)G * K * DSUB, K, DSUB};
    int st = launch_wide<DSUB, __half, TableRows>(tables, whitener, search_tables, tr, (int64_t)S * K, H, G, (int64_t)K * DSUB,
                                                  (int64_t)K * DSUB, (int64_t)S * G * K * DSUB, (int64_t)S * G * K * DSUB, stream);
    if (st != TACVQ_OK) return st;
    StateRows sr{sxb, sxt, 0, 0, T, D, (int64_t)H * T};
    if (x_dtype == TACVQ_F16)
        return launch_wide<DSUB, __half, StateRows>((const __half *)x, whitener, search_rows, sr, (int64_t)B * T, H, G, DSUB, DSUB,
                                                    sxh, (int64_t)T * D, stream);
    return launch_wide<DSUB, float, StateRows>((const float *)x, whitener, search_rows, sr, (int64_t)B * T, H, G, DSUB, DSUB, sxh,
                                               (int64_t)T * D, stream);
}

int whiten_dispatch(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt, const __half *tables,
                    const float *whitener, float *search_tables, float *search_rows, int B, int H, int T, int D, int G,
                    int S, int K, cudaStream_t stream) {
    const int d = D / G;
    // the tiled kernels read rows and matrices in 16-byte pieces
    const bool aligned = (((uintptr_t)search_rows | (uintptr_t)search_tables) & 15) == 0;
    if (aligned && d == 128) return whiten_wide<128>(x, x_dtype, sxb, sxh, sxt, tables, whitener, search_tables, search_rows, B, H, T, D, G, S, K, stream);
    if (aligned && d == 64) return whiten_wide<64>(x, x_dtype, sxb, sxh, sxt, tables, whitener, search_tables, search_rows, B, H, T, D, G, S, K, stream);
    if (aligned && d == 32) return whiten_wide<32>(x, x_dtype, sxb, sxh, sxt, tables, whitener, search_tables, search_rows, B, H, T, D, G, S, K, stream);
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
