// Encode kernels: greedy residual nearest-codeword search with all stages fused.
//
// Two kernels cover the geometry family (G groups, S stages, d = D/G, K <= 256 codewords):
//   encode_small  d <= 16   one thread owns TPT rows of one (head, group); the stage tables of that
//                           (head, group) live in shared memory as fp32 and are read as warp
//                           broadcasts; residual, running minimum and reconstruction stay in registers.
//   encode_large  d >= 32   a register-tiled fp32 GEMM per stage (4 rows x 16 codewords per thread),
//                           residual tile and stage table in shared memory, the contraction index
//                           outermost so every dot product is still one FMA chain from element 0.
// Both are FFMA-bound by design: an exact fp32 distance is what decides a code.
//
// Reference statements: src/jointkv/closed_loop_vq.py:52-76 (search), :343-395 (stage recursion),
// src/jointkv/cq_tac.py:86-105 (grouped one-stage form).

#include "common.cuh"
#include "encode_rows.cuh"

#ifndef TACVQ_ENCODE_TC
#define TACVQ_ENCODE_TC 1  // 8-wide groups go to the tensor-core filtered kernel (encode_tc.cu)
#endif

namespace tacvq {

int encode_tc8_launch(const EncodeArgs &a);
int encode_tc_large_launch(const EncodeArgs &a);

// ------------------------------------------------------------------------------------------------
// d <= 16
// ------------------------------------------------------------------------------------------------

template <int DSUB, int TPT, typename XT, typename TT>
__global__ void __launch_bounds__(128)
encode_small_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const TT *__restrict__ tables,
                    const float *__restrict__ sqnorm_in, uint8_t *__restrict__ codes, void *__restrict__ recon,
                    int recon_dtype, const __half *__restrict__ recon_tables, int B, int H, int T, int G, int S, int K,
                    int64_t t0, int64_t T_cap) {
    extern __shared__ __align__(16) float smem[];
    float *tab = smem;                       // [S][K][DSUB]
    float *nrm = smem + (size_t)S * K * DSUB;  // [S][K]

    const int hg = blockIdx.y;
    const int h = hg / G, g = hg % G;
    const int tid = threadIdx.x;

    for (int idx = tid; idx < S * K * DSUB; idx += blockDim.x) {
        const int i = idx % DSUB;
        const int k = (idx / DSUB) % K;
        const int s = idx / (DSUB * K);
        tab[idx] = to_float<TT>(tables[((((int64_t)h * S + s) * G + g) * K + k) * DSUB + i]);
    }
    __syncthreads();
    for (int idx = tid; idx < S * K; idx += blockDim.x) {
        if (sqnorm_in != nullptr) {
            const int k = idx % K, s = idx / K;
            nrm[idx] = sqnorm_in[(((int64_t)h * S + s) * G + g) * K + k];
        } else {
            const float *row = tab + (size_t)idx * DSUB;
            nrm[idx] = sqnorm_ordered<DSUB>([&](int i) { return row[i]; });
        }
    }
    __syncthreads();

    const int64_t rows = (int64_t)B * T;
    // a block keeps its tables and walks over row tiles, so the table load is paid once per block
    for (int64_t tile = (int64_t)blockIdx.x * (128 * TPT); tile < rows; tile += (int64_t)gridDim.x * (128 * TPT)) {

    float res[TPT][DSUB];
    float dec[TPT][DSUB];
    int64_t row_of[TPT];
#pragma unroll
    for (int j = 0; j < TPT; ++j) {
        const int64_t row = tile + j * 128 + tid;
        row_of[j] = row;
        if (row < rows) {
            const int64_t b = row / T, t = row % T;
            const XT *src = x + b * sxb + (int64_t)h * sxh + t * sxt + (int64_t)g * DSUB;
#pragma unroll
            for (int i = 0; i < DSUB; ++i) res[j][i] = to_float<XT>(src[i]);
        } else {
#pragma unroll
            for (int i = 0; i < DSUB; ++i) res[j][i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < DSUB; ++i) dec[j][i] = 0.0f;
    }

    for (int s = 0; s < S; ++s) {
        const float *stab = tab + (size_t)s * K * DSUB;
        const float *snrm = nrm + (size_t)s * K;
        float xx[TPT], best[TPT];
        int arg[TPT];
#pragma unroll
        for (int j = 0; j < TPT; ++j) {
            xx[j] = sqnorm_ordered<DSUB>([&](int i) { return res[j][i]; });
            best[j] = __int_as_float(0x7f800000);
            arg[j] = 0;
        }
#pragma unroll 4
        for (int k = 0; k < K; ++k) {
            float c[DSUB];
#pragma unroll
            for (int i = 0; i < DSUB; ++i) c[i] = stab[k * DSUB + i];
            const float cc = snrm[k];
#pragma unroll
            for (int j = 0; j < TPT; ++j) {
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < DSUB; ++i) dot = __fmaf_rn(res[j][i], c[i], dot);
                const float dist = distance_expr(xx[j], cc, dot);
                if (dist < best[j]) {
                    best[j] = dist;
                    arg[j] = k;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < TPT; ++j) {
            const float *sel = stab + arg[j] * DSUB;
#pragma unroll
            for (int i = 0; i < DSUB; ++i) res[j][i] = __fsub_rn(res[j][i], sel[i]);
            if (recon != nullptr) {
                if (recon_tables == nullptr) {
#pragma unroll
                    for (int i = 0; i < DSUB; ++i) dec[j][i] = __fadd_rn(dec[j][i], sel[i]);
                } else {
                    const __half *plain = recon_tables + ((((int64_t)h * S + s) * G + g) * K + arg[j]) * DSUB;
#pragma unroll
                    for (int i = 0; i < DSUB; ++i) dec[j][i] = __fadd_rn(dec[j][i], __half2float(plain[i]));
                }
            }
            if (row_of[j] < rows) {
                const int64_t b = row_of[j] / T, t = row_of[j] % T;
                codes[((((int64_t)b * H + h) * T_cap + t0 + t) * S + s) * G + g] = (uint8_t)arg[j];
            }
        }
    }

    if (recon != nullptr) {
#pragma unroll
        for (int j = 0; j < TPT; ++j) {
            if (row_of[j] >= rows) continue;
            const int64_t b = row_of[j] / T, t = row_of[j] % T;
            const int64_t o = (((int64_t)b * H + h) * T + t) * ((int64_t)G * DSUB) + (int64_t)g * DSUB;
            if (recon_dtype == TACVQ_F16) {
#pragma unroll
                for (int i = 0; i < DSUB; ++i) store_as<__half>((__half *)recon + o + i, dec[j][i]);
            } else {
#pragma unroll
                for (int i = 0; i < DSUB; ++i) store_as<float>((float *)recon + o + i, dec[j][i]);
            }
        }
    }
    }  // row tiles
}

// ------------------------------------------------------------------------------------------------
// d <= 16, a handful of rows (decode steps): one warp per (row, head, group), lanes share the codewords
// ------------------------------------------------------------------------------------------------
// With only B*T rows (one new token per sequence) the kernel above would leave every thread alone
// with a 256-word scan.  Here lane l scores words l, l+32, ... (ascending, strict '<' keeps the
// lowest index per lane) and the warp takes the lexicographic minimum of (distance, index), which is
// the same first-minimum as a sequential scan.  Arithmetic per distance is identical to the kernels
// above, so the codes are too.

template <int DSUB, typename XT>
__device__ __forceinline__ void encode_row_unit(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt,
                                                const __half *__restrict__ tables, const float *__restrict__ sqnorm_in,
                                                uint8_t *__restrict__ codes, void *__restrict__ recon, int recon_dtype, int H,
                                                int T, int G, int S, int K, int64_t t0, int64_t T_cap, int64_t unit, int lane) {
    const int g = (int)(unit % G);
    const int h = (int)((unit / G) % H);
    const int64_t row = unit / ((int64_t)G * H);
    const int64_t b = row / T, t = row % T;
    const XT *src = x + b * sxb + (int64_t)h * sxh + t * sxt + (int64_t)g * DSUB;
    float res[DSUB], dec[DSUB];
#pragma unroll
    for (int i = 0; i < DSUB; ++i) {
        res[i] = to_float<XT>(src[i]);
        dec[i] = 0.0f;
    }
    for (int s = 0; s < S; ++s) {
        const int64_t base = (((int64_t)h * S + s) * G + g) * K;
        const int arg = nearest_word_in_warp<DSUB>(res, tables + base * DSUB, sqnorm_in ? sqnorm_in + base : nullptr, K, lane);
#pragma unroll
        for (int i = 0; i < DSUB; ++i) {
            const float w = __half2float(tables[(base + arg) * DSUB + i]);
            res[i] = __fsub_rn(res[i], w);
            dec[i] = __fadd_rn(dec[i], w);
        }
        if (lane == 0) codes[((((int64_t)b * H + h) * T_cap + t0 + t) * S + s) * G + g] = (uint8_t)arg;
    }
    if (recon != nullptr && lane == 0) {
        const int64_t o = ((b * H + h) * T + t) * ((int64_t)G * DSUB) + (int64_t)g * DSUB;
#pragma unroll
        for (int i = 0; i < DSUB; ++i) {
            if (recon_dtype == TACVQ_F16) store_as<__half>((__half *)recon + o + i, dec[i]);
            else store_as<float>((float *)recon + o + i, dec[i]);
        }
    }
}

template <int DSUB, typename XT>
__global__ void __launch_bounds__(256)
encode_rows_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const __half *__restrict__ tables,
                   const float *__restrict__ sqnorm_in, uint8_t *__restrict__ codes, void *__restrict__ recon,
                   int recon_dtype, int B, int H, int T, int G, int S, int K, int64_t t0, int64_t T_cap) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= (int64_t)B * T * H * G) return;
    encode_row_unit<DSUB, XT>(x, sxb, sxh, sxt, tables, sqnorm_in, codes, recon, recon_dtype, H, T, G, S, K, t0, T_cap, unit, lane);
}

// One decode step's bookkeeping in a single launch: the new rows of K and of V are encoded in place (a
// warp per (row, head, group) and side, as above) and every row's visible range is set.  The kernel lets
// its successor start at once (programmatic dependent launch): a successor that needs these outputs
// waits for this grid by itself.
template <int DSUB, typename XT>
__global__ void __launch_bounds__(256)
decode_prologue_kernel(const XT *__restrict__ k_rows, const XT *__restrict__ v_rows, int64_t sxb, int64_t sxh, int64_t sxt,
                       const __half *__restrict__ ktab, const __half *__restrict__ vtab, uint8_t *__restrict__ kcodes,
                       uint8_t *__restrict__ vcodes, int32_t *__restrict__ seq_start, int32_t *__restrict__ seq_end, int start,
                       int end, int B, int H, int T, int G, int S, int K, int64_t t0, int64_t T_cap) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (blockIdx.x == 0) {
        for (int b = threadIdx.x; b < B; b += blockDim.x) {
            seq_start[b] = start;
            seq_end[b] = end;
        }
    }
    const int lane = threadIdx.x & 31;
    const int64_t units = (int64_t)B * T * H * G;
    int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const bool value_side = unit >= units;
    if (value_side) unit -= units;
    if (unit >= units) return;
    encode_row_unit<DSUB, XT>(value_side ? v_rows : k_rows, sxb, sxh, sxt, value_side ? vtab : ktab, nullptr,
                              value_side ? vcodes : kcodes, nullptr, TACVQ_F16, H, T, G, S, K, t0, T_cap, unit, lane);
}

template <int DSUB, typename XT>
static int launch_prologue(const void *k_rows, const void *v_rows, int64_t sxb, int64_t sxh, int64_t sxt, const __half *ktab,
                           const __half *vtab, uint8_t *kcodes, uint8_t *vcodes, int32_t *seq_start, int32_t *seq_end,
                           int start, int end, int B, int H, int T, int G, int S, int K, int64_t t0, int64_t T_cap,
                           cudaStream_t stream) {
    const int64_t units = (int64_t)B * T * H * G;
    decode_prologue_kernel<DSUB, XT><<<(unsigned)((2 * units + 7) / 8), 256, 0, stream>>>(
        (const XT *)k_rows, (const XT *)v_rows, sxb, sxh, sxt, ktab, vtab, kcodes, vcodes, seq_start, seq_end, start, end, B, H,
        T, G, S, K, t0, T_cap);
    return launch_status();
}

template <int DSUB, typename XT>
static int launch_rows(const EncodeArgs &a) {
    const int64_t units = (int64_t)a.B * a.T * a.H * a.G;
    encode_rows_kernel<DSUB, XT><<<(unsigned)((units + 7) / 8), 256, 0, a.stream>>>(
        (const XT *)a.x, a.sxb, a.sxh, a.sxt, (const __half *)a.tables, a.sqnorm, a.codes, a.recon, a.recon_dtype, a.B, a.H,
        a.T, a.G, a.S, a.K, a.t0, a.T_cap);
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// d >= 32
// ------------------------------------------------------------------------------------------------

constexpr int kLargeRows = 128;   // rows (tokens) per block
constexpr int kLargeThreads = 512;

template <int DSUB>
struct LargeLayout {
    static constexpr int kStride = DSUB + 4;  // floats; keeps 16-byte rows and spreads rows over banks
    static constexpr size_t kResFloats = (size_t)kLargeRows * kStride;
    static constexpr size_t kTabFloats = (size_t)kMaxWords * kStride;
    static constexpr size_t bytes(int S) {
        return (kResFloats + kTabFloats + kMaxWords + kLargeRows) * sizeof(float) + (size_t)kLargeRows * sizeof(int) +
               (size_t)kLargeRows * S;
    }
};

template <int DSUB, typename XT, typename TT>
__global__ void __launch_bounds__(kLargeThreads)
encode_large_kernel(const XT *__restrict__ x, int64_t sxb, int64_t sxh, int64_t sxt, const TT *__restrict__ tables,
                    const float *__restrict__ sqnorm_in, uint8_t *__restrict__ codes, void *__restrict__ recon,
                    int recon_dtype, const __half *__restrict__ recon_tables, int B, int H, int T, int G, int S, int K,
                    int64_t t0, int64_t T_cap) {
    using L = LargeLayout<DSUB>;
    constexpr int STR = L::kStride;
    extern __shared__ __align__(16) float smem[];
    float *res = smem;                      // [rows][STR]
    float *tab = res + L::kResFloats;       // [256][STR]
    float *nrm = tab + L::kTabFloats;       // [256]
    float *xxs = nrm + kMaxWords;           // [rows]
    int *pick = (int *)(xxs + kLargeRows);  // [rows]
    uint8_t *hist = (uint8_t *)(pick + kLargeRows);  // [rows][S] codes chosen so far

    const int hg = blockIdx.y;
    const int h = hg / G, g = hg % G;
    const int tid = threadIdx.x;
    const int tx = tid & 15;   // codeword lane: owns words tx, tx+16, ...
    const int ty = tid >> 4;   // row lane: owns rows 4*ty .. 4*ty+3
    const int64_t rows = (int64_t)B * T;
    const int64_t tile = (int64_t)blockIdx.x * kLargeRows;

    for (int idx = tid; idx < kLargeRows * DSUB; idx += kLargeThreads) {
        const int r = idx / DSUB, i = idx % DSUB;
        const int64_t row = tile + r;
        float v = 0.0f;
        if (row < rows) {
            const int64_t b = row / T, t = row % T;
            v = to_float<XT>(x[b * sxb + (int64_t)h * sxh + t * sxt + (int64_t)g * DSUB + i]);
        }
        res[r * STR + i] = v;
    }

    for (int s = 0; s < S; ++s) {
        __syncthreads();  // residual tile settled; previous stage's table no longer read
        const TT *src = tables + (((int64_t)h * S + s) * G + g) * (int64_t)K * DSUB;
        for (int idx = tid; idx < kMaxWords * DSUB; idx += kLargeThreads) {
            const int k = idx / DSUB, i = idx % DSUB;
            tab[k * STR + i] = (k < K) ? to_float<TT>(src[(int64_t)k * DSUB + i]) : 0.0f;
        }
        __syncthreads();
        if (tid < kMaxWords) {
            const float *row = tab + tid * STR;
            float v;
            if (tid >= K) v = __int_as_float(0x7f800000);  // padding words can never win
            else if (sqnorm_in != nullptr) v = sqnorm_in[(((int64_t)h * S + s) * G + g) * K + tid];
            else v = sqnorm_ordered_rt(row, DSUB);
            nrm[tid] = v;
        }
        if (tid < kLargeRows) xxs[tid] = sqnorm_ordered_rt(res + tid * STR, DSUB);
        __syncthreads();

        float acc[4][16];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int w = 0; w < 16; ++w) acc[a][w] = 0.0f;

#pragma unroll 1
        for (int i = 0; i < DSUB; i += 4) {
            float4 xv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) xv[a] = *reinterpret_cast<const float4 *>(res + (ty * 4 + a) * STR + i);
#pragma unroll
            for (int w = 0; w < 16; ++w) {
                const float4 cv = *reinterpret_cast<const float4 *>(tab + (tx + 16 * w) * STR + i);
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    float v = acc[a][w];
                    v = __fmaf_rn(xv[a].x, cv.x, v);
                    v = __fmaf_rn(xv[a].y, cv.y, v);
                    v = __fmaf_rn(xv[a].z, cv.z, v);
                    v = __fmaf_rn(xv[a].w, cv.w, v);
                    acc[a][w] = v;
                }
            }
        }

#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const float xx = xxs[ty * 4 + a];
            float best = __int_as_float(0x7f800000);
            int arg = tx;
#pragma unroll
            for (int w = 0; w < 16; ++w) {
                const int k = tx + 16 * w;
                const float dist = distance_expr(xx, nrm[k], acc[a][w]);
                if (dist < best) {
                    best = dist;
                    arg = k;
                }
            }
            // lowest (distance, index) among the 16 codeword lanes of this row (a half warp)
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, off);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
                if (ob < best || (ob == best && oa < arg)) {
                    best = ob;
                    arg = oa;
                }
            }
            if (tx == 0) pick[ty * 4 + a] = arg < K ? arg : 0;
        }
        __syncthreads();

        for (int idx = tid; idx < kLargeRows * DSUB; idx += kLargeThreads) {
            const int r = idx / DSUB, i = idx % DSUB;
            res[r * STR + i] = __fsub_rn(res[r * STR + i], tab[pick[r] * STR + i]);
        }
        if (tid < kLargeRows) {
            const int64_t row = tile + tid;
            hist[tid * S + s] = (uint8_t)pick[tid];
            if (row < rows) {
                const int64_t b = row / T, t = row % T;
                codes[((((int64_t)b * H + h) * T_cap + t0 + t) * S + s) * G + g] = (uint8_t)pick[tid];
            }
        }
    }

    if (recon != nullptr) {
        __syncthreads();
        const __half *plain = recon_tables;
        for (int idx = tid; idx < kLargeRows * DSUB; idx += kLargeThreads) {
            const int r = idx / DSUB, i = idx % DSUB;
            const int64_t row = tile + r;
            if (row >= rows) continue;
            float sum = 0.0f;
            for (int s = 0; s < S; ++s) {
                const int code = hist[r * S + s];
                sum = __fadd_rn(sum, __half2float(plain[((((int64_t)h * S + s) * G + g) * K + code) * DSUB + i]));
            }
            const int64_t b = row / T, t = row % T;
            const int64_t o = (((int64_t)b * H + h) * T + t) * ((int64_t)G * DSUB) + (int64_t)g * DSUB + i;
            if (recon_dtype == TACVQ_F16) store_as<__half>((__half *)recon + o, sum);
            else store_as<float>((float *)recon + o, sum);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host-side dispatch
// ------------------------------------------------------------------------------------------------

template <int DSUB, int TPT, typename XT, typename TT>
static int launch_small(const EncodeArgs &a) {
    const size_t smem = ((size_t)a.S * a.K * DSUB + (size_t)a.S * a.K) * sizeof(float);
    auto kernel = encode_small_kernel<DSUB, TPT, XT, TT>;
    if (smem > 48 * 1024) {
        if (smem > 227 * 1024) return TACVQ_ERR_UNSUPPORTED;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int64_t rows = (int64_t)a.B * a.T;
    // about 8 resident blocks per SM in total; each block walks over the row tiles of its (head, group)
    int64_t tiles = (rows + 128 * TPT - 1) / (128 * TPT);
    const int64_t want = (148 * 8 + a.H * a.G - 1) / (a.H * a.G);
    if (tiles > want) tiles = want;
    dim3 grid((unsigned)tiles, (unsigned)(a.H * a.G));
    // The search tables are the plain tables unless a whitened search is running.
    const __half *plain = a.tables_f32 ? a.recon_tables : nullptr;
    kernel<<<grid, 128, smem, a.stream>>>((const XT *)a.x, a.sxb, a.sxh, a.sxt, (const TT *)a.tables, a.sqnorm, a.codes,
                                          a.recon, a.recon_dtype, plain, a.B, a.H, a.T, a.G, a.S, a.K, a.t0, a.T_cap);
    return launch_status();
}

template <int DSUB, typename XT, typename TT>
static int launch_large(const EncodeArgs &a) {
    const size_t smem = LargeLayout<DSUB>::bytes(a.S);
    auto kernel = encode_large_kernel<DSUB, XT, TT>;
    if (smem > 227 * 1024) return TACVQ_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int64_t rows = (int64_t)a.B * a.T;
    dim3 grid((unsigned)((rows + kLargeRows - 1) / kLargeRows), (unsigned)(a.H * a.G));
    kernel<<<grid, kLargeThreads, smem, a.stream>>>((const XT *)a.x, a.sxb, a.sxh, a.sxt, (const TT *)a.tables, a.sqnorm,
                                                    a.codes, a.recon, a.recon_dtype, a.recon_tables, a.B, a.H, a.T, a.G,
                                                    a.S, a.K, a.t0, a.T_cap);
    return launch_status();
}

constexpr int kFewRows = 32;  // at or below this many rows a warp per (row, head, group) wins

template <typename XT, typename TT>
static int dispatch_d(const EncodeArgs &a) {
    if constexpr (sizeof(TT) == 2) {
        if ((int64_t)a.B * a.T <= kFewRows) {
            switch (a.D / a.G) {
                case 4: return launch_rows<4, XT>(a);
                case 8: return launch_rows<8, XT>(a);
                case 16: return launch_rows<16, XT>(a);
                default: break;
            }
        }
        if (TACVQ_ENCODE_TC && (a.D / a.G == 8 || a.D / a.G == 4)) {
            const int st = encode_tc8_launch(a);
            if (st != TACVQ_ERR_UNSUPPORTED) return st;
        }
        if (TACVQ_ENCODE_TC && a.D / a.G >= 32) {
            const int st = encode_tc_large_launch(a);
            if (st != TACVQ_ERR_UNSUPPORTED) return st;
        }
    }
    switch (a.D / a.G) {
        case 1: return launch_small<1, 4, XT, TT>(a);
        case 2: return launch_small<2, 4, XT, TT>(a);
        case 3: return launch_small<3, 4, XT, TT>(a);
        case 4: return launch_small<4, 4, XT, TT>(a);
        case 5: return launch_small<5, 4, XT, TT>(a);
        case 6: return launch_small<6, 4, XT, TT>(a);
        case 7: return launch_small<7, 4, XT, TT>(a);
        case 8: return launch_small<8, 4, XT, TT>(a);
        case 16: return launch_small<16, 2, XT, TT>(a);
        case 32: return launch_large<32, XT, TT>(a);
        case 64: return launch_large<64, XT, TT>(a);
        case 128: return launch_large<128, XT, TT>(a);
        default: return TACVQ_ERR_UNSUPPORTED;
    }
}

// Returns TACVQ_ERR_UNSUPPORTED when the step is not a handful of rows of narrow groups; the caller then
// makes the three separate launches.
int decode_prologue_dispatch(const void *k_rows, const void *v_rows, int rows_dtype, int64_t sxb, int64_t sxh, int64_t sxt,
                             const __half *ktab, const __half *vtab, uint8_t *kcodes, uint8_t *vcodes, int32_t *seq_start,
                             int32_t *seq_end, int start, int end, int B, int H, int T, int D, int G, int S, int K, int64_t t0,
                             int64_t T_cap, cudaStream_t stream) {
    if ((int64_t)B * T > kFewRows) return TACVQ_ERR_UNSUPPORTED;
#define TACVQ_CASE(N)                                                                                                          \
    case N:                                                                                                                    \
        return rows_dtype == TACVQ_F16                                                                                         \
                   ? launch_prologue<N, __half>(k_rows, v_rows, sxb, sxh, sxt, ktab, vtab, kcodes, vcodes, seq_start, seq_end, \
                                                start, end, B, H, T, G, S, K, t0, T_cap, stream)                               \
                   : launch_prologue<N, float>(k_rows, v_rows, sxb, sxh, sxt, ktab, vtab, kcodes, vcodes, seq_start, seq_end,  \
                                               start, end, B, H, T, G, S, K, t0, T_cap, stream);
    switch (D / G) {
        TACVQ_CASE(4)
        TACVQ_CASE(8)
        TACVQ_CASE(16)
        default: return TACVQ_ERR_UNSUPPORTED;
    }
#undef TACVQ_CASE
}

int encode_dispatch(const EncodeArgs &a) {
    if (a.x_dtype == TACVQ_F16) {
        return a.tables_f32 ? dispatch_d<__half, float>(a) : dispatch_d<__half, __half>(a);
    }
    return a.tables_f32 ? dispatch_d<float, float>(a) : dispatch_d<float, __half>(a);
}

}  // namespace tacvq
