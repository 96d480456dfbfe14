// C ABI of libtacvq.so: argument validation on the host, then dispatch to the kernels.
// Declarations and the per-function contract live in include/tacvq.h.

#include <atomic>

#include "common.cuh"

namespace tacvq {

int encode_dispatch(const EncodeArgs &a);
int decode_dispatch(const uint8_t *codes, const __half *tables, void *out, int out_dtype, int B, int H, int T, int D,
                    int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream);
int codeword_grad_dispatch(const uint8_t *codes, const float *grad_out, float *grad_tables, int B, int H, int T, int D,
                           int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, cudaStream_t stream);
int table_sqnorm_dispatch(const __half *tables, float *out, int64_t words, int d, cudaStream_t stream);
int tensor_memory_timeouts(unsigned int *out);
int whiten_dispatch(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt, const __half *tables,
                    const float *whitener, float *search_tables, float *search_rows, int B, int H, int T, int D, int G,
                    int S, int K, cudaStream_t stream);
int attn_generic_splits(int B, int Hkv, int64_t T_cap, int sms);
int attn_generic_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                          const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part, int B,
                          int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits, cudaStream_t stream);
int attn_combine_dispatch(const float *states, int n_parts, __half *out, float *merged, int64_t rows, int D,
                          cudaStream_t stream);
bool attn_fullwidth_supported(int Hq, int Hkv, int D, int G, int S, int K);
int attn_fullwidth_splits(int B, int Hkv, int64_t T_cap, int sms);
int attn_fullwidth_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                            const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, float *part,
                            __half *out, float *state_out, int B, int Hq, int Hkv, int S, int64_t T_cap, int splits,
                            cudaStream_t stream);
bool attn_gsrq_supported(int Hq, int Hkv, int D, int G, int S, int K);
size_t attn_gsrq_workspace_bytes(int B, int Hq, int Hkv, int D, int sms);
int attn_gsrq_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                       const __half *vtab, const int32_t *seq_start, const int32_t *seq_end, void *workspace,
                       __half *out, float *state_out, int B, int Hq, int Hkv, int64_t T_cap, int sms,
                       cudaStream_t stream, const GsrqNewToken *fresh = nullptr);
int decode_prologue_dispatch(const void *k_rows, const void *v_rows, int rows_dtype, int64_t sxb, int64_t sxh, int64_t sxt,
                             const __half *ktab, const __half *vtab, uint8_t *kcodes, uint8_t *vcodes, int32_t *seq_start,
                             int32_t *seq_end, int start, int end, int B, int H, int T, int D, int G, int S, int K, int64_t t0,
                             int64_t T_cap, cudaStream_t stream);

int attn_rotary_splits(int B, int Hkv, int64_t T_cap, int sms);
bool attn_rotary_staged_supported(int Hq, int Hkv, int D, int G, int S, int K);
int attn_rotary_staged_splits(int B, int Hkv, int64_t T_cap, int sms);
int attn_rotary_staged_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                                const __half *vtab, const __half *rope, const int32_t *seq_start, const int32_t *seq_end,
                                float *part, int B, int Hq, int Hkv, int G, int S, int64_t T_cap, int splits,
                                cudaStream_t stream);
int rope_table_dispatch(__half *table, int64_t tokens, int D, double theta, int64_t first, cudaStream_t stream);
int attn_rotary_dispatch(const __half *q, const uint8_t *kcodes, const uint8_t *vcodes, const __half *ktab,
                         const __half *vtab, const __half *rope, const int32_t *seq_start, const int32_t *seq_end,
                         float *part, int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap, int splits,
                         cudaStream_t stream);

constexpr int kGenericMaxSplits = 64;

// Per-device caches below are atomics: first calls from several host threads may race, and every
// racer stores the same value.
static int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// the specialised scan keeps a work prefix over at most 512 batch rows in shared memory and reads its
// query rows and tables in 16-byte pieces; other calls are served by the generic kernel
static bool gsrq_batch_ok(int B, int Hkv) { return B <= 512 && (int64_t)B * Hkv <= 1024; }
static bool gsrq_aligned(const void *q, const void *ktab, const void *vtab) {
    return (((uintptr_t)q | (uintptr_t)ktab | (uintptr_t)vtab) & 15) == 0;
}

static bool dtype_ok(int t) { return t == TACVQ_F16 || t == TACVQ_F32; }

static bool sub_dim_ok(int d) { return (d >= 1 && d <= 8) || d == 16 || d == 32 || d == 64 || d == 128; }

static int check_code_geometry(int B, int H, int T, int D, int G, int S, int K, int64_t t0, int64_t T_cap) {
    if (B < 0 || T < 0 || H <= 0 || D <= 0 || G <= 0 || S <= 0 || K <= 0 || K > kMaxWords) return TACVQ_ERR_GEOMETRY;
    if (D % G != 0) return TACVQ_ERR_GEOMETRY;
    if (t0 < 0 || T_cap < 0 || t0 + T > T_cap) return TACVQ_ERR_RANGE;
    return TACVQ_OK;
}

__global__ void set_ranges_kernel(int32_t *seq_start, int32_t *seq_end, int B, int start, int end) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) {
        seq_start[i] = start;
        seq_end[i] = end;
    }
}

// Scratch for tacvq_attn_decode_static: lives in the library image, so every GPU that loads the
// library carries these 16 MiB until the process exits.  In host code the name of a __device__ array
// is only a handle; the address a kernel may use comes from cudaGetSymbolAddress, asked once per
// device while that device is current.
constexpr size_t kStaticScratchBytes = (size_t)16 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static int static_scratch_for_current_device(void **ptr) {
    // The address is valid for the life of the device's primary context; a cudaDeviceReset invalidates it
    // (and everything else this library has set up on that device).
    static std::atomic<void *> cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return TACVQ_ERR_DEVICE;
    void *p = cached[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        cached[dev].store(p, std::memory_order_release);
    }
    *ptr = p;
    return TACVQ_OK;
}

}  // namespace tacvq

using namespace tacvq;

extern "C" {

int tacvq_version(void) { return TACVQ_ABI_VERSION; }

const char *tacvq_status_string(int status) {
    switch (status) {
        case TACVQ_OK: return "ok";
        case TACVQ_ERR_NULL: return "a required pointer is NULL";
        case TACVQ_ERR_GEOMETRY: return "inconsistent geometry";
        case TACVQ_ERR_DTYPE: return "unknown dtype tag";
        case TACVQ_ERR_RANGE: return "token range outside the code buffer";
        case TACVQ_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
        case TACVQ_ERR_UNSUPPORTED: return "no kernel built for this geometry";
        case TACVQ_ERR_ALIGN: return "pointer or stride alignment";
        case TACVQ_ERR_DEVICE: return "device is not compute capability 10.x";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

int tacvq_table_sqnorm(const uint16_t *tables_f16, float *out, int64_t words, int d, tacvq_stream_t stream) {
    if (!tables_f16 || !out) return TACVQ_ERR_NULL;
    if (words < 0 || d <= 0 || d > 128) return TACVQ_ERR_GEOMETRY;
    return table_sqnorm_dispatch((const __half *)tables_f16, out, words, d, (cudaStream_t)stream);
}

int tacvq_encode_tensor_memory_timeouts(unsigned int *count) {
    if (!count) return TACVQ_ERR_NULL;
    return tensor_memory_timeouts(count);
}

int tacvq_encode(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt, const uint16_t *tables_f16,
                 const float *table_sqnorm, uint8_t *codes, void *recon, int recon_dtype, int B, int H, int T, int D,
                 int G, int S, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream) {
    if (!dtype_ok(x_dtype) || (recon && !dtype_ok(recon_dtype))) return TACVQ_ERR_DTYPE;
    const int g = check_code_geometry(B, H, T, D, G, S, K, t0, T_cap);
    if (g != TACVQ_OK) return g;
    if (!sub_dim_ok(D / G)) return TACVQ_ERR_UNSUPPORTED;
    if ((int64_t)B * T == 0) return TACVQ_OK;  // nothing to encode: pointers of empty tensors may be NULL
    if (!x || !tables_f16 || !codes) return TACVQ_ERR_NULL;
    if (sxb < 0 || sxh < 0 || sxt < D) return TACVQ_ERR_GEOMETRY;
    EncodeArgs a{x, x_dtype, sxb, sxh, sxt, tables_f16, false, table_sqnorm, codes, recon, recon_dtype,
                 (const __half *)tables_f16, B, H, T, D, G, S, K, t0, T_cap, (cudaStream_t)stream};
    return encode_dispatch(a);
}

int tacvq_encode_whitened(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt,
                          const uint16_t *tables_f16, const float *whitener, float *search_tables,
                          float *search_rows, uint8_t *codes, void *recon, int recon_dtype, int B, int H, int T, int D,
                          int G, int S, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream) {
    if (!dtype_ok(x_dtype) || (recon && !dtype_ok(recon_dtype))) return TACVQ_ERR_DTYPE;
    const int g = check_code_geometry(B, H, T, D, G, S, K, t0, T_cap);
    if (g != TACVQ_OK) return g;
    if (!sub_dim_ok(D / G)) return TACVQ_ERR_UNSUPPORTED;
    if ((int64_t)B * T == 0) return TACVQ_OK;
    if (!x || !tables_f16 || !codes || !whitener || !search_tables || !search_rows) return TACVQ_ERR_NULL;
    if (sxb < 0 || sxh < 0 || sxt < D) return TACVQ_ERR_GEOMETRY;
    int st = whiten_dispatch(x, x_dtype, sxb, sxh, sxt, (const __half *)tables_f16, whitener, search_tables,
                             search_rows, B, H, T, D, G, S, K, (cudaStream_t)stream);
    if (st != TACVQ_OK) return st;
    EncodeArgs a{search_rows, TACVQ_F32, (int64_t)H * T * D, (int64_t)T * D, (int64_t)D, search_tables, true, nullptr,
                 codes, recon, recon_dtype, (const __half *)tables_f16, B, H, T, D, G, S, K, t0, T_cap,
                 (cudaStream_t)stream};
    return encode_dispatch(a);
}

int tacvq_decode(const uint8_t *codes, const uint16_t *tables_f16, void *out, int out_dtype, int B, int H, int T,
                 int D, int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream) {
    if (!dtype_ok(out_dtype)) return TACVQ_ERR_DTYPE;
    const int g = check_code_geometry(B, H, T, D, G, S, K, t0, T_cap);
    if (g != TACVQ_OK) return g;
    if (S_use < 0 || S_use > S) return TACVQ_ERR_GEOMETRY;
    if ((int64_t)B * T == 0) return TACVQ_OK;
    if (!codes || !tables_f16 || !out) return TACVQ_ERR_NULL;
    return decode_dispatch(codes, (const __half *)tables_f16, out, out_dtype, B, H, T, D, G, S, S_use, K, t0, T_cap,
                           (cudaStream_t)stream);
}

int tacvq_codeword_grad(const uint8_t *codes, const float *grad_out, float *grad_tables, int B, int H, int T, int D,
                        int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream) {
    if (!codes || !grad_out || !grad_tables) return TACVQ_ERR_NULL;
    const int g = check_code_geometry(B, H, T, D, G, S, K, t0, T_cap);
    if (g != TACVQ_OK) return g;
    if (S_use < 0 || S_use > S) return TACVQ_ERR_GEOMETRY;
    return codeword_grad_dispatch(codes, grad_out, grad_tables, B, H, T, D, G, S, S_use, K, t0, T_cap,
                                  (cudaStream_t)stream);
}

static int check_attn_geometry(int B, int Hq, int Hkv, int D, int G, int S, int K) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || G <= 0 || S <= 0) return TACVQ_ERR_GEOMETRY;
    if (Hq % Hkv != 0 || D % G != 0) return TACVQ_ERR_GEOMETRY;
    const int rep = Hq / Hkv;
    if (K != 256 || D % 32 != 0 || D > 256) return TACVQ_ERR_UNSUPPORTED;
    if (rep != 1 && rep != 2 && rep != 4 && rep != 8) return TACVQ_ERR_UNSUPPORTED;
    if ((D / G) % (D / 32) != 0) return TACVQ_ERR_UNSUPPORTED;  // a lane's channels stay inside one group
    return TACVQ_OK;
}

size_t tacvq_attn_workspace_bytes(int B, int Hq, int Hkv, int D, int G, int S) {
    if (check_attn_geometry(B, Hq, Hkv, D, G, S, 256) != TACVQ_OK) return 0;
    size_t generic = (size_t)kGenericMaxSplits * B * Hq * (D + 2) * sizeof(float);
    size_t fast = (attn_gsrq_supported(Hq, Hkv, D, G, S, 256) && gsrq_batch_ok(B, Hkv)) ? attn_gsrq_workspace_bytes(B, Hq, Hkv, D, sm_count()) : 0;
    size_t need = generic > fast ? generic : fast;
    return (need + 255) & ~(size_t)255;
}

int tacvq_attn_decode(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes, const uint16_t *ktab_f16,
                      const uint16_t *vtab_f16, const int32_t *seq_start, const int32_t *seq_end, void *workspace,
                      size_t workspace_bytes, uint16_t *out_f16, float *state_out, int B, int Hq, int Hkv, int D,
                      int G, int S, int K, int64_t T_cap, tacvq_stream_t stream) {
    if (!q_f16 || !kcodes || !vcodes || !ktab_f16 || !vtab_f16) return TACVQ_ERR_NULL;
    if (!out_f16 && !state_out) return TACVQ_ERR_NULL;
    const int g = check_attn_geometry(B, Hq, Hkv, D, G, S, K);
    if (g != TACVQ_OK) return g;
    if (T_cap < 0 || T_cap > 0x7fffffff) return TACVQ_ERR_RANGE;
    if (!workspace || ((uintptr_t)workspace & 255) != 0 || workspace_bytes < tacvq_attn_workspace_bytes(B, Hq, Hkv, D, G, S))
        return TACVQ_ERR_WORKSPACE;
    if ((((uintptr_t)kcodes | (uintptr_t)vcodes) & 15) != 0) return TACVQ_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    if (attn_gsrq_supported(Hq, Hkv, D, G, S, K) && gsrq_batch_ok(B, Hkv) && gsrq_aligned(q_f16, ktab_f16, vtab_f16)) {
        const int fast = attn_gsrq_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                            (const __half *)vtab_f16, seq_start, seq_end, workspace, (__half *)out_f16,
                                            state_out, B, Hq, Hkv, T_cap, sm_count(), s);
        if (fast != TACVQ_ERR_UNSUPPORTED) return fast;  // sizes beyond the specialised scan: the generic kernel below
    }
    int splits = attn_generic_splits(B, Hkv, T_cap, sm_count());
    if (attn_fullwidth_supported(Hq, Hkv, D, G, S, K) && (((uintptr_t)ktab_f16 | (uintptr_t)vtab_f16) & 15) == 0) {
        splits = attn_fullwidth_splits(B, Hkv, T_cap, sm_count());
        if (splits <= kGenericMaxSplits) {
            // a single block per pair writes the result itself; several blocks leave partial states to merge
            int fw = attn_fullwidth_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                             (const __half *)vtab_f16, seq_start, seq_end, (float *)workspace,
                                             (__half *)out_f16, state_out, B, Hq, Hkv, S, T_cap, splits, s);
            if (fw != TACVQ_OK || splits == 1) return fw;
            return attn_combine_dispatch((const float *)workspace, splits, (__half *)out_f16, state_out, (int64_t)B * Hq, D, s);
        }
        splits = attn_generic_splits(B, Hkv, T_cap, sm_count());
    }
    if (attn_rotary_staged_supported(Hq, Hkv, D, G, S, K) && (((uintptr_t)ktab_f16 | (uintptr_t)vtab_f16) & 15) == 0) {
        // head_dim 128 in pieces of 8 channels, at most two stages (e.g. one-stage grouped CQ): score table and
        // value tables in shared memory, two passes (the staged kernel of attn_rotary.cu without its rotary step)
        const int staged = attn_rotary_staged_splits(B, Hkv, T_cap, sm_count());
        if (staged > 0) {
            int st = attn_rotary_staged_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                                 (const __half *)vtab_f16, nullptr, seq_start, seq_end, (float *)workspace,
                                                 B, Hq, Hkv, G, S, T_cap, staged, s);
            if (st != TACVQ_OK) return st;
            return attn_combine_dispatch((const float *)workspace, staged, (__half *)out_f16, state_out, (int64_t)B * Hq, D, s);
        }
    }
    int st = attn_generic_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                   (const __half *)vtab_f16, seq_start, seq_end, (float *)workspace, B, Hq, Hkv, D, G,
                                   S, K, T_cap, splits, s);
    if (st != TACVQ_OK) return st;
    return attn_combine_dispatch((const float *)workspace, splits, (__half *)out_f16, state_out, (int64_t)B * Hq, D, s);
}

int tacvq_rope_table(uint16_t *table_f16, int64_t T, int D, double theta, int64_t first_position, tacvq_stream_t stream) {
    if (T < 0 || D <= 0 || (D & 1) != 0 || !(theta > 0.0) || first_position < 0) return TACVQ_ERR_GEOMETRY;
    if (D > 256) return TACVQ_ERR_UNSUPPORTED;
    if (T == 0) return TACVQ_OK;
    if (!table_f16) return TACVQ_ERR_NULL;
    if (((uintptr_t)table_f16 & 15) != 0) return TACVQ_ERR_ALIGN;
    return rope_table_dispatch((__half *)table_f16, T, D, theta, first_position, (cudaStream_t)stream);
}

int tacvq_attn_decode_rotary(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes,
                             const uint16_t *ktab_f16, const uint16_t *vtab_f16, const uint16_t *rope_table,
                             const int32_t *seq_start, const int32_t *seq_end, void *workspace, size_t workspace_bytes,
                             uint16_t *out_f16, float *state_out, int B, int Hq, int Hkv, int D, int G, int S, int K,
                             int64_t T_cap, tacvq_stream_t stream) {
    if (!q_f16 || !kcodes || !vcodes || !ktab_f16 || !vtab_f16 || !rope_table) return TACVQ_ERR_NULL;
    if (!out_f16 && !state_out) return TACVQ_ERR_NULL;
    const int g = check_attn_geometry(B, Hq, Hkv, D, G, S, K);
    if (g != TACVQ_OK) return g;
    if (D < 64) return TACVQ_ERR_UNSUPPORTED;
    if (T_cap < 0 || T_cap > 0x7fffffff) return TACVQ_ERR_RANGE;
    if (!workspace || ((uintptr_t)workspace & 255) != 0 || workspace_bytes < tacvq_attn_workspace_bytes(B, Hq, Hkv, D, G, S))
        return TACVQ_ERR_WORKSPACE;
    if (((uintptr_t)rope_table & 3) != 0) return TACVQ_ERR_ALIGN;  // the staged kernel wants 16 bytes and is skipped otherwise
    cudaStream_t s = (cudaStream_t)stream;
    if (attn_rotary_staged_supported(Hq, Hkv, D, G, S, K) && (((uintptr_t)ktab_f16 | (uintptr_t)vtab_f16 | (uintptr_t)rope_table) & 15) == 0) {
        const int staged = attn_rotary_staged_splits(B, Hkv, T_cap, sm_count());
        if (staged > 0) {
        int st = attn_rotary_staged_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                             (const __half *)vtab_f16, (const __half *)rope_table, seq_start, seq_end,
                                             (float *)workspace, B, Hq, Hkv, G, S, T_cap, staged, s);
        if (st != TACVQ_OK) return st;
        return attn_combine_dispatch((const float *)workspace, staged, (__half *)out_f16, state_out, (int64_t)B * Hq, D, s);
        }
    }
    const int splits = attn_rotary_splits(B, Hkv, T_cap, sm_count());
    int st = attn_rotary_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16, (const __half *)vtab_f16,
                                  (const __half *)rope_table, seq_start, seq_end, (float *)workspace, B, Hq, Hkv, D, G, S, K,
                                  T_cap, splits, s);
    if (st != TACVQ_OK) return st;
    return attn_combine_dispatch((const float *)workspace, splits, (__half *)out_f16, state_out, (int64_t)B * Hq, D, s);
}

int tacvq_set_ranges(int32_t *seq_start, int32_t *seq_end, int B, int start, int end, tacvq_stream_t stream) {
    if (!seq_start || !seq_end) return TACVQ_ERR_NULL;
    if (B <= 0 || start < 0 || end < start) return TACVQ_ERR_GEOMETRY;
    set_ranges_kernel<<<(B + 255) / 256, 256, 0, (cudaStream_t)stream>>>(seq_start, seq_end, B, start, end);
    return launch_status();
}

int tacvq_decode_step(const uint16_t *q_f16, const void *k_rows, const void *v_rows, int rows_dtype,
                      const uint16_t *ktab_f16, const uint16_t *vtab_f16, uint8_t *kcodes, uint8_t *vcodes,
                      int32_t *seq_start, int32_t *seq_end, int64_t length, int64_t window, void *workspace,
                      size_t workspace_bytes, uint16_t *out_f16, float *state_out, int B, int Hq, int Hkv, int D, int G,
                      int S, int K, int T_new, int64_t T_cap, tacvq_stream_t stream) {
    if (!k_rows || !v_rows || !seq_start || !seq_end) return TACVQ_ERR_NULL;
    if (length < 0 || window < 0 || T_new <= 0 || length + T_new > T_cap) return TACVQ_ERR_RANGE;
    const int64_t row = (int64_t)T_new * D;
    {
        // Fast path: one launch encodes both sides and sets the ranges, and the attention kernels that do
        // not read its results start while it runs.  Every argument check of the separate calls is made first.
        const int64_t new_end = length + T_new;
        const int64_t new_start = (window > 0 && new_end > window) ? new_end - window : 0;
        const bool plain = dtype_ok(rows_dtype) && q_f16 && ktab_f16 && vtab_f16 && kcodes && vcodes && (out_f16 || state_out) &&
                           check_code_geometry(B, Hkv, T_new, D, G, S, K, length, T_cap) == TACVQ_OK &&
                           check_attn_geometry(B, Hq, Hkv, D, G, S, K) == TACVQ_OK && T_cap <= 0x7fffffff && workspace &&
                           ((uintptr_t)workspace & 255) == 0 && workspace_bytes >= tacvq_attn_workspace_bytes(B, Hq, Hkv, D, G, S) &&
                           (((uintptr_t)kcodes | (uintptr_t)vcodes) & 15) == 0;
        if (plain) {
            cudaStream_t s = (cudaStream_t)stream;
            const bool gsrq = attn_gsrq_supported(Hq, Hkv, D, G, S, K) && gsrq_batch_ok(B, Hkv) && gsrq_aligned(q_f16, ktab_f16, vtab_f16);
            if (gsrq && T_new == 1 && ((((uintptr_t)k_rows | (uintptr_t)v_rows) & 15) == 0)) {
                // benchmark geometry, one new token: the table preparation encodes the token and sets the ranges
                // itself, so the whole step is two launches
                const GsrqNewToken token = {k_rows, v_rows, rows_dtype == TACVQ_F32 ? 1 : 0, kcodes, vcodes, seq_start, seq_end,
                                            (int)new_start, (int)new_end, (long long)length, (long long)T_cap};
                const int fast = attn_gsrq_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                                    (const __half *)vtab_f16, seq_start, seq_end, workspace, (__half *)out_f16,
                                                    state_out, B, Hq, Hkv, T_cap, sm_count(), s, &token);
                if (fast != TACVQ_ERR_UNSUPPORTED) return fast;
            }
            const int pro = decode_prologue_dispatch(k_rows, v_rows, rows_dtype, (int64_t)Hkv * row, row, D, (const __half *)ktab_f16,
                                                     (const __half *)vtab_f16, kcodes, vcodes, seq_start, seq_end, (int)new_start,
                                                     (int)new_end, B, Hkv, T_new, D, G, S, K, length, T_cap, s);
            if (pro == TACVQ_OK) {
                if (gsrq) {
                    const int fast = attn_gsrq_dispatch((const __half *)q_f16, kcodes, vcodes, (const __half *)ktab_f16,
                                                        (const __half *)vtab_f16, seq_start, seq_end, workspace,
                                                        (__half *)out_f16, state_out, B, Hq, Hkv, T_cap, sm_count(), s);
                    if (fast != TACVQ_ERR_UNSUPPORTED) return fast;
                }
                return tacvq_attn_decode(q_f16, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end, workspace,
                                         workspace_bytes, out_f16, state_out, B, Hq, Hkv, D, G, S, K, T_cap, stream);
            }
            if (pro != TACVQ_ERR_UNSUPPORTED) return pro;
        }
    }
    int st = tacvq_encode(k_rows, rows_dtype, (int64_t)Hkv * row, row, D, ktab_f16, nullptr, kcodes, nullptr, TACVQ_F16, B,
                          Hkv, T_new, D, G, S, K, length, T_cap, stream);
    if (st != TACVQ_OK) return st;
    st = tacvq_encode(v_rows, rows_dtype, (int64_t)Hkv * row, row, D, vtab_f16, nullptr, vcodes, nullptr, TACVQ_F16, B, Hkv,
                      T_new, D, G, S, K, length, T_cap, stream);
    if (st != TACVQ_OK) return st;
    const int64_t end = length + T_new;
    const int64_t start = (window > 0 && end > window) ? end - window : 0;
    st = tacvq_set_ranges(seq_start, seq_end, B, (int)start, (int)end, stream);
    if (st != TACVQ_OK) return st;
    return tacvq_attn_decode(q_f16, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end, workspace, workspace_bytes,
                             out_f16, state_out, B, Hq, Hkv, D, G, S, K, T_cap, stream);
}

// The device address of a host buffer that kernels may dereference in place (pinned or registered memory), or
// nullptr when the buffer is ordinary pageable memory or lives on the device.
static void *device_view_of_host(const void *host) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (attr.type != cudaMemoryTypeHost) return nullptr;
    return attr.devicePointer;
}

int tacvq_decode_step_host(const void *host_rows, void *dev_rows, int rows_dtype, const uint16_t *ktab_f16,
                           const uint16_t *vtab_f16, uint8_t *kcodes, uint8_t *vcodes, int32_t *seq_start, int32_t *seq_end,
                           int64_t length, int64_t window, void *workspace, size_t workspace_bytes, uint16_t *dev_out,
                           void *host_out, int B, int Hq, int Hkv, int D, int G, int S, int K, int T_new, int64_t T_cap,
                           int synchronize, tacvq_stream_t stream) {
    if (!host_rows || !host_out) return TACVQ_ERR_NULL;
    if (!dtype_ok(rows_dtype)) return TACVQ_ERR_DTYPE;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || T_new <= 0) return TACVQ_ERR_GEOMETRY;
    const size_t q_bytes = (size_t)B * Hq * D * sizeof(uint16_t);
    const size_t kv_bytes = (size_t)B * Hkv * T_new * D * (rows_dtype == TACVQ_F16 ? 2 : 4);
    if ((q_bytes & 15) != 0 || (kv_bytes & 15) != 0) return TACVQ_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    // Without a landing buffer the kernels read the rows where they lie (the prologue and the table preparation
    // each read them once, over the host link), and without dev_out the merging blocks store to host_out.
    const unsigned char *rows = (const unsigned char *)dev_rows;
    if (!rows) {
        rows = (const unsigned char *)device_view_of_host(host_rows);
        if (!rows) return TACVQ_ERR_NULL;
    } else {
        e = cudaMemcpyAsync(dev_rows, host_rows, q_bytes + 2 * kv_bytes, cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) return (int)e;
    }
    if (((uintptr_t)rows & 15) != 0) return TACVQ_ERR_ALIGN;
    uint16_t *out = dev_out;
    if (!out) {
        out = (uint16_t *)device_view_of_host(host_out);
        if (!out) return TACVQ_ERR_NULL;
    }
    const int st = tacvq_decode_step((const uint16_t *)rows, rows + q_bytes, rows + q_bytes + kv_bytes, rows_dtype, ktab_f16,
                                     vtab_f16, kcodes, vcodes, seq_start, seq_end, length, window, workspace, workspace_bytes,
                                     out, nullptr, B, Hq, Hkv, D, G, S, K, T_new, T_cap, stream);
    if (st != TACVQ_OK) return st;
    if (dev_out) {
        e = cudaMemcpyAsync(host_out, dev_out, q_bytes, cudaMemcpyDeviceToHost, s);
        if (e != cudaSuccess) return (int)e;
    }
    if (synchronize) {
        e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return (int)e;
    }
    return TACVQ_OK;
}

size_t tacvq_attn_static_scratch_bytes(void) { return kStaticScratchBytes; }

int tacvq_attn_decode_static(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes,
                             const uint16_t *ktab_f16, const uint16_t *vtab_f16, const int32_t *seq_start,
                             const int32_t *seq_end, uint16_t *out_f16, float *state_out, int B, int Hq, int Hkv, int D,
                             int G, int S, int K, int64_t T_cap, tacvq_stream_t stream) {
    const int g = check_attn_geometry(B, Hq, Hkv, D, G, S, K);
    if (g != TACVQ_OK) return g;
    if (tacvq_attn_workspace_bytes(B, Hq, Hkv, D, G, S) > kStaticScratchBytes) return TACVQ_ERR_WORKSPACE;
    void *scratch = nullptr;
    const int st = static_scratch_for_current_device(&scratch);
    if (st != TACVQ_OK) return st;
    return tacvq_attn_decode(q_f16, kcodes, vcodes, ktab_f16, vtab_f16, seq_start, seq_end, scratch, kStaticScratchBytes,
                             out_f16, state_out, B, Hq, Hkv, D, G, S, K, T_cap, stream);
}

int tacvq_attn_combine(const float *states, int n_parts, uint16_t *out_f16, float *merged, int B, int Hq, int D,
                       tacvq_stream_t stream) {
    if (!states || (!out_f16 && !merged)) return TACVQ_ERR_NULL;
    if (n_parts <= 0 || B <= 0 || Hq <= 0 || D <= 0) return TACVQ_ERR_GEOMETRY;
    return attn_combine_dispatch(states, n_parts, (__half *)out_f16, merged, (int64_t)B * Hq, D, (cudaStream_t)stream);
}

}  // extern "C"
