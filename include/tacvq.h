/*
 * tacvq.h - C ABI of libtacvq.so: hard residual GSRQ/CQ KV-cache quantization on B200 (sm_100a).
 *
 * The reference project (wrb1371/tac-vq-kv-cache) is pure Python and has no FFI of its own; its
 * boundary is a set of Python callables.  Each entry point below names the reference callable whose
 * forward arithmetic it replaces (paths are inside the reference project).  A Python binding that
 * keeps the reference's signatures on top of these entry points ships in the package
 * (tac_vq_kv_cache_b200/jointkv); any other host language can bind the same symbols.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".  The library never
 *     allocates or frees device memory; scratch space is passed in by the caller.
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns
 *     without synchronising.  NULL is the legacy default stream.
 *   - Return value: 0 on success; < 0 an argument error found on the host before anything was
 *     launched (see enum tacvq_status); > 0 a cudaError_t from a launch.  No call aborts or prints.
 *   - Canonical layouts (row-major, innermost last):
 *       states  [B, H, T, D]          fp16 or fp32; D = G*d contiguous, other strides given in elements
 *       tables  [H, S, G, K, d]       fp16 "deployed" codewords (the fp16 round trip of the masters)
 *       codes   [B, H, T_cap, S, G]   uint8; the reference's [B,H,T,S] (G=1) and [B,H,T,G] (S=1)
 *                                     layouts are this one with a unit axis dropped
 *     H = KV heads, G = channel groups, S = residual stages, K <= 256 codewords, d = D/G.
 *   - Arithmetic contract for a code (closed_loop_vq.py:66-75, cq_tac.py:86-96): fp32 distance
 *     (|x|^2 + |c_k|^2) - 2*(x.c_k) in that association; x.c_k one fused-multiply-add chain from
 *     element 0; squared norms from separately rounded products (order documented in
 *     csrc/common.cuh); lowest index wins a tie.
 */
#ifndef TACVQ_H
#define TACVQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TACVQ_ABI_VERSION 1

#if defined(__GNUC__)
#define TACVQ_API __attribute__((visibility("default")))
#else
#define TACVQ_API
#endif

enum tacvq_dtype { TACVQ_F16 = 0, TACVQ_F32 = 1 };

enum tacvq_status {
    TACVQ_OK = 0,
    TACVQ_ERR_NULL = -1,        /* a required pointer is NULL */
    TACVQ_ERR_GEOMETRY = -2,    /* sizes inconsistent (D != G*d, Hq % Hkv, non-positive extent ...) */
    TACVQ_ERR_DTYPE = -3,       /* dtype tag is not a tacvq_dtype */
    TACVQ_ERR_RANGE = -4,       /* token offset/extent outside the code buffer */
    TACVQ_ERR_WORKSPACE = -5,   /* scratch buffer missing, too small or misaligned */
    TACVQ_ERR_UNSUPPORTED = -6, /* geometry valid but no kernel is built for it */
    TACVQ_ERR_ALIGN = -7,       /* a pointer or stride breaks the stated alignment */
    TACVQ_ERR_DEVICE = -8       /* current device is not compute capability 10.x */
};

typedef void *tacvq_stream_t;

/* ABI version of the loaded library (TACVQ_ABI_VERSION at build time). */
TACVQ_API int tacvq_version(void);

/* Static, human-readable text for a status returned by any call below. */
TACVQ_API const char *tacvq_status_string(int status);

/*
 * Squared norms of all codewords, out[words] fp32, words = H*S*G*K, in the library's documented
 * order.  Replaces `table.square().sum(dim=-1)` (closed_loop_vq.py:66; cq_tac.py:86).
 */
TACVQ_API int tacvq_table_sqnorm(const uint16_t *tables_f16, float *out, int64_t words, int d, tacvq_stream_t stream);

/*
 * Diagnostic of the wide-group encode (d = 64, 128), whose approximate scores are tensor-core products
 * (tcgen05) kept in tensor memory: *count = how many times, on the current device since the library was
 * loaded, a block stopped waiting for those products and re-evaluated every pair of the stage instead,
 * or stopped waiting for a table copy of the copy engine (TMA) and copied the table itself, plus the number
 * of launches that could not get a tensor map for their tables at all (codes stay exact either way).  Synchronises the device.  Expected value: 0.  No counterpart in the
 * reference.
 */
TACVQ_API int tacvq_encode_tensor_memory_timeouts(unsigned int *count);

/*
 * Encode: greedy residual nearest-codeword search, all S stages fused, groups independent.
 * Replaces the forward of hard_residual_vq_exits (closed_loop_vq.py:235-410, G=1) and of
 * hard_grouped_cq (cq_tac.py:33-114, S=1), including _nearest_indices (closed_loop_vq.py:52-76).
 *
 *   x, x_dtype         states [B,H,T,D]; strides sxb,sxh,sxt in elements, last axis contiguous;
 *                      base and strides such that every row starts 16-byte aligned
 *   tables_f16         [H,S,G,K,d]
 *   table_sqnorm       NULL (computed inside) or [H,S,G,K] fp32 supplied by the caller
 *                      (tacvq_table_sqnorm); for d >= 32 supplying it saves every 128-row block
 *                      from recomputing the norms of its 256 words
 *   codes              [B,H,T_cap,S,G]; rows t0 .. t0+T-1 are written, the rest is untouched
 *   recon, recon_dtype NULL, or [B,H,T,D] contiguous receiving sum_s word_s (fp32 sum in stage
 *                      order, one final cast) - the reference's exit at depth S
 *   d = D/G must be one of 1..8, 16, 32, 64, 128.
 *
 * The codes are those of a full scan in the library's fp32 order (first minimum wins).  For
 * d = 4, 8, 32, 64, 128 with 16-byte aligned tables the scan is filtered: tensor cores score every
 * word, and only the words within a proven error margin of a row's best score are re-evaluated in
 * that exact order, which cannot change the result.
 */
TACVQ_API int tacvq_encode(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt, const uint16_t *tables_f16,
                 const float *table_sqnorm, uint8_t *codes, void *recon, int recon_dtype, int B, int H, int T, int D,
                 int G, int S, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream);

/*
 * Encode with a whitened assignment geometry.  Replaces the `assignment_whiteners` branch of
 * hard_residual_vq_exits (closed_loop_vq.py:312-320, 384-390: one [D,D] matrix per head, G must
 * be 1 there) and the `selector_whiteners` branch of hard_grouped_cq (cq_tac.py:80-85: one [d,d]
 * matrix per (head, group), S must be 1 there).  The search runs on W.x against W-transformed
 * words and subtracts transformed words; codes index the plain tables, recon uses plain words.
 *
 *   whitener           [H,G,d,d] fp32, row-major (y_i = sum_j W[i][j] x_j)
 *   search_tables      [H,S,G,K,d] fp32 scratch: receives the transformed words (caller-owned)
 *   search_rows        [B,H,T,D] fp32 scratch: receives the transformed rows (caller-owned)
 */
TACVQ_API int tacvq_encode_whitened(const void *x, int x_dtype, int64_t sxb, int64_t sxh, int64_t sxt,
                          const uint16_t *tables_f16, const float *whitener, float *search_tables,
                          float *search_rows, uint8_t *codes, void *recon, int recon_dtype, int B, int H, int T, int D,
                          int G, int S, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream);

/*
 * Decode: rebuild rows t0 .. t0+T-1 from stored codes using the first S_use stages.
 * Replaces _gather_words + the fp32 stage sum (closed_loop_vq.py:127-139, 376-381, 398-403),
 * _gather_group_words (cq_tac.py:21-30) and frozen_assignment_u16_reconstruction
 * (experiments/train_pure_uniform16_closed_loop_vq.py:395-442).   out [B,H,T,D] contiguous.
 */
TACVQ_API int tacvq_decode(const uint8_t *codes, const uint16_t *tables_f16, void *out, int out_dtype, int B, int H, int T,
                 int D, int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream);

/*
 * Gradient of the hard forward with respect to the codeword masters: grad_tables[h,s,g,code,:] +=
 * grad_out[b,h,t,g*d:(g+1)*d] for every stage s < S_use (the straight-through edge through the
 * fp16 round trip has unit gain: closed_loop_vq.py:298, 376-381; cq_tac.py:77, 98-99).
 * grad_tables [H,S,G,K,d] fp32 is accumulated into (caller zeroes it); grad_out [B,H,T,D] fp32 contiguous.
 */
TACVQ_API int tacvq_codeword_grad(const uint8_t *codes, const float *grad_out, float *grad_tables, int B, int H, int T, int D,
                        int G, int S, int S_use, int K, int64_t t0, int64_t T_cap, tacvq_stream_t stream);

/*
 * Bytes of scratch tacvq_attn_decode needs for this geometry (host computation, no CUDA call
 * besides a device-attribute query).  0 on invalid geometry.
 */
TACVQ_API size_t tacvq_attn_workspace_bytes(int B, int Hq, int Hkv, int D, int G, int S);

/*
 * One decode step of attention computed directly on the stored codes: per-query look-up table of
 * q . codeword, score = sum of table entries addressed by the K codes, softmax, V accumulated
 * from the V codes, sequence split across thread blocks and merged by log-sum-exp.
 * Replaces the decode branch of the reference's attention_forward
 * (experiments_followup_mistral/evaluate_mistral_longbench.py:112-122) together with the dense
 * decoded window LayerCache keeps for it (:53-70); rotary embedding is NOT applied here.
 *
 *   q_f16              [B,Hq,D] fp16, already multiplied by the softmax scale
 *   kcodes, vcodes     [B,Hkv,T_cap,S,G] uint8 (16-byte aligned)
 *   ktab_f16, vtab_f16 [Hkv,S,G,K,d] fp16
 *   seq_start, seq_end NULL or int32 [B]: row b attends tokens [seq_start[b], seq_end[b]);
 *                      NULL means 0 resp. T_cap.  An empty range yields out = 0, m = -inf, l = 0.
 *   workspace          scratch of at least tacvq_attn_workspace_bytes(...) bytes, 256-byte aligned
 *   out_f16            NULL or [B,Hq,D] fp16: acc / l
 *   state_out          NULL or [B,Hq,2+D] fp32: (m, l, acc[D]) with l = sum exp(s-m), acc = sum exp(s-m) v
 *                      - the partial softmax state that ranks exchange when the sequence is split
 *                      across GPUs.  m (natural log units) is the reference the sums are taken
 *                      against: never above the maximum score and at most 8 ln 2 below it; m + ln l
 *                      (the log-sum-exp) and acc / l do not depend on it
 *   Hq % Hkv == 0, Hq/Hkv <= 8, K == 256, D % 32 == 0, D <= 256.
 */
TACVQ_API int tacvq_attn_decode(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes, const uint16_t *ktab_f16,
                      const uint16_t *vtab_f16, const int32_t *seq_start, const int32_t *seq_end, void *workspace,
                      size_t workspace_bytes, uint16_t *out_f16, float *state_out, int B, int Hq, int Hkv, int D,
                      int G, int S, int K, int64_t T_cap, tacvq_stream_t stream);

/*
 * Fill seq_start[0..B) = start and seq_end[0..B) = end on the stream: the visible range of a batch
 * whose sequences advance in lockstep, i.e. LayerCache.visible() of the reference
 * (experiments_followup_mistral/evaluate_mistral_longbench.py:62-70) for every row at once.
 */
TACVQ_API int tacvq_set_ranges(int32_t *seq_start, int32_t *seq_end, int B, int start, int end, tacvq_stream_t stream);

/*
 * One decode step of one layer in a single call: encode the new token rows of K and V into the code
 * buffers at position `length` (tacvq_encode, in place), set every row's visible range to the last
 * `window` tokens (window = 0: all stored tokens), attend.  Replaces the body of the reference's decode
 * adapter per layer: cache.codec(...) + LayerCache.append + LayerCache.visible + attention
 * (experiments_followup_mistral/evaluate_mistral_longbench.py:94-98, 112-122), without its torch.cat
 * of the code tensors and without a decoded fp16 window.
 *
 *   k_rows, v_rows       [B,Hkv,T_new,D] contiguous, fp16 or fp32 (rows_dtype)
 *   kcodes, vcodes       [B,Hkv,T_cap,S,G]; rows length .. length+T_new-1 are written
 *   seq_start, seq_end   int32 [B] device scratch that receives the visible range
 *   length               tokens already stored per sequence (host value; sequences advance in lockstep)
 * All other arguments as in tacvq_attn_decode.
 */
TACVQ_API int tacvq_decode_step(const uint16_t *q_f16, const void *k_rows, const void *v_rows, int rows_dtype,
                                const uint16_t *ktab_f16, const uint16_t *vtab_f16, uint8_t *kcodes, uint8_t *vcodes,
                                int32_t *seq_start, int32_t *seq_end, int64_t length, int64_t window, void *workspace,
                                size_t workspace_bytes, uint16_t *out_f16, float *state_out, int B, int Hq, int Hkv,
                                int D, int G, int S, int K, int T_new, int64_t T_cap, tacvq_stream_t stream);

/*
 * tacvq_decode_step for a host that holds the new token's rows and wants the result in HOST memory: one call
 * enqueues the host-to-device copy of the rows, the decode step and the device-to-host copy of the result,
 * and optionally waits for the stream.  It covers one iteration of the reference's generation loop around
 * its per-layer adapter (experiments_followup_mistral/evaluate_mistral_longbench.py:156-197 calls the model
 * once per token; :94-98, 112-122 is the per-layer body), for hosts that drive a layer from another process
 * or language and pay per call.
 *
 *   host_rows     host buffer (pinned for an asynchronous copy): q [B,Hq,D] fp16, then the new K rows
 *                 [B,Hkv,T_new,D], then the new V rows, K and V in rows_dtype, packed back to back
 *   dev_rows      device buffer of the same size, 16-byte aligned: the landing place of host_rows;
 *                 NULL: no copy is enqueued and the kernels read host_rows in place over the host link, which
 *                 needs host_rows to be page-locked (cudaHostAlloc / cudaHostRegister) and 16-byte aligned;
 *                 pageable memory is refused with TACVQ_ERR_NULL before anything is launched
 *   dev_out       device [B,Hq,D] fp16;  host_out  host buffer of the same size receiving it;
 *                 dev_out NULL: the attention kernel stores the result straight into host_out (page-locked)
 *   synchronize   non-zero: return after the stream has finished (host_out is valid on return)
 * Other arguments and status codes as tacvq_decode_step.
 */
TACVQ_API int tacvq_decode_step_host(const void *host_rows, void *dev_rows, int rows_dtype, const uint16_t *ktab_f16,
                                     const uint16_t *vtab_f16, uint8_t *kcodes, uint8_t *vcodes, int32_t *seq_start,
                                     int32_t *seq_end, int64_t length, int64_t window, void *workspace,
                                     size_t workspace_bytes, uint16_t *dev_out, void *host_out, int B, int Hq, int Hkv,
                                     int D, int G, int S, int K, int T_new, int64_t T_cap, int synchronize,
                                     tacvq_stream_t stream);

/*
 * tacvq_attn_decode for callers that must not allocate device memory.  It has no counterpart in the
 * reference.  Some hosts of this library cannot call cudaMalloc at the point where they need
 * attention: a plugin running inside another runtime's memory pool, a callback on a thread that is
 * not allowed to touch the allocator, a process whose device memory was handed out in full at start-up.
 * For them the scratch is a fixed 16 MiB array inside the library image
 * (tacvq_attn_static_scratch_bytes() returns that figure); the caller passes only inputs and outputs.
 * After the set-up call described below a call allocates and frees nothing, on the device or through any library.
 *
 *   - Limit: geometries whose tacvq_attn_workspace_bytes(...) exceeds 16 MiB are refused with
 *     TACVQ_ERR_WORKSPACE (nothing is launched).  The benchmark geometry at batch 8 needs 8.1 MiB.
 *   - The first call on each device is a set-up call: the CUDA runtime loads this library's kernels and the
 *     array onto that device when they are first used, and the call looks up the array's device address
 *     (one cudaGetSymbolAddress with that device current, kept for later calls; first calls from several
 *     host threads may overlap, they store the same address).  Make one warm-up call per device at
 *     start-up, outside any stream capture; calls after it allocate nothing.  A cudaDeviceReset
 *     invalidates the address together with everything else the library has set up on that device.
 *   - All calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *     (different streams without ordering between them) race on it.  Calls on one stream are safe.
 *     The array keeps the previous call's contents; nothing in it has to start at zero, because
 *     every word a call reads is written earlier by the same call.
 *   - Every GPU that loads the library holds the 16 MiB until the process ends.
 * Arguments, results and status codes are those of tacvq_attn_decode without the workspace pair.
 */
TACVQ_API size_t tacvq_attn_static_scratch_bytes(void);
TACVQ_API int tacvq_attn_decode_static(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes,
                                       const uint16_t *ktab_f16, const uint16_t *vtab_f16, const int32_t *seq_start,
                                       const int32_t *seq_end, uint16_t *out_f16, float *state_out, int B, int Hq,
                                       int Hkv, int D, int G, int S, int K, int64_t T_cap, tacvq_stream_t stream);

/*
 * Log-sum-exp merge of n_parts partial softmax states [n_parts,B,Hq,2+D] fp32 (for example the
 * all-gathered per-GPU states of a sequence-split decode): M = max m_r, L = sum l_r e^(m_r-M),
 * A = sum acc_r e^(m_r-M).  out_f16 (NULL or [B,Hq,D]) receives A/L; merged (NULL or [B,Hq,2+D])
 * receives (M, L, A).  Softmax attention itself: src/jointkv/local_attention.py:673-679.
 */
TACVQ_API int tacvq_attn_combine(const float *states, int n_parts, uint16_t *out_f16, float *merged, int B, int Hq, int D,
                       tacvq_stream_t stream);

/*
 * cos/sin table of the rotary position embedding: row t holds D/2 cosines, then D/2 sines, of the
 * angles (first_position + t) * theta^(-2i/D), i < D/2, as fp16: inverse frequencies, angles and
 * cos/sin in fp32, one rounding to fp16.  Replaces `self.rotary_emb(visible_k, all_positions)` of the reference's decode branch
 * (experiments_followup_mistral/evaluate_mistral_longbench.py:115-117; default rope type of
 * transformers' MistralRotaryEmbedding).  A caller that has its model's own cos/sin may fill the
 * table itself.
 *
 *   table_f16          [T][2][D/2] fp16, 16-byte aligned;  D <= 256, D even
 */
TACVQ_API int tacvq_rope_table(uint16_t *table_f16, int64_t T, int D, double theta, int64_t first_position,
                               tacvq_stream_t stream);

/*
 * tacvq_attn_decode for codes of PRE-rotary keys, as the reference stores them: every rebuilt fp16
 * key row t is rotated with rope_table[t] ("rotate_half" pairing of channel c with c +- D/2;
 * k*cos + rotate_half(k)*sin with fp16 products and sum, as apply_rotary_pos_emb does on the fp16
 * window) before its dot product with q.  Replaces evaluate_mistral_longbench.py:112-122 including
 * the rotary step (:113-118).
 *
 *   q_f16              [B,Hq,D] fp16, already rotated at the query's own position and multiplied by
 *                      the softmax scale
 *   rope_table         [T_cap][2][D/2] from tacvq_rope_table (row index = token index in the code buffers)
 *   other arguments, workspace size and results as for tacvq_attn_decode; D in {64, 128, 256}.
 */
TACVQ_API int tacvq_attn_decode_rotary(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes,
                                       const uint16_t *ktab_f16, const uint16_t *vtab_f16, const uint16_t *rope_table,
                                       const int32_t *seq_start, const int32_t *seq_end, void *workspace,
                                       size_t workspace_bytes, uint16_t *out_f16, float *state_out, int B, int Hq,
                                       int Hkv, int D, int G, int S, int K, int64_t T_cap, tacvq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TACVQ_H */
