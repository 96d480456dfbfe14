/*
 * Plain-C restatement of the hard residual GSRQ/CQ path (TEST INFRASTRUCTURE ONLY).
 *
 * It is the scalar, order-explicit twin of oracle/jointkv_oracle.py: the same
 * algorithm, but with every floating-point summation order written out, so that
 * the CUDA kernels (which use the same orders) can be required to agree with it
 * bit for bit, while it is itself compared with the torch restatement and with
 * the golden vectors produced by the reference.  Nothing in the product links
 * or loads this file; tests, the smoke check and the CPU-baseline leg of the
 * benchmark do.
 *
 * Reference statements followed (paths inside the reference project):
 *   src/jointkv/closed_loop_vq.py:66-75   distance (|x|^2 + |c|^2) - 2 x.c, first-minimum argmin
 *   src/jointkv/closed_loop_vq.py:298     tables used through their fp16 round trip
 *   src/jointkv/closed_loop_vq.py:376-383 decoded += word ; residual -= word   (fp32)
 *   src/jointkv/closed_loop_vq.py:398-403 cast of the fp32 sum to the state dtype
 *   src/jointkv/cq_tac.py:86-105          the one-stage grouped form of the same search
 *   experiments_followup_mistral/evaluate_mistral_longbench.py:112-122
 *                                         decode step = softmax(q K^T) V over the rebuilt window
 *
 * Summation orders (observed from the reference's CPU library calls and fixed here):
 *   x.c      one fused-multiply-add chain, element 0 first, starting from 0
 *            (what the batched GEMM does for every output when rows >= 2);
 *   |v|^2    products rounded to fp32, then added:
 *              d <= 8            left to right;
 *              d = 16, 24        eight running lanes (element i -> lane i mod 8),
 *                                lanes then added left to right;
 *              d multiple of 32  four sets of eight lanes (element i -> set (i/8) mod 4,
 *                                lane i mod 8), sets added ((0+1)+2)+3 per lane,
 *                                lanes then added left to right.
 *
 * Build: gcc -O2 -fPIC -shared -fopenmp -mf16c -mfma -ffp-contract=off (see oracle/build.py).
 */

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 half_t;

enum { TACVQ_F16 = 0, TACVQ_F32 = 1 };

static float sqnorm_ordered(const float *v, int d) {
    if (d <= 8 || (d % 8) != 0) {
        float acc = 0.0f;
        for (int i = 0; i < d; ++i) {
            float p = v[i] * v[i];
            acc = acc + p;
        }
        return acc;
    }
    float lane[8];
    if (d % 32 != 0) { /* 16 or 24: one set of lanes */
        for (int j = 0; j < 8; ++j) lane[j] = v[j] * v[j];
        for (int i = 8; i < d; ++i) {
            float p = v[i] * v[i];
            lane[i & 7] = lane[i & 7] + p;
        }
    } else {
        float set[4][8];
        for (int s = 0; s < 4; ++s)
            for (int j = 0; j < 8; ++j) set[s][j] = 0.0f;
        for (int i = 0; i < d; ++i) {
            float p = v[i] * v[i];
            set[(i >> 3) & 3][i & 7] = set[(i >> 3) & 3][i & 7] + p;
        }
        for (int j = 0; j < 8; ++j) lane[j] = ((set[0][j] + set[1][j]) + set[2][j]) + set[3][j];
    }
    float acc = lane[0];
    for (int j = 1; j < 8; ++j) acc = acc + lane[j];
    return acc;
}

static inline float load_state(const void *x, int dtype, int64_t i) {
    return dtype == TACVQ_F16 ? (float)((const half_t *)x)[i] : ((const float *)x)[i];
}

/* Squared norms of every codeword, [H,S,G,K], in the order above. */
int tacvq_oracle_table_sqnorm(const uint16_t *tables_f16, float *out, int64_t words, int d) {
    const half_t *tab = (const half_t *)tables_f16;
#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < words; ++w) {
        float tmp[512];
        for (int i = 0; i < d; ++i) tmp[i] = (float)tab[w * d + i];
        out[w] = sqnorm_ordered(tmp, d);
    }
    return 0;
}

/*
 * Encode rows x[B,H,T,D] (contiguous) against tables_f16[H,S,G,K,d] (d = D/G).
 * codes[B,H,T_cap,S,G] written at token offset t0; recon (optional) [B,H,T,D].
 */
int tacvq_oracle_encode(const void *x, int x_dtype, const uint16_t *tables_f16, uint8_t *codes, void *recon,
                        int recon_dtype, int B, int H, int T, int D, int G, int S, int K, int64_t t0,
                        int64_t T_cap) {
    if (G <= 0 || D % G != 0 || K <= 0 || K > 256 || D / G > 512) return -1;
    const int d = D / G;
    const half_t *tab = (const half_t *)tables_f16;
    const int64_t words = (int64_t)H * S * G * K;
    float *tabf = (float *)malloc(sizeof(float) * words * d);
    float *norm = (float *)malloc(sizeof(float) * words);
    if (!tabf || !norm) return -2;
    for (int64_t i = 0; i < words * d; ++i) tabf[i] = (float)tab[i];
    for (int64_t w = 0; w < words; ++w) norm[w] = sqnorm_ordered(tabf + w * d, d);

    const int64_t rows = (int64_t)B * H * T;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int t = (int)(row % T);
        const int h = (int)((row / T) % H);
        const int b = (int)(row / ((int64_t)T * H));
        float res[512], dec[512];
        for (int g = 0; g < G; ++g) {
            for (int i = 0; i < d; ++i) {
                res[i] = load_state(x, x_dtype, row * D + g * d + i);
                dec[i] = 0.0f;
            }
            for (int s = 0; s < S; ++s) {
                const int64_t base = (((int64_t)h * S + s) * G + g) * K;
                const float xx = sqnorm_ordered(res, d);
                float best = 0.0f;
                int arg = 0;
                for (int k = 0; k < K; ++k) {
                    const float *c = tabf + (base + k) * d;
                    float dot = 0.0f;
                    for (int i = 0; i < d; ++i) dot = fmaf(res[i], c[i], dot);
                    float lhs = xx + norm[base + k];
                    float dist = lhs - 2.0f * dot;
                    if (k == 0 || dist < best) {
                        best = dist;
                        arg = k;
                    }
                }
                const float *c = tabf + (base + arg) * d;
                for (int i = 0; i < d; ++i) {
                    dec[i] = dec[i] + c[i];
                    res[i] = res[i] - c[i];
                }
                codes[((((int64_t)b * H + h) * T_cap + t0 + t) * S + s) * G + g] = (uint8_t)arg;
            }
            if (recon) {
                for (int i = 0; i < d; ++i) {
                    if (recon_dtype == TACVQ_F16)
                        ((half_t *)recon)[row * D + g * d + i] = (half_t)dec[i];
                    else
                        ((float *)recon)[row * D + g * d + i] = dec[i];
                }
            }
        }
    }
    free(tabf);
    free(norm);
    return 0;
}

/*
 * Encode with a whitened assignment geometry (closed_loop_vq.py:312-320, 384-390: one [D,D] matrix per head,
 * G = 1; cq_tac.py:80-85: one [d,d] matrix per (head, group), S = 1).  whitener[H,G,d,d] row-major:
 *   search row   y_i = sum_j W[i][j] x_j          search word  c'_i = sum_j c_j W[i][j]
 * each one fused-multiply-add chain over j ascending, starting from 0.  The search runs on y against c'
 * (norms of c' and of the running search residual in the order above) and subtracts the selected c';
 * codes index the plain tables and the reconstruction sums plain fp16 words.
 */
int tacvq_oracle_encode_whitened(const void *x, int x_dtype, const uint16_t *tables_f16, const float *whitener,
                                 uint8_t *codes, void *recon, int recon_dtype, int B, int H, int T, int D, int G,
                                 int S, int K, int64_t t0, int64_t T_cap) {
    if (G <= 0 || D % G != 0 || K <= 0 || K > 256 || D / G > 512) return -1;
    const int d = D / G;
    const half_t *tab = (const half_t *)tables_f16;
    const int64_t words = (int64_t)H * S * G * K;
    float *tabf = (float *)malloc(sizeof(float) * words * d);   /* plain words */
    float *tabw = (float *)malloc(sizeof(float) * words * d);   /* transformed words */
    float *norm = (float *)malloc(sizeof(float) * words);
    if (!tabf || !tabw || !norm) return -2;
    for (int64_t i = 0; i < words * d; ++i) tabf[i] = (float)tab[i];
#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < words; ++w) {
        const int g = (int)((w / K) % G);
        const int h = (int)(w / ((int64_t)K * G * S));
        const float *mat = whitener + ((int64_t)h * G + g) * d * d;
        for (int i = 0; i < d; ++i) {
            float acc = 0.0f;
            for (int j = 0; j < d; ++j) acc = fmaf(tabf[w * d + j], mat[i * d + j], acc);
            tabw[w * d + i] = acc;
        }
        norm[w] = sqnorm_ordered(tabw + w * d, d);
    }
    const int64_t rows = (int64_t)B * H * T;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int t = (int)(row % T);
        const int h = (int)((row / T) % H);
        const int b = (int)(row / ((int64_t)T * H));
        float raw[512], res[512], dec[512];
        for (int g = 0; g < G; ++g) {
            const float *mat = whitener + ((int64_t)h * G + g) * d * d;
            for (int i = 0; i < d; ++i) {
                raw[i] = load_state(x, x_dtype, row * D + g * d + i);
                dec[i] = 0.0f;
            }
            for (int i = 0; i < d; ++i) {
                float acc = 0.0f;
                for (int j = 0; j < d; ++j) acc = fmaf(mat[i * d + j], raw[j], acc);
                res[i] = acc;
            }
            for (int s = 0; s < S; ++s) {
                const int64_t base = (((int64_t)h * S + s) * G + g) * K;
                const float xx = sqnorm_ordered(res, d);
                float best = 0.0f;
                int arg = 0;
                for (int k = 0; k < K; ++k) {
                    const float *c = tabw + (base + k) * d;
                    float dot = 0.0f;
                    for (int i = 0; i < d; ++i) dot = fmaf(res[i], c[i], dot);
                    float lhs = xx + norm[base + k];
                    float dist = lhs - 2.0f * dot;
                    if (k == 0 || dist < best) {
                        best = dist;
                        arg = k;
                    }
                }
                const float *cw = tabw + (base + arg) * d, *cp = tabf + (base + arg) * d;
                for (int i = 0; i < d; ++i) {
                    dec[i] = dec[i] + cp[i];
                    res[i] = res[i] - cw[i];
                }
                codes[((((int64_t)b * H + h) * T_cap + t0 + t) * S + s) * G + g] = (uint8_t)arg;
            }
            if (recon) {
                for (int i = 0; i < d; ++i) {
                    if (recon_dtype == TACVQ_F16)
                        ((half_t *)recon)[row * D + g * d + i] = (half_t)dec[i];
                    else
                        ((float *)recon)[row * D + g * d + i] = dec[i];
                }
            }
        }
    }
    free(tabf);
    free(tabw);
    free(norm);
    return 0;
}

/* Rebuild rows from codes[B,H,T_cap,S,G] (tokens t0..t0+T) using the first S_use stages. */
int tacvq_oracle_decode(const uint8_t *codes, const uint16_t *tables_f16, void *out, int out_dtype, int B, int H,
                        int T, int D, int G, int S, int S_use, int K, int64_t t0, int64_t T_cap) {
    if (G <= 0 || D % G != 0 || S_use > S) return -1;
    const int d = D / G;
    const half_t *tab = (const half_t *)tables_f16;
    const int64_t rows = (int64_t)B * H * T;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int t = (int)(row % T);
        const int h = (int)((row / T) % H);
        const int b = (int)(row / ((int64_t)T * H));
        const uint8_t *cd = codes + (((int64_t)b * H + h) * T_cap + t0 + t) * S * G;
        for (int g = 0; g < G; ++g) {
            for (int i = 0; i < d; ++i) {
                float acc = 0.0f;
                for (int s = 0; s < S_use; ++s) {
                    int code = cd[s * G + g];
                    acc = acc + (float)tab[((((int64_t)h * S + s) * G + g) * K + code) * d + i];
                }
                if (out_dtype == TACVQ_F16)
                    ((half_t *)out)[row * D + g * d + i] = (half_t)acc;
                else
                    ((float *)out)[row * D + g * d + i] = acc;
            }
        }
    }
    return 0;
}

/*
 * Decode-step attention over codes.  q[B,Hq,D] fp16 (pre-scaled), codes [B,Hkv,T_cap,S,G],
 * tables fp16 [Hkv,S,G,K,d].  Rows rebuilt as fp16 (as the reference's decoded window holds
 * them), scores and sums in double.  state[B,Hq,2+D] = (m, l, acc[D]) in fp32; out fp16 [B,Hq,D]
 * (either may be NULL).  Empty range: m=-inf, l=0, acc=0, out=0.
 */
int tacvq_oracle_attn(const uint16_t *q_f16, const uint8_t *kcodes, const uint8_t *vcodes, const uint16_t *ktab_f16,
                      const uint16_t *vtab_f16, const int32_t *seq_start, const int32_t *seq_end, float *state,
                      uint16_t *out_f16, int B, int Hq, int Hkv, int D, int G, int S, int K, int64_t T_cap) {
    if (Hkv <= 0 || Hq % Hkv != 0 || G <= 0 || D % G != 0 || D > 512) return -1;
    const int d = D / G, rep = Hq / Hkv;
    const half_t *q = (const half_t *)q_f16;
    const half_t *ktab = (const half_t *)ktab_f16, *vtab = (const half_t *)vtab_f16;
    int status = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv, h = bh % Hkv;
        const int lo = seq_start ? seq_start[b] : 0;
        const int hi = seq_end ? seq_end[b] : (int)T_cap;
        const int n = hi > lo ? hi - lo : 0;
        float *krow = (float *)malloc(sizeof(float) * (size_t)D * 2);
        double *score = (double *)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1) * rep);
        double *acc = (double *)calloc((size_t)rep * D, sizeof(double));
        if (!krow || !score || !acc) {
            status = -2;
            free(krow); free(score); free(acc);
            continue;
        }
        float *vrow = krow + D;
        double m[64], l[64];
        for (int r = 0; r < rep; ++r) { m[r] = -INFINITY; l[r] = 0.0; }
        for (int t = 0; t < n; ++t) {
            const uint8_t *cd = kcodes + (((int64_t)b * Hkv + h) * T_cap + lo + t) * S * G;
            for (int g = 0; g < G; ++g)
                for (int i = 0; i < d; ++i) {
                    float a = 0.0f;
                    for (int s = 0; s < S; ++s)
                        a = a + (float)ktab[((((int64_t)h * S + s) * G + g) * K + cd[s * G + g]) * d + i];
                    krow[g * d + i] = (float)(half_t)a;
                }
            for (int r = 0; r < rep; ++r) {
                const half_t *qr = q + ((int64_t)b * Hq + h * rep + r) * D;
                double sc = 0.0;
                for (int i = 0; i < D; ++i) sc += (double)(float)qr[i] * (double)krow[i];
                score[(size_t)t * rep + r] = sc;
                if (sc > m[r]) m[r] = sc;
            }
        }
        for (int t = 0; t < n; ++t) {
            const uint8_t *cd = vcodes + (((int64_t)b * Hkv + h) * T_cap + lo + t) * S * G;
            for (int g = 0; g < G; ++g)
                for (int i = 0; i < d; ++i) {
                    float a = 0.0f;
                    for (int s = 0; s < S; ++s)
                        a = a + (float)vtab[((((int64_t)h * S + s) * G + g) * K + cd[s * G + g]) * d + i];
                    vrow[g * d + i] = (float)(half_t)a;
                }
            for (int r = 0; r < rep; ++r) {
                double p = exp(score[(size_t)t * rep + r] - m[r]);
                l[r] += p;
                double *ar = acc + (size_t)r * D;
                for (int i = 0; i < D; ++i) ar[i] += p * (double)vrow[i];
            }
        }
        for (int r = 0; r < rep; ++r) {
            const int64_t o = (int64_t)b * Hq + h * rep + r;
            if (state) {
                float *st = state + o * (2 + D);
                st[0] = (float)m[r];
                st[1] = (float)l[r];
                for (int i = 0; i < D; ++i) st[2 + i] = (float)acc[(size_t)r * D + i];
            }
            if (out_f16)
                for (int i = 0; i < D; ++i)
                    ((half_t *)out_f16)[o * D + i] = (half_t)(float)(l[r] > 0.0 ? acc[(size_t)r * D + i] / l[r] : 0.0);
        }
        free(krow); free(score); free(acc);
    }
    return status;
}

/* Merge n_parts states [n_parts,B*Hq,2+D] -> out fp16 [B*Hq,D] and/or merged state [B*Hq,2+D]. */
int tacvq_oracle_merge(const float *states, int n_parts, int64_t rows, int D, float *merged, uint16_t *out_f16) {
    for (int64_t r = 0; r < rows; ++r) {
        double top = -INFINITY;
        for (int p = 0; p < n_parts; ++p) {
            double m = states[((int64_t)p * rows + r) * (2 + D)];
            if (m > top) top = m;
        }
        double l = 0.0;
        double acc[512];
        for (int i = 0; i < D; ++i) acc[i] = 0.0;
        for (int p = 0; p < n_parts; ++p) {
            const float *st = states + ((int64_t)p * rows + r) * (2 + D);
            if (isinf(st[0]) && st[0] < 0) continue;
            double w = exp((double)st[0] - top);
            l += w * st[1];
            for (int i = 0; i < D; ++i) acc[i] += w * st[2 + i];
        }
        if (merged) {
            float *o = merged + r * (2 + D);
            o[0] = (float)top;
            o[1] = (float)l;
            for (int i = 0; i < D; ++i) o[2 + i] = (float)acc[i];
        }
        if (out_f16)
            for (int i = 0; i < D; ++i) ((half_t *)out_f16)[r * D + i] = (half_t)(float)(l > 0.0 ? acc[i] / l : 0.0);
    }
    return 0;
}
