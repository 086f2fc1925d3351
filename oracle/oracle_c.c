/* CPU oracle, C/OpenMP edition (TEST INFRASTRUCTURE ONLY).
 *
 * The same fp32 restatement of the reference kernels' arithmetic as oracle.py,
 * written in C so that it can be timed on host cores as the CPU baseline and
 * used as the checker at sizes numpy would take too long on.  Only the tests,
 * the smoke check and the benchmark's CPU-baseline / reference legs may load it;
 * the shipped library never does.
 *
 * Parity status: the reference (sizzlecar/triton-rs) holds no numeric test,
 * golden vector or runnable build for the int4 GEMMs, attention, RoPE or the
 * kv-cache append -- "parity unpinned" for those; this file follows the kernel
 * sources cited at each function.  The f32 glue is pinned by the inputs and
 * tolerances of crates/triton-runtime/examples/run_rms_norm.rs:34-37,71-87 and
 * run_fused_add_rms_norm.rs:32-34,73-94 (checked in tests/test_oracle.py).
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp, x86-64-v3 so the binary runs on
 * any AVX2 host).  fp16 storage type is _Float16; all arithmetic is float.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

int oc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* torchrun exports OMP_NUM_THREADS=1: callers that want every core say so here. */
void oc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline float r16(float x) { return (float)(f16)x; }

/* nibble position of column j (0..7) inside a packed word.
 * GPTQ qzeros: straight (w4a16_gptq_gemm_typed.rs:155-162).
 * AWQ: order[j] = j/2 + (j%2)*4 (awq_gemm_int4_typed.rs:137-151). */
static inline int awq_slot(int j) { return (j >> 1) + ((j & 1) << 2); }

#define NB 64 /* column block per task */

/* C[m,n] = sum_k A[m,k] * ((q[k,n] - zero[k/G,n]) * s[k/G,n]), fp32 accumulate.
 * GPTQ layout: qweight [K/8,N], nibble i of a word is row 8r+i
 * (w4a16_gptq_gemm_typed.rs:167-173,209-260).  qzeros [K/G,N/8] straight order,
 * effective zero = nibble + zero_offset (:223-236); qzeros == NULL -> zero 8
 * (ferrum_dequant_int4_sym.rs:60).  a is fp32 [M,K] (already widened). */
/* faithful != 0: the dequantised weight is rounded to fp16 before the product, as the
 * reference does ahead of its MMA (w4a16_gptq_gemm_typed.rs:256-260: truncf of the
 * f32 product (q - z) * s); faithful == 0: the product stays in fp32 (the grading oracle). */
void oc_gptq_gemm_ex(const float *a, const int32_t *qweight, const f16 *scales,
                     const int32_t *qzeros, float *c, int M, int N, int K, int G,
                     int zero_offset, int faithful) {
    int nblocks = (N + NB - 1) / NB;
#pragma omp parallel for schedule(dynamic, 1)
    for (int nb = 0; nb < nblocks; ++nb) {
        int n0 = nb * NB, nw = N - n0 < NB ? N - n0 : NB;
        float acc[64][NB];
        float wrow[NB], sc[NB], zf[NB];
        for (int m0 = 0; m0 < M; m0 += 64) {
            int mw = M - m0 < 64 ? M - m0 : 64;
            for (int m = 0; m < mw; ++m)
                for (int j = 0; j < nw; ++j) acc[m][j] = 0.f;
            for (int k = 0; k < K; ++k) {
                if (k % G == 0) {
                    int g = k / G;
                    for (int j = 0; j < nw; ++j) {
                        int n = n0 + j;
                        sc[j] = (float)scales[(size_t)g * N + n];
                        int z = 8;
                        if (qzeros) {
                            uint32_t zw = (uint32_t)qzeros[(size_t)g * (N / 8) + n / 8];
                            z = (int)((zw >> (4 * (n % 8))) & 0xF) + zero_offset;
                        }
                        zf[j] = (float)z;
                    }
                }
                const int32_t *qrow = qweight + (size_t)(k / 8) * N + n0;
                int sh = 4 * (k % 8);
                for (int j = 0; j < nw; ++j) {
                    int q = (int)(((uint32_t)qrow[j] >> sh) & 0xF);
                    wrow[j] = ((float)q - zf[j]) * sc[j];
                }
                if (faithful)
                    for (int j = 0; j < nw; ++j) wrow[j] = r16(wrow[j]);
                for (int m = 0; m < mw; ++m) {
                    float av = a[(size_t)(m0 + m) * K + k];
                    for (int j = 0; j < nw; ++j) acc[m][j] += av * wrow[j];
                }
            }
            for (int m = 0; m < mw; ++m)
                for (int j = 0; j < nw; ++j) c[(size_t)(m0 + m) * N + n0 + j] = acc[m][j];
        }
    }
}

void oc_gptq_gemm(const float *a, const int32_t *qweight, const f16 *scales,
                  const int32_t *qzeros, float *c, int M, int N, int K, int G,
                  int zero_offset) {
    oc_gptq_gemm_ex(a, qweight, scales, qzeros, c, M, N, K, G, zero_offset, 0);
}

/* AWQ layout: qweight [K,N/8], qzeros [K/G,N/8], both with the AWQ nibble order,
 * no +1 on zeros (awq_gemm_int4_typed.rs:137-151,183-222).  `faithful` as above
 * (awq_gemm_int4_typed.rs:222-227 rounds the dequantised tile to T the same way). */
void oc_awq_gemm_ex(const float *a, const int32_t *qweight, const f16 *scales,
                    const int32_t *qzeros, float *c, int M, int N, int K, int G, int faithful) {
    int nblocks = (N + NB - 1) / NB;
#pragma omp parallel for schedule(dynamic, 1)
    for (int nb = 0; nb < nblocks; ++nb) {
        int n0 = nb * NB, nw = N - n0 < NB ? N - n0 : NB;
        float acc[64][NB];
        float wrow[NB], sc[NB], zf[NB];
        for (int m0 = 0; m0 < M; m0 += 64) {
            int mw = M - m0 < 64 ? M - m0 : 64;
            for (int m = 0; m < mw; ++m)
                for (int j = 0; j < nw; ++j) acc[m][j] = 0.f;
            for (int k = 0; k < K; ++k) {
                if (k % G == 0) {
                    int g = k / G;
                    for (int j = 0; j < nw; ++j) {
                        int n = n0 + j;
                        sc[j] = (float)scales[(size_t)g * N + n];
                        uint32_t zw = (uint32_t)qzeros[(size_t)g * (N / 8) + n / 8];
                        zf[j] = (float)((zw >> (4 * awq_slot(n % 8))) & 0xF);
                    }
                }
                const int32_t *qrow = qweight + (size_t)k * (N / 8);
                for (int j = 0; j < nw; ++j) {
                    int n = n0 + j;
                    int q = (int)(((uint32_t)qrow[n / 8] >> (4 * awq_slot(n % 8))) & 0xF);
                    wrow[j] = ((float)q - zf[j]) * sc[j];
                }
                if (faithful)
                    for (int j = 0; j < nw; ++j) wrow[j] = r16(wrow[j]);
                for (int m = 0; m < mw; ++m) {
                    float av = a[(size_t)(m0 + m) * K + k];
                    for (int j = 0; j < nw; ++j) acc[m][j] += av * wrow[j];
                }
            }
            for (int m = 0; m < mw; ++m)
                for (int j = 0; j < nw; ++j) c[(size_t)(m0 + m) * N + n0 + j] = acc[m][j];
        }
    }
}

void oc_awq_gemm(const float *a, const int32_t *qweight, const f16 *scales,
                 const int32_t *qzeros, float *c, int M, int N, int K, int G) {
    oc_awq_gemm_ex(a, qweight, scales, qzeros, c, M, N, K, G, 0);
}

void oc_f16_to_f32(const f16 *x, float *y, size_t n) {
#pragma omp parallel for
    for (size_t i = 0; i < n; ++i) y[i] = (float)x[i];
}

void oc_round_f16(float *x, size_t n) {
#pragma omp parallel for
    for (size_t i = 0; i < n; ++i) x[i] = r16(x[i]);
}

/* Batched GQA decode attention over a head-major cache [B,Hkv,max_len,D] with
 * per-sequence lengths: online softmax with m=-1e30, l=0 start, tile by tile
 * (attention.rs:198-272 for the head-major addressing and the tile loop;
 * :287-289 names per-sequence lengths as the follow-up).  q fp32 [B,Hq,D]. */
void oc_batched_decode_attention_hm(const float *q, const f16 *kc, const f16 *vc,
                                    const int32_t *lens, float *out, int B, int Hq,
                                    int Hkv, int D, int max_len, float scale) {
    int grp = Hq / Hkv;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < Hq; ++h) {
            int kvh = h / grp;
            const f16 *kb = kc + ((size_t)b * Hkv + kvh) * (size_t)max_len * D;
            const f16 *vb = vc + ((size_t)b * Hkv + kvh) * (size_t)max_len * D;
            const float *qv = q + ((size_t)b * Hq + h) * D;
            float *o = out + ((size_t)b * Hq + h) * D;
            float acc[512];
            for (int d = 0; d < D; ++d) acc[d] = 0.f;
            float m = -1e30f, l = 0.f;
            int len = lens[b];
            enum { T = 64 };
            float s[T];
            for (int p0 = 0; p0 < len; p0 += T) {
                int tw = len - p0 < T ? len - p0 : T;
                float tmax = -1e30f;
                for (int t = 0; t < tw; ++t) {
                    const f16 *kr = kb + (size_t)(p0 + t) * D;
                    float dot = 0.f;
                    for (int d = 0; d < D; ++d) dot += qv[d] * (float)kr[d];
                    s[t] = dot * scale;
                    if (s[t] > tmax) tmax = s[t];
                }
                float mn = m > tmax ? m : tmax;
                float alpha = expf(m - mn);
                for (int d = 0; d < D; ++d) acc[d] *= alpha;
                l *= alpha;
                for (int t = 0; t < tw; ++t) {
                    float p = expf(s[t] - mn);
                    l += p;
                    const f16 *vr = vb + (size_t)(p0 + t) * D;
                    for (int d = 0; d < D; ++d) acc[d] += p * (float)vr[d];
                }
                m = mn;
            }
            for (int d = 0; d < D; ++d) o[d] = acc[d] / l;
        }
}

/* y = x * rsqrt(mean(x^2)+eps) * w (norms.rs:16-41). */
void oc_rms_norm(const float *x, const f16 *w, float *y, int rows, int n, float eps) {
#pragma omp parallel for
    for (int r = 0; r < rows; ++r) {
        const float *xr = x + (size_t)r * n;
        float ss = 0.f;
        for (int i = 0; i < n; ++i) ss += xr[i] * xr[i];
        float inv = 1.0f / sqrtf(ss * (1.0f / (float)n) + eps);
        for (int i = 0; i < n; ++i) y[(size_t)r * n + i] = xr[i] * inv * (float)w[i];
    }
}

/* out[b,i] = silu(g)*u, gate = first `inter` of the row, up = second
 * (elementwise.rs:188-212). */
void oc_silu_mul_interleaved(const float *gu, float *out, int rows, int inter) {
#pragma omp parallel for
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < inter; ++i) {
            float g = gu[(size_t)r * 2 * inter + i];
            float u = gu[(size_t)r * 2 * inter + inter + i];
            out[(size_t)r * inter + i] = g / (expf(-g) + 1.0f) * u;
        }
}

/* half-split pairs (i, i+D/2), per-token position (positional.rs:94-129). In place. */
void oc_rope_full(float *x, const float *cos_t, const float *sin_t, const int32_t *pos,
                  int tokens, int heads, int D) {
    int half = D / 2;
#pragma omp parallel for
    for (int t = 0; t < tokens; ++t)
        for (int h = 0; h < heads; ++h) {
            float *v = x + ((size_t)t * heads + h) * D;
            const float *c = cos_t + (size_t)pos[t] * half;
            const float *s = sin_t + (size_t)pos[t] * half;
            for (int i = 0; i < half; ++i) {
                float x0 = v[i], x1 = v[i + half];
                v[i] = x0 * c[i] - x1 * s[i];
                v[i + half] = x1 * c[i] + x0 * s[i];
            }
        }
}

/* One Llama-shape decode layer on hidden [B,H] (fp16 in, fp32 out), every
 * intermediate the CUDA path stores as fp16 rounded at that point.  Weights are
 * GPTQ (qweight, scales, qzeros) for qkv, o, gate_up, down.  Caches head-major
 * [B,Hkv,max_len,D], appended at pos[b]; attention over pos[b]+1 entries.
 *
 * faithful != 0 reproduces the reference's extra roundings: the dequantised weight
 * rounded to fp16 before the product (w4a16_gptq_gemm_typed.rs:256-260) and the second
 * norm computed from the unrounded fp32 sum x + o while residual_out is that sum
 * rounded to fp16 (norms.rs:208-219).  faithful == 0 keeps the weight product in fp32
 * and norms the rounded residual.
 *
 * stages, when not NULL, is an array of 10 pointers (each may be NULL) that receive the
 * fp16-rounded intermediates as fp32: n1 [B,H], qkv [B,(Hq+2Hkv)D], q after RoPE
 * [B,Hq,D], attention out [B,Hq,D], o [B,H], h1 [B,H], n2 [B,H], gate_up [B,2I],
 * act [B,I], down [B,H]. */
void oc_decode_layer_ex(const f16 *hidden, float *out, int B, int H, int Hq, int Hkv, int D,
                        int I, int G, int zero_offset, float eps, const f16 *ln1,
                        const f16 *ln2, const int32_t *qkv_qw, const f16 *qkv_sc,
                        const int32_t *qkv_qz, const int32_t *o_qw, const f16 *o_sc,
                        const int32_t *o_qz, const int32_t *gu_qw, const f16 *gu_sc,
                        const int32_t *gu_qz, const int32_t *dn_qw, const f16 *dn_sc,
                        const int32_t *dn_qz, const float *cos_t, const float *sin_t,
                        const int32_t *pos, f16 *kc, f16 *vc, int max_len, int faithful,
                        float *const *stages) {
    int NQKV = (Hq + 2 * Hkv) * D;
    size_t bh = (size_t)B * H;
    float *x = malloc(bh * 4), *n1 = malloc(bh * 4), *qkv = malloc((size_t)B * NQKV * 4);
    float *q = malloc((size_t)B * Hq * D * 4), *k = malloc((size_t)B * Hkv * D * 4);
    float *att = malloc((size_t)B * Hq * D * 4), *o = malloc(bh * 4), *h1 = malloc(bh * 4);
    float *gu = malloc((size_t)B * 2 * I * 4), *act = malloc((size_t)B * I * 4);
    float *dn = malloc(bh * 4), *sum = malloc(bh * 4);
    int32_t *lens = malloc((size_t)B * 4);
#define OC_STAGE(i, src, n) \
    if (stages && stages[i]) memcpy(stages[i], src, (size_t)(n) * 4)
    oc_f16_to_f32(hidden, x, bh);
    oc_rms_norm(x, ln1, n1, B, H, eps);
    oc_round_f16(n1, bh);
    OC_STAGE(0, n1, bh);
    oc_gptq_gemm_ex(n1, qkv_qw, qkv_sc, qkv_qz, qkv, B, NQKV, H, G, zero_offset, faithful);
    oc_round_f16(qkv, (size_t)B * NQKV);
    OC_STAGE(1, qkv, (size_t)B * NQKV);
    for (int b = 0; b < B; ++b) {
        memcpy(q + (size_t)b * Hq * D, qkv + (size_t)b * NQKV, (size_t)Hq * D * 4);
        memcpy(k + (size_t)b * Hkv * D, qkv + (size_t)b * NQKV + Hq * D, (size_t)Hkv * D * 4);
    }
    oc_rope_full(q, cos_t, sin_t, pos, B, Hq, D);
    oc_rope_full(k, cos_t, sin_t, pos, B, Hkv, D);
    oc_round_f16(q, (size_t)B * Hq * D);
    OC_STAGE(2, q, (size_t)B * Hq * D);
    for (int b = 0; b < B; ++b) {
        lens[b] = pos[b] + 1;
        for (int h = 0; h < Hkv; ++h) {
            f16 *kd = kc + (((size_t)b * Hkv + h) * max_len + pos[b]) * D;
            f16 *vd = vc + (((size_t)b * Hkv + h) * max_len + pos[b]) * D;
            const float *vs = qkv + (size_t)b * NQKV + (Hq + Hkv) * D + h * D;
            for (int d = 0; d < D; ++d) {
                kd[d] = (f16)k[((size_t)b * Hkv + h) * D + d];
                vd[d] = (f16)vs[d];
            }
        }
    }
    oc_batched_decode_attention_hm(q, kc, vc, lens, att, B, Hq, Hkv, D, max_len,
                                   1.0f / sqrtf((float)D));
    oc_round_f16(att, (size_t)B * Hq * D);
    OC_STAGE(3, att, (size_t)B * Hq * D);
    oc_gptq_gemm_ex(att, o_qw, o_sc, o_qz, o, B, H, Hq * D, G, zero_offset, faithful);
    oc_round_f16(o, bh);
    OC_STAGE(4, o, bh);
    for (size_t i = 0; i < bh; ++i) {
        sum[i] = x[i] + o[i];
        h1[i] = r16(sum[i]);
    }
    OC_STAGE(5, h1, bh);
    oc_rms_norm(faithful ? sum : h1, ln2, n1, B, H, eps);
    oc_round_f16(n1, bh);
    OC_STAGE(6, n1, bh);
    oc_gptq_gemm_ex(n1, gu_qw, gu_sc, gu_qz, gu, B, 2 * I, H, G, zero_offset, faithful);
    oc_round_f16(gu, (size_t)B * 2 * I);
    OC_STAGE(7, gu, (size_t)B * 2 * I);
    oc_silu_mul_interleaved(gu, act, B, I);
    oc_round_f16(act, (size_t)B * I);
    OC_STAGE(8, act, (size_t)B * I);
    oc_gptq_gemm_ex(act, dn_qw, dn_sc, dn_qz, dn, B, H, I, G, zero_offset, faithful);
    oc_round_f16(dn, bh);
    OC_STAGE(9, dn, bh);
#undef OC_STAGE
    for (size_t i = 0; i < bh; ++i) out[i] = h1[i] + dn[i];
    free(x); free(n1); free(qkv); free(q); free(k); free(att); free(o); free(h1);
    free(gu); free(act); free(dn); free(sum); free(lens);
}

/* The reference-faithful chain (the one every layer-level comparison uses). */
void oc_decode_layer(const f16 *hidden, float *out, int B, int H, int Hq, int Hkv, int D,
                     int I, int G, int zero_offset, float eps, const f16 *ln1,
                     const f16 *ln2, const int32_t *qkv_qw, const f16 *qkv_sc,
                     const int32_t *qkv_qz, const int32_t *o_qw, const f16 *o_sc,
                     const int32_t *o_qz, const int32_t *gu_qw, const f16 *gu_sc,
                     const int32_t *gu_qz, const int32_t *dn_qw, const f16 *dn_sc,
                     const int32_t *dn_qz, const float *cos_t, const float *sin_t,
                     const int32_t *pos, f16 *kc, f16 *vc, int max_len) {
    oc_decode_layer_ex(hidden, out, B, H, Hq, Hkv, D, I, G, zero_offset, eps, ln1, ln2, qkv_qw,
                       qkv_sc, qkv_qz, o_qw, o_sc, o_qz, gu_qw, gu_sc, gu_qz, dn_qw, dn_sc, dn_qz,
                       cos_t, sin_t, pos, kc, vc, max_len, 1, NULL);
}

/* Fused MoE as the benchmark's config 3 specifies it (the reference has no MoE kernel; the parts
 * follow its conventions: GPTQ layout with the symmetric zero-point 8 of
 * ferrum_dequant_int4_sym.rs:60, gate|up half-split rows of elementwise.rs:199-206).
 * Routing: top-k by logit, ties to the lowest expert index; weights exp(x - max) renormalised
 * over the chosen k (softmax's denominator cancels).  x [T,H] fp16, logits [T,E] fp32,
 * w13 [E,H/8,2I] + scales [E,H/G,2I], w2 [E,I/8,H] + scales [E,I/G,H]; out [T,H] fp32 =
 * sum_j w[t,j] * (silu(g) * u) W2_e, the intermediate rounded to fp16 between the GEMMs.
 * topk_ids_out [T,k] / topk_w_out [T,k] / mag_out [T,H] may be NULL; mag_out receives
 * sum_j |w[t,j] * y_j|, the magnitude of the summands behind every output element. */
void oc_fused_moe_gptq(const f16 *x, const float *logits, const int32_t *w13_q, const f16 *w13_s,
                       const int32_t *w2_q, const f16 *w2_s, float *out, int T, int H, int E,
                       int top_k, int I, int G, int faithful, int32_t *topk_ids_out,
                       float *topk_w_out, float *mag_out) {
    int32_t *ids = malloc((size_t)T * top_k * 4);
    float *wts = malloc((size_t)T * top_k * 4);
    for (int t = 0; t < T; ++t) {
        const float *l = logits + (size_t)t * E;
        float mx = l[0];
        for (int e = 1; e < E; ++e) mx = l[e] > mx ? l[e] : mx;
        float sum = 0.f;
        for (int j = 0; j < top_k; ++j) {
            int best = -1;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int jj = 0; jj < j; ++jj) taken |= ids[(size_t)t * top_k + jj] == e;
                if (!taken && (best < 0 || l[e] > l[best])) best = e;
            }
            ids[(size_t)t * top_k + j] = best;
            wts[(size_t)t * top_k + j] = expf(l[best] - mx);
            sum += wts[(size_t)t * top_k + j];
        }
        for (int j = 0; j < top_k; ++j) wts[(size_t)t * top_k + j] /= sum;
    }
    if (topk_ids_out) memcpy(topk_ids_out, ids, (size_t)T * top_k * 4);
    if (topk_w_out) memcpy(topk_w_out, wts, (size_t)T * top_k * 4);
    memset(out, 0, (size_t)T * H * 4);
    if (mag_out) memset(mag_out, 0, (size_t)T * H * 4);
    int *rows = malloc((size_t)T * top_k * sizeof(int));
    float *xa = malloc((size_t)T * H * 4), *gu = malloc((size_t)T * 2 * I * 4);
    float *act = malloc((size_t)T * I * 4), *y = malloc((size_t)T * H * 4);
    for (int e = 0; e < E; ++e) {
        int cnt = 0;
        for (int p = 0; p < T * top_k; ++p)
            if (ids[p] == e) rows[cnt++] = p;   /* pair order = token order (stable) */
        if (!cnt) continue;
        for (int r = 0; r < cnt; ++r)
            oc_f16_to_f32(x + (size_t)(rows[r] / top_k) * H, xa + (size_t)r * H, H);
        oc_gptq_gemm_ex(xa, w13_q + (size_t)e * (H / 8) * 2 * I, w13_s + (size_t)e * (H / G) * 2 * I, NULL,
                        gu, cnt, 2 * I, H, G, 0, faithful);
        oc_silu_mul_interleaved(gu, act, cnt, I);
        oc_round_f16(act, (size_t)cnt * I);
        oc_gptq_gemm_ex(act, w2_q + (size_t)e * (I / 8) * H, w2_s + (size_t)e * (I / G) * H, NULL, y, cnt,
                        H, I, G, 0, faithful);
        for (int r = 0; r < cnt; ++r) {
            float w = wts[rows[r]];
            float *o = out + (size_t)(rows[r] / top_k) * H;
            for (int i = 0; i < H; ++i) o[i] += w * y[(size_t)r * H + i];
            if (mag_out) {
                float *mg = mag_out + (size_t)(rows[r] / top_k) * H;
                for (int i = 0; i < H; ++i) mg[i] += fabsf(w * y[(size_t)r * H + i]);
            }
        }
    }
    free(ids); free(wts); free(rows); free(xa); free(gu); free(act); free(y);
}
