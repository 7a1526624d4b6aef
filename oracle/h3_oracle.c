/* CPU oracle for the MiniMax-H3 DiT denoiser forward: see h3_oracle.h.
 *
 * TEST INFRASTRUCTURE ONLY; never part of the shipped compute path.
 *
 * Build: gcc -O3 -mavx2 -mfma -ffp-contract=off -fopenmp -shared -fPIC
 * (-ffp-contract=off keeps `a*b+c` as two roundings wherever the reference's
 * CPU test references write it that way; explicit fmaf() stays fused).
 */
#include "h3_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

void h3o_set_threads(int count) {
#ifdef _OPENMP
    if (count > 0) omp_set_num_threads(count);
#else
    (void)count;
#endif
}

int h3o_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ bf16 */

float h3o_bf16_to_f32(uint16_t value) {
    uint32_t bits = (uint32_t)value << 16;
    float result;
    memcpy(&result, &bits, sizeof(result));
    return result;
}

uint16_t h3o_f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

static inline float widen(uint16_t v) { return h3o_bf16_to_f32(v); }
static inline uint16_t narrow(float v) { return h3o_f32_to_bf16(v); }
static inline float bf_round(float v) { return widen(narrow(v)); }

void h3o_widen(float *out, const uint16_t *in, size_t count) {
    for (size_t i = 0; i < count; i++) out[i] = widen(in[i]);
}

void h3o_narrow(uint16_t *out, const float *in, size_t count) {
    for (size_t i = 0; i < count; i++) out[i] = narrow(in[i]);
}

/* ------------------------------------------------------------------- rng */

uint32_t h3o_rng_u32(h3o_rng *rng) {
    uint64_t old = rng->state;
    rng->state = old * UINT64_C(6364136223846793005) + rng->increment;
    uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
    uint32_t rot = (uint32_t)(old >> 59u);
    return (xorshifted >> rot) | (xorshifted << ((32u - rot) & 31u));
}

void h3o_rng_seed(h3o_rng *rng, uint64_t seed) {
    rng->state = 0;
    rng->spare = 0.0f;
    rng->has_spare = 0;
    rng->increment = (seed << 1u) | 1u;
    (void)h3o_rng_u32(rng);
    rng->state += seed ^ UINT64_C(0x9e3779b97f4a7c15);
    (void)h3o_rng_u32(rng);
}

float h3o_rng_normal(h3o_rng *rng) {
    if (rng->has_spare) {
        rng->has_spare = 0;
        return rng->spare;
    }
    double u1 = ((double)h3o_rng_u32(rng) + 1.0) / 4294967297.0;
    double u2 = ((double)h3o_rng_u32(rng) + 0.5) / 4294967296.0;
    double radius = sqrt(-2.0 * log(u1));
    double angle = 2.0 * 3.14159265358979323846 * u2;
    rng->spare = (float)(radius * sin(angle));
    rng->has_spare = 1;
    return (float)(radius * cos(angle));
}

void h3o_fill_normal_f32(float *values, size_t count, uint64_t seed,
                         float mean, float std) {
    h3o_rng rng;
    h3o_rng_seed(&rng, seed);
    for (size_t i = 0; i < count; i++)
        values[i] = mean + std * h3o_rng_normal(&rng);
}

void h3o_fill_normal_bf16(uint16_t *values, size_t count, uint64_t seed,
                          float mean, float std) {
    h3o_rng rng;
    h3o_rng_seed(&rng, seed);
    for (size_t i = 0; i < count; i++)
        values[i] = narrow(mean + std * h3o_rng_normal(&rng));
}

uint64_t h3o_named_seed(uint64_t seed, const char *name) {
    uint64_t hash = UINT64_C(0xcbf29ce484222325);
    for (const unsigned char *p = (const unsigned char *)name; *p; p++) {
        hash ^= *p;
        hash *= UINT64_C(0x100000001b3);
    }
    return seed ^ hash;
}

/* ---------------------------------------------------------------- linear */

/* out[r][c] = bias[c] then fmaf over k in increasing order: the summation
 * order of ref_linear_f32 and of the reference's one-thread-per-output hand
 * kernel. Vectorised across a block of rows so every output keeps its own
 * sequential chain. */
#define RB 32
#define CB 64
static void gemm_rows_seq(float *out, size_t out_stride, const float *x_f32,
                          const uint16_t *x_bf16, size_t x_stride,
                          const float *w_f32, const uint16_t *w_bf16,
                          const float *bias, uint32_t rows, uint32_t in_dim,
                          uint32_t out_dim) {
    if (!rows || !out_dim) return;
    uint32_t row_blocks = (rows + RB - 1) / RB;
    uint32_t col_blocks = (out_dim + CB - 1) / CB;
    long tasks = (long)row_blocks * col_blocks;
#pragma omp parallel
    {
        float *xt = (float *)aligned_alloc(64, (size_t)(in_dim ? in_dim : 1) *
                                                   RB * sizeof(float));
        long cached_rb = -1;
        /* consecutive tasks share a row block, so each thread transposes it rarely */
#pragma omp for schedule(dynamic, 4)
        for (long task = 0; task < tasks; task++) {
            uint32_t rb = (uint32_t)(task / col_blocks);
            uint32_t cb = (uint32_t)(task % col_blocks);
            uint32_t r0 = rb * RB;
            uint32_t live = rows - r0 < RB ? rows - r0 : RB;
            if (cached_rb != (long)rb) {
                for (uint32_t k = 0; k < in_dim; k++)
                    for (uint32_t i = 0; i < RB; i++) {
                        float v = 0.0f;
                        if (i < live) {
                            size_t idx = (size_t)(r0 + i) * x_stride + k;
                            v = x_f32 ? x_f32[idx] : widen(x_bf16[idx]);
                        }
                        xt[(size_t)k * RB + i] = v;
                    }
                cached_rb = rb;
            }
            uint32_t c_end = (cb + 1) * CB < out_dim ? (cb + 1) * CB : out_dim;
            for (uint32_t c = cb * CB; c < c_end; c++) {
                float acc[RB];
                float start = bias ? bias[c] : 0.0f;
                for (uint32_t i = 0; i < RB; i++) acc[i] = start;
                if (w_f32) {
                    const float *w = w_f32 + (size_t)c * in_dim;
                    for (uint32_t k = 0; k < in_dim; k++) {
                        float wk = w[k];
                        const float *col = xt + (size_t)k * RB;
#pragma omp simd
                        for (uint32_t i = 0; i < RB; i++)
                            acc[i] = fmaf(col[i], wk, acc[i]);
                    }
                } else {
                    const uint16_t *w = w_bf16 + (size_t)c * in_dim;
                    for (uint32_t k = 0; k < in_dim; k++) {
                        float wk = widen(w[k]);
                        const float *col = xt + (size_t)k * RB;
#pragma omp simd
                        for (uint32_t i = 0; i < RB; i++)
                            acc[i] = fmaf(col[i], wk, acc[i]);
                    }
                }
                for (uint32_t i = 0; i < live; i++)
                    out[(size_t)(r0 + i) * out_stride + c] = acc[i];
            }
        }
        free(xt);
    }
}

void h3o_linear_f32(float *out, const float *in, const float *weight,
                    const float *bias, uint32_t rows, uint32_t in_dim,
                    uint32_t out_dim) {
    gemm_rows_seq(out, out_dim, in, NULL, in_dim, weight, NULL, bias, rows,
                  in_dim, out_dim);
}

void h3o_linear_bf16(uint16_t *out, const uint16_t *in, const uint16_t *weight,
                     const uint16_t *bias, uint32_t rows, uint32_t in_dim,
                     uint32_t out_dim) {
    size_t count = (size_t)rows * out_dim;
    if (!count) return;
    float *acc = (float *)malloc(count * sizeof(float));
    float *fbias = NULL;
    if (bias) {
        fbias = (float *)malloc((size_t)out_dim * sizeof(float));
        h3o_widen(fbias, bias, out_dim);
    }
    gemm_rows_seq(acc, out_dim, NULL, in, in_dim, NULL, weight, fbias, rows,
                  in_dim, out_dim);
#pragma omp parallel for
    for (size_t i = 0; i < count; i++) out[i] = narrow(acc[i]);
    free(acc);
    free(fbias);
}

/* ----------------------------------------------------------- elementwise */

static inline float silu(float x) { return x / (1.0f + expf(-x)); }

void h3o_silu_f32(float *out, const float *in, size_t count) {
    for (size_t i = 0; i < count; i++) out[i] = silu(in[i]);
}

void h3o_silu_bf16(uint16_t *out, const uint16_t *in, size_t count) {
    for (size_t i = 0; i < count; i++) out[i] = narrow(silu(widen(in[i])));
}

void h3o_add_bf16(uint16_t *out, const uint16_t *a, const uint16_t *b,
                  size_t count) {
    for (size_t i = 0; i < count; i++)
        out[i] = narrow(widen(a[i]) + widen(b[i]));
}

void h3o_sub_bf16(uint16_t *out, const uint16_t *a, const uint16_t *b,
                  size_t count) {
    for (size_t i = 0; i < count; i++)
        out[i] = narrow(widen(a[i]) - widen(b[i]));
}

void h3o_swiglu_bf16(uint16_t *out, const uint16_t *fused, uint32_t rows,
                     uint32_t width) {
#pragma omp parallel for
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < width; c++) {
            float gate = widen(fused[(size_t)r * width * 2 + c]);
            float up = widen(fused[(size_t)r * width * 2 + width + c]);
            out[(size_t)r * width + c] = narrow(silu(gate) * up);
        }
}

void h3o_mlp_bf16(uint16_t *out, const uint16_t *in, const uint16_t *fc1,
                  const uint16_t *fc2, uint32_t rows, uint32_t in_dim,
                  uint32_t hidden, uint32_t out_dim) {
    uint16_t *fused = (uint16_t *)malloc((size_t)rows * hidden * 2 * 2 + 2);
    uint16_t *act = (uint16_t *)malloc((size_t)rows * hidden * 2 + 2);
    h3o_linear_bf16(fused, in, fc1, NULL, rows, in_dim, hidden * 2);
    h3o_swiglu_bf16(act, fused, rows, hidden);
    h3o_linear_bf16(out, act, fc2, NULL, rows, hidden, out_dim);
    free(fused);
    free(act);
}

/* ---------------------------------------------------------------- adaLN */

void h3o_adaln_f32(float *out, const float *in, const float *norm,
                   const float *modulation, const uint32_t *row_map,
                   uint32_t rows, uint32_t width, uint32_t slots,
                   uint32_t shift_slot, uint32_t scale_slot, float eps) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *x = in + (size_t)r * width;
        float ss = 0.0f;
        for (uint32_t c = 0; c < width; c++) ss += x[c] * x[c];
        float inv = 1.0f / sqrtf(ss / (float)width + eps);
        size_t base = (size_t)row_map[r] * slots * width;
        for (uint32_t c = 0; c < width; c++) {
            float normalized = x[c] * inv * norm[c];
            float shift = modulation[base + (size_t)shift_slot * width + c];
            float scale = modulation[base + (size_t)scale_slot * width + c];
            out[(size_t)r * width + c] = normalized * (1.0f + scale) + shift;
        }
    }
}

static float row_inverse_rms(const uint16_t *x, uint32_t width, float eps) {
    float ss = 0.0f;
    for (uint32_t c = 0; c < width; c++) {
        float v = widen(x[c]);
        ss += v * v;
    }
    return 1.0f / sqrtf(ss / (float)width + eps);
}

static void adaln_row(uint16_t *out, const uint16_t *x, float inv,
                      const uint16_t *norm, const uint16_t *shift,
                      const uint16_t *scale, uint32_t width) {
    for (uint32_t c = 0; c < width; c++) {
        float normalized = widen(x[c]) * inv * widen(norm[c]);
        out[c] = narrow(normalized * (1.0f + widen(scale[c])) + widen(shift[c]));
    }
}

void h3o_adaln_bf16(uint16_t *out, const uint16_t *in, const uint16_t *norm,
                    const uint16_t *modulation, const uint32_t *row_map,
                    uint32_t rows, uint32_t width, uint32_t slots,
                    uint32_t shift_slot, uint32_t scale_slot, float eps) {
#pragma omp parallel for
    for (uint32_t r = 0; r < rows; r++) {
        const uint16_t *x = in + (size_t)r * width;
        float inv = row_inverse_rms(x, width, eps);
        size_t base = (size_t)row_map[r] * slots * width;
        adaln_row(out + (size_t)r * width, x, inv, norm,
                  modulation + base + (size_t)shift_slot * width,
                  modulation + base + (size_t)scale_slot * width, width);
    }
}

void h3o_rms_norm_bf16(uint16_t *out, const uint16_t *in, const uint16_t *norm,
                       uint32_t rows, uint32_t width, float eps) {
#pragma omp parallel for
    for (uint32_t r = 0; r < rows; r++) {
        const uint16_t *x = in + (size_t)r * width;
        float inv = row_inverse_rms(x, width, eps);
        for (uint32_t c = 0; c < width; c++) {
            float normalized = widen(x[c]) * inv;
            out[(size_t)r * width + c] = narrow(normalized * widen(norm[c]));
        }
    }
}

void h3o_gate_f32(float *out, const float *residual, const float *branch,
                  const float *modulation, const uint32_t *row_map,
                  uint32_t rows, uint32_t width, uint32_t slots,
                  uint32_t gate_slot) {
    for (uint32_t r = 0; r < rows; r++) {
        size_t base = (size_t)row_map[r] * slots * width;
        for (uint32_t c = 0; c < width; c++) {
            float gate = modulation[base + (size_t)gate_slot * width + c];
            size_t i = (size_t)r * width + c;
            out[i] = residual[i] + branch[i] * gate;
        }
    }
}

void h3o_gate_bf16(uint16_t *out, const uint16_t *residual,
                   const uint16_t *branch, const uint16_t *modulation,
                   const uint32_t *row_map, uint32_t rows, uint32_t width,
                   uint32_t slots, uint32_t gate_slot) {
#pragma omp parallel for
    for (uint32_t r = 0; r < rows; r++) {
        size_t base = (size_t)row_map[r] * slots * width;
        for (uint32_t c = 0; c < width; c++) {
            float gate = widen(modulation[base + (size_t)gate_slot * width + c]);
            size_t i = (size_t)r * width + c;
            out[i] = narrow(widen(residual[i]) + widen(branch[i]) * gate);
        }
    }
}

void h3o_gate_adaln_bf16(uint16_t *gated, uint16_t *out,
                         const uint16_t *residual, const uint16_t *branch,
                         const uint16_t *norm, const uint16_t *gate_modulation,
                         const uint16_t *norm_modulation,
                         const uint32_t *row_map, uint32_t rows,
                         uint32_t width, uint32_t slots, uint32_t gate_slot,
                         uint32_t shift_slot, uint32_t scale_slot, float eps) {
#pragma omp parallel
    {
        uint16_t *row = (uint16_t *)malloc((size_t)width * sizeof(uint16_t) + 2);
#pragma omp for
        for (uint32_t r = 0; r < rows; r++) {
            size_t base = (size_t)row_map[r] * slots * width;
            for (uint32_t c = 0; c < width; c++) {
                float gate = widen(
                    gate_modulation[base + (size_t)gate_slot * width + c]);
                size_t i = (size_t)r * width + c;
                row[c] = narrow(widen(residual[i]) + widen(branch[i]) * gate);
            }
            float inv = row_inverse_rms(row, width, eps);
            memcpy(gated + (size_t)r * width, row,
                   (size_t)width * sizeof(uint16_t));
            adaln_row(out + (size_t)r * width, row, inv, norm,
                      norm_modulation + base + (size_t)shift_slot * width,
                      norm_modulation + base + (size_t)scale_slot * width,
                      width);
        }
        free(row);
    }
}

void h3o_adaln_linear_bf16(uint16_t *out, float *inverse, const uint16_t *in,
                           const uint16_t *norm, const uint16_t *modulation,
                           const uint32_t *row_map, const uint16_t *weight,
                           const uint16_t *bias, uint32_t rows, uint32_t width,
                           uint32_t out_dim, uint32_t slots,
                           uint32_t shift_slot, uint32_t scale_slot,
                           float eps) {
    uint16_t *normed = (uint16_t *)malloc((size_t)rows * width * 2 + 2);
    for (uint32_t r = 0; r < rows; r++) {
        const uint16_t *x = in + (size_t)r * width;
        float inv = row_inverse_rms(x, width, eps);
        if (inverse) inverse[r] = inv;
        size_t base = (size_t)row_map[r] * slots * width;
        adaln_row(normed + (size_t)r * width, x, inv, norm,
                  modulation + base + (size_t)shift_slot * width,
                  modulation + base + (size_t)scale_slot * width, width);
    }
    h3o_linear_bf16(out, normed, weight, bias, rows, width, out_dim);
    free(normed);
}

/* ------------------------------------------------------------- attention */

void h3o_qkv_rope_bf16(uint16_t *q, uint16_t *k, uint16_t *v,
                       const uint16_t *qkv, const uint16_t *q_norm,
                       const uint16_t *k_norm, const uint16_t *rope_cos,
                       const uint16_t *rope_sin, uint32_t seq, uint32_t heads,
                       uint32_t hd, uint32_t rope_half, int grouped,
                       float eps) {
    size_t inner = (size_t)heads * hd;
#pragma omp parallel for
    for (uint32_t row = 0; row < seq; row++)
        for (uint32_t head = 0; head < heads; head++) {
            size_t row_base = (size_t)row * inner * 3;
            size_t qb, kb, vb;
            if (grouped) {
                qb = row_base + (size_t)head * hd * 3;
                kb = qb + hd;
                vb = kb + hd;
            } else {
                qb = row_base + (size_t)head * hd;
                kb = qb + inner;
                vb = qb + inner * 2;
            }
            float qs = 0.0f, ks = 0.0f;
            for (uint32_t d = 0; d < hd; d++) {
                float qv = widen(qkv[qb + d]), kv = widen(qkv[kb + d]);
                qs = fmaf(qv, qv, qs);
                ks = fmaf(kv, kv, ks);
            }
            float qi = 1.0f / sqrtf(qs / (float)hd + eps);
            float ki = 1.0f / sqrtf(ks / (float)hd + eps);
            for (uint32_t d = 0; d < hd; d++) {
                float q0 = widen(qkv[qb + d]) * qi * widen(q_norm[d]);
                float k0 = widen(qkv[kb + d]) * ki * widen(k_norm[d]);
                if (d < rope_half) {
                    uint32_t p = d + rope_half;
                    float q1 = widen(qkv[qb + p]) * qi * widen(q_norm[p]);
                    float k1 = widen(qkv[kb + p]) * ki * widen(k_norm[p]);
                    float c = widen(rope_cos[(size_t)row * rope_half + d]);
                    float s = widen(rope_sin[(size_t)row * rope_half + d]);
                    q0 = q0 * c - q1 * s;
                    k0 = k0 * c - k1 * s;
                } else if (d < rope_half * 2) {
                    uint32_t p = d - rope_half;
                    float q1 = widen(qkv[qb + p]) * qi * widen(q_norm[p]);
                    float k1 = widen(qkv[kb + p]) * ki * widen(k_norm[p]);
                    float c = widen(rope_cos[(size_t)row * rope_half + p]);
                    float s = widen(rope_sin[(size_t)row * rope_half + p]);
                    q0 = q0 * c + q1 * s;
                    k0 = k0 * c + k1 * s;
                }
                size_t o = ((size_t)row * heads + head) * hd + d;
                q[o] = narrow(q0);
                k[o] = narrow(k0);
                v[o] = qkv[vb + d];
            }
        }
}

/* sparse_ptr/sparse_idx: optional block-sparse mask in the form h3_gpu_sdpa_set_sparse takes
 * (h3_gpu.h:44-51; walked by the reference kernel at h3_cuda_attention.cu:1652-1673): CSR over
 * 64-key tiles per 128-row query block; a query row attends exactly the keys of its block's
 * listed tiles. NULL = dense. */
static void sdpa_core(uint16_t *out, const uint16_t *q, const uint16_t *k,
                      const uint16_t *v, uint32_t seq, uint32_t heads,
                      uint32_t hd, float scale, int head_major, int round_p,
                      uint32_t row_begin, uint32_t row_end,
                      const uint32_t *sparse_ptr, const uint32_t *sparse_idx) {
    if (!seq || !heads || !hd || row_begin >= row_end) return;
    uint32_t padded = (seq + 15u) & ~15u;
#pragma omp parallel
    {
        /* per-thread head-local copies: K transposed [d][key], V [key][d] */
        float *kt = (float *)aligned_alloc(64, (size_t)hd * padded * 4);
        float *vf = (float *)aligned_alloc(64, (size_t)padded * hd * 4);
        float *scores = (float *)aligned_alloc(64, (size_t)padded * 4);
        float *acc = (float *)aligned_alloc(64, ((size_t)hd * 4 + 63) & ~(size_t)63);
        unsigned char *keep = (unsigned char *)malloc(padded);
#pragma omp for schedule(dynamic, 1)
        for (uint32_t h = 0; h < heads; h++) {
            for (uint32_t j = 0; j < padded; j++)
                for (uint32_t d = 0; d < hd; d++) {
                    float kv = 0.0f, vv = 0.0f;
                    if (j < seq) {
                        size_t idx = ((size_t)j * heads + h) * hd + d;
                        kv = widen(k[idx]);
                        vv = widen(v[idx]);
                    }
                    kt[(size_t)d * padded + j] = kv;
                    vf[(size_t)j * hd + d] = vv;
                }
            for (uint32_t i = row_begin; i < row_end; i++) {
                const uint16_t *qp = q + ((size_t)i * heads + h) * hd;
                for (uint32_t j = 0; j < padded; j++) scores[j] = 0.0f;
                for (uint32_t d = 0; d < hd; d++) {
                    float qd = widen(qp[d]);
                    const float *krow = kt + (size_t)d * padded;
#pragma omp simd
                    for (uint32_t j = 0; j < padded; j++)
                        scores[j] = fmaf(qd, krow[j], scores[j]);
                }
                if (sparse_ptr) {
                    /* keep the scores of the listed tiles, everything else becomes -inf */
                    uint32_t qb = i / 128u;
                    for (uint32_t j = 0; j < seq; j++) keep[j] = 0;
                    for (uint32_t e = sparse_ptr[qb]; e < sparse_ptr[qb + 1]; e++)
                        for (uint32_t j = sparse_idx[e] * 64u; j < sparse_idx[e] * 64u + 64u && j < seq; j++)
                            keep[j] = 1;
                    for (uint32_t j = 0; j < seq; j++)
                        if (!keep[j]) scores[j] = -INFINITY;
                }
                float mx = -INFINITY;
                for (uint32_t j = 0; j < seq; j++) {
                    scores[j] = scores[j] * scale;
                    if (scores[j] > mx) mx = scores[j];
                }
                /* a row whose block lists no tile attends nothing: probabilities and sum are 0
                 * and the row is written as zeros (h3_cuda_attention.cu:1790,1800) */
                float sum = 0.0f;
                for (uint32_t j = 0; j < seq; j++) {
                    scores[j] = mx == -INFINITY ? 0.0f : expf(scores[j] - mx);
                    sum += scores[j];
                }
                float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                for (uint32_t d = 0; d < hd; d++) acc[d] = 0.0f;
                for (uint32_t j = 0; j < seq; j++) {
                    float p = round_p ? bf_round(scores[j]) : scores[j] * inv;
                    const float *vrow = vf + (size_t)j * hd;
#pragma omp simd
                    for (uint32_t d = 0; d < hd; d++)
                        acc[d] = fmaf(p, vrow[d], acc[d]);
                }
                for (uint32_t d = 0; d < hd; d++) {
                    float value = round_p ? acc[d] * inv : acc[d];
                    size_t o = head_major ? ((size_t)h * seq + i) * hd + d
                                          : ((size_t)i * heads + h) * hd + d;
                    out[o] = narrow(value);
                }
            }
        }
        free(kt);
        free(vf);
        free(scores);
        free(acc);
        free(keep);
    }
}

void h3o_sdpa_bf16_rows(uint16_t *out, const uint16_t *q, const uint16_t *k,
                        const uint16_t *v, uint32_t seq, uint32_t heads,
                        uint32_t hd, float scale, int head_major, int round_p,
                        uint32_t row_begin, uint32_t row_end) {
    sdpa_core(out, q, k, v, seq, heads, hd, scale, head_major, round_p, row_begin, row_end,
              NULL, NULL);
}

void h3o_sdpa_bf16_sparse(uint16_t *out, const uint16_t *q, const uint16_t *k,
                          const uint16_t *v, uint32_t seq, uint32_t heads,
                          uint32_t hd, float scale, int head_major, int round_p,
                          const uint32_t *sparse_ptr, const uint32_t *sparse_idx) {
    sdpa_core(out, q, k, v, seq, heads, hd, scale, head_major, round_p, 0, seq, sparse_ptr,
              sparse_idx);
}

void h3o_sdpa_bf16(uint16_t *out, const uint16_t *q, const uint16_t *k,
                   const uint16_t *v, uint32_t seq, uint32_t heads,
                   uint32_t hd, float scale, int head_major, int round_p) {
    h3o_sdpa_bf16_rows(out, q, k, v, seq, heads, hd, scale, head_major,
                       round_p, 0, seq);
}

/* ------------------------------------------------------ patch/euler/etc. */

void h3o_patch_linear_bf16(uint16_t *out, const float *in, const float *weight,
                           const float *bias, const uint32_t *row_map,
                           uint32_t offset_rows, uint32_t rows,
                           uint32_t in_dim, uint32_t out_dim) {
    size_t count = (size_t)rows * out_dim;
    if (!count) return;
    float *acc = (float *)malloc(count * sizeof(float));
    gemm_rows_seq(acc, out_dim, in, NULL, in_dim, weight, NULL, bias, rows,
                  in_dim, out_dim);
    for (uint32_t r = 0; r < rows; r++) {
        size_t dst = row_map ? row_map[r] : (size_t)offset_rows + r;
        for (uint32_t c = 0; c < out_dim; c++)
            out[dst * out_dim + c] = narrow(acc[(size_t)r * out_dim + c]);
    }
    free(acc);
}

void h3o_euler_bf16(float *sample, const uint16_t *last,
                    const uint16_t *previous, size_t count, float delta,
                    float ratio) {
    for (size_t i = 0; i < count; i++) {
        float lv = widen(last[i]);
        float velocity = fmaf(ratio, lv - widen(previous[i]), lv);
        sample[i] = fmaf(delta, velocity, sample[i]);
    }
}

void h3o_cfg_combine_bf16(uint16_t *out, const uint16_t *cond, const uint16_t *uncond,
                          size_t count, float guidance) {
    for (size_t i = 0; i < count; i++) {
        float u = h3o_bf16_to_f32(uncond[i]);
        out[i] = h3o_f32_to_bf16(fmaf(guidance, h3o_bf16_to_f32(cond[i]) - u, u));
    }
}

void h3o_token_pool_bf16(uint16_t *out, const uint16_t *in, uint16_t *original,
                         uint16_t *baseline, const uint32_t *baseline_indices,
                         const uint32_t *pairs, uint32_t rows, uint32_t width) {
    for (uint32_t r = 0; r < rows; r++) {
        uint32_t a = pairs[2 * r], b = pairs[2 * r + 1];
        for (uint32_t c = 0; c < width; c++) {
            uint16_t first = in[(size_t)a * width + c];
            original[(size_t)a * width + c] = first;
            uint16_t pooled = first;
            if (a != b) {
                uint16_t second = in[(size_t)b * width + c];
                original[(size_t)b * width + c] = second;
                pooled = narrow((widen(first) + widen(second)) * 0.5f);
            }
            out[(size_t)r * width + c] = pooled;
            if (baseline_indices[r] != 0xffffffffu)
                baseline[(size_t)baseline_indices[r] * width + c] = pooled;
        }
    }
}

void h3o_token_expand_delta_bf16(uint16_t *out, const uint16_t *original,
                                 const uint16_t *reduced,
                                 const uint16_t *baseline,
                                 const uint32_t *baseline_indices,
                                 const uint32_t *parents, uint32_t rows,
                                 uint32_t width, uint32_t exact_prefix_rows,
                                 float update_scale) {
    for (uint32_t r = 0; r < rows; r++) {
        uint32_t parent = parents[r];
        uint32_t brow = baseline_indices[parent];
        int direct = r < exact_prefix_rows || brow == 0xffffffffu;
        for (uint32_t c = 0; c < width; c++) {
            uint16_t value = reduced[(size_t)parent * width + c];
            if (!direct) {
                float update = widen(value) -
                               widen(baseline[(size_t)brow * width + c]);
                value = narrow(widen(original[(size_t)r * width + c]) +
                               update_scale * update);
            }
            out[(size_t)r * width + c] = value;
        }
    }
}

void h3o_time_features(float *features, const float *times, uint32_t rows) {
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t i = 0; i < 128; i++) {
            float frequency = expf(-logf(10000.0f) * (float)i / 128.0f);
            float angle = times[r] * frequency;
            features[(size_t)r * 256 + i] = cosf(angle);
            features[(size_t)r * 256 + 128 + i] = sinf(angle);
        }
}

void h3o_rope_tables(uint16_t *cos_out, uint16_t *sin_out,
                     const float *positions, const float *inv_freq,
                     uint32_t rows) {
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t axis = 0; axis < 3; axis++)
            for (uint32_t f = 0; f < 16; f++) {
                float angle = positions[(size_t)r * 3 + axis] * inv_freq[f];
                cos_out[(size_t)r * 48 + axis * 16 + f] = narrow(cosf(angle));
                sin_out[(size_t)r * 48 + axis * 16 + f] = narrow(sinf(angle));
            }
}

/* ----------------------------------------------------------------- block */

void h3o_dit_block(uint16_t *hidden, const h3o_block_weights *w,
                   const uint32_t *row_map, const uint16_t *rope_cos,
                   const uint16_t *rope_sin, const h3o_block_shape *s,
                   uint16_t *dump_mod_attention, uint16_t *dump_attention,
                   uint16_t *dump_attention_output, uint16_t *dump_mod_mlp) {
    uint32_t rows = s->rows, width = s->width;
    size_t inner = (size_t)s->heads * s->head_dim;
    size_t act = (size_t)rows * width;
    uint16_t *mod = (uint16_t *)malloc(act * 2 + 2);
    uint16_t *qkv = (uint16_t *)malloc((size_t)rows * inner * 3 * 2 + 2);
    uint16_t *q = (uint16_t *)malloc((size_t)rows * inner * 2 + 2);
    uint16_t *k = (uint16_t *)malloc((size_t)rows * inner * 2 + 2);
    uint16_t *v = (uint16_t *)malloc((size_t)rows * inner * 2 + 2);
    uint16_t *attn = (uint16_t *)malloc((size_t)rows * inner * 2 + 2);
    uint16_t *branch = (uint16_t *)malloc(act * 2 + 2);

    h3o_adaln_bf16(mod, hidden, w->norm1, w->modulation, row_map, rows, width,
                   6, 0, 1, s->eps);
    if (dump_mod_attention) memcpy(dump_mod_attention, mod, act * 2);
    h3o_linear_bf16(qkv, mod, w->qkv_weight, NULL, rows, width,
                    (uint32_t)(inner * 3));
    h3o_qkv_rope_bf16(q, k, v, qkv, w->q_norm, w->k_norm, rope_cos, rope_sin,
                      rows, s->heads, s->head_dim, s->rope_half, 1, s->eps);
    h3o_sdpa_bf16(attn, q, k, v, rows, s->heads, s->head_dim, s->scale, 0,
                  s->round_p);
    if (dump_attention) memcpy(dump_attention, attn, (size_t)rows * inner * 2);
    h3o_linear_bf16(branch, attn, w->out_weight, NULL, rows, (uint32_t)inner,
                    width);
    if (dump_attention_output) memcpy(dump_attention_output, branch, act * 2);
    h3o_gate_adaln_bf16(hidden, mod, hidden, branch, w->norm2, w->modulation,
                        w->modulation, row_map, rows, width, 6, 2, 3, 4,
                        s->eps);
    if (dump_mod_mlp) memcpy(dump_mod_mlp, mod, act * 2);
    h3o_mlp_bf16(branch, mod, w->fc1_weight, w->fc2_weight, rows, width,
                 s->ffn, width);
    h3o_gate_bf16(hidden, hidden, branch, w->modulation, row_map, rows, width,
                  6, 5);

    free(mod); free(qkv); free(q); free(k); free(v); free(attn); free(branch);
}

/* ------------------------------------- video-VAE decoder F32 row operations */

void h3o_rms_norm_f32(float *out, const float *in, const float *weight,
                      uint32_t rows, uint32_t width, float eps) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *x = in + (size_t)r * width;
        float ss = 0.0f;
        for (uint32_t c = 0; c < width; c++) ss += x[c] * x[c];
        float inv = 1.0f / sqrtf(ss / (float)width + eps);
        for (uint32_t c = 0; c < width; c++)
            out[(size_t)r * width + c] = x[c] * inv * weight[c];
    }
}

void h3o_layer_norm_f32(float *out, const float *in, const float *weight,
                        const float *bias, uint32_t rows, uint32_t width, float eps) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *x = in + (size_t)r * width;
        float sum = 0.0f;
        for (uint32_t c = 0; c < width; c++) sum += x[c];
        float mean = sum / (float)width;
        float vs = 0.0f;
        for (uint32_t c = 0; c < width; c++) {
            float d = x[c] - mean;
            vs += d * d;
        }
        float inv = 1.0f / sqrtf(vs / (float)width + eps);
        for (uint32_t c = 0; c < width; c++)
            out[(size_t)r * width + c] = (x[c] - mean) * inv * weight[c] + bias[c];
    }
}

void h3o_scale_add_f32(float *out, const float *residual, const float *branch,
                       const float *scale, uint32_t rows, uint32_t width) {
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < width; c++) {
            size_t i = (size_t)r * width + c;
            out[i] = residual[i] + branch[i] * scale[c];
        }
}

void h3o_swiglu_f32(float *out, const float *fused, uint32_t rows, uint32_t width) {
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < width; c++) {
            float gate = fused[(size_t)r * width * 2 + c];
            float up = fused[(size_t)r * width * 2 + width + c];
            out[(size_t)r * width + c] = gate / (1.0f + expf(-gate)) * up;
        }
}

void h3o_video_qkv_rope_f32(float *q, float *k, float *v, const float *qkv,
                            const float *rope_cos, const float *rope_sin,
                            uint32_t seq, uint32_t heads, uint32_t hd,
                            uint32_t rope_half, float eps) {
    for (uint32_t row = 0; row < seq; row++)
        for (uint32_t head = 0; head < heads; head++) {
            size_t unit = (size_t)row * heads + head;
            const float *qi = qkv + unit * hd * 3, *ki = qi + hd, *vi = ki + hd;
            float qs = 0.0f, ks = 0.0f;
            for (uint32_t d = 0; d < hd; d++) {
                qs = fmaf(qi[d], qi[d], qs);
                ks = fmaf(ki[d], ki[d], ks);
            }
            float q_inv = 1.0f / sqrtf(qs / (float)hd + eps);
            float k_inv = 1.0f / sqrtf(ks / (float)hd + eps);
            for (uint32_t dim = 0; dim < hd; dim++) {
                float q0 = qi[dim] * q_inv, k0 = ki[dim] * k_inv;
                if (dim < rope_half) {
                    uint32_t pair = dim + rope_half;
                    float q1 = qi[pair] * q_inv, k1 = ki[pair] * k_inv;
                    float c = rope_cos[(size_t)row * rope_half + dim];
                    float s = rope_sin[(size_t)row * rope_half + dim];
                    q0 = q0 * c - q1 * s;
                    k0 = k0 * c - k1 * s;
                } else if (dim < rope_half * 2) {
                    uint32_t pair = dim - rope_half;
                    float q1 = qi[pair] * q_inv, k1 = ki[pair] * k_inv;
                    float c = rope_cos[(size_t)row * rope_half + pair];
                    float s = rope_sin[(size_t)row * rope_half + pair];
                    q0 = q0 * c + q1 * s;
                    k0 = k0 * c + k1 * s;
                }
                q[unit * hd + dim] = q0;
                k[unit * hd + dim] = k0;
                v[unit * hd + dim] = vi[dim];
            }
        }
}

void h3o_sdpa_f32(float *out, const float *q, const float *k, const float *v,
                  uint32_t seq, uint32_t heads, uint32_t hd, float scale) {
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t i = 0; i < seq; i++) {
            float *scores = (float *)malloc((size_t)seq * sizeof(float));
            const float *qp = q + ((size_t)i * heads + h) * hd;
            float mx = -INFINITY;
            for (uint32_t j = 0; j < seq; j++) {
                const float *kp = k + ((size_t)j * heads + h) * hd;
                float dot = 0.0f;
                for (uint32_t d = 0; d < hd; d++) dot = fmaf(qp[d], kp[d], dot);
                scores[j] = dot * scale;
                if (scores[j] > mx) mx = scores[j];
            }
            float sum = 0.0f;
            for (uint32_t j = 0; j < seq; j++) {
                scores[j] = expf(scores[j] - mx);
                sum += scores[j];
            }
            float inv = 1.0f / sum;
            for (uint32_t d = 0; d < hd; d++) {
                float acc = 0.0f;
                for (uint32_t j = 0; j < seq; j++)
                    acc = fmaf(scores[j] * inv, v[((size_t)j * heads + h) * hd + d], acc);
                out[((size_t)i * heads + h) * hd + d] = acc;
            }
            free(scores);
        }
}
