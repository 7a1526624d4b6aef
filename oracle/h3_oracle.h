/* CPU oracle for the MiniMax-H3 DiT denoiser forward.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the arithmetic
 * the reference defines for the DiT block path. The shipped library never
 * links, loads or calls it; only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg do, and only as the checker / baseline.
 *
 * The reference has no CPU implementation of the DiT; its CPU arithmetic for
 * these ops lives in the "independent CPU reference" functions of its CUDA
 * test programs. Every function below names the reference lines it follows.
 * Parity status: PINNED. The restatement is compared bit-for-bit against those
 * reference functions (compiled from the reference tree into oracle/_ref/ by
 * build_ref.py) and against committed golden vectors generated from them.
 *
 * Conventions: BF16 is raw uint16_t, widened exactly, narrowed round-to-nearest
 * even with the reference's integer formula; sums are F32; weights are
 * [out][in] row-major; activations are row-major with rows = tokens.
 */
#ifndef H3_ORACLE_H
#define H3_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* h3_cuda_internal.h:244-253, tests/test_cuda_dit.c:12-23 */
float h3o_bf16_to_f32(uint16_t value);
uint16_t h3o_f32_to_bf16(float value);
void h3o_widen(float *out, const uint16_t *in, size_t count);
void h3o_narrow(uint16_t *out, const float *in, size_t count);

/* PCG32 + Box-Muller, h3_host.c:496-530 */
typedef struct {
    uint64_t state;
    uint64_t increment;
    float spare;
    int has_spare;
} h3o_rng;
void h3o_rng_seed(h3o_rng *rng, uint64_t seed);
uint32_t h3o_rng_u32(h3o_rng *rng);
float h3o_rng_normal(h3o_rng *rng);
/* values[i] = mean + std * normal; one sequential stream per call */
void h3o_fill_normal_f32(float *values, size_t count, uint64_t seed,
                         float mean, float std);
void h3o_fill_normal_bf16(uint16_t *values, size_t count, uint64_t seed,
                          float mean, float std);
/* seed ^ FNV-1a(name): independent stream per named tensor */
uint64_t h3o_named_seed(uint64_t seed, const char *name);

/* tests/test_cuda_core.c:174-184 (sequential fmaf from the bias), rounded as
 * h3_cuda_core.cu:358-371 */
void h3o_linear_f32(float *out, const float *in, const float *weight,
                    const float *bias, uint32_t rows, uint32_t in_dim,
                    uint32_t out_dim);
void h3o_linear_bf16(uint16_t *out, const uint16_t *in, const uint16_t *weight,
                     const uint16_t *bias, uint32_t rows, uint32_t in_dim,
                     uint32_t out_dim);

/* tests/test_cuda_core.c:154,351-359; h3_cuda_core.cu:104-114 */
void h3o_swiglu_bf16(uint16_t *out, const uint16_t *fused, uint32_t rows,
                     uint32_t width);
void h3o_silu_bf16(uint16_t *out, const uint16_t *in, size_t count);
void h3o_silu_f32(float *out, const float *in, size_t count);
void h3o_add_bf16(uint16_t *out, const uint16_t *a, const uint16_t *b,
                  size_t count);
void h3o_sub_bf16(uint16_t *out, const uint16_t *a, const uint16_t *b,
                  size_t count);

/* MLP with the CUDA route's rounding points (fc1 output and SwiGLU output each
 * rounded to BF16), h3_cuda_core.cu:1067-1110 */
void h3o_mlp_bf16(uint16_t *out, const uint16_t *in, const uint16_t *fc1,
                  const uint16_t *fc2, uint32_t rows, uint32_t in_dim,
                  uint32_t hidden, uint32_t out_dim);

/* tests/test_cuda_dit.c:134-160 (ref_adaln), rounded as h3_cuda_dit.cu:141-175 */
void h3o_adaln_bf16(uint16_t *out, const uint16_t *in, const uint16_t *norm,
                    const uint16_t *modulation, const uint32_t *row_map,
                    uint32_t rows, uint32_t width, uint32_t slots,
                    uint32_t shift_slot, uint32_t scale_slot, float eps);
void h3o_adaln_f32(float *out, const float *in, const float *norm,
                   const float *modulation, const uint32_t *row_map,
                   uint32_t rows, uint32_t width, uint32_t slots,
                   uint32_t shift_slot, uint32_t scale_slot, float eps);
/* h3_cuda_core.cu:184-210 */
void h3o_rms_norm_bf16(uint16_t *out, const uint16_t *in, const uint16_t *norm,
                       uint32_t rows, uint32_t width, float eps);
/* tests/test_cuda_dit.c:162-175 (ref_gate), h3_cuda_dit.cu:261-276 */
void h3o_gate_bf16(uint16_t *out, const uint16_t *residual,
                   const uint16_t *branch, const uint16_t *modulation,
                   const uint32_t *row_map, uint32_t rows, uint32_t width,
                   uint32_t slots, uint32_t gate_slot);
void h3o_gate_f32(float *out, const float *residual, const float *branch,
                  const float *modulation, const uint32_t *row_map,
                  uint32_t rows, uint32_t width, uint32_t slots,
                  uint32_t gate_slot);
/* tests/test_cuda_dit.c:395-416, h3_cuda_dit.cu:281-332: the gated row is
 * rounded to BF16, stored, and the rounded row is normalised. gated/out may
 * alias residual/branch. */
void h3o_gate_adaln_bf16(uint16_t *gated, uint16_t *out,
                         const uint16_t *residual, const uint16_t *branch,
                         const uint16_t *norm, const uint16_t *gate_modulation,
                         const uint16_t *norm_modulation,
                         const uint32_t *row_map, uint32_t rows,
                         uint32_t width, uint32_t slots, uint32_t gate_slot,
                         uint32_t shift_slot, uint32_t scale_slot, float eps);
/* tests/test_cuda_dit.c:293-326, h3_cuda_dit.cu:179-259 */
void h3o_adaln_linear_bf16(uint16_t *out, float *inverse, const uint16_t *in,
                           const uint16_t *norm, const uint16_t *modulation,
                           const uint32_t *row_map, const uint16_t *weight,
                           const uint16_t *bias, uint32_t rows, uint32_t width,
                           uint32_t out_dim, uint32_t slots,
                           uint32_t shift_slot, uint32_t scale_slot, float eps);

/* tests/test_cuda_attention.c:120-174 (ref_qkv_rope, weighted norm), output
 * rounded as h3_cuda_attention.cu:199-236. grouped=1: row = [head][q,k,v][hd];
 * grouped=0: row = [q heads][k heads][v heads]. rope tables are BF16 [seq, half]. */
void h3o_qkv_rope_bf16(uint16_t *q, uint16_t *k, uint16_t *v,
                       const uint16_t *qkv, const uint16_t *q_norm,
                       const uint16_t *k_norm, const uint16_t *rope_cos,
                       const uint16_t *rope_sin, uint32_t seq, uint32_t heads,
                       uint32_t head_dim, uint32_t rope_half, int grouped,
                       float eps);
/* tests/test_cuda_attention.c:204-242 (ref_sdpa, non-causal, batch 1).
 * round_p=0: exact softmax as the test reference. round_p=1: probabilities are
 * rounded to BF16 before P.V and the row sum uses the unrounded values, the
 * rounding boundary of the reference's tensor-core path
 * (h3_cuda_attention.cu:1189-1194,1526-1528). q/k/v are [seq][heads][hd]. */
void h3o_sdpa_bf16(uint16_t *out, const uint16_t *q, const uint16_t *k,
                   const uint16_t *v, uint32_t seq, uint32_t heads,
                   uint32_t head_dim, float scale, int head_major, int round_p);
/* Same, restricted to query rows [row_begin, row_end) (bounded CPU samples). */
void h3o_sdpa_bf16_rows(uint16_t *out, const uint16_t *q, const uint16_t *k,
                        const uint16_t *v, uint32_t seq, uint32_t heads,
                        uint32_t head_dim, float scale, int head_major,
                        int round_p, uint32_t row_begin, uint32_t row_end);

/* h3_cuda_core.cu:374-403: F32 rows x F32 weight + bias -> BF16, written at
 * (row_map ? row_map[r] : offset_rows + r). */
/* attention under a block-sparse mask: CSR over 64-key tiles per 128-row query block, the form
 * h3_gpu_sdpa_set_sparse takes (h3_gpu.h:44-51, h3_cuda_attention.cu:1652-1673) */
void h3o_sdpa_bf16_sparse(uint16_t *out, const uint16_t *q, const uint16_t *k,
                          const uint16_t *v, uint32_t seq, uint32_t heads,
                          uint32_t hd, float scale, int head_major, int round_p,
                          const uint32_t *sparse_ptr, const uint32_t *sparse_idx);
void h3o_patch_linear_bf16(uint16_t *out, const float *in, const float *weight,
                           const float *bias, const uint32_t *row_map,
                           uint32_t offset_rows, uint32_t rows,
                           uint32_t in_dim, uint32_t out_dim);
/* h3_cuda_dit.cu:536-548 */
void h3o_euler_bf16(float *sample, const uint16_t *last,
                    const uint16_t *previous, size_t count, float delta,
                    float ratio);
/* h3_cuda_dit.cu:336-365 / 437-467 (token reduction pool / expand) */
/* classifier-free guidance combine of the B200 library's h3x_cfg_combine_bf16 (no reference
 * counterpart): out = bf16(fmaf(guidance, cond - uncond, uncond)) */
void h3o_cfg_combine_bf16(uint16_t *out, const uint16_t *cond, const uint16_t *uncond,
                          size_t count, float guidance);
void h3o_token_pool_bf16(uint16_t *out, const uint16_t *in, uint16_t *original,
                         uint16_t *baseline, const uint32_t *baseline_indices,
                         const uint32_t *pairs, uint32_t rows, uint32_t width);
void h3o_token_expand_delta_bf16(uint16_t *out, const uint16_t *original,
                                 const uint16_t *reduced,
                                 const uint16_t *baseline,
                                 const uint32_t *baseline_indices,
                                 const uint32_t *parents, uint32_t rows,
                                 uint32_t width, uint32_t exact_prefix_rows,
                                 float update_scale);

/* h3_dit_schedule.c:148-157: 256 sinusoidal features of t = 1 - sigma. */
void h3o_time_features(float *features, const float *times, uint32_t rows);
/* h3_dit.c:916-928: cos/sin(position[axis] * inv_freq[f]) -> BF16 [rows, 48];
 * positions are F32 [rows][3] (t, h, w); inv_freq has 16 entries. */
void h3o_rope_tables(uint16_t *cos_out, uint16_t *sin_out,
                     const float *positions, const float *inv_freq,
                     uint32_t rows);

/* One DiT block in the order of run_block (h3_dit.c:2008-2180), unfused as in
 * tests/test_real_dit_block.c:294-350: adaLN(0,1) -> QKV -> norm+RoPE -> SDPA ->
 * out-proj -> gate(2)+adaLN(3,4) -> fc1 -> SwiGLU -> fc2 -> gate(5).
 * hidden is updated in place. Optional stage dumps may be NULL. */
typedef struct {
    const uint16_t *norm1, *norm2;       /* [width] */
    const uint16_t *qkv_weight;          /* [3*heads*hd, width] */
    const uint16_t *q_norm, *k_norm;     /* [hd] */
    const uint16_t *out_weight;          /* [width, heads*hd] */
    const uint16_t *fc1_weight;          /* [2*ffn, width] */
    const uint16_t *fc2_weight;          /* [width, ffn] */
    const uint16_t *modulation;          /* [mod_rows, 6, width] */
} h3o_block_weights;
typedef struct {
    uint32_t rows, width, heads, head_dim, ffn, rope_half;
    float eps, scale;
    int round_p;
} h3o_block_shape;
void h3o_dit_block(uint16_t *hidden, const h3o_block_weights *w,
                   const uint32_t *row_map, const uint16_t *rope_cos,
                   const uint16_t *rope_sin, const h3o_block_shape *shape,
                   uint16_t *dump_mod_attention, uint16_t *dump_attention,
                   uint16_t *dump_attention_output, uint16_t *dump_mod_mlp);

/* ---- F32 operations of the video-VAE decoder's transformer (h3_video_vae.c:425-461). Each
 * restates the CPU reference the reference's own tests check its kernels against. ---------- */
/* tests/test_cuda_core.c:419-428 */
void h3o_rms_norm_f32(float *out, const float *in, const float *weight,
                      uint32_t rows, uint32_t width, float eps);
/* tests/test_cuda_core.c:466-482 */
void h3o_layer_norm_f32(float *out, const float *in, const float *weight,
                        const float *bias, uint32_t rows, uint32_t width, float eps);
/* tests/test_cuda_core.c:296-299 */
void h3o_scale_add_f32(float *out, const float *residual, const float *branch,
                       const float *scale, uint32_t rows, uint32_t width);
/* tests/test_cuda_core.c:351-359 */
void h3o_swiglu_f32(float *out, const float *fused, uint32_t rows, uint32_t width);
/* tests/test_cuda_attention.c:120-185 with grouped = 1, weighted = 0 */
void h3o_video_qkv_rope_f32(float *q, float *k, float *v, const float *qkv,
                            const float *rope_cos, const float *rope_sin,
                            uint32_t seq, uint32_t heads, uint32_t hd,
                            uint32_t rope_half, float eps);
/* tests/test_cuda_attention.c:204-242 (non-causal, [row][head][dim] output) */
void h3o_sdpa_f32(float *out, const float *q, const float *k, const float *v,
                  uint32_t seq, uint32_t heads, uint32_t hd, float scale);

int h3o_threads(void);
/* OpenMP threads used from now on (a launcher may have exported OMP_NUM_THREADS=1) */
void h3o_set_threads(int count);

#ifdef __cplusplus
}
#endif
#endif
