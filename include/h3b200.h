/* h3b200 — B200 (sm_100a) device backend for the MiniMax-H3 DiT denoiser forward.
 *
 * This is the C ABI of libh3b200.so. The h3_gpu_* entry points have the names,
 * argument order and return convention of the reference's device API
 * (reference h3_gpu.h), so reference host code (h3_dit.c, h3_dit_schedule.c,
 * h3_weights.c) compiled against the reference header links against this
 * library unchanged. Each group below cites the reference declaration
 * (h3_gpu.h:line) and the reference CUDA implementation it replaces.
 *
 * Conventions (reference h3_cuda_internal.h:126-185, h3_gpu_cuda.cu:871-911):
 *   - every op returns 1 on success and 0 on failure; the message is read
 *     with h3_gpu_error(); constructors return NULL on failure;
 *   - ops fail unless issued between h3_gpu_begin() and h3_gpu_submit();
 *   - work is enqueued in order on one stream; h3_gpu_submit() waits for it
 *     and reports asynchronous failures;
 *   - BF16 is raw uint16_t (exact widening, round-to-nearest-even narrowing),
 *     sums are F32, weights are [out][in] row-major, activations row-major
 *     with rows = tokens, offsets are in elements.
 *
 * Entry points of the reference API that are not on the DiT path (VAE
 * convolutions, Qwen encoders, Metal-only int8/NAX routes) are exported too,
 * as stubs that fail with a message, so that a full libh3 still links; this
 * follows the reference's own practice (h3_cuda_dit.cu:1072-1216).
 */
#ifndef H3B200_H
#define H3B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- types: h3_gpu.h:7-33 ------------------------------------------- */
/* When the reference's own header was included first (its guard is H3_GPU_H), its type
 * definitions are used and every prototype below is checked against its declaration by the
 * compiler: a mismatch in any argument or return type is a compile error. */
#ifndef H3_GPU_H
typedef struct h3_gpu h3_gpu;
typedef struct h3_gpu_tensor h3_gpu_tensor;

typedef enum { H3_GPU_F32 = 0, H3_GPU_BF16, H3_GPU_I8, H3_GPU_U32 } h3_gpu_dtype;

typedef struct {
    uint64_t allocated_bytes, live_bytes, peak_live_bytes, tensor_allocations;
    uint64_t direct_dispatches;     /* hand kernels                        */
    uint64_t mps_linear_dispatches; /* dense projections (tensor-core GEMM) */
    uint64_t mps_conv_dispatches;
    uint64_t mps_sdpa_dispatches;   /* attention calls                      */
    uint64_t blit_copies, submissions;
    double command_encode_seconds, command_wait_seconds, gpu_seconds;
} h3_gpu_stats;
#endif /* H3_GPU_H */

/* ---- context: h3_gpu.h:35-51,100-110; h3_gpu_cuda.cu:80-170,871-933 --- */
h3_gpu *h3_gpu_create(const char *unused_shader_path, char *error, size_t error_size);
void h3_gpu_free(h3_gpu *gpu);
int h3_gpu_is_m5(const h3_gpu *gpu);                /* 0 */
int h3_gpu_has_nax_mlp(const h3_gpu *gpu);          /* 0 */
int h3_gpu_has_int8_mlp(const h3_gpu *gpu);         /* 0 */
int h3_gpu_prefers_gpu_sampler(const h3_gpu *gpu);  /* 1 */
/* Block-sparse attention mask (h3_gpu.h:44-51, h3_cuda_attention.cu:1812-1857): CSR over
 * 64-row K/V tiles per 128-row query block, applied to head_dim-128 attention calls whose row
 * count equals rows (other calls stay dense); NULL ptr clears; same validation as the
 * reference. The lists are regrouped for the 256-row x 128-key tiles of the tensor-core
 * kernel; a tile listed twice for one block counts once. */
int h3_gpu_sdpa_set_sparse(h3_gpu *gpu, const uint32_t *ptr, size_t ptr_count,
                           const uint32_t *idx, size_t idx_count, uint32_t rows);
int h3_gpu_begin(h3_gpu *gpu);
int h3_gpu_continue(h3_gpu *gpu);
int h3_gpu_submit(h3_gpu *gpu);
const char *h3_gpu_error(const h3_gpu *gpu);
int h3_gpu_get_stats(const h3_gpu *gpu, h3_gpu_stats *stats);
void h3_gpu_profile_set_label(h3_gpu *gpu, const char *label);
void h3_gpu_profile_mark(h3_gpu *gpu, const char *phase);

/* ---- tensors: h3_gpu.h:53-98; h3_gpu_cuda.cu:199-870 ----------------- */
h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_i8(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *gpu, const float *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *gpu, const uint16_t *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_load_bf16(h3_gpu *gpu, const char *path, uint64_t file_offset,
                                       size_t elements);
h3_gpu_tensor *h3_gpu_tensor_load_f32(h3_gpu *gpu, const char *path, uint64_t file_offset,
                                      size_t elements);
/* Both fill an existing tensor from a file on a private copy stream and return when the data
 * is on the device; they may run on an I/O thread while the context's thread issues kernels on
 * other tensors (h3_gpu.h:66-78). read_file orders its first copy after the work already queued
 * on the context's stream, so kernels that still read the old contents finish first.
 * stream_file does not wait (it is the double-buffer path that must overlap the running block,
 * h3_dit.c:2355-2433): its target must be idle on the context's stream when it is called.
 * Either way, work on a stream other than the context's is the caller's to order. */
int h3_gpu_tensor_read_file_bf16(h3_gpu_tensor *tensor, const char *path, uint64_t file_offset,
                                 size_t elements, char *error, size_t error_size);
int h3_gpu_tensor_stream_file_bf16(h3_gpu_tensor *tensor, const char *path, uint64_t file_offset,
                                   size_t elements, char *error, size_t error_size);
void h3_gpu_tensor_free(h3_gpu_tensor *tensor);
size_t h3_gpu_tensor_elements(const h3_gpu_tensor *tensor);
h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *tensor);
int h3_gpu_tensor_read_f32(const h3_gpu_tensor *tensor, float *values, size_t elements);
int h3_gpu_tensor_read_f32_range(const h3_gpu_tensor *tensor, size_t source_offset, float *values,
                                 size_t elements);
int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *tensor, uint16_t *values, size_t elements);
int h3_gpu_tensor_write_f32(h3_gpu_tensor *tensor, const float *values, size_t elements);
int h3_gpu_tensor_write_f32_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                  const float *values, size_t elements);
int h3_gpu_tensor_write_bf16(h3_gpu_tensor *tensor, const uint16_t *values, size_t elements);
int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                   const uint16_t *values, size_t elements);

/* ---- dense projections: h3_gpu.h:112-135,302-312; h3_cuda_core.cu:886-1140,
 *      h3_cuda_gemm.cu:442-575. out = bf16(x . W^T + bias), F32 accumulate. -- */
int h3_gpu_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                       const h3_gpu_tensor *weight, const h3_gpu_tensor *bias, uint32_t rows,
                       uint32_t input_dim, uint32_t output_dim);
int h3_gpu_linear_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                      const h3_gpu_tensor *weight, const h3_gpu_tensor *bias, uint32_t rows,
                      uint32_t input_dim, uint32_t output_dim);
/* fc1 -> SwiGLU (gate = first hidden_dim columns, up = last) -> fc2, each
 * stage rounded to BF16. */
int h3_gpu_mlp_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                    const h3_gpu_tensor *fc1_weight, const h3_gpu_tensor *fc2_weight,
                    uint32_t rows, uint32_t input_dim, uint32_t hidden_dim, uint32_t output_dim);
/* F32 rows x F32 weight (+bias) -> BF16 rows, optionally placed at a row
 * offset or scattered through a row map (patch embedding into `hidden`). */
int h3_gpu_patch_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                             const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                             uint32_t rows, uint32_t input_dim, uint32_t output_dim);
int h3_gpu_patch_linear_bf16_offset(h3_gpu *gpu, h3_gpu_tensor *output, size_t output_offset,
                                    const h3_gpu_tensor *input, size_t input_offset,
                                    const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                    uint32_t rows, uint32_t input_dim, uint32_t output_dim);
int h3_gpu_patch_linear_bf16_map(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                 const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                 const h3_gpu_tensor *row_map, uint32_t output_rows,
                                 uint32_t rows, uint32_t input_dim, uint32_t output_dim);

/* ---- adaLN / gate / final head: h3_gpu.h:154-166,387-430;
 *      h3_cuda_dit.cu:94-332,550-795 ------------------------------------ */
int h3_gpu_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                      const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *modulation,
                      const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                      uint32_t slots, uint32_t shift_slot, uint32_t scale_slot, float epsilon);
int h3_gpu_adaln_bf16_offset(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                             size_t input_offset, const h3_gpu_tensor *norm_weight,
                             const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
                             uint32_t rows, uint32_t width, uint32_t slots, uint32_t shift_slot,
                             uint32_t scale_slot, float epsilon);
int h3_gpu_adaln_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                     const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *modulation,
                     const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width, uint32_t slots,
                     uint32_t shift_slot, uint32_t scale_slot, float epsilon);
int h3_gpu_gate_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                     const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                     const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width, uint32_t slots,
                     uint32_t gate_slot);
int h3_gpu_gate_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                    const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                    const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width, uint32_t slots,
                    uint32_t gate_slot);
/* gated_residual = bf16(residual + branch*gate); output = adaLN(gated_residual).
 * gated_residual may alias residual. */
int h3_gpu_gate_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *gated_residual, h3_gpu_tensor *output,
                           const h3_gpu_tensor *residual, const h3_gpu_tensor *branch,
                           const h3_gpu_tensor *norm_weight,
                           const h3_gpu_tensor *gate_modulation,
                           const h3_gpu_tensor *norm_modulation, const h3_gpu_tensor *row_map,
                           uint32_t rows, uint32_t width, uint32_t slots, uint32_t gate_slot,
                           uint32_t shift_slot, uint32_t scale_slot, float epsilon);
/* final head: adaLN rounded to BF16, then Linear(width -> output_dim)+bias;
 * also stores the per-row inverse RMS (F32). */
int h3_gpu_adaln_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, h3_gpu_tensor *inverse,
                             const h3_gpu_tensor *input, size_t input_offset,
                             const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *modulation,
                             const h3_gpu_tensor *row_map, const h3_gpu_tensor *weight,
                             const h3_gpu_tensor *bias, uint32_t rows, uint32_t width,
                             uint32_t output_dim, uint32_t slots, uint32_t shift_slot,
                             uint32_t scale_slot, float epsilon);

/* ---- QKV split + per-head RMSNorm + RoPE, attention: h3_gpu.h:444-482,504-514;
 *      h3_cuda_attention.cu:173-351,2622-2779,2933-3123 ------------------- */
int h3_gpu_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                         h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                         const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                         const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                         uint32_t sequence, uint32_t heads, uint32_t head_dim,
                         uint32_t rope_half, float epsilon);
int h3_gpu_grouped_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                                 h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                                 const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                 const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                 uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                 uint32_t rope_half, float epsilon);
int h3_gpu_grouped_qkv_linear_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                                        h3_gpu_tensor *value, h3_gpu_tensor *qkv,
                                        const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                                        const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                        const h3_gpu_tensor *rope_cos,
                                        const h3_gpu_tensor *rope_sin, uint32_t rows,
                                        uint32_t input_dim, uint32_t heads, uint32_t head_dim,
                                        uint32_t rope_half, float epsilon);
/* non-causal softmax(q k^T * scale) v over all `sequence` rows, per head;
 * q/k/v are [row][head][head_dim]; output likewise, or [head][row][head_dim]. */
int h3_gpu_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                     const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                     uint32_t heads, uint32_t head_dim, float scale);
int h3_gpu_sdpa_bf16_head_major_output(h3_gpu *gpu, h3_gpu_tensor *output,
                                       const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                       const h3_gpu_tensor *value, uint32_t sequence,
                                       uint32_t heads, uint32_t head_dim, float scale);

/* ---- F32 operations of the video-VAE decoder's transformer, the step after the DiT
 *      (h3_video_vae.c:425-461 run_block, 492-519 run_decoder): h3_gpu.h:150-197;
 *      h3_cuda_core.cu:57-66,92-103,161-182,212-250,609-628,673-684,720-772;
 *      h3_cuda_attention.cu:125-170,2657-2682,2990-3013,3125-3131.
 *      Together with h3_gpu_linear_f32 above and the tensor / copy calls they are every device
 *      call that file makes. Row ops are F32 throughout; the projections (reduction >= 1024)
 *      run on the BF16 tensor cores as hi/lo splits where the reference uses TF32; attention
 *      with head_dim 64 or 128 rounds q, k, v to BF16 as the reference does. -- */
/* y = x * rsqrt(mean(x^2) + eps) * weight */
int h3_gpu_rms_norm_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                        const h3_gpu_tensor *weight, uint32_t rows, uint32_t width, float epsilon);
/* y = (x - mean) * rsqrt(var + eps) * weight + bias */
int h3_gpu_layer_norm_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                          const h3_gpu_tensor *weight, const h3_gpu_tensor *bias, uint32_t rows,
                          uint32_t width, float epsilon);
/* out = residual + branch * scale[column] */
int h3_gpu_scale_add_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                         const h3_gpu_tensor *branch, const h3_gpu_tensor *scale, uint32_t rows,
                         uint32_t width);
/* fused rows are [gate (width) | up (width)]; out = gate / (1 + exp(-gate)) * up */
int h3_gpu_swiglu_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *fused,
                      uint32_t rows, uint32_t width);
/* fused rows are [head][q | k | v][head_dim]; q, k: unweighted RMS norm over the head, then RoPE
 * on dims [0, 2 * rope_half) with pairs (d, d + rope_half); v copied. Tables [row][rope_half]. */
int h3_gpu_video_qkv_rope_f32(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                              h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                              const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                              uint32_t sequence, uint32_t heads, uint32_t head_dim,
                              uint32_t rope_half, float epsilon);
/* non-causal attention, F32 tensors [row][head][head_dim] */
int h3_gpu_sdpa_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                    const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                    uint32_t heads, uint32_t head_dim, float scale);

/* ---- elementwise / row ops: h3_gpu.h:136-149,365-370,515-517,551-556,616-622;
 *      h3_cuda_core.cu:15-210, h3_gpu_cuda.cu:937-1030, h3_cuda_dit.cu:536-548 -- */
int h3_gpu_swiglu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *fused,
                       uint32_t rows, uint32_t width);
int h3_gpu_silu_mul_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *gate,
                         const h3_gpu_tensor *up, uint32_t elements);
int h3_gpu_silu_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                    uint32_t elements);
int h3_gpu_silu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                     uint32_t elements);
int h3_gpu_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                         const h3_gpu_tensor *weight, uint32_t rows, uint32_t width,
                         float epsilon);
int h3_gpu_add_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *left,
                    const h3_gpu_tensor *right, uint32_t elements);
int h3_gpu_sub_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *left,
                    const h3_gpu_tensor *right, uint32_t elements);
int h3_gpu_cast_f32_to_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                            uint32_t elements);
int h3_gpu_cast_bf16_to_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                            uint32_t elements);
int h3_gpu_copy_bf16(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                     const h3_gpu_tensor *source, size_t source_offset, size_t elements);
int h3_gpu_copy_f32(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                    const h3_gpu_tensor *source, size_t source_offset, size_t elements);
/* sample += delta * (last + ratio * (last - previous)); F32 sample, BF16 velocities */
int h3_gpu_euler_bf16(h3_gpu *gpu, h3_gpu_tensor *sample, size_t sample_offset,
                      const h3_gpu_tensor *last, const h3_gpu_tensor *previous,
                      uint32_t elements, float delta, float ratio);

/* ---- token reduction: h3_gpu.h:557-613; h3_cuda_dit.cu:336-534,797-1049 -- */
int h3_gpu_token_pool_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                           size_t input_offset, h3_gpu_tensor *original, size_t original_offset,
                           h3_gpu_tensor *baseline, size_t baseline_offset,
                           const h3_gpu_tensor *baseline_indices, const h3_gpu_tensor *pairs,
                           uint32_t input_rows, uint32_t rows, uint32_t baseline_rows,
                           uint32_t width);
int h3_gpu_token_pool_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *residual, h3_gpu_tensor *output,
                                 const h3_gpu_tensor *input, size_t input_offset,
                                 h3_gpu_tensor *original, size_t original_offset,
                                 h3_gpu_tensor *baseline, size_t baseline_offset,
                                 const h3_gpu_tensor *baseline_indices,
                                 const h3_gpu_tensor *pairs, const h3_gpu_tensor *norm_weight,
                                 const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
                                 uint32_t input_rows, uint32_t rows, uint32_t baseline_rows,
                                 uint32_t width, uint32_t slots, uint32_t shift_slot,
                                 uint32_t scale_slot, float epsilon);
int h3_gpu_token_expand_delta_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                   const h3_gpu_tensor *original, size_t original_offset,
                                   const h3_gpu_tensor *reduced, const h3_gpu_tensor *baseline,
                                   size_t baseline_offset,
                                   const h3_gpu_tensor *baseline_indices,
                                   const h3_gpu_tensor *parents, uint32_t rows,
                                   uint32_t reduced_rows, uint32_t baseline_rows, uint32_t width,
                                   uint32_t exact_prefix_rows, float update_scale);
int h3_gpu_token_expand_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *residual, h3_gpu_tensor *output,
                                   const h3_gpu_tensor *original, size_t original_offset,
                                   const h3_gpu_tensor *reduced, const h3_gpu_tensor *baseline,
                                   size_t baseline_offset,
                                   const h3_gpu_tensor *baseline_indices,
                                   const h3_gpu_tensor *parents,
                                   const h3_gpu_tensor *norm_weight,
                                   const h3_gpu_tensor *modulation,
                                   const h3_gpu_tensor *row_map, uint32_t rows,
                                   uint32_t reduced_rows, uint32_t baseline_rows, uint32_t width,
                                   uint32_t exact_prefix_rows, float update_scale, uint32_t slots,
                                   uint32_t shift_slot, uint32_t scale_slot, float epsilon);

/* ---- device probe: h3_cuda.h:9; h3_gpu_cuda.cu:47-79 ----------------------
 * h3_cuda_probe is what the reference's pipeline calls (h3.c:465, tests/test_h3.c:385); its
 * struct belongs to the pipeline header h3.h (guard H3_H, h3.h:132-146), so it is declared
 * here with the same layout only when that header was not included first. Fields as the
 * reference fills them: device name, "sm_XY", host RAM, device memory twice, and zeros for
 * the three Apple-only fields. */
#ifndef H3_H
typedef struct {
    char name[128];
    char architecture[128];
    uint64_t physical_memory;
    uint64_t recommended_working_set;
    uint64_t max_buffer_length;
    int apple_gpu_family;
    int metal4;
    int unified_memory;
} h3_device_info;
#endif
int h3_cuda_probe(h3_device_info *info, char *error, size_t error_size);
/* The same probe with the fields a CUDA host wants (SM count, compute capability). */
typedef struct {
    char name[256];
    uint64_t total_memory;
    int compute_major, compute_minor, multiprocessors;
} h3b200_device_info;
int h3b200_probe(h3b200_device_info *info, char *error, size_t error_size);

/* ====================================================================== *
 * Extensions (no counterpart in the reference, which is single-device and
 * single-stream). They let a host process that owns device memory and
 * streams (one process per GPU) drive the same ops, and provide the
 * sequence-parallel (Ulysses) layout changes around attention.
 * ====================================================================== */

/* Select the device for contexts created afterwards by this thread
 * (the reference hard-wires device 0, h3_gpu_cuda.cu:98-99). */
int h3x_set_device(int device);
/* Enqueue all later work of this context on `cuda_stream` (a cudaStream_t;
 * NULL = the legacy default stream, which is what the reference uses). */
int h3x_set_stream(h3_gpu *gpu, void *cuda_stream);
/* Non-owning tensor over caller-owned device memory (not freed with the tensor). */
h3_gpu_tensor *h3x_tensor_wrap(h3_gpu *gpu, void *device_pointer, size_t elements,
                               h3_gpu_dtype dtype);
void *h3x_tensor_device_pointer(const h3_gpu_tensor *tensor);
/* Last asynchronous kernel status word (0 = ok), read after h3_gpu_submit(). */
int h3x_kernel_status(h3_gpu *gpu);
/* Every device-side wait is bounded: a kernel that sees no progress for its budget records a
 * status, returns normally, and the next h3_gpu_submit() fails with a message (the context
 * stays usable and the status word is cleared). Budgets are in SM clock cycles; a value <= 0
 * keeps the current one. kernel_cycles bounds the pipeline waits inside the GEMM and attention
 * kernels (default 2e9, about a second); barrier_cycles bounds h3x_peer_barrier, which also
 * absorbs the skew between ranks (default 2e10). Not allowed inside a command. */
int h3x_set_wait_budget_cycles(h3_gpu *gpu, long long kernel_cycles, long long barrier_cycles);

/* Ulysses exchange layout. `packed` holds, for each of `world` peers p, the
 * contiguous block [rows_local][heads/world][head_dim] of heads
 * [p*heads/world, (p+1)*heads/world) taken from src = [rows_local][heads][head_dim].
 * After an all-to-all of equal blocks, rank r holds [world][rows_local][heads/world][hd]
 * = all rows of its head slice, row-sharded order preserved. */
int h3x_ulysses_pack_heads(h3_gpu *gpu, h3_gpu_tensor *packed, const h3_gpu_tensor *src,
                           uint32_t rows_local, uint32_t heads, uint32_t head_dim,
                           uint32_t world);
/* Inverse for the attention output: src = [world][rows_local][heads/world][hd]
 * (after the return all-to-all) -> dst = [rows_local][heads][hd]. */
int h3x_ulysses_unpack_heads(h3_gpu *gpu, h3_gpu_tensor *dst, const h3_gpu_tensor *src,
                             uint32_t rows_local, uint32_t heads, uint32_t head_dim,
                             uint32_t world);

/* Sequence parallelism with the exchange fused into the producing kernels (peer stores over
 * NVLink instead of pack + all-to-all + unpack). Every rank owns symmetric buffers that all
 * peers can address (e.g. torch symmetric memory, cudaIpc or cuMemMap; the caller supplies
 * the pointers as seen from THIS process):
 *   q/k/v gathered buffers  [world * rows_local][heads / world][head_dim]   (rows in global order)
 *   attention output buffer [rows_local][heads][head_dim]
 * h3x_grouped_qkv_linear_rope_push: the QKV projection's epilogue (head norm + RoPE) writes
 *   each head's q/k/v row straight into the gathered buffers of the rank that owns that head.
 * h3x_sdpa_push: attention over this rank's heads; the epilogue writes each output row
 *   straight into the output buffer of the rank that owns that row.
 * Only plain global stores go to peer memory; every TMA load reads local memory. The caller
 * orders the phases across ranks (a barrier on the stream after each of the two calls). */
typedef struct {
    uint32_t world, rank, rows_local;
    void *q[8], *k[8], *v[8];   /* gathered q/k/v buffer of every rank */
    void *o[8];                 /* attention output buffer of every rank */
    void *flags[8];             /* barrier words of every rank: 16 x uint32, zero-initialised */
} h3x_ulysses_peers;
int h3x_grouped_qkv_linear_rope_push(h3_gpu *gpu, const h3x_ulysses_peers *peers,
                                     const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                                     const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                     const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                     uint32_t rows, uint32_t input_dim, uint32_t heads,
                                     uint32_t head_dim, uint32_t rope_half, float epsilon);
int h3x_sdpa_push(h3_gpu *gpu, const h3x_ulysses_peers *peers, const h3_gpu_tensor *query,
                  const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                  uint32_t heads_total, uint32_t head_dim, float scale);
/* Barrier across the ranks on this context's stream: one small kernel that raises this rank's
 * epoch in every peer's flag words (release, system scope) and waits until every peer's epoch
 * arrived in its own. Each rank must run on its own GPU. The wait is bounded (about 10 s of
 * GPU clock unless h3x_set_wait_budget_cycles changed it); when it runs out the kernel status
 * word becomes non-zero and submit fails. */
int h3x_peer_barrier(h3_gpu *gpu, const h3x_ulysses_peers *peers);
/* Device memory that other processes on the node can map (CUDA IPC). alloc returns a zeroed
 * cudaMalloc block and fills the 64-byte handle to send to the peers; open maps a peer's block
 * into this process (peer access is enabled on first use); close unmaps; free releases. */
void *h3x_peer_alloc(h3_gpu *gpu, size_t bytes, void *handle64);
void *h3x_peer_open(h3_gpu *gpu, const void *handle64);
int h3x_peer_close(h3_gpu *gpu, void *mapped);
int h3x_peer_free(h3_gpu *gpu, void *block);

/* Classifier-free guidance combine (the reference has no guidance pass; formula fixed here):
 * out[i] = bf16(uncond[i] + guidance * (cond[i] - uncond[i])), evaluated as one F32 fused
 * multiply-add of the F32 difference. out may alias either input. */
int h3x_cfg_combine_bf16(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *cond,
                         const h3_gpu_tensor *uncond, uint32_t elements, float guidance);

/* The MLP's up projection with its activation, as one op (the first stage of h3_gpu_mlp_bf16,
 * h3_cuda_core.cu:1050-1110, exposed so that a host can time it or keep the activation):
 * fused = bf16(input . fc1^T) with fc1 = [gate rows | up rows] of hidden_dim each, then
 * output[r][c] = bf16(silu(fused[r][c]) * fused[r][hidden_dim + c]); output is [rows][hidden_dim].
 * Counted as one projection. */
int h3x_linear_swiglu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                           const h3_gpu_tensor *fc1_weight, uint32_t rows, uint32_t input_dim,
                           uint32_t hidden_dim);

/* Declares that an F32 tensor serves as a projection weight (on != 0) or no longer does (0).
 * h3_gpu_linear_f32 keeps the scaled FP16 rows of such a weight between calls instead of
 * converting it every time; tensors made by h3_gpu_tensor_load_f32 / h3_gpu_tensor_from_f32 are
 * declared so already. Every call of this library that writes the tensor drops the rows; after a
 * write this library cannot see (a wrapped tensor written by its owner) call this with on again.
 * The F32 norms (h3_gpu_rms_norm_f32, h3_gpu_layer_norm_f32) likewise leave the FP16 rows of their
 * output beside a tensor this library allocated, for the projection that reads it next; they
 * are dropped the same way, and H3B_NO_HALF_ROWS=1 switches that off for a host that writes such
 * tensors through their device pointers. */
int h3x_tensor_keep_half_rows(h3_gpu_tensor *tensor, int on);

/* Final head (adaLN + projection) for callers that must not allocate device memory.
 * No counterpart in the reference: its final head always draws its scratch from a
 * grow-only cudaMalloc'd workspace.
 *
 * Who needs this: a host that has handed all device memory to its own pool before the
 * denoiser runs (a serving process that pre-partitions HBM, so a late cudaMalloc can fail
 * or stall behind the driver's allocation lock), or that calls from a thread where
 * driver allocations are forbidden for latency reasons. h3_gpu_adaln_linear_bf16 grows a
 * cudaMalloc'd workspace on demand; this variant never calls cudaMalloc / cudaFree or any
 * allocating library routine. The caller still passes every input and output tensor.
 *
 * The intermediate (the BF16-rounded adaLN rows, rows * width elements) lives in a fixed
 * 8 MiB array inside the library image, so rows * width may not exceed 4 Mi elements
 * (4,194,304; e.g. 780 rows at the model width 5376); larger calls are rejected with a
 * message and must use h3_gpu_adaln_linear_bf16. Each GPU that loads the library holds
 * those 8 MiB until the process exits.
 *
 * The first call on a device looks up the array's device address (once per device, with
 * the context's device current on the calling thread); make that first call before any
 * stream capture begins. All calls on a device share the one array: it keeps the previous
 * call's contents, which is harmless because every element the projection reads is
 * rewritten first, but two calls whose kernels overlap on the GPU (different streams or
 * contexts on the same device) race on it and must be serialised by the caller.
 * Arguments, results and error behaviour are otherwise those of h3_gpu_adaln_linear_bf16. */
int h3x_adaln_linear_bf16_noalloc(h3_gpu *gpu, h3_gpu_tensor *output, h3_gpu_tensor *inverse,
                                  const h3_gpu_tensor *input, size_t input_offset,
                                  const h3_gpu_tensor *norm_weight,
                                  const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
                                  const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                  uint32_t rows, uint32_t width, uint32_t output_dim,
                                  uint32_t slots, uint32_t shift_slot, uint32_t scale_slot,
                                  float epsilon);

#ifdef __cplusplus
}
#endif
#endif /* H3B200_H */
