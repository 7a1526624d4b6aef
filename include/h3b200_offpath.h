/* Entry points of the reference device API (reference h3_gpu.h) that lie outside the DiT denoiser
 * path. libh3b200.so exports them so that a complete libh3 links against it; each one fails with
 * a message (returns 0, text from h3_gpu_error). The reference does the same for the ops its CUDA
 * backend lacks (h3_cuda_dit.cu:1072-1216). Declared here with their full argument lists so the
 * compiler checks the library's definitions, and, when the reference header is included in the
 * same translation unit, checks these lists against the reference's declarations.
 * Parameter names are omitted: nothing is read from them. */
#ifndef H3B200_OFFPATH_H
#define H3B200_OFFPATH_H

#include "h3b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Metal 4 TensorOps / int8 routes: the capability probes answer 0, so the model layer never
 * takes them */
int h3_gpu_quantize_weight_int8(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t);
int h3_gpu_linear_int8_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t,
    int);
int h3_gpu_linear_int8_head_major_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t,
    uint32_t, uint32_t);
int h3_gpu_mlp_int8_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor
    *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t,
    uint32_t, uint32_t, int, int, int, int);
int h3_gpu_mlp_nax_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t);
int h3_gpu_gate_adaln_quantize_int8(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t, float);
int h3_gpu_grouped_qkv_linear_rope_int8(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float, int, int, int, int);

/* audio / video VAE, Qwen text / vision encoders, F32 diagnosis ops */
int h3_gpu_conv1d_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int h3_gpu_conv1d_stride_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor
    *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t);
int h3_gpu_conv_transpose1d_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t);
int h3_gpu_conv3d_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t, uint32_t, uint32_t);
int h3_gpu_weight_norm_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t);
int h3_gpu_add_scaled_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    float, float, uint32_t);
int h3_gpu_alias_free_snake_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t,
    uint32_t, uint32_t);
int h3_gpu_snake1d_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t, uint32_t);
int h3_gpu_audio_qkv_split_f32(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t,
    uint32_t, uint32_t, uint32_t);
int h3_gpu_audio_attention_pool_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t,
    uint32_t, uint32_t, uint32_t, uint32_t);
int h3_gpu_sdpa_causal_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float);
int h3_gpu_geglu_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t);
int h3_gpu_clip_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, float, float);
int h3_gpu_vae_encoder_pad_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t,
    uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int h3_gpu_vae_encoder_group_norm_silu_f32(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, float);
int h3_gpu_qkv_rope_f32(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float);
int h3_gpu_embedding_bf16(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t, uint32_t);
int h3_gpu_gelu_bf16(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, int);
int h3_gpu_layer_norm_bf16(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, uint32_t, uint32_t, float);
int h3_gpu_head_rms_norm_bf16(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t,
    uint32_t, float);
int h3_gpu_vision_qkv_rope_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t,
    uint32_t);
int h3_gpu_text_qk_rope_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float);
int h3_gpu_rope_text_bf16(h3_gpu *, h3_gpu_tensor *, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t);
int h3_gpu_gqa_causal_bf16(h3_gpu *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float);

#ifdef __cplusplus
}
#endif
#endif /* H3B200_OFFPATH_H */
