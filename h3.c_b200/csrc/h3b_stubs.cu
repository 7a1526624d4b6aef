/* Entry points of the reference device API that are not on the DiT denoiser
 * path (VAE convolutions, Qwen text/vision encoders, F32 diagnosis ops and the
 * Metal-only int8 / NAX routes). They are exported so that a complete libh3
 * still links against this library, and fail with a message when called; the
 * reference does the same for the ops its CUDA backend lacks
 * (h3_cuda_dit.cu:1072-1216).
 *
 * Every one of these functions takes the context as its first argument and
 * returns int; the remaining arguments are ignored, so the definitions keep
 * only the first parameter (with the C calling convention the caller owns the
 * argument area, so the extra arguments are harmless).
 */
#include "h3b_common.cuh"

#define H3B_NOT_ON_DIT_PATH(name)                                                        \
    extern "C" int name(h3_gpu *gpu) {                                                   \
        return h3b_fail(gpu, #name " is outside the DiT path and is not provided by "    \
                                   "libh3b200");                                         \
    }

/* Metal 4 TensorOps / NAX int8 routes. The capability probes answer 0, so the model
 * layer never takes them; the message keeps the wording the reference's own test looks
 * for (tests/test_cuda_dit.c:771-817). */
#define H3B_METAL_ONLY(name)                                                             \
    extern "C" int name(h3_gpu *gpu) {                                                   \
        return h3b_fail(gpu, #name " is a Metal-only route and is not available in the " \
                                   "CUDA backend");                                      \
    }
H3B_METAL_ONLY(h3_gpu_quantize_weight_int8)
H3B_METAL_ONLY(h3_gpu_linear_int8_bf16)
H3B_METAL_ONLY(h3_gpu_linear_int8_head_major_bf16)
H3B_METAL_ONLY(h3_gpu_mlp_int8_bf16)
H3B_METAL_ONLY(h3_gpu_mlp_nax_bf16)
H3B_METAL_ONLY(h3_gpu_gate_adaln_quantize_int8)
H3B_METAL_ONLY(h3_gpu_grouped_qkv_linear_rope_int8)
/* audio / video VAE */
H3B_NOT_ON_DIT_PATH(h3_gpu_conv1d_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_conv1d_stride_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_conv_transpose1d_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_conv3d_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_weight_norm_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_add_scaled_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_alias_free_snake_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_snake1d_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_audio_qkv_split_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_audio_attention_pool_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_sdpa_causal_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_geglu_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_clip_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_vae_encoder_pad_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_vae_encoder_group_norm_silu_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_video_qkv_rope_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_sdpa_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_qkv_rope_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_rms_norm_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_layer_norm_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_scale_add_f32)
H3B_NOT_ON_DIT_PATH(h3_gpu_swiglu_f32)
/* Qwen text / vision encoders */
H3B_NOT_ON_DIT_PATH(h3_gpu_embedding_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_gelu_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_layer_norm_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_head_rms_norm_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_vision_qkv_rope_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_text_qk_rope_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_rope_text_bf16)
H3B_NOT_ON_DIT_PATH(h3_gpu_gqa_causal_bf16)
