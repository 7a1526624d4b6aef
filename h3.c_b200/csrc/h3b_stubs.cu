/* Entry points of the reference device API that are not on the DiT denoiser
 * path (VAE convolutions, Qwen text/vision encoders, F32 diagnosis ops and the
 * Metal-only int8 / NAX routes). They are exported so that a complete libh3
 * still links against this library, and fail with a message when called; the
 * reference does the same for the ops its CUDA backend lacks
 * (h3_cuda_dit.cu:1072-1216). Every definition carries the full argument list
 * declared in include/h3b200_offpath.h, so a mismatch with the declared C
 * prototype is a compile error.
 */
#include "h3b_common.cuh"
#include "../../include/h3b200_offpath.h"

/* The message keeps the wording the reference's own test looks for
 * (tests/test_cuda_dit.c:771-817). */
static int metal_only(h3_gpu *gpu, const char *name) {
    return h3b_fail(gpu, "%s is a Metal-only route and is not available in the CUDA backend", name);
}

static int off_path(h3_gpu *gpu, const char *name) {
    return h3b_fail(gpu, "%s is outside the DiT path and is not provided by libh3b200", name);
}

extern "C" int h3_gpu_quantize_weight_int8(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t) { return metal_only(gpu, "h3_gpu_quantize_weight_int8"); }
extern "C" int h3_gpu_linear_int8_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor
    *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t,
    uint32_t, int) { return metal_only(gpu, "h3_gpu_linear_int8_bf16"); }
extern "C" int h3_gpu_linear_int8_head_major_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t,
    uint32_t, uint32_t, uint32_t) { return metal_only(gpu, "h3_gpu_linear_int8_head_major_bf16"); }
extern "C" int h3_gpu_mlp_int8_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t,
    uint32_t, uint32_t, uint32_t, int, int, int, int) { return metal_only(gpu,
    "h3_gpu_mlp_int8_bf16"); }
extern "C" int h3_gpu_mlp_nax_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t,
    uint32_t) { return metal_only(gpu, "h3_gpu_mlp_nax_bf16"); }
extern "C" int h3_gpu_gate_adaln_quantize_int8(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t, uint32_t, uint32_t, float) { return metal_only(gpu,
    "h3_gpu_gate_adaln_quantize_int8"); }
extern "C" int h3_gpu_grouped_qkv_linear_rope_int8(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float, int, int, int,
    int) { return metal_only(gpu, "h3_gpu_grouped_qkv_linear_rope_int8"); }
extern "C" int h3_gpu_conv1d_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_conv1d_f32"); }
extern "C" int h3_gpu_conv1d_stride_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_conv1d_stride_f32"); }
extern "C" int h3_gpu_conv_transpose1d_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_conv_transpose1d_f32"); }
extern "C" int h3_gpu_conv3d_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t) { return off_path(gpu,
    "h3_gpu_conv3d_f32"); }
extern "C" int h3_gpu_weight_norm_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_weight_norm_f32"); }
extern "C" int h3_gpu_add_scaled_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, float, float, uint32_t) { return off_path(gpu, "h3_gpu_add_scaled_f32"); }
extern "C" int h3_gpu_alias_free_snake_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_alias_free_snake_f32"); }
extern "C" int h3_gpu_snake1d_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_snake1d_f32"); }
extern "C" int h3_gpu_audio_qkv_split_f32(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t) { return off_path(gpu,
    "h3_gpu_audio_qkv_split_f32"); }
extern "C" int h3_gpu_audio_attention_pool_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t, uint32_t, uint32_t, uint32_t) { return off_path(gpu,
    "h3_gpu_audio_attention_pool_f32"); }
extern "C" int h3_gpu_sdpa_causal_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float) { return
    off_path(gpu, "h3_gpu_sdpa_causal_f32"); }
extern "C" int h3_gpu_geglu_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t) { return off_path(gpu, "h3_gpu_geglu_f32"); }
extern "C" int h3_gpu_clip_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, float,
    float) { return off_path(gpu, "h3_gpu_clip_f32"); }
extern "C" int h3_gpu_vae_encoder_pad_f32(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t,
    uint32_t) { return off_path(gpu, "h3_gpu_vae_encoder_pad_f32"); }
extern "C" int h3_gpu_vae_encoder_group_norm_silu_f32(h3_gpu *gpu, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t,
    uint32_t, uint32_t, uint32_t, float) { return off_path(gpu,
    "h3_gpu_vae_encoder_group_norm_silu_f32"); }
extern "C" int h3_gpu_qkv_rope_f32(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, h3_gpu_tensor *,
    const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *,
    const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float) { return off_path(gpu,
    "h3_gpu_qkv_rope_f32"); }
extern "C" int h3_gpu_embedding_bf16(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, uint32_t, uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_embedding_bf16");
    }
extern "C" int h3_gpu_gelu_bf16(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, int)
    { return off_path(gpu, "h3_gpu_gelu_bf16"); }
extern "C" int h3_gpu_layer_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, float) { return off_path(gpu,
    "h3_gpu_layer_norm_bf16"); }
extern "C" int h3_gpu_head_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *,
    uint32_t, uint32_t, uint32_t, float) { return off_path(gpu, "h3_gpu_head_rms_norm_bf16"); }
extern "C" int h3_gpu_vision_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *,
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t,
    uint32_t, uint32_t, uint32_t) { return off_path(gpu, "h3_gpu_vision_qkv_rope_bf16"); }
extern "C" int h3_gpu_text_qk_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float) { return
    off_path(gpu, "h3_gpu_text_qk_rope_bf16"); }
extern "C" int h3_gpu_rope_text_bf16(h3_gpu *gpu, h3_gpu_tensor *, h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t) { return
    off_path(gpu, "h3_gpu_rope_text_bf16"); }
extern "C" int h3_gpu_gqa_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *, const h3_gpu_tensor *, const
    h3_gpu_tensor *, const h3_gpu_tensor *, uint32_t, uint32_t, uint32_t, uint32_t, float) { return
    off_path(gpu, "h3_gpu_gqa_causal_bf16"); }
