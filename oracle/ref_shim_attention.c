/* Exports the reference's own CPU references for QKV-norm-RoPE and SDPA.
 * TEST INFRASTRUCTURE ONLY; see ref_shim_dit.c for the mechanism. */
#define main ref_attention_tests_main
#include "test_cuda_attention.c"
#undef main

void refcpu_qkv_rope(const float *qkv, const float *qw, const float *kw,
                     const float *rc, const float *rs, float *q, float *k,
                     float *v, uint32_t seq, uint32_t heads, uint32_t hd,
                     uint32_t rope_half, int grouped, int weighted, float eps) {
    ref_qkv_rope(qkv, qw, kw, rc, rs, q, k, v, seq, heads, hd, rope_half,
                 grouped, weighted, eps);
}

void refcpu_sdpa(const float *q, const float *k, const float *v, float *out,
                 uint32_t batch, uint32_t seq, uint32_t heads, uint32_t hd,
                 float scale, int causal, int head_major) {
    ref_sdpa(q, k, v, out, batch, seq, heads, hd, scale, causal, head_major);
}
