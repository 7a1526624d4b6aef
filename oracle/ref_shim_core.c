/* Exports the reference's own CPU references for linear / SiLU / SwiGLU.
 * TEST INFRASTRUCTURE ONLY; see ref_shim_dit.c for the mechanism. */
#define main ref_core_tests_main
#include "test_cuda_core.c"
#undef main

void refcpu_linear_f32(const float *in, const float *w, const float *b,
                       float *out, uint32_t rows, uint32_t in_dim,
                       uint32_t out_dim) {
    ref_linear_f32(in, w, b, out, rows, in_dim, out_dim);
}

void refcpu_swiglu(const float *fused, float *out, uint32_t rows,
                   uint32_t width) {
    ref_swiglu(fused, out, rows, width);
}

float refcpu_silu(float x) { return ref_silu(x); }

/* F32 norms of the video-VAE decoder (tests/test_cuda_core.c ref_rms_norm, ref_layer_norm) */
void refcpu_rms_norm(const float *in, const float *w, float *out, uint32_t rows,
                     uint32_t width, float eps) {
    ref_rms_norm(in, w, out, rows, width, eps);
}

void refcpu_layer_norm(const float *in, const float *w, const float *b, float *out,
                       uint32_t rows, uint32_t width, float eps) {
    ref_layer_norm(in, w, b, out, rows, width, eps);
}
