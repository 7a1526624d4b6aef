/* Exports the reference's own CPU references for the DiT fused ops.
 * TEST INFRASTRUCTURE ONLY. The reference's test program is compiled in place
 * (it is included, not copied) with its entry point renamed, and thin wrappers
 * make its file-local reference functions callable. */
#define main ref_dit_tests_main
#include "test_cuda_dit.c"
#undef main

void refcpu_adaln(const float *in, const float *w, const float *mod,
                  const uint32_t *row_map, float *out, uint32_t rows,
                  uint32_t width, uint32_t slots, uint32_t shift_slot,
                  uint32_t scale_slot, float eps) {
    ref_adaln(in, w, mod, row_map, out, rows, width, slots, shift_slot,
              scale_slot, eps);
}

void refcpu_gate(const float *res, const float *branch, const float *mod,
                 const uint32_t *row_map, float *out, uint32_t rows,
                 uint32_t width, uint32_t slots, uint32_t gate_slot) {
    ref_gate(res, branch, mod, row_map, out, rows, width, slots, gate_slot);
}

uint16_t refcpu_f32_to_bf16(float value) { return host_f32_to_bf16(value); }
float refcpu_bf16_to_f32(uint16_t value) { return host_bf16_to_f32(value); }
