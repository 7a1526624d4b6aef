/* Internal declarations shared by the translation units of libh3b200.so. */
#pragma once

#include "../../include/h3b200.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

/* The first five members keep the order the reference's CUDA tensor has
 * (h3_cuda_internal.h:20-26): one reference test builds offset views by
 * re-declaring that struct (tests/test_cuda_core.c:749-763). */
struct h3_gpu_tensor {
    void *data;
    size_t elements;
    size_t bytes;
    h3_gpu_dtype dtype;
    struct h3_gpu *owner;
    int external;  /* wraps caller-owned memory: never freed or cached */
    /* F32 tensors created with contents (file loads, from_f32) may serve as projection weights:
     * h3_gpu_linear_f32 keeps their rows as scaled FP16 + one F32 scale per row here (see
     * h3b_gemm_f32_half). The norms, whose result usually feeds a projection, leave the same form
     * beside their output. Dropped by h3b_written() whenever
     * this library writes the tensor, and with the tensor. */
    int keeps_half = 0;
    void *half_rows = nullptr;      /* [rows][k] FP16, then rows F32 inverse scales */
    size_t half_bytes = 0;
    uint32_t half_k = 0;
};
/* the tensor's data is about to change: forget what was derived from it */
void h3b_written(h3_gpu_tensor *tensor);

/* Device-side status word written by kernels whose bounded waits expire. */
enum : int {
    H3B_STATUS_OK = 0,
    H3B_STATUS_GEMM_TIMEOUT = 1,
    H3B_STATUS_ATTN_TIMEOUT = 2,
    H3B_STATUS_PEER_TIMEOUT = 3,
};

struct h3b_pinned_slot {
    void *host = nullptr;
    size_t bytes = 0;
    cudaEvent_t done = nullptr;
    bool pending = false;
};

struct h3b_loader;                  /* pinned ring + copy stream of the file loads */
void h3b_loader_free(h3b_loader *loader);
struct h3b_op_profile;              /* per-op device timing, on when H3_PROFILE=2 */
void h3b_profile_record(struct h3_gpu *gpu, const char *what);

struct h3_gpu {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;  /* nullptr = legacy default stream */
    int active = 0;                 /* between begin and submit */
    char error[512] = {0};
    h3_gpu_stats stats = {};
    double command_start = 0.0;

    /* grow-only scratch for intermediates of composite ops (MLP, final head) */
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    /* F32 partial tiles + counters of the GEMMs' split tail round (allocated by the first
     * launch that splits; at most `workers` partial tiles of 128 KiB per 128 rows) */
    static constexpr size_t kSplitScratchBytes = size_t(40) << 20;
    static constexpr size_t kSplitCounterBytes = 4096;
    void *split_scratch = nullptr;
    int split_counters_dirty = 1;   /* the counter words must be cleared before the next split launch */
    int allocation_barred = 0;      /* set while an entry point that must not allocate runs */

    /* exact-size cache of freed device blocks; reuse is ordered by the stream */
    std::unordered_multimap<size_t, void *> cache;
    size_t cache_bytes = 0;
    size_t cache_limit = 0;

    /* pinned staging ring for host -> device writes */
    static constexpr int kSlots = 4;
    static constexpr size_t kSlotMax = size_t(32) << 20;
    h3b_pinned_slot slots[kSlots];
    unsigned next_slot = 0;

    int *status_device = nullptr;   /* kernel status word */
    int status_seen = 0;
    /* budgets of the bounded device-side waits, in SM clock cycles (h3x_set_wait_budget_cycles):
     * pipeline waits inside the GEMM and attention kernels (~1 s), and the cross-rank barrier,
     * which also has to absorb the skew between ranks (~10 s) */
    long long wait_cycles = 2000000000ll;
    long long barrier_cycles = 20000000000ll;

    /* Block-sparse attention mask (h3_gpu_sdpa_set_sparse), regrouped for the tensor-core
     * kernel: one list per CTA (256 query rows = two 128-row query blocks) of steps over
     * 128-key tiles; a step word = key tile index | 4 mask bits << 28, bit 2*t + h set when
     * query block t of the CTA attends the 64-key half h of the tile. */
    uint32_t sparse_rows = 0;
    uint32_t *sparse_cta_ptr = nullptr;   /* device, ctas + 1 offsets */
    uint32_t *sparse_steps = nullptr;     /* device */
    /* the same mask per 128-row query block, for the kernel with one query tile per CTA: a step
     * word = key tile index | 2 mask bits << 28, bit h set when the block attends the 64-key
     * half h of the tile */
    uint32_t *sparse_block_ptr = nullptr;    /* device, query blocks + 1 offsets */
    uint32_t *sparse_block_steps = nullptr;  /* device */

    char profile_label[128] = {0};
    double profile_mark = 0.0;
    h3b_loader *loader = nullptr;   /* created by the first file load */
    h3b_op_profile *op_profile = nullptr;
};

double h3b_now();

inline size_t h3b_item_size(h3_gpu_dtype dtype) {
    return dtype == H3_GPU_BF16 ? 2 : dtype == H3_GPU_I8 ? 1 : 4;
}

inline int h3b_fail(h3_gpu *gpu, const char *format, ...) {
    if (gpu) {
        va_list args;
        va_start(args, format);
        vsnprintf(gpu->error, sizeof(gpu->error), format, args);
        va_end(args);
    }
    return 0;
}

inline int h3b_fail_cuda(h3_gpu *gpu, const char *what, cudaError_t status) {
    return h3b_fail(gpu, "CUDA %s failed: %s", what, cudaGetErrorString(status));
}

/* Which statistics counter a launch belongs to (reference h3_cuda_internal.h:142-156). */
enum h3b_kind { H3B_DIRECT = 0, H3B_LINEAR = 1, H3B_CONV = 2, H3B_SDPA = 3 };

inline int h3b_launched(h3_gpu *gpu, const char *what, h3b_kind kind = H3B_DIRECT) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return h3b_fail_cuda(gpu, what, status);
    if (gpu->op_profile) h3b_profile_record(gpu, what);
    switch (kind) {
        case H3B_LINEAR: gpu->stats.mps_linear_dispatches++; break;
        case H3B_CONV: gpu->stats.mps_conv_dispatches++; break;
        case H3B_SDPA: gpu->stats.mps_sdpa_dispatches++; break;
        default: gpu->stats.direct_dispatches++; break;
    }
    return 1;
}

inline int h3b_need_command(h3_gpu *gpu) {
    if (!gpu || !gpu->active) return h3b_fail(gpu, "no active command buffer");
    return 1;
}

inline int h3b_need(h3_gpu *gpu, const h3_gpu_tensor *t, h3_gpu_dtype dtype, size_t elements,
                    const char *label) {
    if (!t || t->dtype != dtype) return h3b_fail(gpu, "%s tensor has the wrong dtype", label);
    if (t->elements < elements) return h3b_fail(gpu, "%s tensor is too small", label);
    return 1;
}

void *h3b_workspace(h3_gpu *gpu, size_t bytes);

template <class T>
inline T *h3b_ptr(const h3_gpu_tensor *t, size_t offset = 0) {
    return reinterpret_cast<T *>(t->data) + offset;
}

inline bool h3b_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

/* ---- device helpers --------------------------------------------------- */
#ifdef __CUDACC__
__device__ __forceinline__ float h3b_widen(uint16_t v) {
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
}
/* round to nearest even with the reference's integer formula */
__device__ __forceinline__ uint16_t h3b_narrow(float v) {
    uint32_t bits = __float_as_uint(v);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return static_cast<uint16_t>(bits >> 16);
}
__device__ __forceinline__ uint32_t h3b_narrow2(float lo, float hi) {
    return static_cast<uint32_t>(h3b_narrow(lo)) | (static_cast<uint32_t>(h3b_narrow(hi)) << 16);
}
__device__ __forceinline__ float h3b_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float h3b_hi(uint32_t packed) {
    return __uint_as_float(packed & 0xffff0000u);
}
__device__ __forceinline__ float h3b_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
#endif

/* ---- cross-unit entry points ------------------------------------------ */
/* C[rows,n] = X[rows,k] . W[n,k]^T (+bias) with BF16 in/out and F32 accumulate.
 * Picks the tcgen05 kernel when the shape allows it, else the SIMT kernel. */
enum h3b_gemm_epilogue {
    H3B_EPI_STORE = 0,    /* out[r][c] = bf16(acc + bias[c])                          */
    H3B_EPI_SWIGLU = 1,   /* W = [gate rows | up rows]; out[r][c] = swiglu, n = hidden */
    H3B_EPI_QKV_ROPE = 2, /* grouped QKV: per-head RMSNorm + RoPE, writes q/k/v directly   */
    H3B_EPI_STORE_F32 = 3, /* out[r][c] = acc + bias[c], F32 output and bias                */
};
/* Fused QKV projection + per-head RMSNorm + RoPE for head_dim 128, rope_half 48, grouped
 * layout. Returns -1 when the shape cannot take the fused kernel (caller runs the two-step
 * route), else 1/0 like every op. */
int h3b_qkv_rope_gemm(h3_gpu *gpu, uint16_t *q, uint16_t *k, uint16_t *v, const uint16_t *x,
                      const uint16_t *w, const uint16_t *q_norm, const uint16_t *k_norm,
                      const uint16_t *rope_cos, const uint16_t *rope_sin, uint32_t rows,
                      uint32_t in_dim, uint32_t heads, float eps,
                      const h3x_ulysses_peers *peers = nullptr);
int h3b_gemm_bf16(h3_gpu *gpu, uint16_t *out, const uint16_t *x, const uint16_t *w,
                  const uint16_t *bias, uint32_t rows, uint32_t k, uint32_t n,
                  h3b_gemm_epilogue epilogue, const char *what);
int h3b_swiglu_launch(h3_gpu *gpu, uint16_t *out, const uint16_t *fused, uint32_t rows,
                      uint32_t width);
int h3b_qkv_rope_launch(h3_gpu *gpu, uint16_t *q, uint16_t *k, uint16_t *v, const uint16_t *qkv,
                        const uint16_t *qn, const uint16_t *kn, const uint16_t *rc,
                        const uint16_t *rs, uint32_t seq, uint32_t heads, uint32_t hd,
                        uint32_t rope_half, int grouped, float eps);
bool h3b_tensor_map_available();
/* F32 projection on the 16-bit tensor cores: C[rows,n] = X[rows,k] . W[n,k]^T (+bias), all F32 in
 * memory. Every row of X and of W is scaled by a power of two that brings its largest
 * magnitude to [2^13, 2^14) and rounded to FP16 (10 mantissa bits, the same as the TF32 format the
 * reference uses for this call, h3_cuda_gemm.cu:242-254, but rounded to nearest instead of
 * truncated, and at twice TF32's tensor rate); the epilogue multiplies the F32 accumulator by the
 * two inverse scales (exact) and adds the bias. The weight's FP16 rows are kept with the weight
 * tensor when it was created with contents. Returns -1 when the shape cannot take this route
 * (caller runs the exact F32 kernel). */
int h3b_gemm_f32_half(h3_gpu *gpu, float *out, const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                      const float *bias, uint32_t rows, uint32_t k, uint32_t n);
/* scaled FP16 rows beside an activation tensor, written by the op that produces it (h3b_f32ops.cu) */
uint16_t *h3b_half_rows_attach(h3_gpu *gpu, h3_gpu_tensor *t, size_t rows, uint32_t k, float **inverse);

void *h3b_device_alloc(h3_gpu *gpu, size_t bytes);           /* the tensors' block cache */
void h3b_device_release(h3_gpu *gpu, void *data, size_t bytes);
/* conversion kernels (h3b_f32ops.cu) */
void h3b_f32_to_bf16_pad3(h3_gpu *gpu, const float *const in[3], uint16_t *const out[3], size_t units,
                          uint32_t dims, uint32_t padded);
void h3b_bf16_to_f32_unpad(h3_gpu *gpu, const uint16_t *in, float *out, size_t units, uint32_t dims,
                           uint32_t padded);
/* F32 [rows][k] -> FP16 [rows][k] scaled per row by a power of two, inverse scales to `inverse` */
void h3b_scale_rows_f16(h3_gpu *gpu, const float *in, uint16_t *out, float *inverse, size_t rows, uint32_t k);
