/* F32 row operations of the video-VAE decoder's transformer (the step after the DiT on the
 * reference's pipeline): RMSNorm, LayerNorm, residual + branch * scale, SwiGLU, and the QKV
 * split with unweighted per-head RMS norm and RoPE. They replace h3k_rms_norm_f32,
 * h3k_layer_norm_f32, h3k_scale_add_f32, h3k_swiglu_f32 (h3_cuda_core.cu:57-66, 92-103,
 * 161-182, 212-250) and h3k_video_qkv_rope_f32 (h3_cuda_attention.cu:125-170) behind the same
 * entry points, with the reference's argument checks (h3_cuda_core.cu:609-628, 673-684,
 * 720-772; h3_cuda_attention.cu:2657-2682).
 *
 * All of them are bandwidth-bound: 16-byte accesses where width and pointers allow, one CTA
 * per row for the norms (the row is read from HBM once and again from L1 for the second and
 * third pass), everything F32 like the reference (its tests hold these to 1e-5).
 *
 * The same file holds the small conversion kernels the F32 attention and F32 projection
 * routes need (F32 -> BF16 with head padding, BF16 -> F32, F32 rows -> scaled FP16 rows).
 */
#include "h3b_common.cuh"

#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <initializer_list>

namespace {

constexpr int kRowThreads = 256;

inline unsigned blocks_for(size_t count, unsigned threads) {
    return unsigned((count + threads - 1) / threads);
}

inline bool aligned16(std::initializer_list<const void *> pointers) {
    for (const void *p : pointers)
        if (reinterpret_cast<uintptr_t>(p) & 15u) return false;
    return true;
}

/* sum over the CTA; every thread gets the result */
__device__ __forceinline__ float cta_sum(float value, float *scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) value += __shfl_xor_sync(0xffffffffu, value, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                       /* scratch may still be read from the previous call */
    if (lane == 0) scratch[warp] = value;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; w++) total += scratch[w];
    return total;
}

/* y = x * rsqrt(mean(x^2) + eps) * weight */
template <bool VEC>
__global__ void __launch_bounds__(kRowThreads)
h3b_rms_norm_f32_kernel(const float *__restrict__ input, const float *__restrict__ weight,
                        float *__restrict__ output, uint32_t width, float epsilon) {
    __shared__ float scratch[kRowThreads / 32];
    const float *x = input + size_t(blockIdx.x) * width;
    float *y = output + size_t(blockIdx.x) * width;
    float local = 0.0f;
    if (VEC) {
        for (uint32_t i = threadIdx.x; i < width / 4; i += kRowThreads) {
            const float4 v = reinterpret_cast<const float4 *>(x)[i];
            local = fmaf(v.x, v.x, local); local = fmaf(v.y, v.y, local);
            local = fmaf(v.z, v.z, local); local = fmaf(v.w, v.w, local);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < width; i += kRowThreads) local = fmaf(x[i], x[i], local);
    }
    const float inverse = 1.0f / sqrtf(cta_sum(local, scratch) / float(width) + epsilon);
    if (VEC) {
        for (uint32_t i = threadIdx.x; i < width / 4; i += kRowThreads) {
            const float4 v = reinterpret_cast<const float4 *>(x)[i];
            const float4 w = __ldg(reinterpret_cast<const float4 *>(weight) + i);
            reinterpret_cast<float4 *>(y)[i] =
                make_float4(v.x * inverse * w.x, v.y * inverse * w.y, v.z * inverse * w.z, v.w * inverse * w.w);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < width; i += kRowThreads) y[i] = x[i] * inverse * weight[i];
    }
}

/* y = (x - mean) * rsqrt(var + eps) * weight + bias, variance of the centred values */
template <bool VEC>
__global__ void __launch_bounds__(kRowThreads)
h3b_layer_norm_f32_kernel(const float *__restrict__ input, const float *__restrict__ weight,
                          const float *__restrict__ bias, float *__restrict__ output, uint32_t width,
                          float epsilon) {
    __shared__ float scratch[kRowThreads / 32];
    const float *x = input + size_t(blockIdx.x) * width;
    float *y = output + size_t(blockIdx.x) * width;
    float local = 0.0f;
    if (VEC) {
        for (uint32_t i = threadIdx.x; i < width / 4; i += kRowThreads) {
            const float4 v = reinterpret_cast<const float4 *>(x)[i];
            local += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < width; i += kRowThreads) local += x[i];
    }
    const float mean = cta_sum(local, scratch) / float(width);
    local = 0.0f;
    if (VEC) {
        for (uint32_t i = threadIdx.x; i < width / 4; i += kRowThreads) {
            const float4 v = reinterpret_cast<const float4 *>(x)[i];
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            local = fmaf(a, a, local); local = fmaf(b, b, local);
            local = fmaf(c, c, local); local = fmaf(d, d, local);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < width; i += kRowThreads) {
            const float a = x[i] - mean;
            local = fmaf(a, a, local);
        }
    }
    const float inverse = 1.0f / sqrtf(cta_sum(local, scratch) / float(width) + epsilon);
    if (VEC) {
        for (uint32_t i = threadIdx.x; i < width / 4; i += kRowThreads) {
            const float4 v = reinterpret_cast<const float4 *>(x)[i];
            const float4 w = __ldg(reinterpret_cast<const float4 *>(weight) + i);
            const float4 b = __ldg(reinterpret_cast<const float4 *>(bias) + i);
            reinterpret_cast<float4 *>(y)[i] =
                make_float4((v.x - mean) * inverse * w.x + b.x, (v.y - mean) * inverse * w.y + b.y,
                            (v.z - mean) * inverse * w.z + b.z, (v.w - mean) * inverse * w.w + b.w);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < width; i += kRowThreads)
            y[i] = (x[i] - mean) * inverse * weight[i] + bias[i];
    }
}

/* out = residual + branch * scale[column] */
template <bool VEC>
__global__ void h3b_scale_add_f32_kernel(const float *__restrict__ residual, const float *__restrict__ branch,
                                         const float *__restrict__ scale, float *__restrict__ output,
                                         size_t items, uint32_t width) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= items) return;
    if (VEC) {
        const uint32_t column = uint32_t((i * 4) % width);
        const float4 r = reinterpret_cast<const float4 *>(residual)[i];
        const float4 b = reinterpret_cast<const float4 *>(branch)[i];
        const float4 s = __ldg(reinterpret_cast<const float4 *>(scale + column));
        reinterpret_cast<float4 *>(output)[i] =
            make_float4(r.x + b.x * s.x, r.y + b.y * s.y, r.z + b.z * s.z, r.w + b.w * s.w);
    } else {
        output[i] = residual[i] + branch[i] * scale[i % width];
    }
}

__device__ __forceinline__ float silu_times(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }

/* fused rows are [gate (width) | up (width)]; out = silu(gate) * up */
template <bool VEC>
__global__ void h3b_swiglu_f32_kernel(const float *__restrict__ fused, float *__restrict__ output, size_t items,
                                      uint32_t width) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= items) return;
    if (VEC) {
        const size_t row = (i * 4) / width;
        const uint32_t column = uint32_t((i * 4) % width);
        const float *base = fused + row * width * 2;
        const float4 g = *reinterpret_cast<const float4 *>(base + column);
        const float4 u = *reinterpret_cast<const float4 *>(base + width + column);
        reinterpret_cast<float4 *>(output)[i] =
            make_float4(silu_times(g.x, u.x), silu_times(g.y, u.y), silu_times(g.z, u.z), silu_times(g.w, u.w));
    } else {
        const size_t row = i / width;
        const uint32_t column = uint32_t(i % width);
        output[i] = silu_times(fused[row * width * 2 + column], fused[row * width * 2 + width + column]);
    }
}

/* One warp per (row, head). Fused rows are [head][q | k | v][dim]; q and k get an unweighted RMS
 * norm over the head, then RoPE on the first 2 * rope_half dims (pairs (d, d + rope_half)); v is
 * copied. */
__global__ void __launch_bounds__(256)
h3b_video_qkv_rope_f32_kernel(const float *__restrict__ qkv, const float *__restrict__ rope_cos,
                              const float *__restrict__ rope_sin, float *__restrict__ query,
                              float *__restrict__ key, float *__restrict__ value, uint32_t sequence,
                              uint32_t heads, uint32_t head_dim, uint32_t rope_half, float epsilon) {
    const size_t unit = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31;
    if (unit >= size_t(sequence) * heads) return;
    const uint32_t row = uint32_t(unit / heads);
    const float *q = qkv + unit * head_dim * 3, *k = q + head_dim, *v = k + head_dim;
    float q_sum = 0.0f, k_sum = 0.0f;
    for (uint32_t d = lane; d < head_dim; d += 32) {
        q_sum = fmaf(q[d], q[d], q_sum);
        k_sum = fmaf(k[d], k[d], k_sum);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        q_sum += __shfl_xor_sync(0xffffffffu, q_sum, o);
        k_sum += __shfl_xor_sync(0xffffffffu, k_sum, o);
    }
    const float q_inverse = 1.0f / sqrtf(q_sum / float(head_dim) + epsilon);
    const float k_inverse = 1.0f / sqrtf(k_sum / float(head_dim) + epsilon);
    const float *cosine = rope_cos + size_t(row) * rope_half, *sine = rope_sin + size_t(row) * rope_half;
    float *q_out = query + unit * head_dim, *k_out = key + unit * head_dim, *v_out = value + unit * head_dim;
    for (uint32_t d = lane; d < head_dim; d += 32) {
        float q0 = q[d] * q_inverse, k0 = k[d] * k_inverse;
        if (d < rope_half) {
            const float q1 = q[d + rope_half] * q_inverse, k1 = k[d + rope_half] * k_inverse;
            const float c = cosine[d], s = sine[d];
            q0 = q0 * c - q1 * s;
            k0 = k0 * c - k1 * s;
        } else if (d < rope_half * 2) {
            const float q1 = q[d - rope_half] * q_inverse, k1 = k[d - rope_half] * k_inverse;
            const float c = cosine[d - rope_half], s = sine[d - rope_half];
            q0 = q0 * c + q1 * s;
            k0 = k0 * c + k1 * s;
        }
        q_out[d] = q0;
        k_out[d] = k0;
        v_out[d] = v[d];
    }
}

/* F32 [units][dims] -> BF16 [units][padded], zeros behind the dims (4 output values per thread);
 * blockIdx.y picks one of up to three tensors of the same shape (q, k, v in one launch) */
struct PadCast {
    const float *in[3];
    uint16_t *out[3];
};
__global__ void h3b_f32_to_bf16_pad_kernel(PadCast tensors, size_t units, uint32_t dims, uint32_t padded) {
    /* picked with selects: indexing the parameter arrays with blockIdx.y would move them to local memory */
    const float *__restrict__ in = blockIdx.y == 0 ? tensors.in[0] : blockIdx.y == 1 ? tensors.in[1] : tensors.in[2];
    uint16_t *__restrict__ out = blockIdx.y == 0 ? tensors.out[0] : blockIdx.y == 1 ? tensors.out[1] : tensors.out[2];
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t groups = padded / 4;
    if (i >= units * groups) return;
    const size_t unit = i / groups;
    const uint32_t d = uint32_t(i % groups) * 4;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (d < dims) v = *reinterpret_cast<const float4 *>(in + unit * dims + d);
    *reinterpret_cast<uint2 *>(out + unit * padded + d) =
        make_uint2(uint32_t(h3b_narrow(v.x)) | uint32_t(h3b_narrow(v.y)) << 16,
                   uint32_t(h3b_narrow(v.z)) | uint32_t(h3b_narrow(v.w)) << 16);
}

/* BF16 [units][padded] -> F32 [units][dims] */
__global__ void h3b_bf16_to_f32_unpad_kernel(const uint16_t *__restrict__ in, float *__restrict__ out, size_t units,
                                             uint32_t dims, uint32_t padded) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t groups = dims / 4;
    if (i >= units * groups) return;
    const size_t unit = i / groups;
    const uint32_t d = uint32_t(i % groups) * 4;
    const uint2 v = *reinterpret_cast<const uint2 *>(in + unit * padded + d);
    *reinterpret_cast<float4 *>(out + unit * dims + d) =
        make_float4(h3b_lo(v.x), h3b_hi(v.x), h3b_lo(v.y), h3b_hi(v.y));
}

/* F32 [rows][k] -> FP16 [rows][k], one CTA per row: the row is scaled by the power of two that
 * brings its largest magnitude into [2^13, 2^14) (FP16 tops out at 65,504; values down to 2^-27 of
 * the row's maximum stay normal numbers) and rounded to nearest; inverse[row] undoes the scale. */
__global__ void __launch_bounds__(kRowThreads)
h3b_scale_rows_f16_kernel(const float *__restrict__ in, uint16_t *__restrict__ out, float *__restrict__ inverse,
                          uint32_t k) {
    __shared__ float scratch[kRowThreads / 32];
    const float *x = in + size_t(blockIdx.x) * k;
    uint16_t *y = out + size_t(blockIdx.x) * k;
    float local = 0.0f;
    for (uint32_t i = threadIdx.x; i < k / 4; i += kRowThreads) {
        const float4 v = reinterpret_cast<const float4 *>(x)[i];
        local = fmaxf(fmaxf(local, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = local;
    __syncthreads();
    float largest = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; w++) largest = fmaxf(largest, scratch[w]);
    /* exponent field of the maximum (0 for zero / subnormal rows, 255 for inf / nan: both get scale 1) */
    const int field = int((__float_as_uint(largest) >> 23) & 0xffu);
    int scale_field = 127 + 13 - (field - 127);
    if (field == 0 || field == 255) scale_field = 127;
    scale_field = min(max(scale_field, 1), 253);
    const float scale = __uint_as_float(uint32_t(scale_field) << 23);
    if (threadIdx.x == 0) inverse[blockIdx.x] = __uint_as_float(uint32_t(254 - scale_field) << 23);
    for (uint32_t i = threadIdx.x; i < k / 4; i += kRowThreads) {
        const float4 v = reinterpret_cast<const float4 *>(x)[i];
        const __half2 lo = __floats2half2_rn(v.x * scale, v.y * scale), hi = __floats2half2_rn(v.z * scale, v.w * scale);
        reinterpret_cast<uint2 *>(y)[i] =
            make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
}

/* ---- producers that also leave their rows as scaled FP16 --------------------------------------
 * A projection (h3_gpu_linear_f32 on the tensor cores) needs its input rows as FP16 scaled per row
 * by a power of two. The norms, whose output feeds a projection in the decoder, hold a whole row
 * in registers anyway, so they write that form beside the F32 result and spare the projection its
 * conversion launch (QKV projection 57 -> 47 us at 1,797 rows, the norm itself +0.5 us). The same
 * was tried for SwiGLU and for the attention result and dropped: one CTA per row with a reduction
 * in the middle cost those two as much as the conversion launch saved. PER = 16-byte vectors per
 * thread (row width <= 1024 * PER). */
__device__ __forceinline__ float cta_max(float value, float *scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = value;
    __syncthreads();
    float largest = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; w++) largest = fmaxf(largest, scratch[w]);
    return largest;
}

/* power-of-two scale that brings `largest` into [2^13, 2^14), and its inverse */
__device__ __forceinline__ float half_row_scale(float largest, float *inverse) {
    const int field = int((__float_as_uint(largest) >> 23) & 0xffu);
    int scale_field = 127 + 13 - (field - 127);
    if (field == 0 || field == 255) scale_field = 127;      /* zero / subnormal / inf / nan rows: scale 1 */
    scale_field = min(max(scale_field, 1), 253);
    *inverse = __uint_as_float(uint32_t(254 - scale_field) << 23);
    return __uint_as_float(uint32_t(scale_field) << 23);
}

__device__ __forceinline__ uint2 to_half4(float4 v, float scale) {
    const __half2 lo = __floats2half2_rn(v.x * scale, v.y * scale), hi = __floats2half2_rn(v.z * scale, v.w * scale);
    return make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
}

template <int PER>
__device__ __forceinline__ void store_half_row(const float4 (&y)[PER], uint32_t vectors, uint16_t *half_row,
                                               float *inverse, float *scratch) {
    float largest = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; j++)
        if (threadIdx.x + j * kRowThreads < vectors)
            largest = fmaxf(fmaxf(largest, fmaxf(fabsf(y[j].x), fabsf(y[j].y))), fmaxf(fabsf(y[j].z), fabsf(y[j].w)));
    float undo;
    const float scale = half_row_scale(cta_max(largest, scratch), &undo);
    if (threadIdx.x == 0) *inverse = undo;
#pragma unroll
    for (int j = 0; j < PER; j++)
        if (threadIdx.x + j * kRowThreads < vectors)
            reinterpret_cast<uint2 *>(half_row)[threadIdx.x + j * kRowThreads] = to_half4(y[j], scale);
}

/* RMSNorm (LAYER = false) or LayerNorm with the row held in registers: one read of x, F32 result,
 * and, when half_rows is given, the scaled FP16 row */
template <bool LAYER, int PER>
__global__ void __launch_bounds__(kRowThreads)
h3b_norm_f32_rows_kernel(const float *__restrict__ input, const float *__restrict__ weight,
                         const float *__restrict__ bias, float *__restrict__ output, uint16_t *__restrict__ half_rows,
                         float *__restrict__ inverse, uint32_t width, float epsilon) {
    __shared__ float scratch[kRowThreads / 32];
    const uint32_t vectors = width / 4;
    const float4 *x = reinterpret_cast<const float4 *>(input + size_t(blockIdx.x) * width);
    float4 v[PER];
    float local = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t i = threadIdx.x + j * kRowThreads;
        v[j] = i < vectors ? x[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (LAYER) {
            local += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        } else {
            local = fmaf(v[j].x, v[j].x, local); local = fmaf(v[j].y, v[j].y, local);
            local = fmaf(v[j].z, v[j].z, local); local = fmaf(v[j].w, v[j].w, local);
        }
    }
    float mean = 0.0f;
    if (LAYER) {
        mean = cta_sum(local, scratch) / float(width);
        local = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (threadIdx.x + j * kRowThreads < vectors) {
                const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                local = fmaf(a, a, local); local = fmaf(b, b, local);
                local = fmaf(c, c, local); local = fmaf(d, d, local);
            }
    }
    const float scale = 1.0f / sqrtf(cta_sum(local, scratch) / float(width) + epsilon);
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t i = threadIdx.x + j * kRowThreads;
        if (i < vectors) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(weight) + i);
            if (LAYER) {
                const float4 b = __ldg(reinterpret_cast<const float4 *>(bias) + i);
                v[j] = make_float4((v[j].x - mean) * scale * w.x + b.x, (v[j].y - mean) * scale * w.y + b.y,
                                   (v[j].z - mean) * scale * w.z + b.z, (v[j].w - mean) * scale * w.w + b.w);
            } else {
                v[j] = make_float4(v[j].x * scale * w.x, v[j].y * scale * w.y, v[j].z * scale * w.z, v[j].w * scale * w.w);
            }
            reinterpret_cast<float4 *>(output + size_t(blockIdx.x) * width)[i] = v[j];
        }
    }
    if (half_rows) store_half_row<PER>(v, vectors, half_rows + size_t(blockIdx.x) * width, inverse + blockIdx.x, scratch);
}

/* launches KERNEL<PER> with the smallest PER in {1, 2, 4, 8} that covers `width` */
#define H3B_FOR_ROW_WIDTH(width, CALL)                \
    do {                                              \
        if ((width) <= 1024) { constexpr int PER = 1; CALL; }        \
        else if ((width) <= 2048) { constexpr int PER = 2; CALL; }   \
        else if ((width) <= 4096) { constexpr int PER = 4; CALL; }   \
        else { constexpr int PER = 8; CALL; }                        \
    } while (0)

}  // namespace

/* Room for the scaled FP16 form of `rows` rows of width k beside tensor t (dropped like a weight's
 * rows by h3b_written): null when the rows cannot feed the tensor-core projection route, when t
 * wraps caller-owned memory (writes by its owner would go unseen), or when H3B_NO_HALF_ROWS=1. */
uint16_t *h3b_half_rows_attach(h3_gpu *gpu, h3_gpu_tensor *t, size_t rows, uint32_t k, float **inverse) {
    static const bool off = [] { const char *v = getenv("H3B_NO_HALF_ROWS"); return v && *v && strcmp(v, "0") != 0; }();
    if (off || t->external || k < 1024 || k % 8 != 0 || k > 8192 || t->elements != rows * k ||
        !h3b_aligned16(t->data))
        return nullptr;
    const size_t row_bytes = (rows * k * sizeof(uint16_t) + 255) & ~size_t(255);
    const size_t bytes = row_bytes + ((rows * sizeof(float) + 255) & ~size_t(255));
    t->half_rows = h3b_device_alloc(gpu, bytes);
    if (!t->half_rows) return nullptr;
    t->half_bytes = bytes;
    t->half_k = k;
    *inverse = reinterpret_cast<float *>(static_cast<uint8_t *>(t->half_rows) + row_bytes);
    return static_cast<uint16_t *>(t->half_rows);
}

void h3b_f32_to_bf16_pad3(h3_gpu *gpu, const float *const in[3], uint16_t *const out[3], size_t units,
                          uint32_t dims, uint32_t padded) {
    const size_t items = units * (padded / 4);
    if (!items) return;
    PadCast tensors;
    for (int i = 0; i < 3; i++) {
        tensors.in[i] = in[i];
        tensors.out[i] = out[i];
    }
    h3b_f32_to_bf16_pad_kernel<<<dim3(blocks_for(items, 256), 3), 256, 0, gpu->stream>>>(tensors, units, dims, padded);
}

void h3b_bf16_to_f32_unpad(h3_gpu *gpu, const uint16_t *in, float *out, size_t units, uint32_t dims,
                           uint32_t padded) {
    const size_t items = units * (dims / 4);
    if (items)
        h3b_bf16_to_f32_unpad_kernel<<<blocks_for(items, 256), 256, 0, gpu->stream>>>(in, out, units, dims, padded);
}

void h3b_scale_rows_f16(h3_gpu *gpu, const float *in, uint16_t *out, float *inverse, size_t rows, uint32_t k) {
    if (rows && k)
        h3b_scale_rows_f16_kernel<<<unsigned(rows), kRowThreads, 0, gpu->stream>>>(in, out, inverse, k);
}

/* ================================================================= C ABI */

extern "C" int h3_gpu_rms_norm_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                   const h3_gpu_tensor *weight, uint32_t rows, uint32_t width,
                                   float epsilon) {
    const size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, input, H3_GPU_F32, count, "RMSNorm input") ||
        !h3b_need(gpu, weight, H3_GPU_F32, width, "RMSNorm weight") ||
        !h3b_need(gpu, output, H3_GPU_F32, count, "RMSNorm output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    if (count) {
        const float *x = h3b_ptr<float>(input), *w = h3b_ptr<float>(weight);
        float *y = h3b_ptr<float>(output);
        if (width % 4 == 0 && width <= 8192 && aligned16({x, w, y})) {
            float *inverse = nullptr;
            uint16_t *half_rows = h3b_half_rows_attach(gpu, output, rows, width, &inverse);
            H3B_FOR_ROW_WIDTH(width, (h3b_norm_f32_rows_kernel<false, PER><<<rows, kRowThreads, 0, gpu->stream>>>(
                                         x, w, nullptr, y, half_rows, inverse, width, epsilon)));
        } else if (width % 4 == 0 && aligned16({x, w, y}))
            h3b_rms_norm_f32_kernel<true><<<rows, kRowThreads, 0, gpu->stream>>>(x, w, y, width, epsilon);
        else
            h3b_rms_norm_f32_kernel<false><<<rows, kRowThreads, 0, gpu->stream>>>(x, w, y, width, epsilon);
    }
    return h3b_launched(gpu, "rms_norm_f32");
}

extern "C" int h3_gpu_layer_norm_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                     const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                     uint32_t rows, uint32_t width, float epsilon) {
    const size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, input, H3_GPU_F32, count, "LayerNorm input") ||
        !h3b_need(gpu, weight, H3_GPU_F32, width, "LayerNorm weight") ||
        !h3b_need(gpu, bias, H3_GPU_F32, width, "LayerNorm bias") ||
        !h3b_need(gpu, output, H3_GPU_F32, count, "LayerNorm output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    if (count) {
        const float *x = h3b_ptr<float>(input), *w = h3b_ptr<float>(weight), *b = h3b_ptr<float>(bias);
        float *y = h3b_ptr<float>(output);
        if (width % 4 == 0 && width <= 8192 && aligned16({x, w, b, y})) {
            float *inverse = nullptr;
            uint16_t *half_rows = h3b_half_rows_attach(gpu, output, rows, width, &inverse);
            H3B_FOR_ROW_WIDTH(width, (h3b_norm_f32_rows_kernel<true, PER><<<rows, kRowThreads, 0, gpu->stream>>>(
                                         x, w, b, y, half_rows, inverse, width, epsilon)));
        } else if (width % 4 == 0 && aligned16({x, w, b, y}))
            h3b_layer_norm_f32_kernel<true><<<rows, kRowThreads, 0, gpu->stream>>>(x, w, b, y, width, epsilon);
        else
            h3b_layer_norm_f32_kernel<false><<<rows, kRowThreads, 0, gpu->stream>>>(x, w, b, y, width, epsilon);
    }
    return h3b_launched(gpu, "layer_norm_f32");
}

extern "C" int h3_gpu_scale_add_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                                    const h3_gpu_tensor *branch, const h3_gpu_tensor *scale,
                                    uint32_t rows, uint32_t width) {
    const size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, residual, H3_GPU_F32, count, "scale-add residual") ||
        !h3b_need(gpu, branch, H3_GPU_F32, count, "scale-add branch") ||
        !h3b_need(gpu, scale, H3_GPU_F32, width, "scale-add scale") ||
        !h3b_need(gpu, output, H3_GPU_F32, count, "scale-add output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    if (count) {
        const float *r = h3b_ptr<float>(residual), *b = h3b_ptr<float>(branch), *s = h3b_ptr<float>(scale);
        float *y = h3b_ptr<float>(output);
        if (width % 4 == 0 && aligned16({r, b, s, y}))
            h3b_scale_add_f32_kernel<true><<<blocks_for(count / 4, 256), 256, 0, gpu->stream>>>(r, b, s, y, count / 4,
                                                                                                  width);
        else
            h3b_scale_add_f32_kernel<false><<<blocks_for(count, 256), 256, 0, gpu->stream>>>(r, b, s, y, count, width);
    }
    return h3b_launched(gpu, "scale_add_f32");
}

extern "C" int h3_gpu_swiglu_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *fused,
                                 uint32_t rows, uint32_t width) {
    const size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, fused, H3_GPU_F32, count * 2, "SwiGLU input") ||
        !h3b_need(gpu, output, H3_GPU_F32, count, "SwiGLU output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    if (count) {
        const float *f = h3b_ptr<float>(fused);
        float *y = h3b_ptr<float>(output);
        if (width % 4 == 0 && aligned16({f, y}))
            h3b_swiglu_f32_kernel<true><<<blocks_for(count / 4, 256), 256, 0, gpu->stream>>>(f, y, count / 4, width);
        else
            h3b_swiglu_f32_kernel<false><<<blocks_for(count, 256), 256, 0, gpu->stream>>>(f, y, count, width);
    }
    return h3b_launched(gpu, "swiglu_f32");
}

extern "C" int h3_gpu_video_qkv_rope_f32(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                                         h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                                         const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                         uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                         uint32_t rope_half, float epsilon) {
    const size_t count = size_t(sequence) * heads * head_dim;
    const size_t rope_count = size_t(sequence) * rope_half;
    if (!h3b_need(gpu, qkv, H3_GPU_F32, count * 3, "video QKV") ||
        !h3b_need(gpu, rope_cos, H3_GPU_F32, rope_count, "video RoPE cosine") ||
        !h3b_need(gpu, rope_sin, H3_GPU_F32, rope_count, "video RoPE sine") ||
        !h3b_need(gpu, query, H3_GPU_F32, count, "video query") ||
        !h3b_need(gpu, key, H3_GPU_F32, count, "video key") ||
        !h3b_need(gpu, value, H3_GPU_F32, count, "video value"))
        return 0;
    if (rope_half * 2 > head_dim) return h3b_fail(gpu, "video RoPE spans more than the head dimension");
    if (!h3b_need_command(gpu)) return 0;
    h3b_written(query);
    h3b_written(key);
    h3b_written(value);
    if (count) {
        const size_t threads = size_t(sequence) * heads * 32;
        h3b_video_qkv_rope_f32_kernel<<<blocks_for(threads, 256), 256, 0, gpu->stream>>>(
            h3b_ptr<float>(qkv), h3b_ptr<float>(rope_cos), h3b_ptr<float>(rope_sin), h3b_ptr<float>(query),
            h3b_ptr<float>(key), h3b_ptr<float>(value), sequence, heads, head_dim, rope_half, epsilon);
    }
    return h3b_launched(gpu, "video_qkv_rope_f32");
}
