/* Bandwidth-bound row and elementwise kernels of the DiT block:
 * adaLN, gated residual (+ adaLN of the next sub-layer), RMSNorm, final-head
 * normalisation, SwiGLU/SiLU, add/sub, Euler update, token pooling/restore.
 * Replaces the reference's h3_cuda_dit.cu and the elementwise part of
 * h3_cuda_core.cu behind the same C ABI.
 *
 * Layout: one CTA per row. On the fast path every thread owns up to three
 * 16-byte vectors (8 BF16) of the row, loaded once with 128-bit loads and kept
 * in registers across the reduction, so a fused gate+adaLN touches each input
 * byte once and each output byte once. Sum of squares: per-thread partial ->
 * warp shuffle -> one shared-memory hop. A scalar path with the row cached in
 * shared memory serves odd widths and unaligned offsets (the reference's test
 * shapes); arithmetic and BF16 rounding points are identical on both paths.
 */
#include "h3b_common.cuh"

namespace {

constexpr int kRowThreads = 256;
constexpr int kMaxVecPerThread = 3;           /* 256 * 3 * 8 = 6144 >= 5376 */
constexpr uint32_t kFusedWidthLimit = 5376;   /* reference h3_cuda_dit.cu:763 */
constexpr uint32_t kNoBaseline = 0xffffffffu;

enum RowMode {
    ROW_ADALN,         /* x = input                                        */
    ROW_GATE_ADALN,    /* x = bf16(residual + branch * gate), stored       */
    ROW_POOL_ADALN,    /* x = pooled pair, stored + snapshots              */
    ROW_EXPAND_ADALN,  /* x = restored token, stored                       */
    ROW_RMS_NORM,      /* out = bf16((x * inv) * w)                        */
    ROW_RMS_INVERSE,   /* inverse[row] only                                */
    ROW_ADALN_KEEP,    /* adaLN + inverse[row] (final head)                */
};

struct RowArgs {
    const uint16_t *input;       /* ADALN / RMS: rows x width (already offset)          */
    const uint16_t *residual;    /* GATE_ADALN                                           */
    const uint16_t *branch;      /* GATE_ADALN                                           */
    const uint16_t *gate_mod;    /* GATE_ADALN                                           */
    const uint16_t *norm;        /* [width]                                              */
    const uint16_t *norm_mod;    /* shift/scale table                                    */
    const uint32_t *row_map;
    uint16_t *stored;            /* gated residual / pooled / restored rows              */
    uint16_t *output;
    float *inverse;
    /* token reduction */
    const uint32_t *pairs;
    const uint32_t *parents;
    const uint32_t *baseline_indices;
    uint16_t *original_w;        /* POOL: snapshot of the full grid (already offset)      */
    uint16_t *baseline_w;        /* POOL: pooled baseline rows (already offset)           */
    const uint16_t *original_r;  /* EXPAND (already offset)                              */
    const uint16_t *reduced;
    const uint16_t *baseline_r;  /* EXPAND (already offset)                              */
    uint32_t rows, width, slots, gate_slot, shift_slot, scale_slot, exact_prefix_rows;
    float epsilon, update_scale;
};

struct Vec8 {
    float v[8];
};

__device__ __forceinline__ Vec8 unpack8(const uint4 raw) {
    Vec8 r;
    r.v[0] = h3b_lo(raw.x); r.v[1] = h3b_hi(raw.x);
    r.v[2] = h3b_lo(raw.y); r.v[3] = h3b_hi(raw.y);
    r.v[4] = h3b_lo(raw.z); r.v[5] = h3b_hi(raw.z);
    r.v[6] = h3b_lo(raw.w); r.v[7] = h3b_hi(raw.w);
    return r;
}

__device__ __forceinline__ Vec8 load8(const uint16_t *p) {
    return unpack8(*reinterpret_cast<const uint4 *>(p));
}

__device__ __forceinline__ uint4 pack8(const Vec8 &x) {
    return make_uint4(h3b_narrow2(x.v[0], x.v[1]), h3b_narrow2(x.v[2], x.v[3]),
                      h3b_narrow2(x.v[4], x.v[5]), h3b_narrow2(x.v[6], x.v[7]));
}

__device__ __forceinline__ void store8(uint16_t *p, const Vec8 &x) {
    *reinterpret_cast<uint4 *>(p) = pack8(x);
}

/* round to BF16 and keep the rounded value as F32 */
__device__ __forceinline__ float round_bf(float v) { return h3b_widen(h3b_narrow(v)); }

__device__ __forceinline__ float block_sum(float v, float *scratch) {
    v = h3b_warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int warps = (blockDim.x + 31) >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < warps; w++) total += scratch[w];
    return total;
}

/* Element x[col] of the row before normalisation, with the mode's side effects. */
template <int MODE>
__device__ __forceinline__ float row_value(const RowArgs &a, uint32_t row, uint32_t col,
                                           size_t gate_base, uint32_t first, uint32_t second,
                                           bool direct, uint32_t baseline_row) {
    size_t at = size_t(row) * a.width + col;
    if (MODE == ROW_GATE_ADALN) {
        float gate = h3b_widen(a.gate_mod[gate_base + col]);
        uint16_t g = h3b_narrow(h3b_widen(a.residual[at]) + h3b_widen(a.branch[at]) * gate);
        a.stored[at] = g;
        return h3b_widen(g);
    } else if (MODE == ROW_POOL_ADALN) {
        uint16_t lhs = a.input[size_t(first) * a.width + col];
        a.original_w[size_t(first) * a.width + col] = lhs;
        uint16_t pooled = lhs;
        if (first != second) {
            uint16_t rhs = a.input[size_t(second) * a.width + col];
            a.original_w[size_t(second) * a.width + col] = rhs;
            pooled = h3b_narrow((h3b_widen(lhs) + h3b_widen(rhs)) * 0.5f);
        }
        a.stored[at] = pooled;
        if (baseline_row != kNoBaseline) a.baseline_w[size_t(baseline_row) * a.width + col] = pooled;
        return h3b_widen(pooled);
    } else if (MODE == ROW_EXPAND_ADALN) {
        uint16_t value = a.reduced[size_t(first) * a.width + col];
        if (!direct) {
            float update = h3b_widen(value) -
                           h3b_widen(a.baseline_r[size_t(baseline_row) * a.width + col]);
            value = h3b_narrow(h3b_widen(a.original_r[at]) + a.update_scale * update);
        }
        a.stored[at] = value;
        return h3b_widen(value);
    } else {
        return h3b_widen(a.input[at]);
    }
}

template <int MODE>
__device__ __forceinline__ void row_setup(const RowArgs &a, uint32_t row, uint32_t &first,
                                          uint32_t &second, bool &direct,
                                          uint32_t &baseline_row) {
    first = second = 0;
    direct = true;
    baseline_row = kNoBaseline;
    if (MODE == ROW_POOL_ADALN) {
        first = a.pairs[2 * row];
        second = a.pairs[2 * row + 1];
        baseline_row = a.baseline_indices[row];
    } else if (MODE == ROW_EXPAND_ADALN) {
        first = a.parents[row];
        baseline_row = a.baseline_indices[first];
        direct = row < a.exact_prefix_rows || baseline_row == kNoBaseline;
    }
}

/* Scalar path: any width, any alignment. The row is cached as BF16 in dynamic
 * shared memory when it fits (cached != 0), else re-read from global. */
template <int MODE>
__global__ void h3b_row_scalar(RowArgs a, int cached) {
    extern __shared__ uint16_t row_cache[];
    __shared__ float scratch[32];
    uint32_t row = blockIdx.x;
    if (row >= a.rows) return;
    uint32_t first, second, baseline_row;
    bool direct;
    row_setup<MODE>(a, row, first, second, direct, baseline_row);
    size_t mod_base = 0, gate_base = 0;
    if (MODE != ROW_RMS_NORM && MODE != ROW_RMS_INVERSE)
        mod_base = size_t(a.row_map[row]) * a.slots * a.width;
    if (MODE == ROW_GATE_ADALN) gate_base = mod_base + size_t(a.gate_slot) * a.width;
    float local = 0.0f;
    for (uint32_t col = threadIdx.x; col < a.width; col += blockDim.x) {
        float x = row_value<MODE>(a, row, col, gate_base, first, second, direct, baseline_row);
        if (cached) row_cache[col] = h3b_narrow(x);  /* exact: x is a BF16 value */
        local = fmaf(x, x, local);
    }
    float inv = 1.0f / sqrtf(block_sum(local, scratch) / float(a.width) + a.epsilon);
    if ((MODE == ROW_RMS_INVERSE || MODE == ROW_ADALN_KEEP) && threadIdx.x == 0)
        a.inverse[row] = inv;
    if (MODE == ROW_RMS_INVERSE) return;
    for (uint32_t col = threadIdx.x; col < a.width; col += blockDim.x) {
        float x;
        if (cached) x = h3b_widen(row_cache[col]);
        else if (MODE == ROW_ADALN || MODE == ROW_RMS_NORM || MODE == ROW_ADALN_KEEP)
            x = h3b_widen(a.input[size_t(row) * a.width + col]);
        else
            x = h3b_widen(a.stored[size_t(row) * a.width + col]);
        float w = h3b_widen(a.norm[col]);
        float y;
        if (MODE == ROW_RMS_NORM) {
            y = (x * inv) * w;
        } else {
            float shift = h3b_widen(a.norm_mod[mod_base + size_t(a.shift_slot) * a.width + col]);
            float scale = h3b_widen(a.norm_mod[mod_base + size_t(a.scale_slot) * a.width + col]);
            y = (x * inv * w) * (1.0f + scale) + shift;
        }
        a.output[size_t(row) * a.width + col] = h3b_narrow(y);
    }
}

/* Vector path: width % 8 == 0, width <= 8 * blockDim.x * VPT, 16-byte aligned rows. */
template <int MODE, int VPT>
__global__ void __launch_bounds__(kRowThreads) h3b_row_vector(RowArgs a) {
    __shared__ float scratch[32];
    uint32_t row = blockIdx.x;
    if (row >= a.rows) return;
    uint32_t first, second, baseline_row;
    bool direct;
    row_setup<MODE>(a, row, first, second, direct, baseline_row);
    const uint32_t vectors = a.width >> 3;
    size_t mod_base = 0;
    if (MODE != ROW_RMS_NORM && MODE != ROW_RMS_INVERSE)
        mod_base = size_t(a.row_map[row]) * a.slots * a.width;
    const size_t row_base = size_t(row) * a.width;

    Vec8 x[VPT];
    float local = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        uint32_t vec = threadIdx.x + i * blockDim.x;
        if (vec >= vectors) continue;
        uint32_t col = vec << 3;
        if (MODE == ROW_GATE_ADALN) {
            Vec8 r = load8(a.residual + row_base + col);
            Vec8 b = load8(a.branch + row_base + col);
            Vec8 g = load8(a.gate_mod + mod_base + size_t(a.gate_slot) * a.width + col);
#pragma unroll
            for (int e = 0; e < 8; e++) x[i].v[e] = round_bf(r.v[e] + b.v[e] * g.v[e]);
            store8(a.stored + row_base + col, x[i]);
        } else if (MODE == ROW_POOL_ADALN) {
            uint4 lhs = *reinterpret_cast<const uint4 *>(a.input + size_t(first) * a.width + col);
            *reinterpret_cast<uint4 *>(a.original_w + size_t(first) * a.width + col) = lhs;
            x[i] = load8(reinterpret_cast<const uint16_t *>(&lhs));
            if (first != second) {
                uint4 rhs =
                    *reinterpret_cast<const uint4 *>(a.input + size_t(second) * a.width + col);
                *reinterpret_cast<uint4 *>(a.original_w + size_t(second) * a.width + col) = rhs;
                Vec8 other = load8(reinterpret_cast<const uint16_t *>(&rhs));
#pragma unroll
                for (int e = 0; e < 8; e++) x[i].v[e] = round_bf((x[i].v[e] + other.v[e]) * 0.5f);
            }
            store8(a.stored + row_base + col, x[i]);
            if (baseline_row != kNoBaseline)
                store8(a.baseline_w + size_t(baseline_row) * a.width + col, x[i]);
        } else if (MODE == ROW_EXPAND_ADALN) {
            x[i] = load8(a.reduced + size_t(first) * a.width + col);
            if (!direct) {
                Vec8 base = load8(a.baseline_r + size_t(baseline_row) * a.width + col);
                Vec8 orig = load8(a.original_r + row_base + col);
#pragma unroll
                for (int e = 0; e < 8; e++)
                    x[i].v[e] = round_bf(orig.v[e] + a.update_scale * (x[i].v[e] - base.v[e]));
            }
            store8(a.stored + row_base + col, x[i]);
        } else {
            x[i] = load8(a.input + row_base + col);
        }
#pragma unroll
        for (int e = 0; e < 8; e++) local = fmaf(x[i].v[e], x[i].v[e], local);
    }
    float inv = 1.0f / sqrtf(block_sum(local, scratch) / float(a.width) + a.epsilon);
    if ((MODE == ROW_RMS_INVERSE || MODE == ROW_ADALN_KEEP) && threadIdx.x == 0)
        a.inverse[row] = inv;
    if (MODE == ROW_RMS_INVERSE) return;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        uint32_t vec = threadIdx.x + i * blockDim.x;
        if (vec >= vectors) continue;
        uint32_t col = vec << 3;
        Vec8 w = load8(a.norm + col), y;
        if (MODE == ROW_RMS_NORM) {
#pragma unroll
            for (int e = 0; e < 8; e++) y.v[e] = (x[i].v[e] * inv) * w.v[e];
        } else {
            Vec8 shift = load8(a.norm_mod + mod_base + size_t(a.shift_slot) * a.width + col);
            Vec8 scale = load8(a.norm_mod + mod_base + size_t(a.scale_slot) * a.width + col);
#pragma unroll
            for (int e = 0; e < 8; e++)
                y.v[e] = (x[i].v[e] * inv * w.v[e]) * (1.0f + scale.v[e]) + shift.v[e];
        }
        store8(a.output + row_base + col, y);
    }
}

bool all_aligned16(std::initializer_list<const void *> pointers) {
    for (const void *p : pointers)
        if (p && !h3b_aligned16(p)) return false;
    return true;
}

template <int MODE>
void launch_row(h3_gpu *gpu, const RowArgs &a) {
    bool vec = a.width % 8 == 0 && a.width <= 8u * kRowThreads * kMaxVecPerThread &&
               all_aligned16({a.input, a.residual, a.branch, a.gate_mod, a.norm, a.norm_mod,
                              a.stored, a.output, a.original_w, a.baseline_w, a.original_r,
                              a.reduced, a.baseline_r});
    if (vec) {
        uint32_t vectors = a.width / 8;
        if (vectors <= kRowThreads) {
            int threads = int((vectors + 31) / 32 * 32);
            h3b_row_vector<MODE, 1><<<a.rows, threads, 0, gpu->stream>>>(a);
        } else {
            h3b_row_vector<MODE, kMaxVecPerThread><<<a.rows, kRowThreads, 0, gpu->stream>>>(a);
        }
        return;
    }
    int threads = kRowThreads;
    while (threads > 32 && threads / 2 >= int(a.width)) threads /= 2;
    size_t cache_bytes = size_t(a.width) * sizeof(uint16_t);
    int cached = cache_bytes <= 48 * 1024;
    h3b_row_scalar<MODE><<<a.rows, threads, cached ? cache_bytes : 0, gpu->stream>>>(a, cached);
}

/* ---------------------------------------------------------- elementwise */

enum EltOp { ELT_ADD, ELT_SUB, ELT_SILU, ELT_SILU_MUL };

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

template <int OP>
__device__ __forceinline__ float elt(float a, float b) {
    if (OP == ELT_ADD) return a + b;
    if (OP == ELT_SUB) return a - b;
    if (OP == ELT_SILU) return silu(a);
    return silu(a) * b;
}

template <int OP>
__global__ void h3b_elementwise_bf16(const uint16_t *a, const uint16_t *b, uint16_t *out,
                                     size_t count, int vec) {
    size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i >= count) return;
    if (vec && i + 8 <= count) {
        Vec8 x = load8(a + i), y = x, r;
        if (OP != ELT_SILU) y = load8(b + i);
#pragma unroll
        for (int e = 0; e < 8; e++) r.v[e] = elt<OP>(x.v[e], y.v[e]);
        store8(out + i, r);
    } else {
        size_t end = i + 8 < count ? i + 8 : count;
        for (; i < end; i++)
            out[i] = h3b_narrow(elt<OP>(h3b_widen(a[i]), OP == ELT_SILU ? 0.0f : h3b_widen(b[i])));
    }
}

/* classifier-free guidance: out = bf16(uncond + guidance * (cond - uncond)), one fused
 * multiply-add on the F32 difference */
__global__ void h3b_cfg_combine_kernel(const uint16_t *cond, const uint16_t *uncond, uint16_t *out,
                                       size_t count, float guidance, int vec) {
    size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i >= count) return;
    if (vec && i + 8 <= count) {
        Vec8 c = load8(cond + i), u = load8(uncond + i), r;
#pragma unroll
        for (int e = 0; e < 8; e++) r.v[e] = fmaf(guidance, c.v[e] - u.v[e], u.v[e]);
        store8(out + i, r);
    } else {
        size_t end = i + 8 < count ? i + 8 : count;
        for (; i < end; i++) {
            float u = h3b_widen(uncond[i]);
            out[i] = h3b_narrow(fmaf(guidance, h3b_widen(cond[i]) - u, u));
        }
    }
}

__global__ void h3b_silu_f32_kernel(const float *in, float *out, size_t count) {
    size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) out[i] = silu(in[i]);
}

/* out[r][c] = bf16(silu(fused[r][c]) * fused[r][width + c]) */
__global__ void h3b_swiglu_kernel(const uint16_t *fused, uint16_t *out, uint32_t rows,
                                  uint32_t width, int vec) {
    if (vec) {
        uint32_t per_row = width >> 3;
        size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
        if (idx >= size_t(rows) * per_row) return;
        uint32_t row = uint32_t(idx / per_row), col = uint32_t(idx % per_row) << 3;
        const uint16_t *base = fused + size_t(row) * width * 2;
        Vec8 g = load8(base + col), u = load8(base + width + col), r;
#pragma unroll
        for (int e = 0; e < 8; e++) r.v[e] = silu(g.v[e]) * u.v[e];
        store8(out + size_t(row) * width + col, r);
    } else {
        size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
        if (idx >= size_t(rows) * width) return;
        uint32_t row = uint32_t(idx / width), col = uint32_t(idx % width);
        const uint16_t *base = fused + size_t(row) * width * 2;
        out[idx] = h3b_narrow(silu(h3b_widen(base[col])) * h3b_widen(base[width + col]));
    }
}

template <typename T>
__global__ void h3b_gate_kernel(const T *residual, const T *branch, const T *modulation,
                                const uint32_t *row_map, T *out, uint32_t rows, uint32_t width,
                                uint32_t slots, uint32_t gate_slot, int vec);

template <>
__global__ void h3b_gate_kernel<uint16_t>(const uint16_t *residual, const uint16_t *branch,
                                          const uint16_t *modulation, const uint32_t *row_map,
                                          uint16_t *out, uint32_t rows, uint32_t width,
                                          uint32_t slots, uint32_t gate_slot, int vec) {
    size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec) {
        uint32_t per_row = width >> 3;
        if (idx >= size_t(rows) * per_row) return;
        uint32_t row = uint32_t(idx / per_row), col = uint32_t(idx % per_row) << 3;
        size_t at = size_t(row) * width + col;
        size_t mod = (size_t(row_map[row]) * slots + gate_slot) * width + col;
        Vec8 r = load8(residual + at), b = load8(branch + at), g = load8(modulation + mod), y;
#pragma unroll
        for (int e = 0; e < 8; e++) y.v[e] = r.v[e] + b.v[e] * g.v[e];
        store8(out + at, y);
    } else {
        if (idx >= size_t(rows) * width) return;
        uint32_t row = uint32_t(idx / width), col = uint32_t(idx % width);
        size_t mod = (size_t(row_map[row]) * slots + gate_slot) * width + col;
        out[idx] = h3b_narrow(h3b_widen(residual[idx]) +
                              h3b_widen(branch[idx]) * h3b_widen(modulation[mod]));
    }
}

template <>
__global__ void h3b_gate_kernel<float>(const float *residual, const float *branch,
                                       const float *modulation, const uint32_t *row_map,
                                       float *out, uint32_t rows, uint32_t width, uint32_t slots,
                                       uint32_t gate_slot, int) {
    size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= size_t(rows) * width) return;
    uint32_t row = uint32_t(idx / width), col = uint32_t(idx % width);
    size_t mod = (size_t(row_map[row]) * slots + gate_slot) * width + col;
    out[idx] = residual[idx] + branch[idx] * modulation[mod];
}

/* F32 adaLN (diagnostic path of the reference; one CTA per row). */
__global__ void h3b_adaln_f32_kernel(const float *input, const float *norm,
                                     const float *modulation, const uint32_t *row_map,
                                     float *output, uint32_t rows, uint32_t width, uint32_t slots,
                                     uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    __shared__ float scratch[32];
    uint32_t row = blockIdx.x;
    if (row >= rows) return;
    const float *x = input + size_t(row) * width;
    float local = 0.0f;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) local = fmaf(x[c], x[c], local);
    float inv = 1.0f / sqrtf(block_sum(local, scratch) / float(width) + epsilon);
    size_t base = size_t(row_map[row]) * slots * width;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        float normalized = x[c] * inv * norm[c];
        float shift = modulation[base + size_t(shift_slot) * width + c];
        float scale = modulation[base + size_t(scale_slot) * width + c];
        output[size_t(row) * width + c] = normalized * (1.0f + scale) + shift;
    }
}

__global__ void h3b_euler_kernel(float *sample, const uint16_t *last, const uint16_t *previous,
                                 size_t count, float delta, float ratio) {
    size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float lv = h3b_widen(last[i]);
    float velocity = fmaf(ratio, lv - h3b_widen(previous[i]), lv);
    sample[i] = fmaf(delta, velocity, sample[i]);
}

/* Token pool / expand, unfused forms: VEC = 8 BF16 (one 16-byte vector) per thread when the
 * width is a multiple of 8 and every view is 16-byte aligned, else one element per thread. The
 * arithmetic per element is the reference's (h3_cuda_dit.cu:336-364). */
template <int VEC>
__global__ void h3b_token_pool_kernel(const uint16_t *input, const uint32_t *pairs, uint16_t *out,
                                      uint16_t *baseline, const uint32_t *baseline_indices,
                                      uint16_t *original, uint32_t rows, uint32_t width) {
    const uint32_t per_row = width / VEC;
    size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= size_t(rows) * per_row) return;
    const uint32_t row = uint32_t(idx / per_row), col = uint32_t(idx % per_row) * VEC;
    const uint32_t first = pairs[2 * row], second = pairs[2 * row + 1];
    const uint32_t b = baseline_indices[row];
    const size_t at_first = size_t(first) * width + col, at_out = size_t(row) * width + col;
    if (VEC == 8) {
        const uint4 lhs = *reinterpret_cast<const uint4 *>(input + at_first);
        *reinterpret_cast<uint4 *>(original + at_first) = lhs;
        uint4 pooled = lhs;
        if (first != second) {
            const size_t at_second = size_t(second) * width + col;
            const uint4 rhs = *reinterpret_cast<const uint4 *>(input + at_second);
            *reinterpret_cast<uint4 *>(original + at_second) = rhs;
            const Vec8 l = unpack8(lhs);
            const Vec8 r = unpack8(rhs);
            Vec8 y;
#pragma unroll
            for (int e = 0; e < 8; e++) y.v[e] = (l.v[e] + r.v[e]) * 0.5f;
            pooled = pack8(y);
        }
        *reinterpret_cast<uint4 *>(out + at_out) = pooled;
        if (b != kNoBaseline) *reinterpret_cast<uint4 *>(baseline + size_t(b) * width + col) = pooled;
    } else {
        const uint16_t lhs = input[at_first];
        original[at_first] = lhs;
        uint16_t pooled = lhs;
        if (first != second) {
            const uint16_t rhs = input[size_t(second) * width + col];
            original[size_t(second) * width + col] = rhs;
            pooled = h3b_narrow((h3b_widen(lhs) + h3b_widen(rhs)) * 0.5f);
        }
        out[at_out] = pooled;
        if (b != kNoBaseline) baseline[size_t(b) * width + col] = pooled;
    }
}

template <int VEC>
__global__ void h3b_token_expand_kernel(const uint16_t *original, const uint16_t *reduced,
                                        const uint16_t *baseline,
                                        const uint32_t *baseline_indices, const uint32_t *parents,
                                        uint16_t *out, uint32_t rows, uint32_t width,
                                        uint32_t exact_prefix_rows, float update_scale) {
    const uint32_t per_row = width / VEC;
    size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= size_t(rows) * per_row) return;
    const uint32_t row = uint32_t(idx / per_row), col = uint32_t(idx % per_row) * VEC;
    const uint32_t parent = parents[row];
    const uint32_t b = baseline_indices[parent];
    const bool update = row >= exact_prefix_rows && b != kNoBaseline;
    const size_t at = size_t(row) * width + col, at_parent = size_t(parent) * width + col;
    if (VEC == 8) {
        uint4 value = *reinterpret_cast<const uint4 *>(reduced + at_parent);
        if (update) {
            const Vec8 v = unpack8(value);
            const Vec8 base = load8(baseline + size_t(b) * width + col), o = load8(original + at);
            Vec8 y;
#pragma unroll
            for (int e = 0; e < 8; e++) y.v[e] = o.v[e] + update_scale * (v.v[e] - base.v[e]);
            value = pack8(y);
        }
        *reinterpret_cast<uint4 *>(out + at) = value;
    } else {
        uint16_t value = reduced[at_parent];
        if (update) {
            const float delta = h3b_widen(value) - h3b_widen(baseline[size_t(b) * width + col]);
            value = h3b_narrow(h3b_widen(original[at]) + update_scale * delta);
        }
        out[at] = value;
    }
}

inline unsigned blocks_for(size_t items, int threads) {
    return unsigned((items + threads - 1) / threads);
}

}  // namespace

/* ================================================================= C ABI */

extern "C" int h3_gpu_adaln_bf16_offset(h3_gpu *gpu, h3_gpu_tensor *output,
                                        const h3_gpu_tensor *input, size_t input_offset,
                                        const h3_gpu_tensor *norm_weight,
                                        const h3_gpu_tensor *modulation,
                                        const h3_gpu_tensor *row_map, uint32_t rows,
                                        uint32_t width, uint32_t slots, uint32_t shift_slot,
                                        uint32_t scale_slot, float epsilon) {
    size_t count = size_t(rows) * width;
    if (input_offset > SIZE_MAX - count) return h3b_fail(gpu, "AdaLN input offset is out of range");
    if (!h3b_need(gpu, input, H3_GPU_BF16, input_offset + count, "AdaLN input") ||
        !h3b_need(gpu, norm_weight, H3_GPU_BF16, width, "AdaLN norm") ||
        !h3b_need(gpu, modulation, H3_GPU_BF16, 1, "AdaLN modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "AdaLN row map") ||
        !h3b_need(gpu, output, H3_GPU_BF16, count, "AdaLN output") || !h3b_need_command(gpu))
        return 0;
    if (shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "AdaLN modulation slot is out of range");
    if (count) {
        RowArgs a = {};
        a.input = h3b_ptr<uint16_t>(input, input_offset);
        a.norm = h3b_ptr<uint16_t>(norm_weight);
        a.norm_mod = h3b_ptr<uint16_t>(modulation);
        a.row_map = h3b_ptr<uint32_t>(row_map);
        a.output = h3b_ptr<uint16_t>(output);
        a.rows = rows; a.width = width; a.slots = slots;
        a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
        launch_row<ROW_ADALN>(gpu, a);
    }
    return h3b_launched(gpu, "adaln_bf16");
}

extern "C" int h3_gpu_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                 const h3_gpu_tensor *norm_weight,
                                 const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
                                 uint32_t rows, uint32_t width, uint32_t slots,
                                 uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    return h3_gpu_adaln_bf16_offset(gpu, output, input, 0, norm_weight, modulation, row_map, rows,
                                    width, slots, shift_slot, scale_slot, epsilon);
}

extern "C" int h3_gpu_adaln_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *modulation,
                                const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                                uint32_t slots, uint32_t shift_slot, uint32_t scale_slot,
                                float epsilon) {
    size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, input, H3_GPU_F32, count, "AdaLN input") ||
        !h3b_need(gpu, norm_weight, H3_GPU_F32, width, "AdaLN norm") ||
        !h3b_need(gpu, modulation, H3_GPU_F32, 1, "AdaLN modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "AdaLN row map") ||
        !h3b_need(gpu, output, H3_GPU_F32, count, "AdaLN output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    if (shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "AdaLN modulation slot is out of range");
    if (count)
        h3b_adaln_f32_kernel<<<rows, kRowThreads, 0, gpu->stream>>>(
            h3b_ptr<float>(input), h3b_ptr<float>(norm_weight), h3b_ptr<float>(modulation),
            h3b_ptr<uint32_t>(row_map), h3b_ptr<float>(output), rows, width, slots, shift_slot,
            scale_slot, epsilon);
    return h3b_launched(gpu, "adaln_f32");
}

extern "C" int h3_gpu_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                    const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                                    uint32_t rows, uint32_t width, float epsilon) {
    size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, input, H3_GPU_BF16, count, "RMS norm input") ||
        !h3b_need(gpu, weight, H3_GPU_BF16, width, "RMS norm weight") ||
        !h3b_need(gpu, output, H3_GPU_BF16, count, "RMS norm output") || !h3b_need_command(gpu))
        return 0;
    if (count) {
        RowArgs a = {};
        a.input = h3b_ptr<uint16_t>(input);
        a.norm = h3b_ptr<uint16_t>(weight);
        a.output = h3b_ptr<uint16_t>(output);
        a.rows = rows; a.width = width; a.epsilon = epsilon;
        launch_row<ROW_RMS_NORM>(gpu, a);
    }
    return h3b_launched(gpu, "rms_norm_bf16");
}

template <typename T>
static int gate_common(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                       const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                       const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                       uint32_t slots, uint32_t gate_slot, h3_gpu_dtype dtype, const char *what) {
    size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, residual, dtype, count, "gate residual") ||
        !h3b_need(gpu, branch, dtype, count, "gate branch") ||
        !h3b_need(gpu, modulation, dtype, 1, "gate modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "gate row map") ||
        !h3b_need(gpu, output, dtype, count, "gate output") || !h3b_need_command(gpu))
        return 0;
    if (gate_slot >= slots) return h3b_fail(gpu, "gate modulation slot is out of range");
    if (count) {
        int vec = sizeof(T) == 2 && width % 8 == 0 &&
                  all_aligned16({residual->data, branch->data, modulation->data, output->data});
        size_t items = vec ? count / 8 : count;
        h3b_gate_kernel<T><<<blocks_for(items, 256), 256, 0, gpu->stream>>>(
            h3b_ptr<T>(residual), h3b_ptr<T>(branch), h3b_ptr<T>(modulation),
            h3b_ptr<uint32_t>(row_map), h3b_ptr<T>(output), rows, width, slots, gate_slot, vec);
    }
    return h3b_launched(gpu, what);
}

extern "C" int h3_gpu_gate_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                                const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                                const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                                uint32_t slots, uint32_t gate_slot) {
    return gate_common<uint16_t>(gpu, output, residual, branch, modulation, row_map, rows, width,
                                 slots, gate_slot, H3_GPU_BF16, "gate_bf16");
}

extern "C" int h3_gpu_gate_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                               const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                               const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                               uint32_t slots, uint32_t gate_slot) {
    h3b_written(output);
    return gate_common<float>(gpu, output, residual, branch, modulation, row_map, rows, width,
                              slots, gate_slot, H3_GPU_F32, "gate_f32");
}

extern "C" int h3_gpu_gate_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *gated_residual,
                                      h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                                      const h3_gpu_tensor *branch,
                                      const h3_gpu_tensor *norm_weight,
                                      const h3_gpu_tensor *gate_modulation,
                                      const h3_gpu_tensor *norm_modulation,
                                      const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                                      uint32_t slots, uint32_t gate_slot, uint32_t shift_slot,
                                      uint32_t scale_slot, float epsilon) {
    size_t count = size_t(rows) * width;
    if (!rows || !width || width > kFusedWidthLimit || count > UINT32_MAX)
        return h3b_fail(gpu, "fused gate AdaLN shape is out of range");
    if (gate_slot >= slots || shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "fused gate AdaLN modulation slot is out of range");
    if (!h3b_need(gpu, residual, H3_GPU_BF16, count, "fused gate AdaLN residual") ||
        !h3b_need(gpu, branch, H3_GPU_BF16, count, "fused gate AdaLN branch") ||
        !h3b_need(gpu, norm_weight, H3_GPU_BF16, width, "fused gate AdaLN norm") ||
        !h3b_need(gpu, gate_modulation, H3_GPU_BF16, 1, "fused gate AdaLN gate modulation") ||
        !h3b_need(gpu, norm_modulation, H3_GPU_BF16, 1, "fused gate AdaLN norm modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "fused gate AdaLN row map") ||
        !h3b_need(gpu, gated_residual, H3_GPU_BF16, count, "fused gate AdaLN gated residual") ||
        !h3b_need(gpu, output, H3_GPU_BF16, count, "fused gate AdaLN output") ||
        !h3b_need_command(gpu))
        return 0;
    RowArgs a = {};
    a.residual = h3b_ptr<uint16_t>(residual);
    a.branch = h3b_ptr<uint16_t>(branch);
    a.gate_mod = h3b_ptr<uint16_t>(gate_modulation);
    a.norm = h3b_ptr<uint16_t>(norm_weight);
    a.norm_mod = h3b_ptr<uint16_t>(norm_modulation);
    a.row_map = h3b_ptr<uint32_t>(row_map);
    a.stored = h3b_ptr<uint16_t>(gated_residual);
    a.output = h3b_ptr<uint16_t>(output);
    a.rows = rows; a.width = width; a.slots = slots; a.gate_slot = gate_slot;
    a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
    launch_row<ROW_GATE_ADALN>(gpu, a);
    return h3b_launched(gpu, "gate_adaln_bf16");
}

extern "C" int h3_gpu_adaln_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                        h3_gpu_tensor *inverse, const h3_gpu_tensor *input,
                                        size_t input_offset, const h3_gpu_tensor *norm_weight,
                                        const h3_gpu_tensor *modulation,
                                        const h3_gpu_tensor *row_map,
                                        const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                        uint32_t rows, uint32_t width, uint32_t output_dim,
                                        uint32_t slots, uint32_t shift_slot, uint32_t scale_slot,
                                        float epsilon) {
    size_t in_count = size_t(rows) * width;
    if (input_offset > SIZE_MAX - in_count)
        return h3b_fail(gpu, "fused final head input offset is out of range");
    if (!h3b_need(gpu, input, H3_GPU_BF16, input_offset + in_count, "fused final head input") ||
        !h3b_need(gpu, inverse, H3_GPU_F32, rows, "fused final head inverse RMS") ||
        !h3b_need(gpu, norm_weight, H3_GPU_BF16, width, "fused final head norm") ||
        !h3b_need(gpu, modulation, H3_GPU_BF16, 1, "fused final head modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "fused final head row map") ||
        !h3b_need(gpu, weight, H3_GPU_BF16, size_t(output_dim) * width, "fused final head weight") ||
        !h3b_need(gpu, output, H3_GPU_BF16, size_t(rows) * output_dim, "fused final head output") ||
        (bias && !h3b_need(gpu, bias, H3_GPU_BF16, output_dim, "fused final head bias")) ||
        !h3b_need_command(gpu))
        return 0;
    if (shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "fused final head modulation slot is out of range");
    if (!rows || !width) return h3b_launched(gpu, "adaln_linear_bf16");
    /* adaLN rounded to BF16 into scratch (the reference's rounding point before the
     * dot product, h3_cuda_dit.cu:202-204), then the projection. */
    uint16_t *normed = static_cast<uint16_t *>(h3b_workspace(gpu, in_count * sizeof(uint16_t)));
    if (!normed) return h3b_fail(gpu, "cannot allocate the final head scratch");
    h3b_written(inverse);
    RowArgs a = {};
    a.input = h3b_ptr<uint16_t>(input, input_offset);
    a.norm = h3b_ptr<uint16_t>(norm_weight);
    a.norm_mod = h3b_ptr<uint16_t>(modulation);
    a.row_map = h3b_ptr<uint32_t>(row_map);
    a.output = normed;
    a.inverse = h3b_ptr<float>(inverse);
    a.rows = rows; a.width = width; a.slots = slots;
    a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
    launch_row<ROW_ADALN_KEEP>(gpu, a);
    if (!h3b_launched(gpu, "adaln_linear_bf16 normalisation")) return 0;
    if (!output_dim) return 1;
    return h3b_gemm_bf16(gpu, h3b_ptr<uint16_t>(output), normed, h3b_ptr<uint16_t>(weight),
                         bias ? h3b_ptr<uint16_t>(bias) : nullptr, rows, width, output_dim,
                         H3B_EPI_STORE, "adaln_linear_bf16");
}

/* ------------------------------------------------- final head, no allocation */

/* Scratch for h3x_adaln_linear_bf16_noalloc: the BF16-rounded adaLN rows that sit
 * between the normalisation kernel and the projection. It is part of the library
 * image, so every GPU that loads the library holds these 8 MiB until the process
 * exits. */
constexpr size_t kNoAllocScratchElements = size_t(4) << 20;   /* 4 Mi BF16 = 8 MiB */
static __device__ __align__(256) uint16_t g_noalloc_scratch[kNoAllocScratchElements];

constexpr int kNoAllocMaxDevices = 64;
static uint16_t *g_noalloc_scratch_address[kNoAllocMaxDevices] = {nullptr};

/* `g_noalloc_scratch` named in host code is only a handle for the runtime, not a device
 * address; the address is looked up once per device, with that device current. */
static uint16_t *noalloc_scratch_for(h3_gpu *gpu) {
    int current = -1;
    cudaError_t status = cudaGetDevice(&current);
    if (status != cudaSuccess) {
        h3b_fail_cuda(gpu, "cudaGetDevice", status);
        return nullptr;
    }
    if (current < 0 || current >= kNoAllocMaxDevices) {
        h3b_fail(gpu, "h3x_adaln_linear_bf16_noalloc serves device indices 0..%d; the current device is %d",
                 kNoAllocMaxDevices - 1, current);
        return nullptr;
    }
    if (current != gpu->device) {
        h3b_fail(gpu, "the context's device %d is not the calling thread's current device %d",
                 gpu->device, current);
        return nullptr;
    }
    /* threads of different contexts may make their first call on a device at the same time */
    static std::mutex lookup;
    std::lock_guard<std::mutex> guard(lookup);
    if (!g_noalloc_scratch_address[current]) {
        void *address = nullptr;
        status = cudaGetSymbolAddress(&address, g_noalloc_scratch);
        if (status != cudaSuccess || !address) {
            h3b_fail_cuda(gpu, "cudaGetSymbolAddress(no-allocation scratch)", status);
            return nullptr;
        }
        g_noalloc_scratch_address[current] = static_cast<uint16_t *>(address);
    }
    return g_noalloc_scratch_address[current];
}

extern "C" int h3x_adaln_linear_bf16_noalloc(h3_gpu *gpu, h3_gpu_tensor *output,
                                             h3_gpu_tensor *inverse, const h3_gpu_tensor *input,
                                             size_t input_offset,
                                             const h3_gpu_tensor *norm_weight,
                                             const h3_gpu_tensor *modulation,
                                             const h3_gpu_tensor *row_map,
                                             const h3_gpu_tensor *weight,
                                             const h3_gpu_tensor *bias, uint32_t rows,
                                             uint32_t width, uint32_t output_dim, uint32_t slots,
                                             uint32_t shift_slot, uint32_t scale_slot,
                                             float epsilon) {
    if (!gpu) return 0;
    size_t in_count = size_t(rows) * width;
    if (in_count > kNoAllocScratchElements)
        return h3b_fail(gpu,
                        "h3x_adaln_linear_bf16_noalloc: rows * width = %zu exceeds the built-in "
                        "scratch of %zu elements; use h3_gpu_adaln_linear_bf16 for larger calls",
                        in_count, kNoAllocScratchElements);
    if (input_offset > SIZE_MAX - in_count)
        return h3b_fail(gpu, "fused final head input offset is out of range");
    if (!h3b_need(gpu, input, H3_GPU_BF16, input_offset + in_count, "fused final head input") ||
        !h3b_need(gpu, inverse, H3_GPU_F32, rows, "fused final head inverse RMS") ||
        !h3b_need(gpu, norm_weight, H3_GPU_BF16, width, "fused final head norm") ||
        !h3b_need(gpu, modulation, H3_GPU_BF16, 1, "fused final head modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "fused final head row map") ||
        !h3b_need(gpu, weight, H3_GPU_BF16, size_t(output_dim) * width, "fused final head weight") ||
        !h3b_need(gpu, output, H3_GPU_BF16, size_t(rows) * output_dim, "fused final head output") ||
        (bias && !h3b_need(gpu, bias, H3_GPU_BF16, output_dim, "fused final head bias")) ||
        !h3b_need_command(gpu))
        return 0;
    if (shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "fused final head modulation slot is out of range");
    uint16_t *normed = noalloc_scratch_for(gpu);
    if (!normed) return 0;
    if (!rows || !width) return h3b_launched(gpu, "adaln_linear_bf16_noalloc");
    /* every element of the scratch region that the projection reads is written by the
     * normalisation kernel first, so nothing left over from an earlier call is consumed */
    RowArgs a = {};
    a.input = h3b_ptr<uint16_t>(input, input_offset);
    a.norm = h3b_ptr<uint16_t>(norm_weight);
    a.norm_mod = h3b_ptr<uint16_t>(modulation);
    a.row_map = h3b_ptr<uint32_t>(row_map);
    a.output = normed;
    a.inverse = h3b_ptr<float>(inverse);
    a.rows = rows; a.width = width; a.slots = slots;
    a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
    launch_row<ROW_ADALN_KEEP>(gpu, a);
    if (!h3b_launched(gpu, "adaln_linear_bf16_noalloc normalisation")) return 0;
    if (!output_dim) return 1;
    gpu->allocation_barred = 1;       /* the projection must not create its split-tail scratch here */
    const int done = h3b_gemm_bf16(gpu, h3b_ptr<uint16_t>(output), normed, h3b_ptr<uint16_t>(weight),
                                   bias ? h3b_ptr<uint16_t>(bias) : nullptr, rows, width, output_dim,
                                   H3B_EPI_STORE, "adaln_linear_bf16_noalloc");
    gpu->allocation_barred = 0;
    return done;
}

/* ----------------------------------------------------------- elementwise */

template <int OP>
static int elementwise(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *a,
                       const h3_gpu_tensor *b, uint32_t elements, const char *what) {
    if (!h3b_need(gpu, a, H3_GPU_BF16, elements, what) ||
        (b && !h3b_need(gpu, b, H3_GPU_BF16, elements, what)) ||
        !h3b_need(gpu, output, H3_GPU_BF16, elements, what) || !h3b_need_command(gpu))
        return 0;
    if (elements) {
        int vec = all_aligned16({a->data, b ? b->data : nullptr, output->data});
        h3b_elementwise_bf16<OP><<<blocks_for((size_t(elements) + 7) / 8, 256), 256, 0, gpu->stream>>>(
            h3b_ptr<uint16_t>(a), b ? h3b_ptr<uint16_t>(b) : nullptr, h3b_ptr<uint16_t>(output),
            elements, vec);
    }
    return h3b_launched(gpu, what);
}

extern "C" int h3x_cfg_combine_bf16(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *cond,
                                    const h3_gpu_tensor *uncond, uint32_t elements,
                                    float guidance) {
    if (!gpu) return 0;
    if (!h3b_need(gpu, cond, H3_GPU_BF16, elements, "cfg_combine cond") ||
        !h3b_need(gpu, uncond, H3_GPU_BF16, elements, "cfg_combine uncond") ||
        !h3b_need(gpu, out, H3_GPU_BF16, elements, "cfg_combine output") || !h3b_need_command(gpu))
        return 0;
    if (elements) {
        int vec = all_aligned16({cond->data, uncond->data, out->data});
        h3b_cfg_combine_kernel<<<blocks_for((size_t(elements) + 7) / 8, 256), 256, 0, gpu->stream>>>(
            h3b_ptr<uint16_t>(cond), h3b_ptr<uint16_t>(uncond), h3b_ptr<uint16_t>(out), elements,
            guidance, vec);
    }
    return h3b_launched(gpu, "cfg_combine_bf16");
}

extern "C" int h3_gpu_add_bf16(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *l,
                               const h3_gpu_tensor *r, uint32_t n) {
    if (!r) return h3b_fail(gpu, "add_bf16 tensor has the wrong dtype");
    return elementwise<ELT_ADD>(gpu, out, l, r, n, "add_bf16");
}
extern "C" int h3_gpu_sub_bf16(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *l,
                               const h3_gpu_tensor *r, uint32_t n) {
    if (!r) return h3b_fail(gpu, "sub_bf16 tensor has the wrong dtype");
    return elementwise<ELT_SUB>(gpu, out, l, r, n, "sub_bf16");
}
extern "C" int h3_gpu_silu_bf16(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *in,
                                uint32_t n) {
    return elementwise<ELT_SILU>(gpu, out, in, nullptr, n, "silu_bf16");
}
extern "C" int h3_gpu_silu_mul_bf16(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *gate,
                                    const h3_gpu_tensor *up, uint32_t n) {
    if (!up) return h3b_fail(gpu, "silu_mul_bf16 tensor has the wrong dtype");
    return elementwise<ELT_SILU_MUL>(gpu, out, gate, up, n, "silu_mul_bf16");
}

extern "C" int h3_gpu_silu_f32(h3_gpu *gpu, h3_gpu_tensor *out, const h3_gpu_tensor *in,
                               uint32_t n) {
    if (!h3b_need(gpu, in, H3_GPU_F32, n, "SiLU input") ||
        !h3b_need(gpu, out, H3_GPU_F32, n, "SiLU output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(out);
    if (n)
        h3b_silu_f32_kernel<<<blocks_for(n, 256), 256, 0, gpu->stream>>>(h3b_ptr<float>(in),
                                                                        h3b_ptr<float>(out), n);
    return h3b_launched(gpu, "silu_f32");
}

int h3b_swiglu_launch(h3_gpu *gpu, uint16_t *out, const uint16_t *fused, uint32_t rows,
                      uint32_t width) {
    size_t count = size_t(rows) * width;
    if (count) {
        int vec = width % 8 == 0 && all_aligned16({out, fused});
        h3b_swiglu_kernel<<<blocks_for(vec ? count / 8 : count, 256), 256, 0, gpu->stream>>>(
            fused, out, rows, width, vec);
    }
    return h3b_launched(gpu, "swiglu_bf16");
}

extern "C" int h3_gpu_swiglu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *fused,
                                  uint32_t rows, uint32_t width) {
    size_t count = size_t(rows) * width;
    if (!h3b_need(gpu, fused, H3_GPU_BF16, count * 2, "SwiGLU input") ||
        !h3b_need(gpu, output, H3_GPU_BF16, count, "SwiGLU output") || !h3b_need_command(gpu))
        return 0;
    return h3b_swiglu_launch(gpu, h3b_ptr<uint16_t>(output), h3b_ptr<uint16_t>(fused), rows,
                             width);
}

extern "C" int h3_gpu_euler_bf16(h3_gpu *gpu, h3_gpu_tensor *sample, size_t sample_offset,
                                 const h3_gpu_tensor *last, const h3_gpu_tensor *previous,
                                 uint32_t elements, float delta, float ratio) {
    if (!sample || sample->dtype != H3_GPU_F32 || sample_offset > sample->elements ||
        elements > sample->elements - sample_offset)
        return h3b_fail(gpu, "Euler sample range is out of range");
    if (!h3b_need(gpu, last, H3_GPU_BF16, elements, "Euler last velocity") ||
        !h3b_need(gpu, previous, H3_GPU_BF16, elements, "Euler previous velocity") ||
        !h3b_need_command(gpu))
        return 0;
    h3b_written(sample);
    if (elements)
        h3b_euler_kernel<<<blocks_for(elements, 256), 256, 0, gpu->stream>>>(
            h3b_ptr<float>(sample, sample_offset), h3b_ptr<uint16_t>(last),
            h3b_ptr<uint16_t>(previous), elements, delta, ratio);
    return h3b_launched(gpu, "euler_bf16");
}

/* -------------------------------------------------------- token reduction */

static int view_ok(const h3_gpu_tensor *t, size_t offset, size_t elements) {
    return t && t->dtype == H3_GPU_BF16 && offset <= t->elements &&
           elements <= t->elements - offset;
}

extern "C" int h3_gpu_token_pool_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                      const h3_gpu_tensor *input, size_t input_offset,
                                      h3_gpu_tensor *original, size_t original_offset,
                                      h3_gpu_tensor *baseline, size_t baseline_offset,
                                      const h3_gpu_tensor *baseline_indices,
                                      const h3_gpu_tensor *pairs, uint32_t input_rows,
                                      uint32_t rows, uint32_t baseline_rows, uint32_t width) {
    size_t count = size_t(rows) * width, in_count = size_t(input_rows) * width;
    if (!input_rows || !rows || rows > input_rows || baseline_rows > rows || !width ||
        in_count > UINT32_MAX)
        return h3b_fail(gpu, "token pool shape is out of range");
    if (!view_ok(input, input_offset, in_count))
        return h3b_fail(gpu, "token pool input tensor is too small");
    if (!view_ok(original, original_offset, in_count))
        return h3b_fail(gpu, "token pool original tensor is too small");
    if (!view_ok(baseline, baseline_offset, size_t(baseline_rows) * width))
        return h3b_fail(gpu, "token pool baseline tensor is too small");
    if (!h3b_need(gpu, output, H3_GPU_BF16, count, "token pool output") ||
        !h3b_need(gpu, baseline_indices, H3_GPU_U32, rows, "token pool baseline indices") ||
        !h3b_need(gpu, pairs, H3_GPU_U32, size_t(rows) * 2, "token pool pairs") ||
        !h3b_need_command(gpu))
        return 0;
    const uint16_t *in = h3b_ptr<uint16_t>(input, input_offset);
    uint16_t *out = h3b_ptr<uint16_t>(output), *base = h3b_ptr<uint16_t>(baseline, baseline_offset);
    uint16_t *orig = h3b_ptr<uint16_t>(original, original_offset);
    if (width % 8 == 0 && all_aligned16({in, out, base, orig}))
        h3b_token_pool_kernel<8><<<blocks_for(count / 8, 256), 256, 0, gpu->stream>>>(
            in, h3b_ptr<uint32_t>(pairs), out, base, h3b_ptr<uint32_t>(baseline_indices), orig, rows, width);
    else
        h3b_token_pool_kernel<1><<<blocks_for(count, 256), 256, 0, gpu->stream>>>(
            in, h3b_ptr<uint32_t>(pairs), out, base, h3b_ptr<uint32_t>(baseline_indices), orig, rows, width);
    return h3b_launched(gpu, "token_pool_bf16");
}

extern "C" int h3_gpu_token_pool_adaln_bf16(
    h3_gpu *gpu, h3_gpu_tensor *residual, h3_gpu_tensor *output, const h3_gpu_tensor *input,
    size_t input_offset, h3_gpu_tensor *original, size_t original_offset, h3_gpu_tensor *baseline,
    size_t baseline_offset, const h3_gpu_tensor *baseline_indices, const h3_gpu_tensor *pairs,
    const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *modulation,
    const h3_gpu_tensor *row_map, uint32_t input_rows, uint32_t rows, uint32_t baseline_rows,
    uint32_t width, uint32_t slots, uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    size_t count = size_t(rows) * width, in_count = size_t(input_rows) * width;
    if (!input_rows || !rows || rows > input_rows || !width || width > kFusedWidthLimit ||
        baseline_rows > rows || in_count > UINT32_MAX)
        return h3b_fail(gpu, "fused token pool shape is out of range");
    if (shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "fused token pool modulation slot is out of range");
    if (!view_ok(input, input_offset, in_count))
        return h3b_fail(gpu, "fused token pool input tensor is too small");
    if (!view_ok(original, original_offset, in_count))
        return h3b_fail(gpu, "fused token pool original tensor is too small");
    if (!view_ok(baseline, baseline_offset, size_t(baseline_rows) * width))
        return h3b_fail(gpu, "fused token pool baseline tensor is too small");
    if (!h3b_need(gpu, residual, H3_GPU_BF16, count, "fused token pool residual") ||
        !h3b_need(gpu, baseline_indices, H3_GPU_U32, rows, "fused token pool baseline indices") ||
        !h3b_need(gpu, pairs, H3_GPU_U32, size_t(rows) * 2, "fused token pool pairs") ||
        !h3b_need(gpu, norm_weight, H3_GPU_BF16, width, "fused token pool norm") ||
        !h3b_need(gpu, modulation, H3_GPU_BF16, 1, "fused token pool modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "fused token pool row map") ||
        !h3b_need(gpu, output, H3_GPU_BF16, count, "fused token pool AdaLN output") ||
        !h3b_need_command(gpu))
        return 0;
    RowArgs a = {};
    a.input = h3b_ptr<uint16_t>(input, input_offset);
    a.pairs = h3b_ptr<uint32_t>(pairs);
    a.baseline_indices = h3b_ptr<uint32_t>(baseline_indices);
    a.original_w = h3b_ptr<uint16_t>(original, original_offset);
    a.baseline_w = h3b_ptr<uint16_t>(baseline, baseline_offset);
    a.stored = h3b_ptr<uint16_t>(residual);
    a.norm = h3b_ptr<uint16_t>(norm_weight);
    a.norm_mod = h3b_ptr<uint16_t>(modulation);
    a.row_map = h3b_ptr<uint32_t>(row_map);
    a.output = h3b_ptr<uint16_t>(output);
    a.rows = rows; a.width = width; a.slots = slots;
    a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
    launch_row<ROW_POOL_ADALN>(gpu, a);
    return h3b_launched(gpu, "token_pool_adaln_bf16");
}

extern "C" int h3_gpu_token_expand_delta_bf16(
    h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *original, size_t original_offset,
    const h3_gpu_tensor *reduced, const h3_gpu_tensor *baseline, size_t baseline_offset,
    const h3_gpu_tensor *baseline_indices, const h3_gpu_tensor *parents, uint32_t rows,
    uint32_t reduced_rows, uint32_t baseline_rows, uint32_t width, uint32_t exact_prefix_rows,
    float update_scale) {
    size_t count = size_t(rows) * width;
    if (!rows || !reduced_rows || reduced_rows > rows || baseline_rows > reduced_rows || !width ||
        exact_prefix_rows > reduced_rows || count > UINT32_MAX)
        return h3b_fail(gpu, "token expand shape is out of range");
    if (!view_ok(original, original_offset, count))
        return h3b_fail(gpu, "token expand original tensor is too small");
    if (!view_ok(baseline, baseline_offset, size_t(baseline_rows) * width))
        return h3b_fail(gpu, "token expand baseline tensor is too small");
    if (!h3b_need(gpu, output, H3_GPU_BF16, count, "token expand output") ||
        !h3b_need(gpu, reduced, H3_GPU_BF16, size_t(reduced_rows) * width, "token expand reduced") ||
        !h3b_need(gpu, baseline_indices, H3_GPU_U32, reduced_rows, "token expand baseline indices") ||
        !h3b_need(gpu, parents, H3_GPU_U32, rows, "token expand parents") ||
        !h3b_need_command(gpu))
        return 0;
    const uint16_t *orig = h3b_ptr<uint16_t>(original, original_offset);
    const uint16_t *red = h3b_ptr<uint16_t>(reduced), *base = h3b_ptr<uint16_t>(baseline, baseline_offset);
    uint16_t *out = h3b_ptr<uint16_t>(output);
    if (width % 8 == 0 && all_aligned16({orig, red, base, out}))
        h3b_token_expand_kernel<8><<<blocks_for(count / 8, 256), 256, 0, gpu->stream>>>(
            orig, red, base, h3b_ptr<uint32_t>(baseline_indices), h3b_ptr<uint32_t>(parents), out, rows,
            width, exact_prefix_rows, update_scale);
    else
        h3b_token_expand_kernel<1><<<blocks_for(count, 256), 256, 0, gpu->stream>>>(
            orig, red, base, h3b_ptr<uint32_t>(baseline_indices), h3b_ptr<uint32_t>(parents), out, rows,
            width, exact_prefix_rows, update_scale);
    return h3b_launched(gpu, "token_expand_delta_bf16");
}

extern "C" int h3_gpu_token_expand_adaln_bf16(
    h3_gpu *gpu, h3_gpu_tensor *residual, h3_gpu_tensor *output, const h3_gpu_tensor *original,
    size_t original_offset, const h3_gpu_tensor *reduced, const h3_gpu_tensor *baseline,
    size_t baseline_offset, const h3_gpu_tensor *baseline_indices, const h3_gpu_tensor *parents,
    const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *modulation,
    const h3_gpu_tensor *row_map, uint32_t rows, uint32_t reduced_rows, uint32_t baseline_rows,
    uint32_t width, uint32_t exact_prefix_rows, float update_scale, uint32_t slots,
    uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    size_t count = size_t(rows) * width;
    if (!rows || !reduced_rows || reduced_rows > rows || !width || width > kFusedWidthLimit ||
        baseline_rows > reduced_rows || exact_prefix_rows > reduced_rows || count > UINT32_MAX)
        return h3b_fail(gpu, "fused token AdaLN shape is out of range");
    if (shift_slot >= slots || scale_slot >= slots)
        return h3b_fail(gpu, "fused token AdaLN modulation slot is out of range");
    if (!view_ok(original, original_offset, count))
        return h3b_fail(gpu, "fused token AdaLN original tensor is too small");
    if (!view_ok(baseline, baseline_offset, size_t(baseline_rows) * width))
        return h3b_fail(gpu, "fused token AdaLN baseline tensor is too small");
    if (!h3b_need(gpu, reduced, H3_GPU_BF16, size_t(reduced_rows) * width,
                  "fused token AdaLN reduced input") ||
        !h3b_need(gpu, baseline_indices, H3_GPU_U32, reduced_rows,
                  "fused token AdaLN baseline indices") ||
        !h3b_need(gpu, parents, H3_GPU_U32, rows, "fused token AdaLN parents") ||
        !h3b_need(gpu, residual, H3_GPU_BF16, count, "fused token AdaLN residual") ||
        !h3b_need(gpu, norm_weight, H3_GPU_BF16, width, "fused token AdaLN norm") ||
        !h3b_need(gpu, modulation, H3_GPU_BF16, 1, "fused token AdaLN modulation") ||
        !h3b_need(gpu, row_map, H3_GPU_U32, rows, "fused token AdaLN row map") ||
        !h3b_need(gpu, output, H3_GPU_BF16, count, "fused token AdaLN output") ||
        !h3b_need_command(gpu))
        return 0;
    RowArgs a = {};
    a.original_r = h3b_ptr<uint16_t>(original, original_offset);
    a.reduced = h3b_ptr<uint16_t>(reduced);
    a.baseline_r = h3b_ptr<uint16_t>(baseline, baseline_offset);
    a.baseline_indices = h3b_ptr<uint32_t>(baseline_indices);
    a.parents = h3b_ptr<uint32_t>(parents);
    a.stored = h3b_ptr<uint16_t>(residual);
    a.norm = h3b_ptr<uint16_t>(norm_weight);
    a.norm_mod = h3b_ptr<uint16_t>(modulation);
    a.row_map = h3b_ptr<uint32_t>(row_map);
    a.output = h3b_ptr<uint16_t>(output);
    a.rows = rows; a.width = width; a.slots = slots; a.exact_prefix_rows = exact_prefix_rows;
    a.update_scale = update_scale;
    a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
    launch_row<ROW_EXPAND_ADALN>(gpu, a);
    return h3b_launched(gpu, "token_expand_adaln_bf16");
}
