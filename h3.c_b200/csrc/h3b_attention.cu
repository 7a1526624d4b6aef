/* QKV split + per-head RMSNorm + RoPE, and joint (video+audio+text) non-causal
 * attention. Replaces the reference's h3_cuda_attention.cu for the DiT path
 * behind the same C ABI.
 *
 * Flash attention on the 5th-generation tensor cores (head_dim 128):
 *   grid = (ceil(S/128) query tiles, heads); two CTAs share an SM, so one CTA's
 *   softmax overlaps the other's matrix work.
 *   warp 0     TMA producer: Q tile once, then K/V tiles of 64 keys into a
 *              2-stage ring (3-D tensor maps over [row][head][128], 128-byte
 *              swizzle; rows past S are zero-filled by the copy engine).
 *   warp 1     one thread issues tcgen05.mma: S_j = Q.K_j^T (M128 N64 K128)
 *              into one of two TMEM score buffers, and O += P_j.V_j
 *              (M128 N128 K64, V read as an N-major operand) into a TMEM
 *              accumulator.
 *   warps 2-5  softmax, one query row per thread: read S_j from TMEM, online
 *              max/sum in the exp2 domain, round P to BF16 (the reference's
 *              rounding point before P.V, h3_cuda_attention.cu:1526-1528) and
 *              write it to shared memory in the swizzled K-major layout the
 *              tensor core reads. The running maximum is only raised when it
 *              would grow by more than 2^8, in which case the thread rescales
 *              its O row in TMEM; results are exact either way because the row
 *              sum uses the same maximum.
 *   Every wait is bounded (status H3B_STATUS_ATTN_TIMEOUT, reported by submit).
 *
 * A SIMT flash kernel serves other head sizes (the reference's small test
 * shapes); it follows the same online-softmax recurrence in F32.
 */
#include "h3b_common.cuh"
#include "h3b_sm100.cuh"

#include <cmath>
#include <cstdlib>

namespace {

/* ----------------------------------------------------------- QKV + RoPE */

/* One warp per (row, head), head_dim 128: a lane owns dims 4*lane .. 4*lane+3.
 * RoPE pairs dim d < half with d + half; with half a multiple of 4 the partner
 * values live in lane +- half/4 and travel by shuffle. */
__global__ void __launch_bounds__(256)
h3b_qkv_rope_warp(const uint16_t *qkv, const uint16_t *q_norm, const uint16_t *k_norm,
                  const uint16_t *rope_cos, const uint16_t *rope_sin, uint16_t *q_out,
                  uint16_t *k_out, uint16_t *v_out, uint32_t seq, uint32_t heads,
                  uint32_t rope_half, int grouped, float eps) {
    size_t warp_id = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (warp_id >= size_t(seq) * heads) return;
    const int lane = threadIdx.x & 31;
    const uint32_t row = uint32_t(warp_id / heads), head = uint32_t(warp_id % heads);
    const size_t inner = size_t(heads) * 128;
    const size_t row_base = size_t(row) * inner * 3;
    size_t qb, kb, vb;
    if (grouped) {
        qb = row_base + size_t(head) * 384;
        kb = qb + 128;
        vb = kb + 128;
    } else {
        qb = row_base + size_t(head) * 128;
        kb = qb + inner;
        vb = qb + inner * 2;
    }
    const int d0 = lane * 4;
    uint2 qraw = *reinterpret_cast<const uint2 *>(qkv + qb + d0);
    uint2 kraw = *reinterpret_cast<const uint2 *>(qkv + kb + d0);
    uint2 vraw = *reinterpret_cast<const uint2 *>(qkv + vb + d0);
    float q[4] = {h3b_lo(qraw.x), h3b_hi(qraw.x), h3b_lo(qraw.y), h3b_hi(qraw.y)};
    float k[4] = {h3b_lo(kraw.x), h3b_hi(kraw.x), h3b_lo(kraw.y), h3b_hi(kraw.y)};
    float qs = 0.0f, ks = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        qs = fmaf(q[i], q[i], qs);
        ks = fmaf(k[i], k[i], ks);
    }
    qs = h3b_warp_sum(qs);
    ks = h3b_warp_sum(ks);
    const float qi = 1.0f / sqrtf(qs / 128.0f + eps);
    const float ki = 1.0f / sqrtf(ks / 128.0f + eps);
    uint2 qw = *reinterpret_cast<const uint2 *>(q_norm + d0);
    uint2 kw = *reinterpret_cast<const uint2 *>(k_norm + d0);
    const float qwf[4] = {h3b_lo(qw.x), h3b_hi(qw.x), h3b_lo(qw.y), h3b_hi(qw.y)};
    const float kwf[4] = {h3b_lo(kw.x), h3b_hi(kw.x), h3b_lo(kw.y), h3b_hi(kw.y)};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        q[i] = q[i] * qi * qwf[i];
        k[i] = k[i] * ki * kwf[i];
    }
    const int shift = int(rope_half / 4);
    const bool low = uint32_t(d0) < rope_half;
    const bool high = !low && uint32_t(d0) < 2 * rope_half;
    /* partner lane: +shift for the low half, -shift for the high half */
    int partner = low ? lane + shift : lane - shift;
    partner &= 31;
    float qp[4], kp[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        qp[i] = __shfl_sync(0xffffffffu, q[i], partner);
        kp[i] = __shfl_sync(0xffffffffu, k[i], partner);
    }
    if (low || high) {
        const uint32_t table = uint32_t(d0) - (low ? 0u : rope_half);
        uint2 craw = *reinterpret_cast<const uint2 *>(rope_cos + size_t(row) * rope_half + table);
        uint2 sraw = *reinterpret_cast<const uint2 *>(rope_sin + size_t(row) * rope_half + table);
        const float c[4] = {h3b_lo(craw.x), h3b_hi(craw.x), h3b_lo(craw.y), h3b_hi(craw.y)};
        const float s[4] = {h3b_lo(sraw.x), h3b_hi(sraw.x), h3b_lo(sraw.y), h3b_hi(sraw.y)};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (low) {
                q[i] = q[i] * c[i] - qp[i] * s[i];
                k[i] = k[i] * c[i] - kp[i] * s[i];
            } else {
                q[i] = q[i] * c[i] + qp[i] * s[i];
                k[i] = k[i] * c[i] + kp[i] * s[i];
            }
        }
    }
    const size_t o = (size_t(row) * heads + head) * 128 + d0;
    *reinterpret_cast<uint2 *>(q_out + o) = make_uint2(h3b_narrow2(q[0], q[1]), h3b_narrow2(q[2], q[3]));
    *reinterpret_cast<uint2 *>(k_out + o) = make_uint2(h3b_narrow2(k[0], k[1]), h3b_narrow2(k[2], k[3]));
    *reinterpret_cast<uint2 *>(v_out + o) = vraw;
}

/* Any head size: one warp per (row, head), lanes stride over the dims. */
__global__ void __launch_bounds__(256)
h3b_qkv_rope_generic(const uint16_t *qkv, const uint16_t *q_norm, const uint16_t *k_norm,
                     const uint16_t *rope_cos, const uint16_t *rope_sin, uint16_t *q_out,
                     uint16_t *k_out, uint16_t *v_out, uint32_t seq, uint32_t heads, uint32_t hd,
                     uint32_t rope_half, int grouped, float eps) {
    size_t warp_id = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (warp_id >= size_t(seq) * heads) return;
    const int lane = threadIdx.x & 31;
    const uint32_t row = uint32_t(warp_id / heads), head = uint32_t(warp_id % heads);
    const size_t inner = size_t(heads) * hd;
    const size_t row_base = size_t(row) * inner * 3;
    size_t qb, kb, vb;
    if (grouped) {
        qb = row_base + size_t(head) * hd * 3;
        kb = qb + hd;
        vb = kb + hd;
    } else {
        qb = row_base + size_t(head) * hd;
        kb = qb + inner;
        vb = qb + inner * 2;
    }
    float qs = 0.0f, ks = 0.0f;
    for (uint32_t d = lane; d < hd; d += 32) {
        float qv = h3b_widen(qkv[qb + d]), kv = h3b_widen(qkv[kb + d]);
        qs = fmaf(qv, qv, qs);
        ks = fmaf(kv, kv, ks);
    }
    qs = h3b_warp_sum(qs);
    ks = h3b_warp_sum(ks);
    const float qi = 1.0f / sqrtf(qs / float(hd) + eps);
    const float ki = 1.0f / sqrtf(ks / float(hd) + eps);
    for (uint32_t d = lane; d < hd; d += 32) {
        float q0 = h3b_widen(qkv[qb + d]) * qi * h3b_widen(q_norm[d]);
        float k0 = h3b_widen(qkv[kb + d]) * ki * h3b_widen(k_norm[d]);
        if (d < 2 * rope_half) {
            const bool low = d < rope_half;
            const uint32_t p = low ? d + rope_half : d - rope_half;
            const uint32_t t = low ? d : p;
            float q1 = h3b_widen(qkv[qb + p]) * qi * h3b_widen(q_norm[p]);
            float k1 = h3b_widen(qkv[kb + p]) * ki * h3b_widen(k_norm[p]);
            float c = h3b_widen(rope_cos[size_t(row) * rope_half + t]);
            float s = h3b_widen(rope_sin[size_t(row) * rope_half + t]);
            if (low) {
                q0 = q0 * c - q1 * s;
                k0 = k0 * c - k1 * s;
            } else {
                q0 = q0 * c + q1 * s;
                k0 = k0 * c + k1 * s;
            }
        }
        const size_t o = (size_t(row) * heads + head) * hd + d;
        q_out[o] = h3b_narrow(q0);
        k_out[o] = h3b_narrow(k0);
        v_out[o] = qkv[vb + d];
    }
}

/* ------------------------------------------------------ SIMT flash SDPA */

constexpr int kSimtThreads = 128;
constexpr int kSimtMaxDimsPerThread = 4; /* head_dim <= 512 */

__global__ void __launch_bounds__(kSimtThreads)
h3b_sdpa_simt(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *out,
              uint32_t seq, uint32_t heads, uint32_t hd, float scale, int head_major) {
    extern __shared__ float simt_smem[];
    float *qs = simt_smem;              /* hd          */
    float *ps = simt_smem + hd;         /* kSimtThreads */
    __shared__ float red[kSimtThreads / 32];
    __shared__ float bcast;
    const uint32_t row = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint16_t *qp = q + (size_t(row) * heads + head) * hd;
    for (uint32_t d = tid; d < hd; d += kSimtThreads) qs[d] = h3b_widen(qp[d]);
    __syncthreads();
    float m = -INFINITY, l = 0.0f;
    float acc[kSimtMaxDimsPerThread] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint32_t j0 = 0; j0 < seq; j0 += kSimtThreads) {
        const uint32_t j = j0 + tid;
        float s = -INFINITY;
        if (j < seq) {
            const uint16_t *kp = k + (size_t(j) * heads + head) * hd;
            float dot = 0.0f;
            for (uint32_t d = 0; d < hd; d++) dot = fmaf(qs[d], h3b_widen(kp[d]), dot);
            s = dot * scale;
        }
        float tile_max = s;
#pragma unroll
        for (int o = 16; o; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
        if (lane == 0) red[warp] = tile_max;
        __syncthreads();
        if (tid == 0) {
            float t = red[0];
            for (int w = 1; w < kSimtThreads / 32; w++) t = fmaxf(t, red[w]);
            bcast = t;
        }
        __syncthreads();
        const float m_new = fmaxf(m, bcast);
        const float alpha = expf(m - m_new);   /* 0 on the first tile */
        const float p = j < seq ? expf(s - m_new) : 0.0f;
        ps[tid] = p;
        float tile_sum = h3b_warp_sum(p);
        __syncthreads();                      /* bcast consumed, ps visible */
        if (lane == 0) red[warp] = tile_sum;
        __syncthreads();
        float total = 0.0f;
        for (int w = 0; w < kSimtThreads / 32; w++) total += red[w];
        l = l * alpha + total;
        m = m_new;
        const uint32_t live = min(uint32_t(kSimtThreads), seq - j0);
#pragma unroll
        for (int i = 0; i < kSimtMaxDimsPerThread; i++) {
            const uint32_t d = tid + i * kSimtThreads;
            if (d >= hd) break;
            float a = acc[i] * alpha;
            for (uint32_t t = 0; t < live; t++)
                a = fmaf(ps[t], h3b_widen(v[(size_t(j0 + t) * heads + head) * hd + d]), a);
            acc[i] = a;
        }
        __syncthreads();
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < kSimtMaxDimsPerThread; i++) {
        const uint32_t d = tid + i * kSimtThreads;
        if (d >= hd) break;
        const size_t o = head_major ? (size_t(head) * seq + row) * hd + d
                                    : (size_t(row) * heads + head) * hd + d;
        out[o] = h3b_narrow(acc[i] * inv);
    }
}

/* ------------------------------------------- tensor-core flash attention */

constexpr int AT_Q = 128;               /* query rows per CTA            */
constexpr int AT_KV = 64;               /* keys per tile                 */
constexpr int AT_D = 128;               /* head dim                      */
constexpr int AT_STAGES = 2;
constexpr int AT_THREADS = 192;
constexpr int AT_Q_BYTES = AT_Q * AT_D * 2;      /* 32 KiB: two 64-column boxes */
constexpr int AT_K_BYTES = AT_KV * AT_D * 2;     /* 16 KiB: two boxes           */
constexpr int AT_V_BYTES = AT_KV * AT_D * 2;     /* 16 KiB: two boxes           */
constexpr int AT_P_BYTES = AT_Q * AT_KV * 2;     /* 16 KiB: one box             */
constexpr int AT_STAGE_BYTES = AT_K_BYTES + AT_V_BYTES;
constexpr int AT_BAR_BYTES = 128;
constexpr size_t AT_SMEM = AT_Q_BYTES + AT_STAGES * AT_STAGE_BYTES + AT_P_BYTES + AT_BAR_BYTES;
constexpr uint32_t AT_TMEM_COLS = 256;           /* S0 64 | S1 64 | O 128       */
constexpr float AT_RESCALE_THRESHOLD = 8.0f;     /* log2 units                  */

struct AttnArgs {
    uint16_t *out;
    int *status;
    uint32_t seq, heads;
    float scale_log2;
    int head_major;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

/* N-major (MN-major) B operand: V tile [64 keys][128 dims] held as two boxes of
 * [64 keys][64 dims] with 128-byte swizzle. Along N, 64-element groups are one
 * box (8192 bytes) apart = leading byte offset; along K, groups of 8 keys are
 * 1024 bytes apart = stride byte offset. */
__device__ __forceinline__ uint64_t v_operand_desc(uint32_t smem_addr) {
    uint64_t desc = (smem_addr >> 4) & 0x3fffu;
    desc |= uint64_t(8192 >> 4) << 16;
    desc |= uint64_t(1024 >> 4) << 32;
    desc |= uint64_t(1) << 46;
    desc |= uint64_t(2) << 61;
    return desc;
}

__global__ void __launch_bounds__(AT_THREADS, 2)
h3b_sdpa_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, AttnArgs args) {
    extern __shared__ __align__(1024) uint8_t at_smem[];
    const uint32_t base = smem_u32(at_smem);
    const uint32_t q_smem = base;
    const uint32_t kv_smem = q_smem + AT_Q_BYTES;
    const uint32_t p_smem = kv_smem + AT_STAGES * AT_STAGE_BYTES;
    const uint32_t bars = p_smem + AT_P_BYTES;
    const uint32_t q_full = bars;
    const uint32_t k_full = bars + 8;                  /* 2 */
    const uint32_t v_full = bars + 24;                 /* 2 */
    const uint32_t kv_empty = bars + 40;               /* 2 */
    const uint32_t s_full = bars + 56;                 /* 2 */
    const uint32_t s_empty = bars + 72;                /* 2 */
    const uint32_t p_full = bars + 88;
    const uint32_t pv_done = bars + 96;
    const uint32_t tmem_holder = bars + 104;
    volatile int *stop = reinterpret_cast<volatile int *>(at_smem + (bars - base) + 112);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_tile = blockIdx.x, head = blockIdx.y;
    const uint32_t n_tiles = (args.seq + AT_KV - 1) / AT_KV;

    if ((base & 1023u) != 0) {  /* swizzled tiles need 1024-byte alignment */
        if (threadIdx.x == 0) atomicMax(args.status, int(H3B_STATUS_ATTN_TIMEOUT));
        return;
    }
    if (threadIdx.x == 0) {
        *stop = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, 1);
            mbar_init(s_full + 8 * s, 1);
            mbar_init(s_empty + 8 * s, 4);
        }
        mbar_init(p_full, 4);
        mbar_init(pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, AT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_holder));
    const uint32_t tmem_o = tmem_base + 128;

    if (warp == 0) {
        /* ------------------------------------------------ TMA producer */
        if (lane == 0) {
            mbar_expect_tx(q_full, AT_Q_BYTES);
            tma_load_3d(q_smem, &map_q, q_full, 0, int(head), int(q_tile * AT_Q));
            tma_load_3d(q_smem + AT_Q_BYTES / 2, &map_q, q_full, 64, int(head), int(q_tile * AT_Q));
            for (uint32_t j = 0; j < n_tiles; j++) {
                const uint32_t stage = j & 1, round = j >> 1;
                if (!mbar_wait(kv_empty + 8 * stage, (round & 1) ^ 1, stop)) break;
                const uint32_t k_dst = kv_smem + stage * AT_STAGE_BYTES;
                const uint32_t v_dst = k_dst + AT_K_BYTES;
                const int row0 = int(j * AT_KV);
                mbar_expect_tx(k_full + 8 * stage, AT_K_BYTES);
                tma_load_3d(k_dst, &map_k, k_full + 8 * stage, 0, int(head), row0);
                tma_load_3d(k_dst + AT_K_BYTES / 2, &map_k, k_full + 8 * stage, 64, int(head), row0);
                mbar_expect_tx(v_full + 8 * stage, AT_V_BYTES);
                tma_load_3d(v_dst, &map_v, v_full + 8 * stage, 0, int(head), row0);
                tma_load_3d(v_dst + AT_V_BYTES / 2, &map_v, v_full + 8 * stage, 64, int(head), row0);
            }
        }
    } else if (warp == 1) {
        /* -------------------------------------------------- MMA issuer */
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instruction_desc(AT_Q, AT_KV);
            constexpr uint32_t idesc_pv = instruction_desc(AT_Q, AT_D) | (1u << 16); /* B N-major */
            bool alive = mbar_wait(q_full, 0, stop);
            auto issue_qk = [&](uint32_t j) -> bool {
                const uint32_t stage = j & 1, round = j >> 1;
                if (!mbar_wait(k_full + 8 * stage, round & 1, stop)) return false;
                if (!mbar_wait(s_empty + 8 * stage, (round & 1) ^ 1, stop)) return false;
                tc_fence_after();
                const uint32_t k_src = kv_smem + stage * AT_STAGE_BYTES;
#pragma unroll
                for (int kk = 0; kk < AT_D / 16; kk++) {
                    const uint64_t a = operand_desc(q_smem + (kk >> 2) * (AT_Q_BYTES / 2)) +
                                       uint64_t(2 * (kk & 3));
                    const uint64_t b = operand_desc(k_src + (kk >> 2) * (AT_K_BYTES / 2)) +
                                       uint64_t(2 * (kk & 3));
                    umma_bf16(tmem_base + stage * AT_KV, a, b, idesc_qk, kk != 0);
                }
                umma_commit(s_full + 8 * stage);
                return true;
            };
            if (alive) alive = issue_qk(0);
            for (uint32_t j = 0; alive && j < n_tiles; j++) {
                if (j + 1 < n_tiles && !issue_qk(j + 1)) break;
                const uint32_t stage = j & 1, round = j >> 1;
                if (!mbar_wait(p_full, j & 1, stop)) break;
                if (!mbar_wait(v_full + 8 * stage, round & 1, stop)) break;
                tc_fence_after();
                const uint32_t v_src = kv_smem + stage * AT_STAGE_BYTES + AT_K_BYTES;
#pragma unroll
                for (int kk = 0; kk < AT_KV / 16; kk++) {
                    const uint64_t a = operand_desc(p_smem) + uint64_t(2 * kk);
                    const uint64_t b = v_operand_desc(v_src + kk * 16 * 128);
                    umma_bf16(tmem_o, a, b, idesc_pv, (j | uint32_t(kk)) != 0);
                }
                umma_commit(pv_done);
                umma_commit(kv_empty + 8 * stage);
            }
        }
    } else {
        /* ------------------------------------------------------ softmax */
        const uint32_t quarter = warp & 3;
        const uint32_t local_row = quarter * 32 + lane;
        const uint32_t row = q_tile * AT_Q + local_row;
        const uint32_t lane_base = (quarter * 32) << 16;
        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        for (uint32_t j = 0; alive && j < n_tiles; j++) {
            const uint32_t buf = j & 1, round = j >> 1;
            if (!mbar_wait(s_full + 8 * buf, round & 1, stop)) { alive = false; break; }
            tc_fence_after();
            uint32_t s0[32], s1[32];
            tmem_ld32(tmem_base + lane_base + buf * AT_KV, s0);
            tmem_ld32(tmem_base + lane_base + buf * AT_KV + 32, s1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty + 8 * buf);

            const uint32_t valid = args.seq - j * AT_KV;   /* >= 1; >= 64 except on the last tile */
            float tile_max = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i++) {
                float a = uint32_t(i) < valid ? __uint_as_float(s0[i]) : -INFINITY;
                float b = uint32_t(i + 32) < valid ? __uint_as_float(s1[i]) : -INFINITY;
                s0[i] = __float_as_uint(a);
                s1[i] = __float_as_uint(b);
                tile_max = fmaxf(tile_max, fmaxf(a, b));
            }
            const float m_tile = tile_max * args.scale_log2;
            float alpha = 1.0f;
            bool rescale = false;
            if (m_tile - m_run > AT_RESCALE_THRESHOLD) {   /* also true on the first tile */
                alpha = fast_exp2(m_run - m_tile);         /* exp2(-inf) = 0 on the first tile */
                m_run = m_tile;
                rescale = true;
            }
            float tile_sum = 0.0f;
            uint32_t packed[32];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float p0 = fast_exp2(fmaf(__uint_as_float(s0[2 * i]), args.scale_log2, -m_run));
                float p1 = fast_exp2(fmaf(__uint_as_float(s0[2 * i + 1]), args.scale_log2, -m_run));
                float p2 = fast_exp2(fmaf(__uint_as_float(s1[2 * i]), args.scale_log2, -m_run));
                float p3 = fast_exp2(fmaf(__uint_as_float(s1[2 * i + 1]), args.scale_log2, -m_run));
                tile_sum += (p0 + p1) + (p2 + p3);
                packed[i] = pack_bf16(p0, p1);
                packed[16 + i] = pack_bf16(p2, p3);
            }
            l_run = l_run * alpha + tile_sum;

            if (j > 0) {
                /* P buffer free and O stable once P_{j-1}.V_{j-1} has finished */
                if (!mbar_wait(pv_done, (j - 1) & 1, stop)) { alive = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
                    for (int c = 0; c < AT_D / 32; c++) {
                        uint32_t o[32];
                        tmem_ld32(tmem_o + lane_base + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tmem_o + lane_base + c * 32, o);
                    }
                    tmem_st_wait();
                }
            }
            /* P row: 64 BF16 = 8 chunks of 16 bytes, chunk c of row r at ((c ^ (r & 7)) << 4) */
            const uint32_t p_row = p_smem + local_row * 128;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint32_t addr = p_row + ((uint32_t(c) ^ (local_row & 7u)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                             "r"(packed[4 * c]), "r"(packed[4 * c + 1]), "r"(packed[4 * c + 2]),
                             "r"(packed[4 * c + 3])
                             : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (alive && mbar_wait(pv_done, (n_tiles - 1) & 1, stop)) {
            tc_fence_after();
            const float inv = 1.0f / l_run;
            uint16_t *dst = args.head_major
                                ? args.out + (size_t(head) * args.seq + row) * AT_D
                                : args.out + (size_t(row) * args.heads + head) * AT_D;
#pragma unroll 1
            for (int c = 0; c < AT_D / 32; c++) {
                uint32_t o[32];
                tmem_ld32(tmem_o + lane_base + c * 32, o);
                tmem_ld_wait();
                if (row < args.seq) {
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                        *reinterpret_cast<uint4 *>(dst + c * 32 + v * 8) = w;
                    }
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*stop) {
        if (threadIdx.x == 0) atomicMax(args.status, int(H3B_STATUS_ATTN_TIMEOUT));
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_free(tmem_base, AT_TMEM_COLS);
    }
}

/* [rows][heads][128] BF16 viewed as a 3-D tensor (dim, head, row); box = 64 dims x 1 head x box_rows */
bool make_qkv_map(CUtensorMap *map, const uint16_t *data, uint32_t rows, uint32_t heads,
                  uint32_t box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    cuuint64_t dims[3] = {128, heads, rows};
    cuuint64_t strides[2] = {128 * 2, cuuint64_t(heads) * 128 * 2};
    cuuint32_t box[3] = {64, 1, box_rows};
    cuuint32_t elem[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<uint16_t *>(data), dims,
                  strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sdpa_common(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t seq,
                uint32_t heads, uint32_t hd, float scale, int head_major) {
    size_t count = size_t(seq) * heads * hd;
    if (!seq || !heads || !hd) return h3b_fail(gpu, "SDPA shape is empty");
    if (!h3b_need_command(gpu)) return 0;
    if (!query || !key || !value || !output || query->dtype != H3_GPU_BF16 ||
        key->dtype != H3_GPU_BF16 || value->dtype != H3_GPU_BF16 || output->dtype != H3_GPU_BF16)
        return h3b_fail(gpu, "SDPA tensor dtype mismatch");
    if (query->elements < count || key->elements < count || value->elements < count ||
        output->elements < count)
        return h3b_fail(gpu, "SDPA tensor is too small");
    const char *force = getenv("H3B_SDPA_SIMT");
    bool simt = force && *force && strcmp(force, "0") != 0;
    bool aligned = h3b_aligned16(query->data) && h3b_aligned16(key->data) &&
                   h3b_aligned16(value->data) && h3b_aligned16(output->data);
    if (hd == AT_D && aligned && !simt && scale > 0.0f) {
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(h3b_sdpa_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(AT_SMEM)) != cudaSuccess) {
                cudaGetLastError();
                return h3b_fail(gpu, "cannot reserve shared memory for the attention kernel");
            }
            configured = true;
        }
        CUtensorMap map_q, map_k, map_v;
        if (!make_qkv_map(&map_q, h3b_ptr<uint16_t>(query), seq, heads, AT_Q) ||
            !make_qkv_map(&map_k, h3b_ptr<uint16_t>(key), seq, heads, AT_KV) ||
            !make_qkv_map(&map_v, h3b_ptr<uint16_t>(value), seq, heads, AT_KV))
            return h3b_fail(gpu, "cannot encode the attention tensor maps");
        AttnArgs args;
        args.out = h3b_ptr<uint16_t>(output);
        args.status = gpu->status_device;
        args.seq = seq;
        args.heads = heads;
        args.scale_log2 = scale * 1.4426950408889634f;
        args.head_major = head_major;
        dim3 grid((seq + AT_Q - 1) / AT_Q, heads);
        h3b_sdpa_tc<<<grid, AT_THREADS, AT_SMEM, gpu->stream>>>(map_q, map_k, map_v, args);
        return h3b_launched(gpu, "sdpa_bf16", H3B_SDPA);
    }
    if (hd > uint32_t(kSimtThreads * kSimtMaxDimsPerThread))
        return h3b_fail(gpu, "SDPA head dimension is too large");
    dim3 grid(seq, heads);
    size_t smem = (size_t(hd) + kSimtThreads) * sizeof(float);
    h3b_sdpa_simt<<<grid, kSimtThreads, smem, gpu->stream>>>(
        h3b_ptr<uint16_t>(query), h3b_ptr<uint16_t>(key), h3b_ptr<uint16_t>(value),
        h3b_ptr<uint16_t>(output), seq, heads, hd, scale, head_major);
    return h3b_launched(gpu, "sdpa_bf16", H3B_SDPA);
}

}  // namespace

int h3b_qkv_rope_launch(h3_gpu *gpu, uint16_t *q, uint16_t *k, uint16_t *v, const uint16_t *qkv,
                        const uint16_t *qn, const uint16_t *kn, const uint16_t *rc,
                        const uint16_t *rs, uint32_t seq, uint32_t heads, uint32_t hd,
                        uint32_t rope_half, int grouped, float eps) {
    size_t warps = size_t(seq) * heads;
    if (warps) {
        unsigned blocks = unsigned((warps * 32 + 255) / 256);
        bool aligned8 = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(qkv) |
                          reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn) |
                          reinterpret_cast<uintptr_t>(rc) | reinterpret_cast<uintptr_t>(rs)) & 7u) == 0;
        if (hd == 128 && rope_half % 4 == 0 && aligned8)
            h3b_qkv_rope_warp<<<blocks, 256, 0, gpu->stream>>>(qkv, qn, kn, rc, rs, q, k, v, seq,
                                                              heads, rope_half, grouped, eps);
        else
            h3b_qkv_rope_generic<<<blocks, 256, 0, gpu->stream>>>(qkv, qn, kn, rc, rs, q, k, v, seq,
                                                                 heads, hd, rope_half, grouped, eps);
    }
    return h3b_launched(gpu, "qkv_rope_bf16");
}

/* ================================================================= C ABI */

static int qkv_rope_checked(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                            h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                            const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                            const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                            uint32_t seq, uint32_t heads, uint32_t hd, uint32_t rope_half,
                            int grouped, float eps) {
    size_t count = size_t(seq) * heads * hd;
    size_t rope_count = size_t(seq) * rope_half;
    if (!h3b_need(gpu, qkv, H3_GPU_BF16, count * 3, "QKV input") ||
        !h3b_need(gpu, q_norm, H3_GPU_BF16, hd, "Q norm") ||
        !h3b_need(gpu, k_norm, H3_GPU_BF16, hd, "K norm") ||
        !h3b_need(gpu, rope_cos, H3_GPU_BF16, rope_count, "RoPE cosine") ||
        !h3b_need(gpu, rope_sin, H3_GPU_BF16, rope_count, "RoPE sine") ||
        !h3b_need(gpu, query, H3_GPU_BF16, count, "query") ||
        !h3b_need(gpu, key, H3_GPU_BF16, count, "key") ||
        !h3b_need(gpu, value, H3_GPU_BF16, count, "value"))
        return 0;
    if (rope_half * 2 > hd) return h3b_fail(gpu, "RoPE width exceeds the head dimension");
    if (!h3b_need_command(gpu)) return 0;
    return h3b_qkv_rope_launch(gpu, h3b_ptr<uint16_t>(query), h3b_ptr<uint16_t>(key),
                               h3b_ptr<uint16_t>(value), h3b_ptr<uint16_t>(qkv),
                               h3b_ptr<uint16_t>(q_norm), h3b_ptr<uint16_t>(k_norm),
                               h3b_ptr<uint16_t>(rope_cos), h3b_ptr<uint16_t>(rope_sin), seq, heads,
                               hd, rope_half, grouped, eps);
}

extern "C" int h3_gpu_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                                    h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                                    const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                    const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                    uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                    uint32_t rope_half, float epsilon) {
    return qkv_rope_checked(gpu, query, key, value, qkv, q_norm, k_norm, rope_cos, rope_sin,
                            sequence, heads, head_dim, rope_half, 0, epsilon);
}

extern "C" int h3_gpu_grouped_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                                            h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                                            const h3_gpu_tensor *q_norm,
                                            const h3_gpu_tensor *k_norm,
                                            const h3_gpu_tensor *rope_cos,
                                            const h3_gpu_tensor *rope_sin, uint32_t sequence,
                                            uint32_t heads, uint32_t head_dim, uint32_t rope_half,
                                            float epsilon) {
    return qkv_rope_checked(gpu, query, key, value, qkv, q_norm, k_norm, rope_cos, rope_sin,
                            sequence, heads, head_dim, rope_half, 1, epsilon);
}

extern "C" int h3_gpu_grouped_qkv_linear_rope_bf16(
    h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key, h3_gpu_tensor *value,
    h3_gpu_tensor *qkv, const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
    const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm, const h3_gpu_tensor *rope_cos,
    const h3_gpu_tensor *rope_sin, uint32_t rows, uint32_t input_dim, uint32_t heads,
    uint32_t head_dim, uint32_t rope_half, float epsilon) {
    uint32_t inner = heads * head_dim;
    return h3_gpu_linear_bf16(gpu, qkv, input, weight, nullptr, rows, input_dim, inner * 3) &&
           h3_gpu_grouped_qkv_rope_bf16(gpu, query, key, value, qkv, q_norm, k_norm, rope_cos,
                                        rope_sin, rows, heads, head_dim, rope_half, epsilon);
}

extern "C" int h3_gpu_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                                const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                                uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                float scale) {
    return sdpa_common(gpu, output, query, key, value, sequence, heads, head_dim, scale, 0);
}

extern "C" int h3_gpu_sdpa_bf16_head_major_output(h3_gpu *gpu, h3_gpu_tensor *output,
                                                  const h3_gpu_tensor *query,
                                                  const h3_gpu_tensor *key,
                                                  const h3_gpu_tensor *value, uint32_t sequence,
                                                  uint32_t heads, uint32_t head_dim,
                                                  float scale) {
    return sdpa_common(gpu, output, query, key, value, sequence, heads, head_dim, scale, 1);
}
