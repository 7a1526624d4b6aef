/* QKV split + per-head RMSNorm + RoPE, and joint (video+audio+text) non-causal
 * attention. Replaces the reference's h3_cuda_attention.cu for the DiT path
 * behind the same C ABI.
 *
 * Flash attention on the 5th-generation tensor cores (head_dim 128), two kernels. Calls take
 * h3b_sdpa_tc2 (described at its definition below: one 128-row query tile per CTA, three
 * score buffers, softmax groups alternating over key steps; dense or under a block-sparse
 * mask); with H3B_SDPA_TWO_TILES=1 they take h3b_sdpa_tc:
 *   grid = (ceil(S/256), heads); one CTA per SM works on two 128-row query tiles that
 *   ping-pong: while one tile's softmax runs, the tensor core works for the other, and every
 *   K/V tile fetched into shared memory is used by both.
 *   warp 0      TMA producer: the 256 query rows once, then K tiles (3-stage ring) and V
 *               tiles (2-stage ring) of 128 keys (3-D tensor maps over [row][head][128],
 *               128-byte swizzle; rows past S are zero-filled by the copy engine).
 *   warp 1      issues tcgen05.mma (all lanes run the loop so operands stay warp-uniform,
 *               lane 0 issues): S_t = Q_t.K_j^T (M128 N128 K16 x 8, both operands in smem)
 *               into the tile's TMEM score buffer, and O_t += P_j.V_j (M128 N128 K16 x 8)
 *               with P read from TENSOR MEMORY as the A operand and V as an N-major smem
 *               operand. P_t overwrites the first half of S_t; the next Q.K^T of the tile
 *               is issued right behind P.V, in-order execution protects P.
 *               128-key tiles keep every instruction at N=128: measured here, N=64
 *               instructions reach only ~75 % of the N=128 rate.
 *   warps 2-17  softmax: per query tile 4 lane quarters x 2 key halves. A thread owns one
 *               query row (its TMEM lane) and 64 keys: scores TMEM -> registers, maxima of
 *               the two halves exchanged through shared memory (named barrier of the two
 *               warps), online max/sum in the exp2 domain (ex2.approx), P rounded to BF16
 *               (the reference's rounding point before P.V, h3_cuda_attention.cu:1526-1528)
 *               and stored to TMEM. The running maximum is raised lazily (only when it
 *               would grow by more than 2^8) with an in-TMEM rescale of O; results are exact
 *               either way because the row sum uses the same maximum.
 *   Every wait is bounded (status H3B_STATUS_ATTN_TIMEOUT, reported by submit); the
 *   named barrier of a warp pair also carries a "still running" vote so both leave together.
 *
 * A SIMT flash kernel serves other head sizes (the reference's small test
 * shapes); it follows the same online-softmax recurrence in F32.
 */
#include "h3b_common.cuh"
#include "h3b_sm100.cuh"

#include <cmath>
#include <type_traits>
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

__device__ __forceinline__ float simt_load(const uint16_t *p) { return h3b_widen(*p); }
__device__ __forceinline__ float simt_load(const float *p) { return *p; }
__device__ __forceinline__ void simt_store(uint16_t *p, float v) { *p = h3b_narrow(v); }
__device__ __forceinline__ void simt_store(float *p, float v) { *p = v; }

/* T = uint16_t (BF16) or float: the arithmetic is F32 either way */
template <typename T>
__global__ void __launch_bounds__(kSimtThreads)
h3b_sdpa_simt(const T *q, const T *k, const T *v, T *out,
              uint32_t seq, uint32_t heads, uint32_t hd, float scale, int head_major) {
    extern __shared__ float simt_smem[];
    float *qs = simt_smem;              /* hd          */
    float *ps = simt_smem + hd;         /* kSimtThreads */
    __shared__ float red[kSimtThreads / 32];
    __shared__ float bcast;
    const uint32_t row = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T *qp = q + (size_t(row) * heads + head) * hd;
    for (uint32_t d = tid; d < hd; d += kSimtThreads) qs[d] = simt_load(qp + d);
    __syncthreads();
    float m = -INFINITY, l = 0.0f;
    float acc[kSimtMaxDimsPerThread] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint32_t j0 = 0; j0 < seq; j0 += kSimtThreads) {
        const uint32_t j = j0 + tid;
        float s = -INFINITY;
        if (j < seq) {
            const T *kp = k + (size_t(j) * heads + head) * hd;
            float dot = 0.0f;
            for (uint32_t d = 0; d < hd; d++) dot = fmaf(qs[d], simt_load(kp + d), dot);
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
                a = fmaf(ps[t], simt_load(v + (size_t(j0 + t) * heads + head) * hd + d), a);
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
        simt_store(out + o, acc[i] * inv);
    }
}

/* ------------------------------------------- tensor-core flash attention */

constexpr int AT_QT = 128;              /* rows of one query tile        */
constexpr int AT_TILES = 2;             /* query tiles per CTA           */
constexpr int AT_Q = AT_QT * AT_TILES;  /* query rows per CTA            */
constexpr int AT_KV = 128;              /* keys per tile                 */
constexpr int AT_D = 128;               /* head dim                      */
constexpr int AT_K_STAGES = 3;
constexpr int AT_V_STAGES = 2;
constexpr int AT_SOFTMAX_WARPS = 8 * AT_TILES;   /* per tile: 4 lane quarters x 2 key halves */
constexpr int AT_THREADS = 64 + 32 * AT_SOFTMAX_WARPS;  /* producer, MMA, softmax warps */
constexpr int AT_Q_BYTES = AT_Q * AT_D * 2;      /* 64 KiB: two boxes of [256 rows][64 dims] */
constexpr int AT_K_BYTES = AT_KV * AT_D * 2;     /* 32 KiB: two boxes of [128 keys][64 dims] */
constexpr int AT_V_BYTES = AT_KV * AT_D * 2;     /* 32 KiB: two boxes                        */
constexpr int AT_BAR_BYTES = 256;
constexpr int AT_XCHG_BYTES = AT_TILES * 2 * AT_QT * 4;   /* row maxima / sums between key halves */
constexpr size_t AT_SMEM =
    AT_Q_BYTES + AT_K_STAGES * AT_K_BYTES + AT_V_STAGES * AT_V_BYTES + AT_BAR_BYTES + AT_XCHG_BYTES;
/* Tensor-memory columns (32-bit each, 128 lanes = query rows):
 *   [  0,256)  S_t scores F32 (128 columns per query tile); P_t (BF16 pairs, 64 columns)
 *              overwrites the first half of S_t and is the A operand of P.V
 *   [256,512)  O_t accumulators F32 (128 columns per tile)
 * Keys are taken 128 at a time so that every tcgen05.mma is M128 N128 K16: measured on
 * B200, N=64 instructions run at well under the N=128 rate.                          */
constexpr uint32_t AT_TMEM_COLS = 512;
constexpr uint32_t AT_COL_S = 0, AT_COL_O = 256;
constexpr float AT_RESCALE_THRESHOLD = 8.0f;     /* log2 units */

struct AttnArgs {
    uint16_t *out;
    int *status;
    long long wait_cycles;   /* budget of every bounded wait */
    uint32_t seq, heads;
    float scale_log2;
    int head_major;
    /* sequence-parallel push (world != 0): output row r goes to rank r / rows_local, into
     * [rows_local][heads_total][128] at head head0 + head */
    uint32_t world, rows_local, heads_total, head0;
    uint16_t *peer_o[8];
    /* block-sparse mask: step lists per CTA of two query tiles and per query block (see
     * h3_gpu); NULL = dense */
    const uint32_t *sparse_cta_ptr, *sparse_steps;
    const uint32_t *sparse_block_ptr, *sparse_block_steps;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

/* 8-column forms for the rare rescale of O, which runs while the scores occupy the registers */
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
                   "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
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

/* V tile [128 keys][128 dims] is held as two boxes of [128 keys][64 dims] with 128-byte
 * swizzle and read as an N-major B operand: along N, 64-element groups are one box
 * (16384 bytes) apart = leading byte offset; along K, groups of 8 keys are 1024 bytes
 * apart = stride byte offset; 16 keys (one instruction) are 2048 bytes. */
template <bool PUSH, bool SPARSE>
__global__ void __launch_bounds__(AT_THREADS, 1)
h3b_sdpa_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, AttnArgs args) {
    extern __shared__ __align__(1024) uint8_t at_smem[];
    const uint32_t base = smem_u32(at_smem);
    const uint32_t q_smem = base;
    const uint32_t k_smem = q_smem + AT_Q_BYTES;
    const uint32_t v_smem = k_smem + AT_K_STAGES * AT_K_BYTES;
    const uint32_t bars = v_smem + AT_V_STAGES * AT_V_BYTES;
    const uint32_t q_full = bars;                          /* 1           */
    const uint32_t k_full = bars + 8;                      /* AT_K_STAGES */
    const uint32_t k_empty = k_full + 8 * AT_K_STAGES;     /* AT_K_STAGES */
    const uint32_t v_full = k_empty + 8 * AT_K_STAGES;     /* AT_V_STAGES */
    const uint32_t v_empty = v_full + 8 * AT_V_STAGES;     /* AT_V_STAGES */
    const uint32_t s_full = v_empty + 8 * AT_V_STAGES;     /* [tile] = 2  */
    const uint32_t p_full = s_full + 16;                   /* [tile][early, late] = 4 */
    const uint32_t o_done = p_full + 32;                   /* 1           */
    const uint32_t tmem_holder = o_done + 8;
    volatile int *stop = reinterpret_cast<volatile int *>(at_smem + (tmem_holder + 8 - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_block = blockIdx.x, head = blockIdx.y;
    /* dense: key tiles 0 .. n_tiles-1 in order; sparse: this CTA's step list (never longer than
     * the dense walk, so no defect in the lists can unbound the loops) */
    uint32_t n_tiles = (args.seq + AT_KV - 1) / AT_KV;
    const uint32_t *steps = nullptr;
    if (SPARSE) {
        const uint32_t first = args.sparse_cta_ptr[q_block];
        steps = args.sparse_steps + first;
        n_tiles = min(n_tiles, args.sparse_cta_ptr[q_block + 1] - first);
    }

    if ((base & 1023u) != 0) {  /* swizzled tiles need 1024-byte alignment */
        if (threadIdx.x == 0) atomicMax(args.status, int(H3B_STATUS_ATTN_TIMEOUT));
        return;
    }
    if (threadIdx.x == 0) {
        *stop = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < AT_K_STAGES; s++) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
        }
        for (int s = 0; s < AT_V_STAGES; s++) {
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        for (int t = 0; t < AT_TILES; t++) {
            mbar_init(s_full + 8 * t, 1);
            mbar_init(p_full + 16 * t, 8);
            mbar_init(p_full + 16 * t + 8, 8);
        }
        mbar_init(o_done, 1);
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

    if (warp == 0) {
        /* ------------------------------------------------ TMA producer */
        if (lane == 0) {
            mbar_expect_tx(q_full, AT_Q_BYTES);
            tma_load_3d(q_smem, &map_q, q_full, 0, int(head), int(q_block * AT_Q));
            tma_load_3d(q_smem + AT_Q_BYTES / 2, &map_q, q_full, 64, int(head), int(q_block * AT_Q));
            uint32_t ks = 0, kp = 0, vs = 0, vp = 0;
            for (uint32_t j = 0; j < n_tiles; j++) {
                const int row0 = int((SPARSE ? (steps[j] & 0x0fffffffu) : j) * AT_KV);
                if (!mbar_wait(k_empty + 8 * ks, kp ^ 1, stop, args.wait_cycles)) break;
                mbar_expect_tx(k_full + 8 * ks, AT_K_BYTES);
                tma_load_3d(k_smem + ks * AT_K_BYTES, &map_k, k_full + 8 * ks, 0, int(head), row0);
                tma_load_3d(k_smem + ks * AT_K_BYTES + AT_K_BYTES / 2, &map_k, k_full + 8 * ks, 64,
                            int(head), row0);
                if (++ks == AT_K_STAGES) { ks = 0; kp ^= 1; }
                if (!mbar_wait(v_empty + 8 * vs, vp ^ 1, stop, args.wait_cycles)) break;
                mbar_expect_tx(v_full + 8 * vs, AT_V_BYTES);
                tma_load_3d(v_smem + vs * AT_V_BYTES, &map_v, v_full + 8 * vs, 0, int(head), row0);
                tma_load_3d(v_smem + vs * AT_V_BYTES + AT_V_BYTES / 2, &map_v, v_full + 8 * vs, 64,
                            int(head), row0);
                if (++vs == AT_V_STAGES) { vs = 0; vp ^= 1; }
            }
        }
    } else if (warp == 1) {
        /* -------------------------------------------------- MMA issuer */
        /* all 32 lanes run the loop (warp-uniform control flow and operands); lane 0 issues */
        {
            const uint32_t leader = lane == 0;
            constexpr uint32_t idesc_qk = instruction_desc(AT_QT, AT_KV);
            constexpr uint32_t idesc_pv = instruction_desc(AT_QT, AT_D) | (1u << 16); /* B N-major */
            const uint32_t q_lo0 = desc_lo_kmajor(q_smem);
            const uint32_t k_lo0 = desc_lo_kmajor(k_smem);
            const uint32_t v_lo0 = desc_lo_nmajor(v_smem, AT_V_BYTES / 2);
            /* S_t = Q_t . K_j^T : Q box b holds dims [64b, 64b+64) of all 256 rows, tile t starts
             * 16 KiB into the box; K likewise in two boxes; 32 bytes per 16-dim slice */
            auto issue_qk = [&](uint32_t t, uint32_t k_lo) {
                const uint32_t d = tmem_base + AT_COL_S + t * AT_KV;
                const uint32_t a_lo = q_lo0 + t * ((AT_QT * 128) >> 4);
                umma_ss<false>(d, a_lo, k_lo, idesc_qk, leader);
#pragma unroll
                for (int kk = 1; kk < AT_D / 16; kk++)
                    umma_ss<true>(d, a_lo + (kk >> 2) * ((AT_Q_BYTES / 2) >> 4) + 2 * (kk & 3),
                                  k_lo + (kk >> 2) * ((AT_K_BYTES / 2) >> 4) + 2 * (kk & 3), idesc_qk,
                                  leader);
                umma_commit_if(s_full + 8 * t, leader);
            };
            bool alive = mbar_wait(q_full, 0, stop, args.wait_cycles) && mbar_wait(k_full, 0, stop, args.wait_cycles);
            alive = __all_sync(0xffffffffu, alive);
            if (alive) {
                tc_fence_after();
                issue_qk(0, k_lo0);
                issue_qk(1, k_lo0);
                umma_commit_if(k_empty, leader);
            }
            uint32_t ks = 1 % AT_K_STAGES, kp = (AT_K_STAGES == 1), vs = 0, vp = 0;
            for (uint32_t j = 0; alive && j < n_tiles; j++) {
                const uint32_t v_lo = v_lo0 + vs * (AT_V_BYTES >> 4);
                const uint32_t k_lo_next = k_lo0 + ks * (AT_K_BYTES >> 4);
                const bool more = j + 1 < n_tiles;
#pragma unroll
                for (int t = 0; t < AT_TILES; t++) {
                    /* P_t arrives in two parts: each softmax warp publishes the first 32 of its
                     * 64 keys while it still works on the rest, so the first half of O_t += P_t.V_j
                     * (16-key groups 0,1 and 4,5) overlaps the second half of the exponentials */
                    /* Waits that are normally satisfied long before (the next K tile, this V tile)
                     * come first: a wait in the middle of a run of MMAs lets the short queue of
                     * the tensor pipe run dry, even when the barrier has already flipped. */
                    if (t == 0) {
                        alive = mbar_wait(v_full + 8 * vs, vp, stop, args.wait_cycles);
                        if (alive && more) alive = mbar_wait(k_full + 8 * ks, kp, stop, args.wait_cycles);
                    }
                    alive = __all_sync(0xffffffffu, alive && mbar_wait(p_full + 16 * t, j & 1, stop, args.wait_cycles));
                    if (!alive) break;
                    /* the second part of P_t is usually complete by now: one fence, eight MMAs */
                    const bool late_ready = __all_sync(0xffffffffu, mbar_try(p_full + 16 * t + 8, j & 1));
                    tc_fence_after();
                    /* O_t += P_t . V_j : A = P_t in TMEM (first 64 columns of S_t), 8 columns and
                     * 2048 bytes of V per 16 keys */
                    const uint32_t d = tmem_base + AT_COL_O + t * AT_D;
                    const uint32_t a = tmem_base + AT_COL_S + t * AT_KV;
                    if (j == 0) umma_ts<false>(d, a, v_lo, idesc_pv, leader);
                    else umma_ts<true>(d, a, v_lo, idesc_pv, leader);
                    umma_ts<true>(d, a + 1 * 8, v_lo + 1 * (2048 >> 4), idesc_pv, leader);
                    umma_ts<true>(d, a + 4 * 8, v_lo + 4 * (2048 >> 4), idesc_pv, leader);
                    umma_ts<true>(d, a + 5 * 8, v_lo + 5 * (2048 >> 4), idesc_pv, leader);
                    if (!late_ready) {
                        alive = __all_sync(0xffffffffu, mbar_wait(p_full + 16 * t + 8, j & 1, stop, args.wait_cycles));
                        if (!alive) break;
                        tc_fence_after();
                    }
                    umma_ts<true>(d, a + 2 * 8, v_lo + 2 * (2048 >> 4), idesc_pv, leader);
                    umma_ts<true>(d, a + 3 * 8, v_lo + 3 * (2048 >> 4), idesc_pv, leader);
                    umma_ts<true>(d, a + 6 * 8, v_lo + 6 * (2048 >> 4), idesc_pv, leader);
                    umma_ts<true>(d, a + 7 * 8, v_lo + 7 * (2048 >> 4), idesc_pv, leader);
                    if (t == AT_TILES - 1) umma_commit_if(v_empty + 8 * vs, leader);
                    if (more) {
                        /* the next scores of this tile go straight behind: in-order execution keeps
                         * them from overwriting P_t before P_t.V_j has read it */
                        issue_qk(t, k_lo_next);
                        if (t == AT_TILES - 1) umma_commit_if(k_empty + 8 * ks, leader);
                    }
                }
                if (!alive) break;
                if (++vs == AT_V_STAGES) { vs = 0; vp ^= 1; }
                if (++ks == AT_K_STAGES) { ks = 0; kp ^= 1; }
            }
            if (alive) umma_commit_if(o_done, leader);
        }
    } else {
        /* ------------------------------------------------------ softmax */
        /* 16 warps: query tile (2) x key half (2) x lane quarter (4). A thread owns one query
         * row (its TMEM lane) and 64 of the 128 keys of a tile; the two warps that share a
         * row exchange their maxima through shared memory, so both use the same reference
         * maximum, and keep separate partial row sums that are added at the end. */
        const uint32_t idx = uint32_t(warp - 2);
        const uint32_t tile = idx >> 3, half = (idx >> 2) & 1u;
        const uint32_t quarter = warp & 3;
        const uint32_t local_row = quarter * 32 + lane;
        const uint32_t lane_base = (quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + AT_COL_S + tile * AT_KV + half * 64 + lane_base;
        const uint32_t tmem_p = tmem_base + AT_COL_S + tile * AT_KV + half * 32 + lane_base;
        const uint32_t tmem_o = tmem_base + AT_COL_O + tile * AT_D + lane_base;
        const uint32_t my_s_full = s_full + 8 * tile, my_p_full = p_full + 16 * tile;
        const uint32_t pair_barrier = 1 + tile * 4 + quarter;          /* 64 threads each */
        float *xchg = reinterpret_cast<float *>(at_smem + (bars - base) + AT_BAR_BYTES);
        float *mine = xchg + (tile * 2 + half) * AT_QT + local_row;
        const float *theirs = xchg + (tile * 2 + (half ^ 1u)) * AT_QT + local_row;
        const float scale_log2 = args.scale_log2;

        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        for (uint32_t j = 0; alive && j < n_tiles; j++) {
            /* S_t(j) complete; every earlier MMA of this CTA (P.V of tile j-1 included) too */
            const bool ready = __all_sync(0xffffffffu, mbar_wait(my_s_full, j & 1, stop, args.wait_cycles));
            tc_fence_after();
            /* the loads run even if the wait gave up (tensor-memory reads are always safe), so
             * the score registers have one definition and stay in registers */
            uint32_t s0[32], s1[32];
            tmem_ld32(tmem_s, s0);
            tmem_ld32(tmem_s + 32, s1);
            tmem_ld_wait();
            /* keys of the tile this warp may use: all but the ragged tail of the sequence; none
             * when the block-sparse mask leaves out this (query block, 64-key half) */
            const uint32_t step = SPARSE ? steps[j] : (j | 0xf0000000u);
            const uint32_t valid =
                ((step >> (28 + 2 * tile + half)) & 1u) ? args.seq - (step & 0x0fffffffu) * AT_KV : 0u;
            if (valid < uint32_t(AT_KV)) {
                const uint32_t k0 = half * 64;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (k0 + i >= valid) s0[i] = 0xff800000u;        /* -inf */
                    if (k0 + 32 + i >= valid) s1[i] = 0xff800000u;
                }
            }
            /* three-input max: half the instructions of a pairwise reduction */
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                mx0 = max3_f32(mx0, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
                mx1 = max3_f32(mx1, __uint_as_float(s0[i + 2]), __uint_as_float(s0[i + 3]));
                mx2 = max3_f32(mx2, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
                mx3 = max3_f32(mx3, __uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3]));
            }
            const float mx_half = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            *mine = mx_half;
            /* Pair barrier: after it both key halves have their scores in registers (P may
             * overwrite S) and see each other's maximum. It also carries the "still running"
             * vote, so the two warps of a row always leave the loop in the same iteration. */
            {
                uint32_t both;
                asm volatile(
                    "{\n\t.reg .pred pin, pout;\n\t"
                    "setp.ne.u32 pin, %2, 0;\n\t"
                    "bar.red.and.pred pout, %1, 64, pin;\n\t"
                    "selp.u32 %0, 1, 0, pout;\n\t}"
                    : "=r"(both)
                    : "r"(pair_barrier), "r"(uint32_t(ready))
                    : "memory");
                if (!both) { alive = false; break; }
            }
            const float m_tile = fmaxf(mx_half, *theirs) * scale_log2;
            float alpha = 1.0f;
            bool rescale = false;
            if (m_tile - m_run > AT_RESCALE_THRESHOLD) {   /* also true on the first tile */
                alpha = fast_exp2(m_run - m_tile);         /* exp2(-inf) = 0 on the first tile */
                m_run = m_tile;
                rescale = true;
            }
            if (j > 0 && __any_sync(0xffffffffu, rescale)) {
                /* O_t is stable: P.V of tile j-1 finished before S_t(j) was signalled. Each
                 * key half rescales its own 64 columns of O_t (the decision is identical in
                 * both warps of a row: same maxima, same history). Done before any part of
                 * P_t(j) is published, so no P.V of this step can run ahead of it. */
#pragma unroll 1
                for (int c = 0; c < 8; c++) {
                    uint32_t o[8];
                    tmem_ld8(tmem_o + half * 64 + c * 8, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st8(tmem_o + half * 64 + c * 8, o);
                }
            }
            /* x = s * scale_log2 - m and the row sum run as packed F32 pairs (one instruction
             * per two elements); the exponential itself is scalar (MUFU). The thread's first 32
             * keys are published as soon as they are done (keys 64*half + 2i, +1 -> P column
             * 32*half + i), the other 32 follow. */
            const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
            /* m_run is still -inf only when every score so far was masked: subtract 0 then, so
             * that the masked scores give 2^-inf = 0 and not 2^(inf - inf) */
            const float neg_m = m_run == -INFINITY ? 0.0f : -m_run;
            const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
            uint64_t sum_a = 0, sum_b = 0;                  /* two packed partial sums (+0.0f) */
#pragma unroll
            for (int part = 0; part < 2; part++) {
                const uint32_t(&sv)[32] = part == 0 ? s0 : s1;
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint64_t xa = fma_f32x2(pack_f32x2(__uint_as_float(sv[4 * i]), __uint_as_float(sv[4 * i + 1])),
                                                  scale2, neg_m2);
                    const uint64_t xb = fma_f32x2(pack_f32x2(__uint_as_float(sv[4 * i + 2]), __uint_as_float(sv[4 * i + 3])),
                                                  scale2, neg_m2);
                    float x0, x1, x2, x3;
                    unpack_f32x2(xa, x0, x1);
                    unpack_f32x2(xb, x2, x3);
                    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                    const float p2 = fast_exp2(x2), p3 = fast_exp2(x3);
                    sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
                    sum_b = add_f32x2(sum_b, pack_f32x2(p2, p3));
                    packed[2 * i] = pack_bf16(p0, p1);
                    packed[2 * i + 1] = pack_bf16(p2, p3);
                }
                tmem_st16(tmem_p + part * 16, packed);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(my_p_full + 8 * part);
            }
            float sum0, sum1, sum2, sum3;
            unpack_f32x2(sum_a, sum0, sum1);
            unpack_f32x2(sum_b, sum2, sum3);
            l_run = l_run * alpha + ((sum0 + sum1) + (sum2 + sum3));
        }
        /* total row sum = sum of the two halves' partial sums (same reference maximum) */
        if (alive) *mine = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        /* Epilogue. Every MMA of the CTA has completed once o_done fires, so the Q tiles'
         * shared memory is free: the two warps that share 32 rows stage their halves of the
         * normalised output there (16-byte chunks, chunk index XOR row: no bank conflicts on
         * either side) and then write whole 256-byte rows, two rows per store instruction.
         * Full-line stores matter when the destination is another GPU's memory. */
        const bool finished = alive && mbar_wait(o_done, 0, stop, args.wait_cycles);
        const uint32_t stage = q_smem + (tile * 4 + quarter) * 8192;
        if (finished) {
            tc_fence_after();
            /* a row whose keys are all masked has sum 0 and O = 0: it gets zeros, as in the
             * reference (h3_cuda_attention.cu:1790,1800), not 0 * inf */
            const float l_row = l_run + *theirs;
            const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
#pragma unroll 1
            for (uint32_t c = 0; c < 2; c++) {
                uint32_t o[32];
                tmem_ld32(tmem_o + half * 64 + c * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t v = 0; v < 4; v++) {
                    const uint32_t chunk = half * 8 + c * 4 + v;
                    const uint32_t addr = stage + lane * 256 + ((chunk ^ (lane & 15)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv)),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv)),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv)),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv))
                                 : "memory");
                }
            }
        }
        uint32_t both_finished;
        asm volatile(
            "{\n\t.reg .pred pin, pout;\n\t"
            "setp.ne.u32 pin, %2, 0;\n\t"
            "bar.red.and.pred pout, %1, 64, pin;\n\t"
            "selp.u32 %0, 1, 0, pout;\n\t}"
            : "=r"(both_finished)
            : "r"(pair_barrier), "r"(uint32_t(finished))
            : "memory");
        if (both_finished) {
            const uint32_t row0 = q_block * AT_Q + tile * AT_QT + quarter * 32;
            const uint32_t chunk = lane & 15;
#pragma unroll 1
            for (uint32_t j = 0; j < 8; j++) {
                const uint32_t r = half * 16 + 2 * j + (lane >> 4);
                const uint32_t out_row = row0 + r;
                uint4 val;
                const uint32_t addr = stage + r * 256 + ((chunk ^ (r & 15)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr) : "memory");
                if (out_row < args.seq) {
                    uint16_t *dst;
                    if (PUSH) {
                        const uint32_t owner = min(out_row / args.rows_local, args.world - 1);
                        uint16_t *peer = args.peer_o[0];
#pragma unroll
                        for (uint32_t p = 1; p < 8; p++)
                            if (p == owner) peer = args.peer_o[p];
                        dst = peer + (size_t(out_row - owner * args.rows_local) * args.heads_total +
                                      args.head0 + head) * AT_D;
                    } else {
                        dst = args.head_major ? args.out + (size_t(head) * args.seq + out_row) * AT_D
                                              : args.out + (size_t(out_row) * args.heads + head) * AT_D;
                    }
                    *reinterpret_cast<uint4 *>(dst + chunk * 8) = val;
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

/* ------------------------------------------------------------------------------------------
 * Second form of the tensor-core kernel: ONE 128-row query tile per CTA, THREE score buffers, and
 * two softmax groups that alternate over the KEY steps of the tile.
 *
 *   tensor memory   S[0] | S[1] | S[2] | O  = 3 x 128 + 128 columns (all 512): the scores of step j
 *                   go to S[j % 3]; P(j) (BF16 pairs, 64 columns) overwrites the first half of the
 *                   buffer it came from and is the A operand of O += P(j).V(j).
 *   MMA warp        per step j: O += P(j).V(j), then S[j % 3] = Q.K(j+3)^T into the buffer P(j) was
 *                   just read from (the in-order pipe keeps the two apart). Scores are thus
 *                   three steps ahead of the P.V products: a group that publishes P(j) finds the
 *                   scores of its next step j+2 complete, and no MMA sits in the chain between
 *                   two softmax passes of a group.
 *   softmax         2 groups x 4 warps; a thread owns one query row (its TMEM lane) and all 128
 *                   keys of a step; group g takes the steps j = g, g+2, ... There is no exchange
 *                   inside a row. The two threads that share a row (one per group) hand the
 *                   row's reference maximum back and forth through shared memory: the group of
 *                   step j decides (lazily, threshold 2^8) whether to raise it, rescales O if so
 *                   (after P(j-1).V(j-1) has completed), publishes it and signals the other
 *                   group, whose step j+1 waits for that signal before its own decision. Each
 *                   group keeps its own partial row sum, rescaled whenever it sees a new
 *                   reference; the two are combined at the end.
 *   ring            three stages; stage j % 3 holds what step j of the MMA warp reads, K(j+3) and
 *                   V(j). They also die together: S(j+3) complete means Q.K(j+3)^T is done and,
 *                   issued before it, so is P(j).V(j); a softmax thread that sees those scores
 *                   releases the stage. One barrier per step ("go") collects everything the MMA
 *                   warp waits for: the bytes of the two tiles and the four softmax warps'
 *                   arrivals for P(j). The first three K tiles come with Q.
 * The two-tile kernel above has QK^T -> softmax -> P.V as the serial chain of a tile's step;
 * here nothing of a step waits for another unit's work on the same step but P.V for P. Measured
 * (B200, CUDA events, S = 6,400 x 56 heads / S = 50,476 x 7 heads): 0.97 / 7.1 ms against
 * 1.02-1.08 / 8.4 ms for the two-tile kernel, and with 7 heads at S = 6,400 (a rank's share
 * under 8-way sequence parallelism, twice as many CTAs) 0.175 against 0.25 ms. What bounds a
 * step now is shared-memory traffic: Q and K tiles are read by the tensor core for every MMA
 * (64 KiB per step), V (32 KiB), and TMA writes the next K and V (64 KiB), 160 KiB at 128 bytes
 * per cycle = 1,250 of the ~1,850 cycles a step takes; the two-tile kernel shares K and V between
 * its tiles (128 KiB per tile step) but pays the serial chain. All waits are mbarrier waits with
 * the context's budget (no named barriers: a group that gives up can never leave the other one
 * blocked). Under a block-sparse mask (SPARSE) the key steps are the query block's own list of
 * 128-key tiles instead of all tiles in order, and a 64-key half the block does not attend gets
 * -inf scores; a block that lists nothing runs one step with both halves off and stores zeros.
 * With one query tile per CTA no step is spent on tiles only the neighbouring block lists. Template
 * parameter D: head_dim 128, or 64 (the video-VAE decoder's: tiles of one 64-dim box, four Q.K^T
 * instructions per step, N = 64 for P.V, local output only). */
constexpr int A2_QT = 128, A2_KV = 128;
constexpr int A2_BOX_BYTES = A2_KV * 64 * 2;                /* a TMA box: 128 rows x 64 dims = 16 KiB */
constexpr int A2_STAGES = 3, A2_S_BUFFERS = 3;
constexpr int A2_THREADS = 64 + 32 * 8;                    /* producer, MMA, 2 groups x 4 softmax warps */
/* Q tile, K stage, V stage of head_dim D (128: two boxes, 64: one) */
template <int D>
constexpr int a2_tile_bytes() { return A2_KV * D * 2; }
constexpr int A2_BAR_BYTES = 512;
constexpr int A2_STATE_BYTES = 5 * A2_QT * 4;   /* per row: reference maximum; (sum, its reference) per group */
template <int D>
constexpr size_t a2_smem() { return size_t(1 + 2 * A2_STAGES) * a2_tile_bytes<D>() + A2_BAR_BYTES + A2_STATE_BYTES; }
static_assert(a2_smem<128>() <= 232448, "the step-alternating attention kernel needs at most 227 KiB of shared memory");
constexpr uint32_t A2_COL_S = 0, A2_COL_O = A2_S_BUFFERS * A2_KV;

template <bool PUSH, int D, bool SPARSE = false>
__global__ void __launch_bounds__(A2_THREADS, 1)
h3b_sdpa_tc2(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
             const __grid_constant__ CUtensorMap map_v, AttnArgs args) {
    static_assert(D == 64 || D == 128, "head_dim 64 or 128");
    constexpr int A2_D = D, A2_TILE_BYTES = a2_tile_bytes<D>();
    extern __shared__ __align__(1024) uint8_t at_smem[];
    const uint32_t base = smem_u32(at_smem);
    const uint32_t q_smem = base;
    const uint32_t k_smem = q_smem + A2_TILE_BYTES;
    const uint32_t v_smem = k_smem + A2_STAGES * A2_TILE_BYTES;
    const uint32_t bars = v_smem + A2_STAGES * A2_TILE_BYTES;
    const uint32_t q_full = bars;                              /* 1: Q and K(0)        */
    const uint32_t go = q_full + 8;                            /* [stage] = 3: tiles loaded and P published */
    const uint32_t stage_free = go + 8 * A2_STAGES;            /* [stage] = 3          */
    const uint32_t s_full = stage_free + 8 * A2_STAGES;        /* [buffer] = 3         */
    const uint32_t pv_tail = s_full + 8 * A2_S_BUFFERS;        /* [step parity] = 2    */
    const uint32_t ref_bar = pv_tail + 16;                     /* [deciding group][quarter] = 8 */
    const uint32_t o_done = ref_bar + 64;                      /* 1                    */
    const uint32_t sum_bar = o_done + 8;                       /* [quarter] = 4        */
    const uint32_t out_bar = sum_bar + 32;                     /* [quarter] = 4        */
    const uint32_t k_first = out_bar + 32;                     /* [2]: K(1), K(2) of the prologue */
    const uint32_t tmem_holder = k_first + 16;
    volatile int *stop = reinterpret_cast<volatile int *>(at_smem + (tmem_holder + 8 - base));
    float *state = reinterpret_cast<float *>(at_smem + (bars - base) + A2_BAR_BYTES);
    float *row_reference = state;                              /* [128]: reference maximum (log2 units) */
    float *group_sum = state + A2_QT;                          /* [2][128] */
    float *group_reference = state + 3 * A2_QT;                /* [2][128] */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_block = blockIdx.x, head = blockIdx.y;
    /* dense: key tiles 0 .. n_steps-1 in order; under a block-sparse mask this query block's
     * step list (at least one step, never more than the dense count) */
    uint32_t n_steps = (args.seq + A2_KV - 1) / A2_KV;
    const uint32_t *steps = nullptr;
    if (SPARSE) {
        const uint32_t first = args.sparse_block_ptr[q_block];
        steps = args.sparse_block_steps + first;
        n_steps = min(n_steps, args.sparse_block_ptr[q_block + 1] - first);
    }
    const long long budget = args.wait_cycles;

    if ((base & 1023u) != 0) {  /* swizzled tiles need 1024-byte alignment */
        if (threadIdx.x == 0) atomicMax(args.status, int(H3B_STATUS_ATTN_TIMEOUT));
        return;
    }
    /* one K, V or Q tile (two 64-dim boxes for head_dim 128) */
    auto load = [&](uint32_t smem, const CUtensorMap *map, uint32_t bar, uint32_t row) {
        tma_load_3d(smem, map, bar, 0, int(head), int(row));
        if (D == 128) tma_load_3d(smem + A2_BOX_BYTES, map, bar, 64, int(head), int(row));
    };
    /* first key row of step j */
    auto key_row = [&](uint32_t j) { return (SPARSE ? (steps[j] & 0x0fffffffu) : j) * A2_KV; };
    if (threadIdx.x == 0) {
        *stop = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < A2_STAGES; s++) { mbar_init(go + 8 * s, 5); mbar_init(stage_free + 8 * s, 1); }
        for (int b = 0; b < A2_S_BUFFERS; b++) {
            mbar_init(s_full + 8 * b, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(pv_tail + 8 * b, 1);
            for (int q = 0; q < 4; q++) mbar_init(ref_bar + 32 * b + 8 * q, 1);
        }
        mbar_init(o_done, 1);
        for (int q = 0; q < 4; q++) { mbar_init(sum_bar + 8 * q, 2); mbar_init(out_bar + 8 * q, 2); }
        mbar_init(k_first, 1);
        mbar_init(k_first + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        /* The prologue's loads go out here, before the block-wide barrier, so that their latency
         * runs beside the tensor-memory allocation: the thread that initialised the barriers may
         * use them at once. Q.K(0)^T starts as soon as Q and K(0) are there; K(1) and K(2) have
         * barriers of their own. The V halves of the first three stages are empty from the
         * start: their tiles go out now too (the stage's barrier is told its whole byte count,
         * K(j+3) follows in the producer's loop). */
        const uint32_t first = n_steps < 3 ? n_steps : 3;
        mbar_expect_tx(q_full, 2 * A2_TILE_BYTES);
        load(q_smem, &map_q, q_full, q_block * A2_QT);
        load(k_smem, &map_k, q_full, key_row(0));
        for (uint32_t j = 1; j < first; j++) {
            mbar_expect_tx(k_first + 8 * (j - 1), A2_TILE_BYTES);
            load(k_smem + j * A2_TILE_BYTES, &map_k, k_first + 8 * (j - 1), key_row(j));
        }
        for (uint32_t j = 0; j < first; j++) {
            mbar_expect_tx(go + 8 * j, (j + 3 < n_steps ? 2 : 1) * A2_TILE_BYTES);
            load(v_smem + j * A2_TILE_BYTES, &map_v, go + 8 * j, key_row(j));
        }
    }
    if (threadIdx.x < A2_QT) row_reference[threadIdx.x] = -INFINITY;
    if (warp == 1) tmem_alloc(tmem_holder, AT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_holder));

    if (warp == 0) {
        /* ------------------------------------------------ TMA producer */
        if (lane == 0) {
            for (uint32_t j = 0; j < n_steps; j++) {
                /* the stage is free once S(j) has been seen: Q.K(j)^T and P(j-3).V(j-3) are done */
                const uint32_t stage = j % A2_STAGES;
                const bool ahead = j + 3 < n_steps;
                if (j < 3 && !ahead) continue;            /* nothing left to load for this step */
                if (!mbar_wait(stage_free + 8 * stage, (j / A2_STAGES) & 1u, stop, budget)) break;
                if (j >= 3) mbar_expect_tx(go + 8 * stage, (ahead ? 2 : 1) * A2_TILE_BYTES);
                if (ahead) load(k_smem + stage * A2_TILE_BYTES, &map_k, go + 8 * stage, key_row(j + 3));
                if (j >= 3) load(v_smem + stage * A2_TILE_BYTES, &map_v, go + 8 * stage, key_row(j));
            }
        }
    } else if (warp == 1) {
        /* -------------------------------------------------- MMA issuer */
        /* The issuing warp is the scarcest resource of this kernel: the tensor pipe accepts the
         * next MMA only when the one before has started (an M128 N128 K16 instruction occupies it
         * for 72 cycles, measured), so every cycle this warp spends on anything else is a cycle
         * the pipe idles. Hence: (a) the loop is unrolled by six (two barrier phases x three
         * buffers), which makes every barrier address, phase and descriptor offset a constant;
         * (b) the three barriers of step j+1 are tested (non-blocking) between the MMAs of step j,
         * where the test's latency hides behind the pipe; only a failed test leads to a wait. */
        const uint32_t leader = lane == 0;
        constexpr uint32_t idesc_qk = instruction_desc(A2_QT, A2_KV);
        constexpr uint32_t idesc_pv = instruction_desc(A2_QT, A2_D) | (1u << 16); /* B N-major */
        constexpr uint32_t HALF = A2_BOX_BYTES >> 4, STAGE = A2_TILE_BYTES >> 4;
        constexpr int QK_MMAS = A2_D / 16;       /* 16 dims per instruction */
        const uint32_t q_lo0 = desc_lo_kmajor(q_smem);
        const uint32_t k_lo0 = desc_lo_kmajor(k_smem);
        const uint32_t v_lo0 = desc_lo_nmajor(v_smem, A2_BOX_BYTES);
        const uint32_t tmem_s0 = tmem_base + A2_COL_S, tmem_o = tmem_base + A2_COL_O;
        /* scores of a step into S[buffer] from K stage `stage` (both step % 3) */
        auto issue_qk = [&](uint32_t buffer) {
            const uint32_t d = tmem_s0 + buffer * A2_KV;
            const uint32_t k_lo = k_lo0 + buffer * STAGE;
            umma_ss<false>(d, q_lo0, k_lo, idesc_qk, leader);
#pragma unroll
            for (int kk = 1; kk < A2_D / 16; kk++)
                umma_ss<true>(d, q_lo0 + (kk >> 2) * HALF + 2 * (kk & 3), k_lo + (kk >> 2) * HALF + 2 * (kk & 3),
                              idesc_qk, leader);
            umma_commit_if(s_full + 8 * buffer, leader);
        };
        bool alive = __all_sync(0xffffffffu, mbar_wait(q_full, 0, stop, budget));
        if (alive) {
            tc_fence_after();
            issue_qk(0);
        }
        for (uint32_t j = 1; alive && j < 3 && j < n_steps; j++) {
            alive = __all_sync(0xffffffffu, mbar_wait(k_first + 8 * (j - 1), 0, stop, budget));
            if (alive) {
                tc_fence_after();
                issue_qk(j);
            }
        }
        /* has the barrier of the coming step been seen complete? */
        uint32_t ready = 0;
        /* one step; R = j mod 6 */
        auto step = [&](auto r_const, uint32_t j) -> bool {
            constexpr uint32_t R = decltype(r_const)::value;
            constexpr uint32_t buffer = R % 3, round = (R / 3) & 1u;   /* S/P buffer and ring stage of step j */
            constexpr uint32_t n_buffer = (R + 1) % 3, n_round = ((R + 1) / 3) & 1u;  /* of step j + 1 */
            const bool ahead = j + 3 < n_steps;
            if (!__all_sync(0xffffffffu, ready != 0u) &&
                !__all_sync(0xffffffffu, mbar_wait(go + 8 * buffer, round, stop, budget)))
                return false;
            tc_fence_after();
            const uint32_t v_lo = v_lo0 + buffer * STAGE;
            const uint32_t a = tmem_s0 + buffer * A2_KV;
            /* O += P(j).V(j): 8 P columns and 2048 bytes of V per 16 keys */
            if (j == 0) umma_ts<false>(tmem_o, a, v_lo, idesc_pv, leader);
            else umma_ts<true>(tmem_o, a, v_lo, idesc_pv, leader);
#pragma unroll
            for (uint32_t kk = 1; kk < 8; kk++) umma_ts<true>(tmem_o, a + kk * 8, v_lo + kk * (2048 >> 4), idesc_pv, leader);
            /* a raise of the reference at step j + 1 waits for this product; from here on no later
             * scores imply it */
            if (j + 3 >= n_steps && j + 1 < n_steps) umma_commit_if(pv_tail + 8 * (j & 1u), leader);
            /* S(j+3) = Q.K(j+3)^T into the buffer P(j) has just been read from (in-order pipe) */
            const uint32_t d = tmem_s0 + buffer * A2_KV;
            const uint32_t k_lo = k_lo0 + buffer * STAGE;
            if (ahead) {
                umma_ss<false>(d, q_lo0, k_lo, idesc_qk, leader);
#pragma unroll
                for (int kk = 1; kk < QK_MMAS - 2; kk++)
                    umma_ss<true>(d, q_lo0 + (kk >> 2) * HALF + 2 * (kk & 3), k_lo + (kk >> 2) * HALF + 2 * (kk & 3),
                                  idesc_qk, leader);
            }
            /* the barrier of step j + 1, tested while the pipe still has MMAs to run */
            ready = mbar_test(go + 8 * n_buffer, n_round);
            if (ahead) {
#pragma unroll
                for (int kk = QK_MMAS - 2; kk < QK_MMAS; kk++)
                    umma_ss<true>(d, q_lo0 + (kk >> 2) * HALF + 2 * (kk & 3), k_lo + (kk >> 2) * HALF + 2 * (kk & 3),
                                  idesc_qk, leader);
                umma_commit_if(s_full + 8 * buffer, leader);
            }
            return true;
        };
        for (uint32_t j = 0; alive && j < n_steps; j += 6) {
            alive = step(std::integral_constant<uint32_t, 0>{}, j);
            if (alive && j + 1 < n_steps) alive = step(std::integral_constant<uint32_t, 1>{}, j + 1);
            if (alive && j + 2 < n_steps) alive = step(std::integral_constant<uint32_t, 2>{}, j + 2);
            if (alive && j + 3 < n_steps) alive = step(std::integral_constant<uint32_t, 3>{}, j + 3);
            if (alive && j + 4 < n_steps) alive = step(std::integral_constant<uint32_t, 4>{}, j + 4);
            if (alive && j + 5 < n_steps) alive = step(std::integral_constant<uint32_t, 5>{}, j + 5);
        }
        if (alive) umma_commit_if(o_done, leader);
    } else {
        /* ------------------------------------------------------ softmax */
        const uint32_t group = uint32_t(warp - 2) >> 2, quarter = warp & 3;
        const uint32_t local_row = quarter * 32 + lane;
        const uint32_t lane_base = (quarter * 32) << 16;
        const uint32_t tmem_o = tmem_base + A2_COL_O + lane_base;
        const uint32_t my_ref_bar = ref_bar + 32 * group + 8 * quarter;            /* I signal   */
        const uint32_t their_ref_bar = ref_bar + 32 * (group ^ 1u) + 8 * quarter;  /* I wait for */
        const float scale_log2 = args.scale_log2;
        const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);

        float reference = -INFINITY;     /* the maximum my partial sum is relative to */
        float sum = 0.0f;
        bool alive = true;
        for (uint32_t j = group; alive && j < n_steps; j += 2) {
            const uint32_t buffer = j % A2_S_BUFFERS, round = (j / A2_S_BUFFERS) & 1u;
            const uint32_t tmem_s = tmem_base + A2_COL_S + buffer * A2_KV + lane_base;   /* also P */
            /* key tile of this step and which of its 64-key halves the query block attends
             * (read before the wait, which hides the load) */
            const uint32_t step_word = SPARSE ? steps[j] : (j | 0x30000000u);
            alive = __all_sync(0xffffffffu, mbar_wait(s_full + 8 * buffer, round, stop, budget));
            if (!alive) break;
            tc_fence_after();
            /* S(j) is there, so Q.K(j)^T has finished and, being issued before it, so has
             * P(j-3).V(j-3): the ring stage that held K(j) and V(j-3) is free; one thread says so */
            if (quarter == 0 && lane == 0) mbar_arrive(stage_free + 8 * buffer);
            /* asked early, needed after the maximum: has the other group decided step j - 1? */
            bool ref_ready = j == 0 || mbar_try(their_ref_bar, ((j - 1) >> 1) & 1u);
            uint32_t s[128];
            tmem_ld32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
            tmem_ld32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
            tmem_ld32(tmem_s + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
            tmem_ld32(tmem_s + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
            tmem_ld_wait();
            const uint32_t valid = args.seq - (step_word & 0x0fffffffu) * A2_KV;
            if (valid < uint32_t(A2_KV)) {
#pragma unroll
                for (int i = 0; i < 128; i++)
                    if (uint32_t(i) >= valid) s[i] = 0xff800000u;        /* -inf */
            }
            if (SPARSE) {
                if (!(step_word & 0x10000000u)) {
#pragma unroll
                    for (int i = 0; i < 64; i++) s[i] = 0xff800000u;
                }
                if (!(step_word & 0x20000000u)) {
#pragma unroll
                    for (int i = 64; i < 128; i++) s[i] = 0xff800000u;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
                mx0 = max3_f32(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                mx1 = max3_f32(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                mx2 = max3_f32(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                mx3 = max3_f32(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
            }
            const float m_step = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
            /* the row's reference as the other group left it after step j - 1 */
            if (!__all_sync(0xffffffffu, ref_ready)) {
                alive = __all_sync(0xffffffffu, mbar_wait(their_ref_bar, ((j - 1) >> 1) & 1u, stop, budget));
                if (!alive) break;
            }
            float row_ref = row_reference[local_row];
            const bool raise = m_step - row_ref > AT_RESCALE_THRESHOLD;   /* also true at step 0 */
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                /* O must be at rest: P(j-1).V(j-1) complete, P(j) not published yet. Q.K(j+2)^T is
                 * issued behind P(j-1).V(j-1), so the scores of step j+2 imply it; the last two
                 * steps have barriers of their own */
                alive = __all_sync(0xffffffffu,
                                   j + 2 < n_steps
                                       ? mbar_wait(s_full + 8 * ((j + 2) % A2_S_BUFFERS), ((j + 2) / A2_S_BUFFERS) & 1u,
                                                   stop, budget)
                                       : mbar_wait(pv_tail + 8 * ((j - 1) & 1u), 0, stop, budget));
                if (!alive) break;
                tc_fence_after();
                const float alpha = raise ? fast_exp2(row_ref - m_step) : 1.0f;
#pragma unroll 1
                for (int c = 0; c < A2_D / 32; c++) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(tmem_o + c * 32, o);
                }
                tmem_st_wait_all();
                tc_fence_before();
            }
            if (raise) {
                row_ref = m_step;
                row_reference[local_row] = m_step;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(my_ref_bar);          /* release: the other group may decide */
            /* my partial sum follows the reference */
            if (reference != row_ref) {
                sum *= reference == -INFINITY ? 0.0f : fast_exp2(reference - row_ref);
                reference = row_ref;
            }
            /* a query block whose list is empty has one step with both halves off: its reference
             * stays -inf, and the probabilities must come out 0, not exp2(-inf + inf) */
            const float neg_m = SPARSE && row_ref == -INFINITY ? 0.0f : -row_ref;
            const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
            uint64_t sum_a = 0, sum_b = 0;
#pragma unroll
            for (int chunk = 0; chunk < 4; chunk++) {                /* 32 keys -> 16 P columns */
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int e = 32 * chunk + 4 * i;
                    const uint64_t xa = fma_f32x2(pack_f32x2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])),
                                                  scale2, neg_m2);
                    const uint64_t xb = fma_f32x2(pack_f32x2(__uint_as_float(s[e + 2]), __uint_as_float(s[e + 3])),
                                                  scale2, neg_m2);
                    float x0, x1, x2, x3;
                    unpack_f32x2(xa, x0, x1);
                    unpack_f32x2(xb, x2, x3);
                    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                    const float p2 = fast_exp2(x2), p3 = fast_exp2(x3);
                    sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
                    sum_b = add_f32x2(sum_b, pack_f32x2(p2, p3));
                    packed[2 * i] = pack_bf16(p0, p1);
                    packed[2 * i + 1] = pack_bf16(p2, p3);
                }
                tmem_st16(tmem_s + chunk * 16, packed);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(go + 8 * buffer);
            float s0, s1, s2, s3;
            unpack_f32x2(sum_a, s0, s1);
            unpack_f32x2(sum_b, s2, s3);
            sum += (s0 + s1) + (s2 + s3);
        }
        /* Combine the two groups' partial sums; normalise and store. Every MMA has completed once
         * o_done fires, so the Q tile's shared memory is free for staging the output rows. */
        group_sum[group * A2_QT + local_row] = sum;
        group_reference[group * A2_QT + local_row] = reference;
        __syncwarp();
        if (lane == 0) mbar_arrive(sum_bar + 8 * quarter);
        bool finished = alive && mbar_wait(sum_bar + 8 * quarter, 0, stop, budget) &&
                        mbar_wait(o_done, 0, stop, budget);
        finished = __all_sync(0xffffffffu, finished);
        /* output rows staged in the Q tile's shared memory: 32 rows x D dims BF16 per quarter */
        constexpr uint32_t ROW_BYTES = A2_D * 2, CHUNKS = A2_D / 8;          /* 16-byte pieces per row */
        const uint32_t stage = q_smem + quarter * 32 * ROW_BYTES;
        if (finished) {
            tc_fence_after();
            const float ra = group_reference[local_row], rb = group_reference[A2_QT + local_row];
            const float r = fmaxf(ra, rb);
            float total = 0.0f;
            if (ra != -INFINITY) total += group_sum[local_row] * fast_exp2(ra - r);
            if (rb != -INFINITY) total += group_sum[A2_QT + local_row] * fast_exp2(rb - r);
            const float inv = total > 0.0f ? 1.0f / total : 0.0f;
            /* group g owns output dims [D/2 g, D/2 g + D/2) of its rows */
#pragma unroll 1
            for (uint32_t c = 0; c < A2_D / 64; c++) {
                uint32_t o[32];
                tmem_ld32(tmem_o + group * (A2_D / 2) + c * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t v = 0; v < 4; v++) {
                    const uint32_t chunk = group * (CHUNKS / 2) + c * 4 + v;
                    const uint32_t addr = stage + lane * ROW_BYTES + ((chunk ^ (lane & (CHUNKS - 1))) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv)),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv)),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv)),
                                 "r"(pack_bf16(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv))
                                 : "memory");
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(out_bar + 8 * quarter);
            finished = __all_sync(0xffffffffu, mbar_wait(out_bar + 8 * quarter, 0, stop, budget));
        }
        if (finished) {
            const uint32_t row0 = q_block * A2_QT + quarter * 32;
            constexpr uint32_t ROWS_PER_STORE = 32 / CHUNKS;         /* a warp's store covers whole rows */
            const uint32_t chunk = lane & (CHUNKS - 1);
#pragma unroll 1
            for (uint32_t i = 0; i < 16 / ROWS_PER_STORE; i++) {
                const uint32_t r = group * 16 + ROWS_PER_STORE * i + lane / CHUNKS;
                const uint32_t out_row = row0 + r;
                uint4 val;
                const uint32_t addr = stage + r * ROW_BYTES + ((chunk ^ (r & (CHUNKS - 1))) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr) : "memory");
                if (out_row < args.seq) {
                    uint16_t *dst;
                    if (PUSH) {
                        const uint32_t owner = min(out_row / args.rows_local, args.world - 1);
                        uint16_t *peer = args.peer_o[0];
#pragma unroll
                        for (uint32_t p = 1; p < 8; p++)
                            if (p == owner) peer = args.peer_o[p];
                        dst = peer + (size_t(out_row - owner * args.rows_local) * args.heads_total +
                                      args.head0 + head) * A2_D;
                    } else {
                        dst = args.head_major ? args.out + (size_t(head) * args.seq + out_row) * A2_D
                                              : args.out + (size_t(out_row) * args.heads + head) * A2_D;
                    }
                    *reinterpret_cast<uint4 *>(dst + chunk * 8) = val;
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

/* [rows][heads][hd] BF16 viewed as a 3-D tensor (dim, head, row); box = 64 dims x 1 head x box_rows */
bool make_qkv_map(CUtensorMap *map, const uint16_t *data, uint32_t rows, uint32_t heads,
                  uint32_t box_rows, uint32_t hd = 128) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    cuuint64_t dims[3] = {hd, heads, rows};
    cuuint64_t strides[2] = {cuuint64_t(hd) * 2, cuuint64_t(heads) * hd * 2};
    cuuint32_t box[3] = {64, 1, box_rows};
    cuuint32_t elem[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<uint16_t *>(data), dims,
                  strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sdpa_common(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t seq,
                uint32_t heads, uint32_t hd, float scale, int head_major,
                const h3x_ulysses_peers *peers = nullptr, uint32_t heads_total = 0) {
    size_t count = size_t(seq) * heads * hd;
    if (!seq || !heads || !hd) return h3b_fail(gpu, "SDPA shape is empty");
    if (!h3b_need_command(gpu)) return 0;
    if (!query || !key || !value || (!output && !peers) || query->dtype != H3_GPU_BF16 ||
        key->dtype != H3_GPU_BF16 || value->dtype != H3_GPU_BF16 ||
        (output && output->dtype != H3_GPU_BF16))
        return h3b_fail(gpu, "SDPA tensor dtype mismatch");
    if (query->elements < count || key->elements < count || value->elements < count ||
        (output && output->elements < count))
        return h3b_fail(gpu, "SDPA tensor is too small");
    const char *force = getenv("H3B_SDPA_SIMT");
    bool simt = force && *force && strcmp(force, "0") != 0;
    bool aligned = h3b_aligned16(query->data) && h3b_aligned16(key->data) &&
                   h3b_aligned16(value->data) && (!output || h3b_aligned16(output->data));
    if (peers && !(hd == AT_D && aligned && scale > 0.0f))
        return h3b_fail(gpu, "the push variant of SDPA needs head_dim 128 and aligned tensors");
    /* a registered block-sparse mask applies to calls with its row count (reference
     * h3_cuda_attention.cu:2559-2562); only the tensor-core kernel walks it */
    const bool sparse = gpu->sparse_cta_ptr && gpu->sparse_rows == seq;
    if (sparse && !(hd == AT_D && aligned && !simt && scale > 0.0f))
        return h3b_fail(gpu, "the block-sparse mask needs head_dim 128, aligned tensors and the tensor-core kernel");
    /* head_dim 64 (the video-VAE decoder's): dense, local output, the one-tile kernel only */
    const char *two_tiles = getenv("H3B_SDPA_TWO_TILES");
    const bool narrow = hd == 64 && !peers && !sparse && !(two_tiles && *two_tiles && strcmp(two_tiles, "0") != 0);
    if ((hd == AT_D || narrow) && aligned && !simt && scale > 0.0f) {
        static bool configured_on[64];      /* the attribute is per device */
        static std::mutex configure_mutex;
        std::unique_lock<std::mutex> configure_guard(configure_mutex);
        bool &configured = configured_on[gpu->device & 63];
        if (!configured) {
            bool ok = true;
            for (auto *kernel : {h3b_sdpa_tc<false, false>, h3b_sdpa_tc<false, true>,
                                 h3b_sdpa_tc<true, false>, h3b_sdpa_tc<true, true>})
                ok = ok && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                int(AT_SMEM)) == cudaSuccess;
            for (auto *kernel : {h3b_sdpa_tc2<false, 128, false>, h3b_sdpa_tc2<true, 128, false>,
                                 h3b_sdpa_tc2<false, 128, true>, h3b_sdpa_tc2<true, 128, true>})
                ok = ok && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                int(a2_smem<128>())) == cudaSuccess;
            ok = ok && cudaFuncSetAttribute(h3b_sdpa_tc2<false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(a2_smem<64>())) == cudaSuccess;
            if (!ok) {
                cudaGetLastError();
                return h3b_fail(gpu, "cannot reserve shared memory for the attention kernel");
            }
            configured = true;
        }
        configure_guard.unlock();
        /* the kernel whose softmax groups alternate over key steps, unless H3B_SDPA_TWO_TILES=1
         * asks for the one that alternates over two query tiles */
        const char *pick = getenv("H3B_SDPA_TWO_TILES");
        const bool step_kernel = !(pick && *pick && strcmp(pick, "0") != 0);
        CUtensorMap map_q, map_k, map_v;
        if (!make_qkv_map(&map_q, h3b_ptr<uint16_t>(query), seq, heads, step_kernel ? A2_QT : AT_Q, hd) ||
            !make_qkv_map(&map_k, h3b_ptr<uint16_t>(key), seq, heads, AT_KV, hd) ||
            !make_qkv_map(&map_v, h3b_ptr<uint16_t>(value), seq, heads, AT_KV, hd))
            return h3b_fail(gpu, "cannot encode the attention tensor maps");
        AttnArgs args = {};
        args.out = output ? h3b_ptr<uint16_t>(output) : nullptr;
        if (peers) {
            args.world = peers->world;
            args.rows_local = peers->rows_local;
            args.heads_total = heads_total;
            args.head0 = peers->rank * heads;
            for (uint32_t r = 0; r < peers->world; r++)
                args.peer_o[r] = static_cast<uint16_t *>(peers->o[r]);
        }
        if (sparse) {
            args.sparse_cta_ptr = gpu->sparse_cta_ptr;
            args.sparse_steps = gpu->sparse_steps;
            args.sparse_block_ptr = gpu->sparse_block_ptr;
            args.sparse_block_steps = gpu->sparse_block_steps;
        }
        args.status = gpu->status_device;
        args.wait_cycles = gpu->wait_cycles;
        args.seq = seq;
        args.heads = heads;
        args.scale_log2 = scale * 1.4426950408889634f;
        args.head_major = head_major;
        if (step_kernel) {
            dim3 grid((seq + A2_QT - 1) / A2_QT, heads);
            if (narrow) {
                h3b_sdpa_tc2<false, 64><<<grid, A2_THREADS, a2_smem<64>(), gpu->stream>>>(map_q, map_k, map_v, args);
                return h3b_launched(gpu, "sdpa_bf16", H3B_SDPA);
            }
            auto *kernel = peers ? (sparse ? h3b_sdpa_tc2<true, 128, true> : h3b_sdpa_tc2<true, 128, false>)
                                 : (sparse ? h3b_sdpa_tc2<false, 128, true> : h3b_sdpa_tc2<false, 128, false>);
            kernel<<<grid, A2_THREADS, a2_smem<128>(), gpu->stream>>>(map_q, map_k, map_v, args);
            return h3b_launched(gpu, "sdpa_bf16", H3B_SDPA);
        }
        dim3 grid((seq + AT_Q - 1) / AT_Q, heads);
        auto *kernel = peers ? (sparse ? h3b_sdpa_tc<true, true> : h3b_sdpa_tc<true, false>)
                             : (sparse ? h3b_sdpa_tc<false, true> : h3b_sdpa_tc<false, false>);
        kernel<<<grid, AT_THREADS, AT_SMEM, gpu->stream>>>(map_q, map_k, map_v, args);
        return h3b_launched(gpu, "sdpa_bf16", H3B_SDPA);
    }
    if (hd > uint32_t(kSimtThreads * kSimtMaxDimsPerThread))
        return h3b_fail(gpu, "SDPA head dimension is too large");
    dim3 grid(seq, heads);
    size_t smem = (size_t(hd) + kSimtThreads) * sizeof(float);
    h3b_sdpa_simt<uint16_t><<<grid, kSimtThreads, smem, gpu->stream>>>(
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
    /* Fused route: the projection's epilogue applies the head norm and RoPE and writes
     * query/key/value directly; the caller's qkv scratch is then left untouched (the
     * reference documents it as scratch that a backend may bypass, h3_gpu.h:465-467).
     * Statistics: one projection + one hand kernel, as the two-step route counts. */
    if (head_dim == 128 && rope_half == 48 && rows && heads) {
        size_t count = size_t(rows) * inner, rope_count = size_t(rows) * rope_half;
        if (!h3b_need(gpu, input, H3_GPU_BF16, size_t(rows) * input_dim, "linear input") ||
            !h3b_need(gpu, weight, H3_GPU_BF16, size_t(inner) * 3 * input_dim, "linear weight") ||
            !h3b_need(gpu, qkv, H3_GPU_BF16, count * 3, "linear output") ||
            !h3b_need(gpu, q_norm, H3_GPU_BF16, head_dim, "Q norm") ||
            !h3b_need(gpu, k_norm, H3_GPU_BF16, head_dim, "K norm") ||
            !h3b_need(gpu, rope_cos, H3_GPU_BF16, rope_count, "RoPE cosine") ||
            !h3b_need(gpu, rope_sin, H3_GPU_BF16, rope_count, "RoPE sine") ||
            !h3b_need(gpu, query, H3_GPU_BF16, count, "query") ||
            !h3b_need(gpu, key, H3_GPU_BF16, count, "key") ||
            !h3b_need(gpu, value, H3_GPU_BF16, count, "value") || !h3b_need_command(gpu))
            return 0;
        int fused = h3b_qkv_rope_gemm(gpu, h3b_ptr<uint16_t>(query), h3b_ptr<uint16_t>(key),
                                      h3b_ptr<uint16_t>(value), h3b_ptr<uint16_t>(input),
                                      h3b_ptr<uint16_t>(weight), h3b_ptr<uint16_t>(q_norm),
                                      h3b_ptr<uint16_t>(k_norm), h3b_ptr<uint16_t>(rope_cos),
                                      h3b_ptr<uint16_t>(rope_sin), rows, input_dim, heads, epsilon);
        if (fused == 1) {
            gpu->stats.direct_dispatches++;
            if (!(rows >= 32 && input_dim >= 256 && inner * 3 >= 256)) {
                gpu->stats.mps_linear_dispatches--;
                gpu->stats.direct_dispatches++;
            }
            return 1;
        }
        if (fused == 0) return 0;
    }
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

/* F32 attention (the video-VAE decoder's, head_dim 64). Like the reference (h3_cuda_attention.cu:
 * 2990-3013) head sizes 64 and 128 go through the BF16 tensor-core kernel: q, k and v are rounded
 * to BF16 into scratch (one launch) and the result is widened again.
 * Other head sizes, and H3B_SDPA_F32_EXACT=1 (the reference's H3_CUDA_SDPA_F32_EXACT), take the
 * F32 SIMT kernel. */
extern "C" int h3_gpu_sdpa_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                               const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                               uint32_t sequence, uint32_t heads, uint32_t head_dim, float scale) {
    const size_t count = size_t(sequence) * heads * head_dim;
    if (!sequence || !heads || !head_dim) return h3b_fail(gpu, "SDPA shape is empty");
    if (!h3b_need(gpu, query, H3_GPU_F32, count, "SDPA query") ||
        !h3b_need(gpu, key, H3_GPU_F32, count, "SDPA key") ||
        !h3b_need(gpu, value, H3_GPU_F32, count, "SDPA value") ||
        !h3b_need(gpu, output, H3_GPU_F32, count, "SDPA output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    const char *exact = getenv("H3B_SDPA_F32_EXACT");
    const bool aligned = h3b_aligned16(query->data) && h3b_aligned16(key->data) &&
                         h3b_aligned16(value->data) && h3b_aligned16(output->data);
    if ((head_dim == 64 || head_dim == 128) && aligned && scale > 0.0f && h3b_tensor_map_available() &&
        !(exact && *exact && strcmp(exact, "0") != 0) && !getenv("H3B_SDPA_SIMT")) {
        /* head_dim 64 runs as it is on the one-tile kernel; where that kernel is switched off
         * (H3B_SDPA_TWO_TILES=1) it is padded with zeros to 128: zero dims add nothing to a score,
         * and the output's extra dims are dropped */
        const char *two_tiles = getenv("H3B_SDPA_TWO_TILES");
        const uint32_t run_dim = head_dim == 64 && !(two_tiles && *two_tiles && strcmp(two_tiles, "0") != 0) ? 64 : AT_D;
        const size_t units = size_t(sequence) * heads, padded = units * run_dim;
        uint16_t *scratch = static_cast<uint16_t *>(h3b_workspace(gpu, 4 * padded * sizeof(uint16_t)));
        if (!scratch) return h3b_fail(gpu, "sdpa_f32: cannot allocate the BF16 operands");
        h3_gpu_tensor half[4];
        for (int i = 0; i < 4; i++) {
            half[i] = h3_gpu_tensor{scratch + i * padded, padded, padded * sizeof(uint16_t), H3_GPU_BF16, gpu, 1};
        }
        const float *const sources[3] = {h3b_ptr<float>(query), h3b_ptr<float>(key), h3b_ptr<float>(value)};
        uint16_t *const targets[3] = {scratch, scratch + padded, scratch + 2 * padded};
        h3b_f32_to_bf16_pad3(gpu, sources, targets, units, head_dim, run_dim);
        if (!h3b_launched(gpu, "sdpa_f32 operands")) return 0;
        /* a block-sparse mask registered for the DiT's BF16 attention does not apply here (the
         * reference passes none on this route, h3_cuda_attention.cu:3010) */
        const uint32_t masked_rows = gpu->sparse_rows;
        gpu->sparse_rows = 0;
        const int ok = sdpa_common(gpu, &half[3], &half[0], &half[1], &half[2], sequence, heads, run_dim, scale, 0);
        gpu->sparse_rows = masked_rows;
        if (!ok) return 0;
        h3b_bf16_to_f32_unpad(gpu, scratch + 3 * padded, h3b_ptr<float>(output), units, head_dim, run_dim);
        return h3b_launched(gpu, "sdpa_f32 result");
    }
    if (head_dim > uint32_t(kSimtThreads * kSimtMaxDimsPerThread))
        return h3b_fail(gpu, "SDPA head dimension is too large");
    dim3 grid(sequence, heads);
    const size_t smem = (size_t(head_dim) + kSimtThreads) * sizeof(float);
    h3b_sdpa_simt<float><<<grid, kSimtThreads, smem, gpu->stream>>>(
        h3b_ptr<float>(query), h3b_ptr<float>(key), h3b_ptr<float>(value), h3b_ptr<float>(output), sequence,
        heads, head_dim, scale, 0);
    return h3b_launched(gpu, "sdpa_f32", H3B_SDPA);
}

/* ---- sequence-parallel variants: the exchange is the kernels' own peer stores ---- */

static int peers_ok(h3_gpu *gpu, const h3x_ulysses_peers *peers, uint32_t heads) {
    if (!peers || !peers->world || peers->world > 8 || peers->rank >= peers->world ||
        !peers->rows_local || heads % peers->world)
        return h3b_fail(gpu, "invalid sequence-parallel peer table");
    return 1;
}

extern "C" int h3x_grouped_qkv_linear_rope_push(
    h3_gpu *gpu, const h3x_ulysses_peers *peers, const h3_gpu_tensor *input,
    const h3_gpu_tensor *weight, const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
    const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin, uint32_t rows,
    uint32_t input_dim, uint32_t heads, uint32_t head_dim, uint32_t rope_half, float epsilon) {
    if (!gpu || !peers_ok(gpu, peers, heads)) return 0;
    if (head_dim != 128 || rope_half != 48 || rows > peers->rows_local)
        return h3b_fail(gpu, "the push variant needs head_dim 128, rope_half 48 and rows <= rows_local");
    for (uint32_t r = 0; r < peers->world; r++)
        if (!peers->q[r] || !peers->k[r] || !peers->v[r] || !h3b_aligned16(peers->q[r]) ||
            !h3b_aligned16(peers->k[r]) || !h3b_aligned16(peers->v[r]))
            return h3b_fail(gpu, "peer q/k/v buffers must be non-null and 16-byte aligned");
    uint32_t inner = heads * head_dim;
    if (!h3b_need(gpu, input, H3_GPU_BF16, size_t(rows) * input_dim, "linear input") ||
        !h3b_need(gpu, weight, H3_GPU_BF16, size_t(inner) * 3 * input_dim, "linear weight") ||
        !h3b_need(gpu, q_norm, H3_GPU_BF16, head_dim, "Q norm") ||
        !h3b_need(gpu, k_norm, H3_GPU_BF16, head_dim, "K norm") ||
        !h3b_need(gpu, rope_cos, H3_GPU_BF16, size_t(rows) * rope_half, "RoPE cosine") ||
        !h3b_need(gpu, rope_sin, H3_GPU_BF16, size_t(rows) * rope_half, "RoPE sine") ||
        !h3b_need_command(gpu))
        return 0;
    if (!rows) return 1;
    int fused = h3b_qkv_rope_gemm(gpu, nullptr, nullptr, nullptr, h3b_ptr<uint16_t>(input),
                                  h3b_ptr<uint16_t>(weight), h3b_ptr<uint16_t>(q_norm),
                                  h3b_ptr<uint16_t>(k_norm), h3b_ptr<uint16_t>(rope_cos),
                                  h3b_ptr<uint16_t>(rope_sin), rows, input_dim, heads, epsilon, peers);
    if (fused < 0) return h3b_fail(gpu, "shape not supported by the fused QKV projection kernel");
    if (fused == 1) gpu->stats.direct_dispatches++;
    return fused;
}

extern "C" int h3x_sdpa_push(h3_gpu *gpu, const h3x_ulysses_peers *peers,
                             const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                             const h3_gpu_tensor *value, uint32_t sequence, uint32_t heads_total,
                             uint32_t head_dim, float scale) {
    if (!gpu || !peers_ok(gpu, peers, heads_total)) return 0;
    for (uint32_t r = 0; r < peers->world; r++)
        if (!peers->o[r] || !h3b_aligned16(peers->o[r]))
            return h3b_fail(gpu, "peer output buffers must be non-null and 16-byte aligned");
    if (size_t(peers->rows_local) * peers->world < sequence)
        return h3b_fail(gpu, "rows_local * world does not cover the sequence");
    return sdpa_common(gpu, nullptr, query, key, value, sequence, heads_total / peers->world,
                       head_dim, scale, 0, peers, heads_total);
}
