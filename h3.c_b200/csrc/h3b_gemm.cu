/* Dense projections of the DiT block: C[rows,n] = X[rows,k] . W[n,k]^T (+bias),
 * BF16 operands, F32 accumulation, BF16 result. Replaces the reference's
 * cuBLASLt wrapper (h3_cuda_gemm.cu) and the projection entry points of
 * h3_cuda_core.cu behind the same C ABI.
 *
 * Tensor-core kernel (sm_100a): one persistent CTA per SM walks 128 x 256
 * output tiles. Warp 0 feeds a 4-stage shared-memory ring with TMA
 * (128-byte swizzle, 64-element K slabs, out-of-range rows and columns are
 * zero-filled by the copy engine). One thread of warp 1 issues
 * tcgen05.mma (M128 N256 K16, cta_group::1) with the F32 accumulator in
 * tensor memory; the accumulator is double-buffered (2 x 256 columns) so that
 * warps 2-5 drain tile i (tcgen05.ld, BF16 rounding, 16-byte stores) while the
 * tensor core already works on tile i+1. Tiles are walked in groups of row
 * blocks sized to ~40 MB of X, so the CTAs that run together share operand
 * slabs in L2 and the weight streams from HBM once per group.
 *
 * The same kernel exists for CTA pairs (h3b_gemm_pair: clusters of two,
 * tcgen05.mma.cta_group::2, 256 x 256 tiles, each CTA loads half of the weight
 * tile); it is chosen for problems of up to 8,192 rows when the 256-row
 * granularity costs no extra round of tiles.
 *
 * Epilogue variants: plain store (+bias); SwiGLU for the MLP up projection,
 * where a tile holds 128 gate columns and the matching 128 up columns so the
 * [rows, 2*hidden] intermediate never goes to memory (rounding points as in the
 * reference: the fc1 result is rounded to BF16, then silu(gate)*up is rounded
 * to BF16, h3_cuda_core.cu:1067-1110); and the grouped QKV projection with
 * per-head RMSNorm and RoPE, which writes q, k and v directly (locally or into
 * the owning rank's buffers for sequence parallelism).
 *
 * Every wait on an mbarrier is bounded: a thread that sees no progress for
 * about a second records H3B_STATUS_GEMM_TIMEOUT, tells the rest of the CTA
 * to stop, and the kernel returns normally (h3_gpu_submit reports it).
 *
 * A SIMT kernel (64 x 64 tiles, one sequential fmaf chain per output starting
 * from the bias, so bit-identical to the reference's scalar kernel) serves
 * shapes the TMA path cannot take (k or n not a multiple of 8, unaligned
 * pointers, F32 operands) and problems too small to fill the machine.
 */
#include "h3b_common.cuh"
#include "h3b_sm100.cuh"

#include <cstdlib>

namespace {

/* ------------------------------------------------------ tensor-core GEMM */

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;                 /* one 128-byte swizzle row of BF16 */
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   /* 16 KiB */
constexpr int B_BYTES = BN * BK * 2;   /* 32 KiB */
constexpr int TC_THREADS = 192;
constexpr size_t TC_SMEM = size_t(STAGES) * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
/* the QKV epilogue turns its row-per-thread results into whole-row stores through an
 * 8 KiB staging area per epilogue warp */
constexpr int QKV_STAGE_BYTES = 32 * 256;
constexpr size_t TC_SMEM_QKV = TC_SMEM + 4 * QKV_STAGE_BYTES;

struct TcArgs {
    uint16_t *out;
    const uint16_t *bias;
    /* F32-store epilogue: out and bias point to F32; the accumulator is multiplied by
     * row_scale[row] * col_scale[column] first (either may be null) */
    const float *row_scale, *col_scale;
    int *status;
    long long wait_cycles; /* budget of every bounded wait */
    uint32_t rows;        /* M */
    uint32_t out_cols;    /* stored columns (n, or hidden for SwiGLU) */
    uint32_t k_blocks;
    uint32_t tiles_m, tiles_n;
    uint32_t group_m;     /* row-blocks walked together so their X slabs stay in L2 */
    /* Tail round split along K: the last split_tiles tiles (what is left after the rounds in
     * which every worker has a whole tile) are each computed by `split` workers, every one over
     * 1/split of the K blocks. Workers 1..split-1 of a tile write their F32 partial tile to
     * split_scratch and raise the tile's counter; worker 0 waits for them, adds the partials to
     * its accumulator in a fixed order and runs the epilogue. split_tiles == 0: off. */
    uint32_t split_tiles, split;
    float *split_scratch;         /* [split_tiles][split - 1][tile rows][256] */
    uint32_t *split_counters;     /* [2][split_tiles]: partials delivered, finishing warps done */
    uint32_t up_offset;   /* SwiGLU: weight row of the first up column (= hidden) */
    /* QKV + norm + RoPE epilogue */
    uint16_t *q_out, *k_out, *v_out;
    const uint16_t *q_norm, *k_norm, *rope_cos, *rope_sin;
    uint32_t heads;
    float eps;
    /* sequence-parallel push: head h belongs to rank h / heads_per_rank, whose gathered
     * buffers take this rank's rows at row offset rank * rows_local (world == 0: local) */
    uint32_t world, rank, rows_local, heads_per_rank;
    uint16_t *peer_q[8], *peer_k[8], *peer_v[8];
};

constexpr int ROPE_HALF = 48;   /* the model's RoPE width (h3_dit.c ROPE_HALF) */

/* A and B are BF16 for every epilogue but the F32 store, whose operands are FP16 (format 0 in
 * bits 7-9 and 10-12 of the instruction descriptor instead of 1) */
template <int EPI>
__host__ __device__ constexpr uint32_t operand_formats(uint32_t idesc) {
    return EPI == H3B_EPI_STORE_F32 ? idesc & ~((7u << 7) | (7u << 10)) : idesc;
}

/* One 128-column unit of the grouped QKV row = q, k or v of one head, held by the thread
 * that owns the row: F32 accumulators -> BF16 (the reference rounds the projection first),
 * RMSNorm over the 128 values with the head-norm weight, half-pair RoPE on dims [0,96),
 * BF16 store. Same expression order as the stand-alone kernel. */
__device__ __forceinline__ void qkv_unit_epilogue(const TcArgs &args, uint32_t lane_addr,
                                                  uint32_t unit, uint32_t row, bool row_ok,
                                                  uint32_t stage_smem, uint32_t lane) {
    const uint32_t head = unit / 3, kind = unit % 3;
    /* dst0 = where row 0 of this rank's slice goes for this head; rows are row_stride apart */
    uint16_t *dst0;
    uint32_t row_stride;
    if (args.world) {
        const uint32_t owner = head / args.heads_per_rank, local_head = head % args.heads_per_rank;
        uint16_t *base = kind == 0 ? args.peer_q[owner] : kind == 1 ? args.peer_k[owner] : args.peer_v[owner];
        row_stride = args.heads_per_rank * 128;
        dst0 = base + (size_t(args.rank) * args.rows_local * args.heads_per_rank + local_head) * 128;
    } else {
        row_stride = args.heads * 128;
        dst0 = (kind == 0 ? args.q_out : kind == 1 ? args.k_out : args.v_out) + size_t(head) * 128;
    }
    float x[128];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tmem_ld32(lane_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) x[c * 32 + i] = round_bf16(__uint_as_float(r[i]));
    }
    if (kind != 2) {
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 128; i++) ss = fmaf(x[i], x[i], ss);
        const float inv = 1.0f / sqrtf(ss / 128.0f + args.eps);
        const uint4 *wsrc = reinterpret_cast<const uint4 *>(kind == 0 ? args.q_norm : args.k_norm);
#pragma unroll
        for (int v = 0; v < 16; v++) {
            const uint4 w = __ldg(wsrc + v);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                x[8 * v + 2 * i] = x[8 * v + 2 * i] * inv * h3b_lo(ww[i]);
                x[8 * v + 2 * i + 1] = x[8 * v + 2 * i + 1] * inv * h3b_hi(ww[i]);
            }
        }
        const uint32_t trow = row_ok ? row : 0;
        const uint4 *csrc = reinterpret_cast<const uint4 *>(args.rope_cos + size_t(trow) * ROPE_HALF);
        const uint4 *ssrc = reinterpret_cast<const uint4 *>(args.rope_sin + size_t(trow) * ROPE_HALF);
#pragma unroll
        for (int v = 0; v < ROPE_HALF / 8; v++) {
            const uint4 c4 = __ldg(csrc + v), s4 = __ldg(ssrc + v);
            const uint32_t cw[4] = {c4.x, c4.y, c4.z, c4.w}, sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int d = 8 * v + i;
                const float c = (i & 1) ? h3b_hi(cw[i >> 1]) : h3b_lo(cw[i >> 1]);
                const float s = (i & 1) ? h3b_hi(sw[i >> 1]) : h3b_lo(sw[i >> 1]);
                const float lo = x[d], hi = x[d + ROPE_HALF];
                x[d] = lo * c - hi * s;
                x[d + ROPE_HALF] = hi * c + lo * s;
            }
        }
    }
    /* Each thread holds one 256-byte row. Through the warp's staging area (16-byte chunks,
     * chunk index XOR row so that neither side has bank conflicts) the warp writes two whole
     * rows per store instruction: full 128-byte lines, which matters when the destination is
     * another GPU's memory. */
#pragma unroll
    for (uint32_t v = 0; v < 16; v++) {
        const uint32_t addr = stage_smem + lane * 256 + ((v ^ (lane & 15)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                     "r"(pack_bf16(x[8 * v], x[8 * v + 1])), "r"(pack_bf16(x[8 * v + 2], x[8 * v + 3])),
                     "r"(pack_bf16(x[8 * v + 4], x[8 * v + 5])), "r"(pack_bf16(x[8 * v + 6], x[8 * v + 7]))
                     : "memory");
    }
    __syncwarp();
    const uint32_t row0 = row - lane, chunk = lane & 15;
#pragma unroll
    for (uint32_t j = 0; j < 16; j++) {
        const uint32_t r = 2 * j + (lane >> 4);
        uint4 val;
        const uint32_t addr = stage_smem + r * 256 + ((chunk ^ (r & 15)) << 4);
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr) : "memory");
        if (row0 + r < args.rows)
            *reinterpret_cast<uint4 *>(dst0 + size_t(row0 + r) * row_stride + chunk * 8) = val;
    }
    __syncwarp();
}

/* What a worker does in a given pass over its work: whole tiles first, then (at most) one
 * K slice of a split tile. */
struct WorkItem {
    uint32_t tile, kb0, kb1, slot, part;    /* part: 0 = whole tile or the finishing slice */
    bool split;
};

__device__ __forceinline__ bool next_item(const TcArgs &args, uint32_t worker, uint32_t workers,
                                          uint32_t pass, WorkItem &item) {
    const uint32_t whole = args.tiles_m * args.tiles_n - args.split_tiles;
    const uint32_t tile = worker + pass * workers;
    if (tile < whole) {
        item = {tile, 0u, args.k_blocks, 0u, 0u, false};
        return true;
    }
    /* whole is a multiple of workers whenever split_tiles != 0, so the split slice comes right
     * after the last whole tile of every worker */
    if (!args.split_tiles || tile - worker != whole || worker >= args.split_tiles * args.split) return false;
    const uint32_t slot = worker / args.split, part = worker % args.split;
    item = {whole + slot, part * args.k_blocks / args.split, (part + 1) * args.k_blocks / args.split,
            slot, part, true};
    return true;
}

/* Epilogue side of a split tile for one thread (= one accumulator row). row_in_tile: the row's
 * index inside the tile; tile_rows: 128 (lone CTA) or 256 (CTA pair); arrivals: epilogue warps
 * per worker (4 or 8). Returns true when this thread goes on to the normal epilogue (its
 * accumulator now holds the whole sum), false when it only delivered a partial or gave up.
 * A partial tile is stored as [32-column chunk][16-byte vector of the chunk][row][4 floats], so
 * the 32 threads of a warp (32 consecutive rows) write and read 512 contiguous bytes per
 * instruction although each of them owns a row. Counters: [slot] counts delivered partials,
 * [split_tiles + slot] counts finishing warps that are done; the last of those clears both,
 * so the words are zero again when the kernel ends. */
constexpr uint32_t kMaxSplit = 4;     /* K slices per split tile, at most */

struct SplitCall {     /* passed by value: the kernel's argument block stays in constant memory */
    float *scratch;
    uint32_t *counters;
    long long wait_cycles;
    uint32_t split_tiles, split, slot, part;
};

__device__ __noinline__ bool split_tile_merge(const SplitCall args, uint32_t lane_addr,
                                              uint32_t row_in_tile, uint32_t tile_rows,
                                              uint32_t arrivals, uint32_t lane, volatile int *stop) {
    const size_t tile_vectors = size_t(tile_rows) * (BN / 4);
    uint4 *slot_base = reinterpret_cast<uint4 *>(args.scratch) +
                       size_t(args.slot) * (args.split - 1) * tile_vectors;
    uint32_t *delivered = args.counters + args.slot;
    uint32_t *finished = args.counters + args.split_tiles + args.slot;
    if (args.part != 0) {
        uint4 *dst = slot_base + size_t(args.part - 1) * tile_vectors + row_in_tile;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
            uint32_t r[32];
            tmem_ld32(lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 8; v++)
                __stcg(dst + size_t(c * 8 + v) * tile_rows,
                       make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]));
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(delivered, 1u);
        return false;
    }
    /* the finishing slice: wait for the other slices' partial tiles (bounded) */
    uint32_t ok = 1;
    if (lane == 0) {
        const uint32_t want = (args.split - 1) * arrivals;
        const long long start = clock64();
        for (;;) {
            uint32_t seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(delivered) : "memory");
            if (seen >= want) break;
            if (*stop || clock64() - start > args.wait_cycles) {
                *stop = 1;
                ok = 0;
                break;
            }
            __nanosleep(32);
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return false;
    /* all partials of a 32-column chunk are requested at once (split <= kMaxSplit, so at most
     * 24 vectors in flight per thread): one round trip to L2 per chunk, not one per partial */
#pragma unroll 1
    for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld32(lane_addr + c * 32, r);
        const uint4 *src = slot_base + size_t(c * 8) * tile_rows + row_in_tile;
        uint4 p[kMaxSplit - 1][8];
#pragma unroll
        for (uint32_t part = 0; part < kMaxSplit - 1; part++)
            if (part + 1 < args.split) {
#pragma unroll
                for (int v = 0; v < 8; v++)
                    p[part][v] = __ldcg(src + size_t(part) * tile_vectors + size_t(v) * tile_rows);
            }
        tmem_ld_wait();
#pragma unroll
        for (uint32_t part = 0; part < kMaxSplit - 1; part++)
            if (part + 1 < args.split) {      /* fixed order: slice 1, 2, 3 */
#pragma unroll
                for (int v = 0; v < 8; v++) {
                    r[4 * v] = __float_as_uint(__uint_as_float(r[4 * v]) + __uint_as_float(p[part][v].x));
                    r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + __uint_as_float(p[part][v].y));
                    r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + __uint_as_float(p[part][v].z));
                    r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + __uint_as_float(p[part][v].w));
                }
            }
        tmem_st32(lane_addr + c * 32, r);
    }
    tmem_st_wait_all();
    __syncwarp();
    if (lane == 0 && atomicAdd(finished, 1u) == arrivals - 1) {
        *finished = 0;
        *delivered = 0;
    }
    return true;
}

/* One thread's share of a finished 128 x 256 accumulator tile: its row (TMEM lane) through the
 * epilogue EPI. lane_addr = TMEM address of the row's first column. */
template <int EPI>
__device__ __forceinline__ void tile_epilogue(const TcArgs &args, uint32_t lane_addr, uint32_t row,
                                              bool row_ok, uint32_t n_blk, uint32_t stage_smem,
                                              uint32_t lane) {
                if (EPI == H3B_EPI_QKV_ROPE) {
                    /* the tile's 256 columns are two whole 128-column units of the grouped row */
    #pragma unroll 1
                    for (uint32_t u = 0; u < 2; u++) {
                        const uint32_t unit = n_blk * 2 + u;
                        if (unit < args.heads * 3)
                            qkv_unit_epilogue(args, lane_addr + u * 128, unit, row, row_ok,
                                              stage_smem, lane);
                    }
                } else if (EPI == H3B_EPI_SWIGLU) {
                    uint16_t *dst = args.out + size_t(row) * args.out_cols + n_blk * 128;
    #pragma unroll 1
                    for (int c = 0; c < 4; c++) {
                        uint32_t g[32], u[32];
                        tmem_ld32(lane_addr + c * 32, g);
                        tmem_ld32(lane_addr + 128 + c * 32, u);
                        tmem_ld_wait();
                        uint32_t col0 = n_blk * 128 + c * 32;
                        uint32_t packed[16];
    #pragma unroll
                        for (int i = 0; i < 16; i++) {
                            float g0 = round_bf16(__uint_as_float(g[2 * i]));
                            float g1 = round_bf16(__uint_as_float(g[2 * i + 1]));
                            float u0 = round_bf16(__uint_as_float(u[2 * i]));
                            float u1 = round_bf16(__uint_as_float(u[2 * i + 1]));
                            packed[i] = pack_bf16(g0 / (1.0f + expf(-g0)) * u0,
                                                   g1 / (1.0f + expf(-g1)) * u1);
                        }
                        if (row_ok) {
    #pragma unroll
                            for (int v = 0; v < 4; v++)
                                if (col0 + v * 8 < args.out_cols)
                                    *reinterpret_cast<uint4 *>(dst + c * 32 + v * 8) = make_uint4(
                                        packed[4 * v], packed[4 * v + 1], packed[4 * v + 2],
                                        packed[4 * v + 3]);
                        }
                    }
                } else if (EPI == H3B_EPI_STORE_F32) {
                    /* the accumulator times the two scales (+ F32 bias): `out` and `bias` point to F32.
                     * A thread holds 32 columns of ITS row; stored like that, a warp's store touches 32
                     * rows with 16 bytes each. The 32 x 32 block goes through the warp's staging area
                     * instead (16-byte pieces XOR-swizzled by row, conflict-free both ways) and leaves as
                     * four whole 128-byte row segments per store instruction. */
                    const float *bias = reinterpret_cast<const float *>(args.bias);
                    const float row_scale = args.row_scale && row_ok ? args.row_scale[row] : 1.0f;
                    const uint32_t row0 = row - lane, piece = lane & 7, sub = lane >> 3;
    #pragma unroll 1
                    for (int c = 0; c < BN / 32; c++) {
                        const uint32_t col0 = n_blk * BN + c * 32;
                        if (col0 >= args.out_cols) break;
                        uint32_t r[32];
                        tmem_ld32(lane_addr + c * 32, r);
                        tmem_ld_wait();
    #pragma unroll
                        for (int v = 0; v < 8; v++) {
                            float4 value = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                            if (args.col_scale && col0 + v * 4 < args.out_cols) {
                                const float4 s = __ldg(reinterpret_cast<const float4 *>(args.col_scale + col0 + v * 4));
                                value.x *= row_scale * s.x; value.y *= row_scale * s.y;
                                value.z *= row_scale * s.z; value.w *= row_scale * s.w;
                            }
                            const uint32_t addr = stage_smem + lane * 128 + ((uint32_t(v) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(value.x),
                                         "f"(value.y), "f"(value.z), "f"(value.w) : "memory");
                        }
                        __syncwarp();
                        const uint32_t col = col0 + piece * 4;
                        float4 b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (bias && col < args.out_cols) b = __ldg(reinterpret_cast<const float4 *>(bias + col));
    #pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const uint32_t rr = sub + 4 * i;
                            float4 value;
                            const uint32_t addr = stage_smem + rr * 128 + ((piece ^ (rr & 7)) << 4);
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(value.x), "=f"(value.y), "=f"(value.z), "=f"(value.w) : "r"(addr) : "memory");
                            value.x += b.x; value.y += b.y; value.z += b.z; value.w += b.w;
                            if (row0 + rr < args.rows && col < args.out_cols)
                                *reinterpret_cast<float4 *>(reinterpret_cast<float *>(args.out) +
                                                            size_t(row0 + rr) * args.out_cols + col) = value;
                        }
                        __syncwarp();
                    }
                } else {
                    uint16_t *dst = args.out + size_t(row) * args.out_cols + n_blk * BN;
    #pragma unroll 1
                    for (int c = 0; c < BN / 32; c++) {
                        uint32_t r[32];
                        tmem_ld32(lane_addr + c * 32, r);
                        tmem_ld_wait();
                        uint32_t col0 = n_blk * BN + c * 32;
                        uint32_t packed[16];
                        if (args.bias) {
    #pragma unroll
                            for (int v = 0; v < 4; v++) {
                                uint4 b = make_uint4(0, 0, 0, 0);
                                if (col0 + v * 8 < args.out_cols)
                                    b = __ldg(reinterpret_cast<const uint4 *>(args.bias + col0 + v * 8));
                                const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
    #pragma unroll
                                for (int i = 0; i < 4; i++)
                                    packed[4 * v + i] = pack_bf16(
                                        __uint_as_float(r[8 * v + 2 * i]) + h3b_lo(bw[i]),
                                        __uint_as_float(r[8 * v + 2 * i + 1]) + h3b_hi(bw[i]));
                            }
                        } else {
    #pragma unroll
                            for (int i = 0; i < 16; i++)
                                packed[i] = pack_bf16(__uint_as_float(r[2 * i]),
                                                       __uint_as_float(r[2 * i + 1]));
                        }
                        if (row_ok) {
    #pragma unroll
                            for (int v = 0; v < 4; v++)
                                if (col0 + v * 8 < args.out_cols)
                                    *reinterpret_cast<uint4 *>(dst + c * 32 + v * 8) = make_uint4(
                                        packed[4 * v], packed[4 * v + 1], packed[4 * v + 2],
                                        packed[4 * v + 3]);
                        }
                    }
                }
}

template <int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
h3b_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            TcArgs args) {
    extern __shared__ uint8_t raw_smem[];
    __shared__ int stop_flag;
    const uint32_t base = (smem_u32(raw_smem) + 1023u) & ~1023u;
    const uint32_t a_smem = base;
    const uint32_t b_smem = base + STAGES * A_BYTES;
    const uint32_t bars = b_smem + STAGES * B_BYTES;
    const uint32_t full_bar = bars;                   /* STAGES x 8 */
    const uint32_t empty_bar = bars + 8 * STAGES;     /* STAGES x 8 */
    const uint32_t acc_full = bars + 16 * STAGES;     /* 2 x 8      */
    const uint32_t acc_empty = acc_full + 16;         /* 2 x 8      */
    const uint32_t tmem_holder = acc_empty + 16;      /* 4 bytes    */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *stop = &stop_flag;

    if (threadIdx.x == 0) {
        stop_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(acc_full + 8 * i, 1);
            mbar_init(acc_empty + 8 * i, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_holder));

    const uint32_t group_tiles = args.group_m * args.tiles_n;

    auto tile_coords = [&](uint32_t tile, uint32_t &m_blk, uint32_t &n_blk) {
        uint32_t group = tile / group_tiles, local = tile % group_tiles;
        uint32_t first_m = group * args.group_m;
        uint32_t group_m = min(args.tiles_m - first_m, args.group_m);
        m_blk = first_m + local % group_m;
        n_blk = local / group_m;
    };

    if (warp == 0) {
        /* ---- TMA producer ---- */
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            WorkItem item;
            for (uint32_t pass = 0; alive && next_item(args, blockIdx.x, gridDim.x, pass, item); pass++) {
                uint32_t m_blk, n_blk;
                tile_coords(item.tile, m_blk, n_blk);
                for (uint32_t kb = item.kb0; kb < item.kb1; kb++) {
                    if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, stop, args.wait_cycles)) { alive = false; break; }
                    uint32_t bar = full_bar + 8 * stage;
                    mbar_expect_tx(bar, A_BYTES + B_BYTES);
                    tma_load_2d(a_smem + stage * A_BYTES, &map_a, bar, int(kb * BK), int(m_blk * BM));
                    if (EPI == H3B_EPI_SWIGLU) {
                        /* 128 gate rows then the matching 128 up rows of the weight */
                        tma_load_2d(b_smem + stage * B_BYTES, &map_b, bar, int(kb * BK),
                                    int(n_blk * 128));
                        tma_load_2d(b_smem + stage * B_BYTES + B_BYTES / 2, &map_b, bar,
                                    int(kb * BK), int(args.up_offset + n_blk * 128));
                    } else {
                        tma_load_2d(b_smem + stage * B_BYTES, &map_b, bar, int(kb * BK),
                                    int(n_blk * BN));
                        tma_load_2d(b_smem + stage * B_BYTES + B_BYTES / 2, &map_b, bar,
                                    int(kb * BK), int(n_blk * BN + 128));
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        /* ---- MMA issuer: all lanes run the loop (uniform operands), lane 0 issues ---- */
        {
            const uint32_t leader = lane == 0;
            constexpr uint32_t idesc = operand_formats<EPI>(instruction_desc(BM, BN));
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            const uint32_t a_lo0 = desc_lo_kmajor(a_smem), b_lo0 = desc_lo_kmajor(b_smem);
            bool alive = true;
            WorkItem item;
            for (uint32_t pass = 0; alive && next_item(args, blockIdx.x, gridDim.x, pass, item); pass++) {
                if (!__all_sync(0xffffffffu, mbar_wait(acc_empty + 8 * acc, acc_phase ^ 1, stop, args.wait_cycles))) break;
                tc_fence_after();
                uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = item.kb0; kb < item.kb1; kb++) {
                    if (!__all_sync(0xffffffffu, mbar_wait(full_bar + 8 * stage, phase, stop, args.wait_cycles))) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (A_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (B_BYTES >> 4);
                    /* 16 BF16 along K = 32 bytes = 2 descriptor address units */
                    if (kb == item.kb0) umma_ss<false>(d_tmem, a_lo, b_lo, idesc, leader);
                    else umma_ss<true>(d_tmem, a_lo, b_lo, idesc, leader);
#pragma unroll
                    for (int k = 1; k < BK / 16; k++)
                        umma_ss<true>(d_tmem, a_lo + 2 * k, b_lo + 2 * k, idesc, leader);
                    umma_commit_if(empty_bar + 8 * stage, leader);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!alive) break;
                umma_commit_if(acc_full + 8 * acc, leader);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        /* ---- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31 ---- */
        const uint32_t quarter = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        WorkItem item;
        for (uint32_t pass = 0; next_item(args, blockIdx.x, gridDim.x, pass, item); pass++) {
            uint32_t m_blk, n_blk;
            tile_coords(item.tile, m_blk, n_blk);
            if (!mbar_wait(acc_full + 8 * acc, acc_phase, stop, args.wait_cycles)) break;
            tc_fence_after();
            const uint32_t row = m_blk * BM + quarter * 32 + lane;
            const uint32_t lane_addr = tmem_base + acc * BN + ((quarter * 32) << 16);
            const bool row_ok = row < args.rows;
            if (!item.split ||
                split_tile_merge(SplitCall{args.split_scratch, args.split_counters, args.wait_cycles,
                                           args.split_tiles, args.split, item.slot, item.part},
                                 lane_addr, quarter * 32 + lane, BM, 4, lane, stop))
                tile_epilogue<EPI>(args, lane_addr, row, row_ok, n_blk,
                                   bars + 256 + quarter * QKV_STAGE_BYTES, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (stop_flag) {
        if (threadIdx.x == 0) atomicMax(args.status, int(H3B_STATUS_GEMM_TIMEOUT));
        /* give copies that may still be in flight time to land before the CTA retires */
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_free(tmem_base, 512);
    }
}

/* ---- the same GEMM on CTA pairs ------------------------------------------------------
 * Cluster of two CTAs = one 256 x 256 output tile: CTA r owns rows [128 r, 128 r + 128) of the
 * tile (its own A slab and its own 128 x 256 accumulator in tensor memory) and loads only half
 * of the weight tile (weight rows [128 r, 128 r + 128) of the 256); the even CTA issues
 * tcgen05.mma.cta_group::2 (M = 256), which reads both halves. Per output element the pair
 * pulls 2/3 of the operand bytes a lone CTA needs, and the weight stream, which is what limits
 * the lone-CTA kernel on the large projections, is halved. Barriers: TMA bytes of both CTAs
 * complete on the even CTA's full barrier; the MMA's commits arrive on the empty / accumulator
 * barriers of both CTAs; the epilogue warps of both CTAs arrive on the even CTA's
 * accumulator-free barrier. Every wait is bounded as in the lone-CTA kernel. */
constexpr int PAIR_STAGE_BYTES = A_BYTES + B_BYTES / 2;          /* 32 KiB per CTA and stage */
/* the epilogues that stage rows through shared memory give up a stage for it */
template <int EPI>
constexpr bool stages_rows() { return EPI == H3B_EPI_QKV_ROPE || EPI == H3B_EPI_STORE_F32; }
template <int EPI>
constexpr int pair_stages() { return stages_rows<EPI>() ? 5 : 6; }
template <int EPI>
constexpr size_t pair_smem() {
    return size_t(pair_stages<EPI>()) * PAIR_STAGE_BYTES + 1024 + 256 +
           (stages_rows<EPI>() ? 4 * QKV_STAGE_BYTES : 0);
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
h3b_gemm_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              TcArgs args) {
    constexpr int NS = pair_stages<EPI>();
    extern __shared__ uint8_t raw_smem[];
    __shared__ int stop_flag;
    const uint32_t base = (smem_u32(raw_smem) + 1023u) & ~1023u;
    const uint32_t a_smem = base;
    const uint32_t b_smem = base + NS * A_BYTES;
    const uint32_t bars = b_smem + NS * (B_BYTES / 2);
    const uint32_t full_bar = bars;                   /* NS x 8, used in the even CTA */
    const uint32_t empty_bar = bars + 8 * NS;         /* NS x 8, per CTA              */
    const uint32_t acc_full = bars + 16 * NS;         /* 2 x 8, per CTA               */
    const uint32_t acc_empty = acc_full + 16;         /* 2 x 8, used in the even CTA  */
    const uint32_t tmem_holder = acc_empty + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    volatile int *stop = &stop_flag;

    if (threadIdx.x == 0) {
        stop_flag = 0;
        for (int s = 0; s < NS; s++) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(acc_full + 8 * i, 1);
            mbar_init(acc_empty + 8 * i, 8);          /* 4 epilogue warps x 2 CTAs */
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_holder, 512);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          /* the peer's barriers exist before anything signals them */
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_holder));

    /* tiles_m counts 256-row tiles */
    const uint32_t group_tiles = args.group_m * args.tiles_n;
    auto tile_coords = [&](uint32_t tile, uint32_t &m_blk, uint32_t &n_blk) {
        uint32_t group = tile / group_tiles, local = tile % group_tiles;
        uint32_t first_m = group * args.group_m;
        uint32_t group_m = min(args.tiles_m - first_m, args.group_m);
        m_blk = first_m + local % group_m;
        n_blk = local / group_m;
    };

    if (warp == 0) {
        /* ---- TMA producer (both CTAs): own A rows, own half of the weight tile ---- */
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            WorkItem item;
            for (uint32_t pass = 0; alive && next_item(args, pair, pairs, pass, item); pass++) {
                uint32_t m_blk, n_blk;
                tile_coords(item.tile, m_blk, n_blk);
                const int a_row = int(m_blk * 256 + rank * BM);
                const int b_row = EPI == H3B_EPI_SWIGLU
                                      ? int((rank ? args.up_offset : 0u) + n_blk * 128)
                                      : int(n_blk * BN + rank * 128);
                for (uint32_t kb = item.kb0; kb < item.kb1; kb++) {
                    if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, stop, args.wait_cycles)) { alive = false; break; }
                    const uint32_t bar = cluster_map(full_bar + 8 * stage, 0);
                    if (rank == 0) mbar_expect_tx(full_bar + 8 * stage, 2 * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(a_smem + stage * A_BYTES, &map_a, bar, int(kb * BK), a_row);
                    tma_load_2d_pair(b_smem + stage * (B_BYTES / 2), &map_b, bar, int(kb * BK), b_row);
                    if (++stage == NS) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        /* ---- MMA issuer: the even CTA only ---- */
        if (rank == 0) {
            const uint32_t leader = lane == 0;
            constexpr uint32_t idesc = operand_formats<EPI>(instruction_desc(256, BN));
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            const uint32_t a_lo0 = desc_lo_kmajor(a_smem), b_lo0 = desc_lo_kmajor(b_smem);
            bool alive = true;
            WorkItem item;
            for (uint32_t pass = 0; alive && next_item(args, pair, pairs, pass, item); pass++) {
                if (!__all_sync(0xffffffffu, mbar_wait(acc_empty + 8 * acc, acc_phase ^ 1, stop, args.wait_cycles))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = item.kb0; kb < item.kb1; kb++) {
                    if (!__all_sync(0xffffffffu, mbar_wait(full_bar + 8 * stage, phase, stop, args.wait_cycles))) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (A_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + stage * ((B_BYTES / 2) >> 4);
                    if (kb == item.kb0) umma_ss_pair<false>(d_tmem, a_lo, b_lo, idesc, leader);
                    else umma_ss_pair<true>(d_tmem, a_lo, b_lo, idesc, leader);
#pragma unroll
                    for (int k = 1; k < BK / 16; k++)
                        umma_ss_pair<true>(d_tmem, a_lo + 2 * k, b_lo + 2 * k, idesc, leader);
                    umma_commit_pair_if(empty_bar + 8 * stage, leader);
                    if (++stage == NS) { stage = 0; phase ^= 1; }
                }
                if (!alive) break;
                umma_commit_pair_if(acc_full + 8 * acc, leader);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        /* ---- epilogue (both CTAs): warps 2..5 own TMEM lanes 32*(warp%4) .. +31 ---- */
        const uint32_t quarter = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        WorkItem item;
        for (uint32_t pass = 0; next_item(args, pair, pairs, pass, item); pass++) {
            uint32_t m_blk, n_blk;
            tile_coords(item.tile, m_blk, n_blk);
            if (!mbar_wait(acc_full + 8 * acc, acc_phase, stop, args.wait_cycles)) break;
            tc_fence_after();
            const uint32_t row = m_blk * 256 + rank * BM + quarter * 32 + lane;
            const uint32_t lane_addr = tmem_base + acc * BN + ((quarter * 32) << 16);
            if (!item.split ||
                split_tile_merge(SplitCall{args.split_scratch, args.split_counters, args.wait_cycles,
                                           args.split_tiles, args.split, item.slot, item.part},
                                 lane_addr, rank * BM + quarter * 32 + lane, 2 * BM, 8, lane, stop))
                tile_epilogue<EPI>(args, lane_addr, row, row < args.rows, n_blk,
                                   bars + 256 + quarter * QKV_STAGE_BYTES, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_map(acc_empty + 8 * acc, 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*stop) {
        if (threadIdx.x == 0) atomicMax(args.status, int(H3B_STATUS_GEMM_TIMEOUT));
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
        __syncthreads();
    }
    /* neither CTA may leave (or free tensor memory) while its peer can still signal its barriers
     * or have its shared memory read by an MMA */
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_free_pair(tmem_base, 512);
    }
}

/* ------------------------------------------------------------- SIMT GEMM */

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<uint16_t>(uint16_t v) { return h3b_widen(v); }

template <typename T>
__device__ __forceinline__ void from_f32(T *p, float v);
template <>
__device__ __forceinline__ void from_f32<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void from_f32<uint16_t>(uint16_t *p, float v) { *p = h3b_narrow(v); }

/* 64 x 64 tile, 16 x 16 threads, 4 x 4 outputs per thread. Each output is one
 * fmaf chain over k in increasing order starting from the bias. Output row r is
 * written at row_map[r] when row_map is given. */
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
h3b_gemm_simt(const TIn *x, const TIn *w, const TIn *bias, TOut *out, const uint32_t *row_map,
              uint32_t rows, uint32_t k, uint32_t n) {
    __shared__ float xs[16][65];
    __shared__ float ws[16][65];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint32_t row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t col = col0 + tx + 16 * j;
        float start = (bias && col < n) ? to_f32<TIn>(bias[col]) : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i][j] = start;
    }
    for (uint32_t k0 = 0; k0 < k; k0 += 16) {
        for (int e = threadIdx.x; e < 64 * 16; e += 256) {
            int r = e >> 4, kk = e & 15;
            uint32_t gr = row0 + r, gc = col0 + r, gk = k0 + kk;
            xs[kk][r] = (gr < rows && gk < k) ? to_f32<TIn>(x[size_t(gr) * k + gk]) : 0.0f;
            ws[kk][r] = (gc < n && gk < k) ? to_f32<TIn>(w[size_t(gc) * k + gk]) : 0.0f;
        }
        __syncthreads();
        uint32_t limit = min(16u, k - k0);
        for (uint32_t kk = 0; kk < limit; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t row = row0 + ty + 16 * i;
        if (row >= rows) continue;
        size_t dst_row = row_map ? row_map[row] : row;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t col = col0 + tx + 16 * j;
            if (col < n) from_f32<TOut>(out + dst_row * n + col, acc[i][j]);
        }
    }
}

template <typename TIn, typename TOut>
void launch_simt(h3_gpu *gpu, const TIn *x, const TIn *w, const TIn *bias, TOut *out,
                 const uint32_t *row_map, uint32_t rows, uint32_t k, uint32_t n) {
    dim3 grid((n + 63) / 64, (rows + 63) / 64);
    h3b_gemm_simt<TIn, TOut><<<grid, 256, 0, gpu->stream>>>(x, w, bias, out, row_map, rows, k, n);
}

/* ----------------------------------------------------------- tensor maps */

/* [rows, k] row-major BF16 matrix, box = 64 columns x box_rows rows, 128-byte swizzle */
bool make_map(CUtensorMap *map, const uint16_t *data, uint64_t rows, uint64_t k,
              uint32_t box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    cuuint64_t dims[2] = {k, rows};
    cuuint64_t strides[1] = {k * 2};
    cuuint32_t box[2] = {BK, box_rows};
    cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(data), dims,
                  strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool env_flag(const char *name) {
    const char *v = getenv(name);
    return v && *v && strcmp(v, "0") != 0;
}

/* How many CTA pairs of the paired kernel the device keeps resident at once (0: clusters of two
 * cannot be scheduled, or the kernel cannot get its shared memory); queried once per epilogue. */
template <int EPI>
int max_resident_pairs(int device) {
    /* function attributes and occupancy belong to a device: one answer per device */
    static int per_device[64];
    static bool known[64];
    static std::mutex guard_mutex;      /* contexts on several threads may launch their first GEMM together */
    std::lock_guard<std::mutex> guard(guard_mutex);
    int &pairs = per_device[device & 63];
    if (known[device & 63]) return pairs;
    known[device & 63] = true;
    pairs = 0;
    if (cudaFuncSetAttribute(h3b_gemm_pair<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(pair_smem<EPI>())) != cudaSuccess) {
        cudaGetLastError();
        return pairs;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * 148);
    config.blockDim = dim3(TC_THREADS);
    config.dynamicSmemBytes = pair_smem<EPI>();
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, h3b_gemm_pair<EPI>, &config) != cudaSuccess) {
        cudaGetLastError();
        return pairs;
    }
    pairs = clusters;
    return pairs;
}

/* Decides whether the last, partly filled round of tiles is split along K, and prepares the
 * scratch for it. `workers` = tiles in flight (CTAs or CTA pairs), tile_rows = 128 or 256.
 * Without the split a launch whose tile count is not a multiple of the workers pays a whole
 * round for the leftover tiles (525 pair tiles on 74 pairs: 8 rounds for 7.1 rounds of work);
 * with it the leftover tiles are shared by all workers. Returns false only on an allocation or
 * memset failure. */
bool configure_split(h3_gpu *gpu, TcArgs &args, uint32_t workers, uint32_t tile_rows) {
    args.split_tiles = args.split = 0;
    args.split_scratch = nullptr;
    args.split_counters = nullptr;
    const uint32_t total = args.tiles_m * args.tiles_n;
    if (env_flag("H3B_NO_SPLIT_K") || total <= workers) return true;
    const uint32_t leftover = total % workers;
    if (!leftover) return true;
    uint32_t split = workers / leftover;
    if (split > args.k_blocks / 8) split = args.k_blocks / 8;     /* at least 8 K blocks per slice */
    if (split > kMaxSplit) split = kMaxSplit;     /* more slices shorten the round little and add partial tiles to merge */
    if (split < 2) return true;
    const size_t need = size_t(leftover) * (split - 1) * tile_rows * BN * sizeof(float);
    if (need > h3_gpu::kSplitScratchBytes) return true;
    if (!gpu->split_scratch) {
        if (gpu->allocation_barred) return true;      /* a no-allocation entry point is running */
        void *block = nullptr;
        if (cudaMalloc(&block, h3_gpu::kSplitScratchBytes + h3_gpu::kSplitCounterBytes) != cudaSuccess) {
            cudaGetLastError();
            return true;                              /* no scratch: run without the split */
        }
        gpu->split_scratch = block;
    }
    uint32_t *counters = reinterpret_cast<uint32_t *>(static_cast<char *>(gpu->split_scratch) +
                                                      h3_gpu::kSplitScratchBytes);
    /* the kernels leave the counters at zero; they are cleared here only for the first launch
     * and after a launch that gave up on a wait */
    if (gpu->split_counters_dirty) {
        if (cudaMemsetAsync(counters, 0, h3_gpu::kSplitCounterBytes, gpu->stream) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        gpu->split_counters_dirty = 0;
    }
    args.split_tiles = leftover;
    args.split = split;
    args.split_scratch = static_cast<float *>(gpu->split_scratch);
    args.split_counters = counters;
    return true;
}

template <int EPI>
int launch_tc(h3_gpu *gpu, uint16_t *out, const uint16_t *x, const uint16_t *w,
              const uint16_t *bias, uint32_t rows, uint32_t k, uint32_t weight_rows,
              uint32_t out_cols, uint32_t tiles_n, uint32_t up_offset,
              const TcArgs *extra = nullptr) {
    static bool configured_on[64];      /* the attribute is per device */
    static std::mutex configure_mutex;
    constexpr size_t smem_bytes = stages_rows<EPI>() ? TC_SMEM_QKV : TC_SMEM;
    std::unique_lock<std::mutex> configure_guard(configure_mutex);
    bool &configured = configured_on[gpu->device & 63];
    if (!configured) {
        if (cudaFuncSetAttribute(h3b_gemm_tc<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(smem_bytes)) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        configured = true;
    }
    configure_guard.unlock();
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, x, rows, k, BM) || !make_map(&map_b, w, weight_rows, k, 128)) return 0;
    TcArgs args = {};
    if (extra) args = *extra;
    args.out = out;
    args.bias = bias;
    args.status = gpu->status_device;
    args.wait_cycles = gpu->wait_cycles;
    args.rows = rows;
    args.out_cols = out_cols;
    args.k_blocks = (k + BK - 1) / BK;
    args.tiles_m = (rows + BM - 1) / BM;
    args.tiles_n = tiles_n;
    args.up_offset = up_offset;
    /* Tile walk: all column blocks for a group of row blocks, then the next group. The
     * weight is streamed from HBM once per group, the group's X rows are re-used from L2,
     * so the group is made as tall as ~40 MB of X allows (L2 is 126 MB) and the groups are
     * balanced. Measured with 16-row-block groups: 3.3x the algorithmic DRAM reads. */
    {
        const double slab = double(BM) * k * 2.0;
        uint32_t gm = uint32_t(40.0e6 / slab);
        gm = gm < 4 ? 4 : gm;
        gm = gm > args.tiles_m ? args.tiles_m : gm;
        const uint32_t groups = (args.tiles_m + gm - 1) / gm;
        args.group_m = (args.tiles_m + groups - 1) / groups;
    }
    /* CTA pairs (256 x 256 tiles) when that does not cost an extra round of tiles (a pair tile
     * occupies each of its two SMs as long as a lone 128 x 256 tile; with few rows the 256-row
     * granularity wastes more: 800 rows = 7 lone row blocks but 4 x 256), the device can
     * co-schedule clusters of two, and X fits in L2: measured inside the power-capped step, pairs
     * win at 6,400 rows (258 vs 265 ms per 50-block step), make no difference at 12,619 rows and
     * lose at 50,476 rows (1,070 vs 1,024 ms per 10 blocks), where X streams from HBM as well. */
    const int pairs = max_resident_pairs<EPI>(gpu->device);
    bool pair_size = false;
    if (pairs > 0 && rows > BM) {
        const uint64_t lone_rounds = (uint64_t(args.tiles_m) * tiles_n + gpu->sm_count - 1) / gpu->sm_count;
        const uint64_t pair_rounds = (uint64_t((rows + 2 * BM - 1) / (2 * BM)) * tiles_n + pairs - 1) / pairs;
        pair_size = (rows <= 8192 && pair_rounds <= lone_rounds) || env_flag("H3B_CTA_PAIRS_ALWAYS");
    }
    if (pair_size && pairs > 0 && !env_flag("H3B_NO_CTA_PAIRS")) {
        args.tiles_m = (rows + 2 * BM - 1) / (2 * BM);
        const double slab = 2.0 * BM * k * 2.0;
        uint32_t gm = uint32_t(40.0e6 / slab);
        gm = gm < 2 ? 2 : gm;
        gm = gm > args.tiles_m ? args.tiles_m : gm;
        const uint32_t groups = (args.tiles_m + gm - 1) / gm;
        args.group_m = (args.tiles_m + groups - 1) / groups;
        const uint32_t tiles = args.tiles_m * args.tiles_n;
        const uint32_t workers = tiles < uint32_t(pairs) ? tiles : uint32_t(pairs);
        if (!configure_split(gpu, args, workers, 2 * BM)) return 0;
        h3b_gemm_pair<EPI><<<2 * workers, TC_THREADS, pair_smem<EPI>(), gpu->stream>>>(map_a, map_b, args);
        return 1;
    }
    uint32_t tiles = args.tiles_m * args.tiles_n;
    uint32_t grid = tiles < uint32_t(gpu->sm_count) ? tiles : uint32_t(gpu->sm_count);
    if (!configure_split(gpu, args, grid, BM)) return 0;
    h3b_gemm_tc<EPI><<<grid, TC_THREADS, smem_bytes, gpu->stream>>>(map_a, map_b, args);
    return 1;
}

}  // namespace

bool h3b_tensor_map_available() { return encode_tiled() != nullptr; }

int h3b_gemm_bf16(h3_gpu *gpu, uint16_t *out, const uint16_t *x, const uint16_t *w,
                  const uint16_t *bias, uint32_t rows, uint32_t k, uint32_t n,
                  h3b_gemm_epilogue epilogue, const char *what) {
    /* n is the number of stored columns: for SwiGLU the weight has 2*n rows */
    if (!rows || !n) return h3b_launched(gpu, what, H3B_LINEAR);
    bool aligned = h3b_aligned16(out) && h3b_aligned16(x) && h3b_aligned16(w) &&
                   (!bias || h3b_aligned16(bias));
    bool tc_ok = aligned && k && k % 8 == 0 && n % 8 == 0 && !env_flag("H3B_NO_TENSOR_CORES") &&
                 (epilogue == H3B_EPI_STORE || n % 128 == 0);
    /* tiny problems are latency bound either way; keep them on the exact kernel */
    if (double(rows) * n * k < 32.0 * 256 * 256) tc_ok = false;
    if (tc_ok) {
        int ok = epilogue == H3B_EPI_SWIGLU
                     ? launch_tc<H3B_EPI_SWIGLU>(gpu, out, x, w, nullptr, rows, k, 2 * n, n,
                                                 n / 128, n)
                     : launch_tc<H3B_EPI_STORE>(gpu, out, x, w, bias, rows, k, n, n,
                                                (n + BN - 1) / BN, 0);
        if (ok) return h3b_launched(gpu, what, H3B_LINEAR);
        return h3b_fail(gpu, "%s: cannot set up the tensor-core GEMM (tensor map or launch attribute)", what);
    }
    if (epilogue == H3B_EPI_SWIGLU) {
        uint16_t *fused =
            static_cast<uint16_t *>(h3b_workspace(gpu, size_t(rows) * n * 2 * sizeof(uint16_t)));
        if (!fused) return h3b_fail(gpu, "%s: cannot allocate the MLP scratch", what);
        launch_simt<uint16_t, uint16_t>(gpu, x, w, nullptr, fused, nullptr, rows, k, 2 * n);
        if (!h3b_launched(gpu, what, H3B_LINEAR)) return 0;
        return h3b_swiglu_launch(gpu, out, fused, rows, n);
    }
    launch_simt<uint16_t, uint16_t>(gpu, x, w, bias, out, nullptr, rows, k, n);
    return h3b_launched(gpu, what, H3B_LINEAR);
}

int h3b_gemm_f32_half(h3_gpu *gpu, float *out, const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                      const float *bias, uint32_t rows, uint32_t k, uint32_t n) {
    const float *x = h3b_ptr<float>(input);
    /* the reference sends an F32 projection to the tensor cores from a reduction length of
     * 1,024 on (h3_cuda_gemm.cu:246-251); shorter ones stay exact */
    const float *w = h3b_ptr<float>(weight);
    if (!rows || !n || k < 1024 || k % 8 != 0 || n % 4 != 0 || env_flag("H3B_NO_TENSOR_CORES") ||
        env_flag("H3B_F32_GEMM_EXACT") || !h3b_aligned16(out) || !h3b_aligned16(x) || !h3b_aligned16(w) ||
        (bias && !h3b_aligned16(bias)))
        return -1;
    auto rounded = [](size_t bytes) { return (bytes + 255) & ~size_t(255); };
    const size_t x_bytes = rounded(size_t(rows) * k * sizeof(uint16_t)), x_scale_bytes = rounded(size_t(rows) * sizeof(float));
    const size_t w_bytes = rounded(size_t(n) * k * sizeof(uint16_t)), w_scale_bytes = rounded(size_t(n) * sizeof(float));
    /* the weight's FP16 rows: kept with a tensor that was created with contents, else scratch */
    h3_gpu_tensor *keeper = weight->keeps_half && weight->elements == size_t(n) * k
                                ? const_cast<h3_gpu_tensor *>(weight) : nullptr;
    /* the input's FP16 rows: left beside it by the op that produced it, else converted here */
    const bool ready = input->half_rows && input->half_k == k && input->elements == size_t(rows) * k;
    const size_t x_room = ready ? 0 : x_bytes + x_scale_bytes;
    uint8_t *scratch = static_cast<uint8_t *>(h3b_workspace(gpu, x_room + (keeper ? 0 : w_bytes + w_scale_bytes)));
    if (!scratch) return h3b_fail(gpu, "linear_f32: cannot allocate the FP16 operands");
    uint16_t *x16 = ready ? static_cast<uint16_t *>(input->half_rows) : reinterpret_cast<uint16_t *>(scratch);
    float *x_scale = ready ? reinterpret_cast<float *>(static_cast<uint8_t *>(input->half_rows) + x_bytes)
                           : reinterpret_cast<float *>(scratch + x_bytes);
    uint16_t *w16;
    float *w_scale;
    if (keeper) {
        if (!keeper->half_rows || keeper->half_k != k) {
            h3b_written(keeper);
            keeper->half_rows = h3b_device_alloc(gpu, w_bytes + w_scale_bytes);
            if (!keeper->half_rows) return h3b_fail(gpu, "linear_f32: cannot allocate the weight's FP16 rows");
            keeper->half_bytes = w_bytes + w_scale_bytes;
            keeper->half_k = k;
            h3b_scale_rows_f16(gpu, w, static_cast<uint16_t *>(keeper->half_rows),
                               reinterpret_cast<float *>(static_cast<uint8_t *>(keeper->half_rows) + w_bytes), n, k);
        }
        w16 = static_cast<uint16_t *>(keeper->half_rows);
        w_scale = reinterpret_cast<float *>(static_cast<uint8_t *>(keeper->half_rows) + w_bytes);
    } else {
        w16 = reinterpret_cast<uint16_t *>(scratch + x_room);
        w_scale = reinterpret_cast<float *>(scratch + x_room + w_bytes);
        h3b_scale_rows_f16(gpu, w, w16, w_scale, n, k);
    }
    if (!ready) h3b_scale_rows_f16(gpu, x, x16, x_scale, rows, k);
    if (cudaGetLastError() != cudaSuccess) return h3b_fail(gpu, "linear_f32: operand conversion failed");
    TcArgs extra = {};
    extra.row_scale = x_scale;
    extra.col_scale = w_scale;
    if (!launch_tc<H3B_EPI_STORE_F32>(gpu, reinterpret_cast<uint16_t *>(out), x16, w16,
                                      reinterpret_cast<const uint16_t *>(bias), rows, k, n, n,
                                      (n + BN - 1) / BN, 0, &extra))
        return h3b_fail(gpu, "linear_f32: cannot set up the tensor-core GEMM (tensor map or launch attribute)");
    return 1;
}

int h3b_qkv_rope_gemm(h3_gpu *gpu, uint16_t *q, uint16_t *k, uint16_t *v, const uint16_t *x,
                      const uint16_t *w, const uint16_t *q_norm, const uint16_t *k_norm,
                      const uint16_t *rope_cos, const uint16_t *rope_sin, uint32_t rows,
                      uint32_t in_dim, uint32_t heads, float eps, const h3x_ulysses_peers *peers) {
    const uint32_t n = heads * 3 * 128;
    bool aligned = (peers || (h3b_aligned16(q) && h3b_aligned16(k) && h3b_aligned16(v))) && h3b_aligned16(x) &&
                   h3b_aligned16(w) && h3b_aligned16(q_norm) && h3b_aligned16(k_norm) &&
                   h3b_aligned16(rope_cos) && h3b_aligned16(rope_sin);
    if (!aligned || !rows || !heads || !in_dim || in_dim % 8 != 0 ||
        env_flag("H3B_NO_TENSOR_CORES") || env_flag("H3B_UNFUSED_QKV_ROPE") ||
        double(rows) * n * in_dim < 32.0 * 256 * 256)
        return -1;
    TcArgs extra = {};
    extra.q_out = q; extra.k_out = k; extra.v_out = v;
    extra.q_norm = q_norm; extra.k_norm = k_norm;
    extra.rope_cos = rope_cos; extra.rope_sin = rope_sin;
    extra.heads = heads;
    extra.eps = eps;
    if (peers) {
        extra.world = peers->world;
        extra.rank = peers->rank;
        extra.rows_local = peers->rows_local;
        extra.heads_per_rank = heads / peers->world;
        for (uint32_t r = 0; r < peers->world; r++) {
            extra.peer_q[r] = static_cast<uint16_t *>(peers->q[r]);
            extra.peer_k[r] = static_cast<uint16_t *>(peers->k[r]);
            extra.peer_v[r] = static_cast<uint16_t *>(peers->v[r]);
        }
    }
    if (!launch_tc<H3B_EPI_QKV_ROPE>(gpu, nullptr, x, w, nullptr, rows, in_dim, n, n,
                                     (n + BN - 1) / BN, 0, &extra))
        return h3b_fail(gpu, "cannot set up the fused QKV projection kernel");
    return h3b_launched(gpu, "grouped_qkv_linear_rope_bf16", H3B_LINEAR);
}

/* ================================================================= C ABI */

/* Which counter a projection bumps follows the reference's shape rule
 * (h3_cuda_core.cu:838-841), so the statistics its tests assert are identical. */
static h3b_kind linear_kind(uint32_t rows, uint32_t in_dim, uint32_t out_dim) {
    return rows >= 32 && in_dim >= 256 && out_dim >= 256 ? H3B_LINEAR : H3B_DIRECT;
}

extern "C" int h3_gpu_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                  const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                  uint32_t rows, uint32_t input_dim, uint32_t output_dim) {
    if (!h3b_need(gpu, input, H3_GPU_BF16, size_t(rows) * input_dim, "linear input") ||
        !h3b_need(gpu, weight, H3_GPU_BF16, size_t(output_dim) * input_dim, "linear weight") ||
        !h3b_need(gpu, output, H3_GPU_BF16, size_t(rows) * output_dim, "linear output") ||
        (bias && !h3b_need(gpu, bias, H3_GPU_BF16, output_dim, "linear bias")) ||
        !h3b_need_command(gpu))
        return 0;
    uint64_t before = gpu->stats.mps_linear_dispatches;
    if (!h3b_gemm_bf16(gpu, h3b_ptr<uint16_t>(output), h3b_ptr<uint16_t>(input),
                       h3b_ptr<uint16_t>(weight), bias ? h3b_ptr<uint16_t>(bias) : nullptr, rows,
                       input_dim, output_dim, H3B_EPI_STORE, "linear_bf16"))
        return 0;
    if (linear_kind(rows, input_dim, output_dim) == H3B_DIRECT) {
        gpu->stats.mps_linear_dispatches = before;
        gpu->stats.direct_dispatches++;
    }
    return 1;
}

extern "C" int h3_gpu_linear_f32(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                 const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                                 uint32_t rows, uint32_t input_dim, uint32_t output_dim) {
    if (!h3b_need(gpu, input, H3_GPU_F32, size_t(rows) * input_dim, "linear input") ||
        !h3b_need(gpu, weight, H3_GPU_F32, size_t(output_dim) * input_dim, "linear weight") ||
        !h3b_need(gpu, output, H3_GPU_F32, size_t(rows) * output_dim, "linear output") ||
        (bias && !h3b_need(gpu, bias, H3_GPU_F32, output_dim, "linear bias")) ||
        !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    const int served = h3b_gemm_f32_half(gpu, h3b_ptr<float>(output), input, weight,
                                         bias ? h3b_ptr<float>(bias) : nullptr, rows, input_dim, output_dim);
    if (served == 0) return 0;
    if (served < 0 && rows && output_dim)
        launch_simt<float, float>(gpu, h3b_ptr<float>(input), h3b_ptr<float>(weight),
                                  bias ? h3b_ptr<float>(bias) : nullptr, h3b_ptr<float>(output),
                                  nullptr, rows, input_dim, output_dim);
    return h3b_launched(gpu, "linear_f32", linear_kind(rows, input_dim, output_dim));
}

extern "C" int h3_gpu_mlp_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                               const h3_gpu_tensor *fc1_weight, const h3_gpu_tensor *fc2_weight,
                               uint32_t rows, uint32_t input_dim, uint32_t hidden_dim,
                               uint32_t output_dim) {
    if (!h3b_need(gpu, input, H3_GPU_BF16, size_t(rows) * input_dim, "MLP input") ||
        !h3b_need(gpu, fc1_weight, H3_GPU_BF16, size_t(hidden_dim) * 2 * input_dim, "MLP fc1") ||
        !h3b_need(gpu, fc2_weight, H3_GPU_BF16, size_t(output_dim) * hidden_dim, "MLP fc2") ||
        !h3b_need(gpu, output, H3_GPU_BF16, size_t(rows) * output_dim, "MLP output") ||
        !h3b_need_command(gpu))
        return 0;
    uint64_t linear_before = gpu->stats.mps_linear_dispatches;
    uint64_t direct_before = gpu->stats.direct_dispatches;
    if (rows && hidden_dim && output_dim) {
        size_t act_bytes = (size_t(rows) * hidden_dim * sizeof(uint16_t) + 255) & ~size_t(255);
        size_t fused_bytes = size_t(rows) * hidden_dim * 2 * sizeof(uint16_t);
        /* activated | (unfused route only) fc1 output */
        uint8_t *scratch = static_cast<uint8_t *>(h3b_workspace(gpu, act_bytes + fused_bytes));
        if (!scratch) return h3b_fail(gpu, "cannot allocate the MLP scratch");
        uint16_t *activated = reinterpret_cast<uint16_t *>(scratch);
        if (env_flag("H3B_UNFUSED_MLP")) {
            uint16_t *fused = reinterpret_cast<uint16_t *>(scratch + act_bytes);
            if (!h3b_gemm_bf16(gpu, fused, h3b_ptr<uint16_t>(input), h3b_ptr<uint16_t>(fc1_weight),
                               nullptr, rows, input_dim, hidden_dim * 2, H3B_EPI_STORE, "mlp fc1") ||
                !h3b_swiglu_launch(gpu, activated, fused, rows, hidden_dim))
                return 0;
        } else if (!h3b_gemm_bf16(gpu, activated, h3b_ptr<uint16_t>(input),
                                  h3b_ptr<uint16_t>(fc1_weight), nullptr, rows, input_dim,
                                  hidden_dim, H3B_EPI_SWIGLU, "mlp fc1+swiglu")) {
            return 0;
        }
        if (!h3b_gemm_bf16(gpu, h3b_ptr<uint16_t>(output), activated,
                           h3b_ptr<uint16_t>(fc2_weight), nullptr, rows, hidden_dim, output_dim,
                           H3B_EPI_STORE, "mlp fc2"))
            return 0;
    }
    /* the reference counts an MLP as two projections whatever route ran */
    gpu->stats.mps_linear_dispatches = linear_before + 2;
    gpu->stats.direct_dispatches = direct_before;
    return 1;
}

/* The first stage of h3_gpu_mlp_bf16 on its own: activated = swiglu(x . fc1^T). */
extern "C" int h3x_linear_swiglu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                                      const h3_gpu_tensor *fc1_weight, uint32_t rows,
                                      uint32_t input_dim, uint32_t hidden_dim) {
    if (!h3b_need(gpu, input, H3_GPU_BF16, size_t(rows) * input_dim, "MLP input") ||
        !h3b_need(gpu, fc1_weight, H3_GPU_BF16, size_t(hidden_dim) * 2 * input_dim, "MLP fc1") ||
        !h3b_need(gpu, output, H3_GPU_BF16, size_t(rows) * hidden_dim, "MLP activation") ||
        !h3b_need_command(gpu))
        return 0;
    if (!rows || !hidden_dim) return 1;
    return h3b_gemm_bf16(gpu, h3b_ptr<uint16_t>(output), h3b_ptr<uint16_t>(input),
                         h3b_ptr<uint16_t>(fc1_weight), nullptr, rows, input_dim, hidden_dim,
                         H3B_EPI_SWIGLU, "linear_swiglu_bf16");
}

static int patch_common(h3_gpu *gpu, h3_gpu_tensor *output, size_t output_offset,
                        size_t output_span, const h3_gpu_tensor *input, size_t input_offset,
                        const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                        const h3_gpu_tensor *row_map, uint32_t rows, uint32_t input_dim,
                        uint32_t output_dim, const char *what) {
    /* the reference accepts exactly the model's patch shapes (h3_cuda_core.cu:929-931) */
    if (output_dim != 5376 || (input_dim != 32 && input_dim != 96))
        return h3b_fail(gpu, "unsupported fused patch projection shape");
    size_t in_count = size_t(rows) * input_dim;
    if (input_offset > SIZE_MAX - in_count || output_offset > SIZE_MAX - output_span)
        return h3b_fail(gpu, "fused patch projection offset is out of range");
    if (!h3b_need(gpu, input, H3_GPU_F32, input_offset + in_count, "patch projection input") ||
        !h3b_need(gpu, weight, H3_GPU_F32, size_t(output_dim) * input_dim,
                  "patch projection weight") ||
        !h3b_need(gpu, output, H3_GPU_BF16, output_offset + output_span,
                  "patch projection output") ||
        (row_map && !h3b_need(gpu, row_map, H3_GPU_U32, rows, "patch projection row map")) ||
        (bias && !h3b_need(gpu, bias, H3_GPU_F32, output_dim, "patch projection bias")) ||
        !h3b_need_command(gpu))
        return 0;
    if (rows)
        launch_simt<float, uint16_t>(gpu, h3b_ptr<float>(input, input_offset),
                                     h3b_ptr<float>(weight), bias ? h3b_ptr<float>(bias) : nullptr,
                                     h3b_ptr<uint16_t>(output, output_offset),
                                     row_map ? h3b_ptr<uint32_t>(row_map) : nullptr, rows,
                                     input_dim, output_dim);
    return h3b_launched(gpu, what);
}

extern "C" int h3_gpu_patch_linear_bf16_offset(h3_gpu *gpu, h3_gpu_tensor *output,
                                               size_t output_offset, const h3_gpu_tensor *input,
                                               size_t input_offset, const h3_gpu_tensor *weight,
                                               const h3_gpu_tensor *bias, uint32_t rows,
                                               uint32_t input_dim, uint32_t output_dim) {
    return patch_common(gpu, output, output_offset, size_t(rows) * output_dim, input, input_offset,
                        weight, bias, nullptr, rows, input_dim, output_dim, "patch_linear_bf16");
}

extern "C" int h3_gpu_patch_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                        const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                                        const h3_gpu_tensor *bias, uint32_t rows,
                                        uint32_t input_dim, uint32_t output_dim) {
    return h3_gpu_patch_linear_bf16_offset(gpu, output, 0, input, 0, weight, bias, rows, input_dim,
                                           output_dim);
}

extern "C" int h3_gpu_patch_linear_bf16_map(h3_gpu *gpu, h3_gpu_tensor *output,
                                            const h3_gpu_tensor *input,
                                            const h3_gpu_tensor *weight,
                                            const h3_gpu_tensor *bias,
                                            const h3_gpu_tensor *row_map, uint32_t output_rows,
                                            uint32_t rows, uint32_t input_dim,
                                            uint32_t output_dim) {
    if (!row_map) return h3b_fail(gpu, "patch projection row map tensor has the wrong dtype");
    return patch_common(gpu, output, 0, size_t(output_rows) * output_dim, input, 0, weight, bias,
                        row_map, rows, input_dim, output_dim, "patch_linear_bf16_map");
}
