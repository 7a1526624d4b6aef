/* Inline-PTX wrappers for the sm_100a features the tensor-core kernels use:
 * mbarriers with bounded waits, TMA tile loads, tensor-memory allocation,
 * tcgen05.mma / commit / ld, and the operand / instruction descriptors. */
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace {

/* ------------------------------------------------------------------ PTX */

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

/* Non-blocking look at a phase (try_wait may suspend the thread for a while when the phase is
 * still open; this returns at once). 1 when the phase with this parity has completed. */
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

/* Bounded wait: gives up after `limit` cycles of the SM clock without progress (the context's
 * wait budget, about a second by default). Returns false when the CTA should stop. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *stop,
                                          long long limit) {
    if (mbar_try(bar, parity)) return true;
    long long start = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            if (*stop) return false;
            if (clock64() - start > limit) {
                *stop = 1;
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

/* D[tmem] (+)= A[smem] . B[smem]^T, BF16 in, F32 out, issued by one thread */
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

/* arrive on an mbarrier once every tcgen05.mma issued so far by this thread has finished */
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

/* 32 consecutive F32 columns of this thread's TMEM lane */
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

/* 32 consecutive 32-bit columns of this thread's TMEM lane, written from registers */
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
          "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
          "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
          "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait_all() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

/* Shared-memory operand descriptor: K-major tile of 128-byte rows written by a
 * TMA copy with 128-byte swizzle. Rows sit in groups of 8 (1024 bytes apart =
 * stride byte offset); descriptor version 1 (sm_100); layout code 2 = SW128. */
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
    uint64_t desc = (smem_addr >> 4) & 0x3fffu;
    desc |= uint64_t(1) << 16;              /* leading byte offset: unused with swizzle */
    desc |= uint64_t(1024 >> 4) << 32;      /* stride byte offset                       */
    desc |= uint64_t(1) << 46;              /* descriptor version                       */
    desc |= uint64_t(2) << 61;              /* 128-byte swizzle                         */
    return desc;
}

/* Instruction descriptor: F32 accumulate, BF16 A and B, both K-major, M x N tile. */
__host__ __device__ constexpr uint32_t instruction_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}


/* ---- descriptor words for hot issue loops -----------------------------------------
 * The single thread that issues tcgen05.mma is a scalar instruction stream; building a
 * 64-bit descriptor per instruction costs more than a small MMA takes. The upper word of
 * a descriptor is constant per operand kind and the lower word is (address >> 4) plus the
 * leading-byte-offset field, so a loop only adds a constant to the lower word. */
constexpr uint32_t DESC_HI_SW128 = (1024u >> 4) | (1u << 14) | (2u << 29);   /* SBO | version | SW128 */
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t smem_addr) {
    return ((smem_addr >> 4) & 0x3fffu) | (1u << 16);
}
__device__ __forceinline__ uint32_t desc_lo_nmajor(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr >> 4) & 0x3fffu) | ((lbo_bytes >> 4) << 16);
}

/* The issuing warp runs its loop with all 32 lanes converged, so addresses and descriptor
 * words stay warp-uniform (no per-instruction moves from the vector to the uniform register
 * file); only the tcgen05 instruction itself is predicated on the `leader` lane.
 * D[tmem] (+)= A[smem] . B[smem]; ACC is a compile-time flag. */
template <bool ACC>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                        uint32_t leader = 1) {
    asm volatile(
        "{\n\t.reg .pred p, l;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "setp.ne.u32 l, %6, 0;\n\t"
        "mov.b64 da, {%1, %4};\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "@l tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(DESC_HI_SW128), "n"(ACC ? 1 : 0),
          "r"(leader)
        : "memory");
}

/* D[tmem] (+)= A[tmem] . B[smem] */
template <bool ACC>
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                        uint32_t leader = 1) {
    asm volatile(
        "{\n\t.reg .pred p, l;\n\t.reg .b64 db;\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "setp.ne.u32 l, %6, 0;\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "@l tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(DESC_HI_SW128), "n"(ACC ? 1 : 0),
          "r"(leader)
        : "memory");
}

__device__ __forceinline__ void umma_commit_if(uint32_t bar, uint32_t leader) {
    asm volatile(
        "{\n\t.reg .pred l;\n\tsetp.ne.u32 l, %1, 0;\n\t"
        "@l tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(leader)
        : "memory");
}

/* ---- CTA pairs (cluster of two, tcgen05 cta_group::2) -------------------------------------
 * One tcgen05.mma issued by the even CTA multiplies M = 256 rows (128 from each CTA's shared
 * memory, accumulated in each CTA's own tensor memory) by a B tile whose N rows are split
 * between the two CTAs' shared memory. No TMA multicast is involved: each CTA loads its own
 * halves and reports the bytes to the even CTA's mbarrier. */
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
/* shared::cluster address of `smem_addr` (a shared::cta address of this CTA) in CTA `rank` */
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
                 : "memory");
}
/* TMA load into this CTA's shared memory; completion bytes go to the mbarrier at the given
 * shared::cluster address (the even CTA's barrier) */
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map,
                                                 uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free_pair(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                             uint32_t idesc, uint32_t leader) {
    asm volatile(
        "{\n\t.reg .pred p, l;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "setp.ne.u32 l, %6, 0;\n\t"
        "mov.b64 da, {%1, %4};\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "@l tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(DESC_HI_SW128), "n"(ACC ? 1 : 0),
          "r"(leader)
        : "memory");
}
/* arrive on the mbarrier at the same shared-memory offset in both CTAs of the pair when all
 * MMAs issued so far have completed */
__device__ __forceinline__ void umma_commit_pair_if(uint32_t bar, uint32_t leader) {
    asm volatile(
        "{\n\t.reg .pred l;\n\t.reg .b16 mask;\n\tsetp.ne.u32 l, %1, 0;\n\tmov.b16 mask, 3;\n\t"
        "@l tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], mask;\n\t}"
        ::"r"(bar), "r"(leader)
        : "memory");
}

/* two F32 -> packed BF16x2, round to nearest even (one cvt instruction) */
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

/* Packed pairs of F32 in one 64-bit register: sm_100 executes fma/add on both halves with one
 * instruction (same rounding as the scalar forms). */
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3_f32(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float round_bf16(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}

/* cuTensorMapEncodeTiled, resolved through the runtime so the library does not link libcuda */
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                 const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return EncodeTiled(nullptr);
        }
        return EncodeTiled(p);
    }();
    return fn;
}


}  // namespace
