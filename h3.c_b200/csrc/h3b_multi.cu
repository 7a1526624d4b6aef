/* Sequence-parallel (Ulysses) layout changes around attention. The reference
 * is single-device; these entry points have no counterpart there.
 *
 * Rank r of `world` owns rows_local consecutive rows of every activation.
 * Before attention each rank regroups its [rows_local][heads][hd] Q/K/V into
 * `world` contiguous blocks, block p = heads [p*heads/world, (p+1)*heads/world),
 * and an all-to-all of equal blocks leaves rank r with all rows of its head
 * slice, stored [source rank][rows_local][heads/world][hd] = row order
 * preserved. After attention the inverse exchange and unpack restore
 * [rows_local][heads][hd]. Both kernels move 16 bytes per thread.
 */
#include "h3b_common.cuh"

namespace {

/* pack == true : dst[p][r][hl][v] = src[r][p*hpr + hl][v]
 * pack == false: dst[r][p*hpr + hl][v] = src[p][r][hl][v]        (v = 16-byte vector index) */
__global__ void h3b_ulysses_permute(const uint4 *src, uint4 *dst, uint32_t rows, uint32_t heads,
                                    uint32_t vec_per_head, uint32_t world, int pack) {
    const size_t total = size_t(rows) * heads * vec_per_head;
    const uint32_t hpr = heads / world;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += size_t(gridDim.x) * blockDim.x) {
        const uint32_t v = uint32_t(i % vec_per_head);
        const size_t t = i / vec_per_head;
        const uint32_t head = uint32_t(t % heads), row = uint32_t(t / heads);
        const uint32_t p = head / hpr, hl = head % hpr;
        const size_t packed = ((size_t(p) * rows + row) * hpr + hl) * vec_per_head + v;
        if (pack) dst[packed] = src[i];
        else dst[i] = src[packed];
    }
}

int permute(h3_gpu *gpu, h3_gpu_tensor *dst, const h3_gpu_tensor *src, uint32_t rows,
            uint32_t heads, uint32_t head_dim, uint32_t world, int pack, const char *what) {
    size_t count = size_t(rows) * heads * head_dim;
    if (!world || heads % world != 0 || head_dim % 8 != 0)
        return h3b_fail(gpu, "%s: heads must divide by the world size and head_dim by 8", what);
    if (!h3b_need(gpu, src, H3_GPU_BF16, count, what) || !h3b_need(gpu, dst, H3_GPU_BF16, count, what) ||
        !h3b_need_command(gpu))
        return 0;
    if (!h3b_aligned16(src->data) || !h3b_aligned16(dst->data))
        return h3b_fail(gpu, "%s: tensors must be 16-byte aligned", what);
    if (count) {
        size_t vectors = count / 8;
        unsigned blocks = unsigned((vectors + 255) / 256);
        unsigned cap = unsigned(gpu->sm_count) * 16;
        if (blocks > cap) blocks = cap;
        h3b_ulysses_permute<<<blocks, 256, 0, gpu->stream>>>(
            h3b_ptr<uint4>(src), h3b_ptr<uint4>(dst), rows, heads, head_dim / 8, world, pack);
    }
    return h3b_launched(gpu, what);
}

/* Flag words of one rank: [0, 8) = epoch last announced by rank r, [8] = this rank's own
 * barrier count. One warp; lane r talks to rank r. */
__global__ void h3b_peer_barrier(uint32_t *mine, h3x_ulysses_peers peers, int *status,
                                 long long cycle_limit) {
    __shared__ uint32_t epoch_shared;
    if (threadIdx.x == 0) {
        epoch_shared = mine[8] + 1;
        mine[8] = epoch_shared;
    }
    __syncthreads();
    const uint32_t epoch = epoch_shared;
    if (threadIdx.x < peers.world) {
        uint32_t *theirs = static_cast<uint32_t *>(peers.flags[threadIdx.x]) + peers.rank;
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        const uint32_t *slot = mine + threadIdx.x;
        const long long start = clock64();
        for (;;) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(slot) : "memory");
            if (int32_t(seen - epoch) >= 0) break;
            if (clock64() - start > cycle_limit) {
                atomicExch(status, H3B_STATUS_PEER_TIMEOUT);
                break;
            }
            __nanosleep(64);
        }
    }
}

}  // namespace

extern "C" int h3x_peer_barrier(h3_gpu *gpu, const h3x_ulysses_peers *peers) {
    if (!gpu) return 0;
    if (!peers || !peers->world || peers->world > 8 || peers->rank >= peers->world)
        return h3b_fail(gpu, "invalid sequence-parallel peer table");
    for (uint32_t r = 0; r < peers->world; r++)
        if (!peers->flags[r]) return h3b_fail(gpu, "peer table has no barrier words");
    if (!h3b_need_command(gpu)) return 0;
    h3b_peer_barrier<<<1, 32, 0, gpu->stream>>>(static_cast<uint32_t *>(peers->flags[peers->rank]),
                                                *peers, gpu->status_device, gpu->barrier_cycles);
    return h3b_launched(gpu, "peer_barrier");
}

extern "C" void *h3x_peer_alloc(h3_gpu *gpu, size_t bytes, void *handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!gpu || !bytes || !handle64) {
        h3b_fail(gpu, "peer_alloc needs a size and a handle buffer");
        return nullptr;
    }
    void *block = nullptr;
    cudaError_t status = cudaMalloc(&block, bytes);
    if (status == cudaSuccess) status = cudaMemset(block, 0, bytes);
    if (status == cudaSuccess) status = cudaDeviceSynchronize();
    cudaIpcMemHandle_t handle;
    if (status == cudaSuccess) status = cudaIpcGetMemHandle(&handle, block);
    if (status != cudaSuccess) {
        if (block) cudaFree(block);
        h3b_fail_cuda(gpu, "peer_alloc", status);
        return nullptr;
    }
    memcpy(handle64, &handle, sizeof(handle));
    return block;
}

extern "C" void *h3x_peer_open(h3_gpu *gpu, const void *handle64) {
    if (!gpu || !handle64) return nullptr;
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle64, sizeof(handle));
    void *mapped = nullptr;
    cudaError_t status = cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess);
    if (status != cudaSuccess) {
        h3b_fail_cuda(gpu, "peer_open", status);
        return nullptr;
    }
    return mapped;
}

extern "C" int h3x_peer_close(h3_gpu *gpu, void *mapped) {
    if (!gpu || !mapped) return 0;
    cudaError_t status = cudaIpcCloseMemHandle(mapped);
    return status == cudaSuccess ? 1 : h3b_fail_cuda(gpu, "peer_close", status);
}

extern "C" int h3x_peer_free(h3_gpu *gpu, void *block) {
    if (!gpu || !block) return 0;
    cudaError_t status = cudaFree(block);
    return status == cudaSuccess ? 1 : h3b_fail_cuda(gpu, "peer_free", status);
}

extern "C" int h3x_ulysses_pack_heads(h3_gpu *gpu, h3_gpu_tensor *packed, const h3_gpu_tensor *src,
                                      uint32_t rows_local, uint32_t heads, uint32_t head_dim,
                                      uint32_t world) {
    return permute(gpu, packed, src, rows_local, heads, head_dim, world, 1, "ulysses_pack_heads");
}

extern "C" int h3x_ulysses_unpack_heads(h3_gpu *gpu, h3_gpu_tensor *dst, const h3_gpu_tensor *src,
                                        uint32_t rows_local, uint32_t heads, uint32_t head_dim,
                                        uint32_t world) {
    return permute(gpu, dst, src, rows_local, heads, head_dim, world, 0, "ulysses_unpack_heads");
}
