/* Context, tensors, host<->device traffic, command bracketing, casts and copies
 * of libh3b200.so. Replaces the reference's h3_gpu_cuda.cu behind the same C ABI.
 *
 * Design notes
 *  - One in-order stream per context. By default it is the legacy default
 *    stream, as in the reference, so a host process that also uses another
 *    CUDA library on that stream stays ordered with us; h3x_set_stream()
 *    moves the context to a caller-owned stream (one process per GPU).
 *  - Freed device blocks go to an exact-size cache and are handed out again
 *    without synchronising: reuse is ordered by the stream.
 *  - Host writes go through a small ring of pinned buffers so that the call
 *    can return as soon as the host buffer has been consumed.
 */
#include "h3b_common.cuh"

#include <algorithm>
#include <atomic>
#include <map>
#include <string>
#include <condition_variable>
#include <thread>

#include <cerrno>
#include <cstdlib>
#include <ctime>
#include <fcntl.h>
#include <unistd.h>

static thread_local int g_device = 0;

double h3b_now() {
    timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return double(t.tv_sec) + double(t.tv_nsec) * 1e-9;
}

/* ------------------------------------------------------------ op profile */
/* H3_PROFILE=2: device time per op name. Every launch is followed by an event on the
 * context's stream; at submit the gaps between consecutive events (the stream is in order, so
 * a gap is the op's duration plus any launch bubble before it) are added up per name, and
 * h3_gpu_profile_mark / h3_gpu_free print the table. The reference prints wall and wait time
 * per phase (h3_gpu_cuda.cu:21-45,919-933); this adds where inside a phase the device time
 * goes. Off by default: one event record per launch otherwise. */
struct h3b_op_profile {
    struct Total { double ms = 0.0; uint64_t count = 0; };
    std::vector<cudaEvent_t> pool;
    std::vector<std::pair<const char *, cudaEvent_t>> marks;   /* first = nullptr: command begin */
    std::map<std::string, Total> totals;

    cudaEvent_t take() {
        cudaEvent_t e = nullptr;
        if (!pool.empty()) { e = pool.back(); pool.pop_back(); return e; }
        if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        return e;
    }
    void collect() {       /* the stream has been synchronised */
        cudaEvent_t previous = nullptr;
        for (auto &mark : marks) {
            if (mark.first && previous) {
                float ms = 0.0f;
                if (cudaEventElapsedTime(&ms, previous, mark.second) == cudaSuccess) {
                    Total &t = totals[mark.first];
                    t.ms += ms;
                    t.count++;
                } else {
                    cudaGetLastError();
                }
            }
            previous = mark.second;
        }
        for (auto &mark : marks) pool.push_back(mark.second);
        marks.clear();
    }
    void print(const char *label, const char *phase) {
        if (totals.empty()) return;
        std::vector<std::pair<std::string, Total>> rows(totals.begin(), totals.end());
        std::sort(rows.begin(), rows.end(), [](const auto &a, const auto &b) { return a.second.ms > b.second.ms; });
        double sum = 0.0;
        for (auto &r : rows) sum += r.second.ms;
        fprintf(stderr, "h3b200: [%s] %s: %.3f ms of device time in %zu op names\n", label, phase, sum, rows.size());
        for (auto &r : rows)
            fprintf(stderr, "h3b200:   %-40s %10.3f ms %5.1f %% %8llu launches %9.4f ms each\n", r.first.c_str(),
                    r.second.ms, 100.0 * r.second.ms / (sum > 0 ? sum : 1), (unsigned long long)r.second.count,
                    r.second.ms / double(r.second.count ? r.second.count : 1));
        totals.clear();
    }
    ~h3b_op_profile() {
        for (auto &mark : marks) cudaEventDestroy(mark.second);
        for (cudaEvent_t e : pool) cudaEventDestroy(e);
    }
};

void h3b_profile_record(h3_gpu *gpu, const char *what) {
    h3b_op_profile *p = gpu->op_profile;
    cudaEvent_t e = p->take();
    if (!e) return;
    if (cudaEventRecord(e, gpu->stream) != cudaSuccess) {
        cudaGetLastError();
        p->pool.push_back(e);
        return;
    }
    p->marks.emplace_back(what, e);
}

/* ------------------------------------------------------------ allocator */

static void cache_evict_all(h3_gpu *gpu) {
    for (auto &entry : gpu->cache) cudaFree(entry.second);
    gpu->cache.clear();
    gpu->cache_bytes = 0;
}

static cudaError_t cache_alloc(h3_gpu *gpu, size_t bytes, void **out) {
    auto hit = gpu->cache.find(bytes);
    if (hit != gpu->cache.end()) {
        *out = hit->second;
        gpu->cache.erase(hit);
        gpu->cache_bytes -= bytes;
        return cudaSuccess;
    }
    if (gpu->cache_bytes > gpu->cache_limit) {
        cudaStreamSynchronize(gpu->stream);
        cache_evict_all(gpu);
    }
    cudaError_t status = cudaMalloc(out, bytes);
    if (status != cudaSuccess && !gpu->cache.empty()) {
        cudaGetLastError();
        cudaStreamSynchronize(gpu->stream);
        cache_evict_all(gpu);
        status = cudaMalloc(out, bytes);
    }
    return status;
}

static void cache_release(h3_gpu *gpu, void *data, size_t bytes) {
    gpu->cache.emplace(bytes, data);
    gpu->cache_bytes += bytes;
}

void *h3b_device_alloc(h3_gpu *gpu, size_t bytes) {
    void *data = nullptr;
    if (cache_alloc(gpu, (bytes + 255) & ~size_t(255), &data) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return data;
}

void h3b_device_release(h3_gpu *gpu, void *data, size_t bytes) {
    if (data) cache_release(gpu, data, (bytes + 255) & ~size_t(255));
}

void h3b_written(h3_gpu_tensor *tensor) {
    if (!tensor || !tensor->half_rows) return;
    /* kernels that read the rows may still be queued: the block goes back to the stream-ordered
     * cache, whose next user runs behind them */
    if (tensor->owner) h3b_device_release(tensor->owner, tensor->half_rows, tensor->half_bytes);
    else cudaFree(tensor->half_rows);
    tensor->half_rows = nullptr;
    tensor->half_bytes = 0;
    tensor->half_k = 0;
}

extern "C" int h3x_tensor_keep_half_rows(h3_gpu_tensor *tensor, int on) {
    if (!tensor || tensor->dtype != H3_GPU_F32) return 0;
    h3b_written(tensor);
    tensor->keeps_half = on != 0;
    return 1;
}

void *h3b_workspace(h3_gpu *gpu, size_t bytes) {
    if (!bytes) bytes = 1;
    if (gpu->workspace && bytes <= gpu->workspace_bytes) return gpu->workspace;
    size_t capacity = gpu->workspace_bytes ? gpu->workspace_bytes : (size_t(1) << 20);
    while (capacity < bytes) capacity = capacity > SIZE_MAX / 2 ? bytes : capacity * 2;
    void *fresh = nullptr;
    if (cudaMalloc(&fresh, capacity) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    cudaStreamSynchronize(gpu->stream);  /* kernels in flight may still use the old block */
    cudaFree(gpu->workspace);
    gpu->workspace = fresh;
    gpu->workspace_bytes = capacity;
    return fresh;
}

/* ----------------------------------------------------------- host I/O */

static bool upload(h3_gpu *gpu, void *device, const void *host, size_t bytes) {
    if (!bytes) return true;
    const unsigned char *src = static_cast<const unsigned char *>(host);
    unsigned char *dst = static_cast<unsigned char *>(device);
    while (bytes) {
        size_t chunk = bytes < h3_gpu::kSlotMax ? bytes : h3_gpu::kSlotMax;
        h3b_pinned_slot &slot = gpu->slots[gpu->next_slot++ % h3_gpu::kSlots];
        if (slot.pending) {
            if (cudaEventSynchronize(slot.done) != cudaSuccess) return false;
            slot.pending = false;
        }
        if (slot.bytes < chunk) {
            if (slot.host) cudaFreeHost(slot.host);
            slot.host = nullptr;
            slot.bytes = 0;
            size_t want = chunk < (size_t(1) << 16) ? (size_t(1) << 16) : chunk;
            if (cudaMallocHost(&slot.host, want) != cudaSuccess) {
                cudaGetLastError();
                /* no pinned memory: a pageable copy is staged by the runtime before it returns */
                if (cudaMemcpyAsync(dst, src, chunk, cudaMemcpyHostToDevice, gpu->stream) !=
                    cudaSuccess)
                    return false;
                src += chunk; dst += chunk; bytes -= chunk;
                continue;
            }
            slot.bytes = want;
        }
        if (!slot.done && cudaEventCreateWithFlags(&slot.done, cudaEventDisableTiming) != cudaSuccess)
            return false;
        memcpy(slot.host, src, chunk);
        if (cudaMemcpyAsync(dst, slot.host, chunk, cudaMemcpyHostToDevice, gpu->stream) !=
                cudaSuccess ||
            cudaEventRecord(slot.done, gpu->stream) != cudaSuccess)
            return false;
        slot.pending = true;
        src += chunk; dst += chunk; bytes -= chunk;
    }
    return true;
}

static bool download(const h3_gpu *gpu, void *host, const void *device, size_t bytes) {
    if (!bytes) return true;
    cudaStream_t stream = gpu ? gpu->stream : nullptr;
    if (cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess)
        return false;
    return cudaStreamSynchronize(stream) == cudaSuccess;
}

/* -------------------------------------------------------------- context */

extern "C" int h3x_set_device(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return 0;
    }
    g_device = device;
    return cudaSetDevice(device) == cudaSuccess;
}

extern "C" h3_gpu *h3_gpu_create(const char *, char *error, size_t error_size) {
    auto fail = [&](const char *what, cudaError_t status) -> h3_gpu * {
        if (error && error_size)
            snprintf(error, error_size, "%s: %s", what, cudaGetErrorString(status));
        cudaGetLastError();
        return nullptr;
    };
    int count = 0;
    cudaError_t status = cudaGetDeviceCount(&count);
    if (status != cudaSuccess || count <= 0) {
        if (error && error_size) snprintf(error, error_size, "no CUDA device available");
        cudaGetLastError();
        return nullptr;
    }
    status = cudaSetDevice(g_device);
    if (status == cudaSuccess) status = cudaFree(nullptr);
    if (status != cudaSuccess) return fail("cannot initialize CUDA device", status);
    cudaDeviceProp prop;
    status = cudaGetDeviceProperties(&prop, g_device);
    if (status != cudaSuccess) return fail("cannot query CUDA device", status);
    if (prop.major != 10) {
        if (error && error_size)
            snprintf(error, error_size,
                     "libh3b200 needs an sm_100 (B200) device; device %d is sm_%d%d", g_device,
                     prop.major, prop.minor);
        return nullptr;
    }
    h3_gpu *gpu = new (std::nothrow) h3_gpu();
    if (!gpu) {
        if (error && error_size) snprintf(error, error_size, "out of memory");
        return nullptr;
    }
    gpu->device = g_device;
    gpu->sm_count = prop.multiProcessorCount;
    size_t available = 0, total = 0;
    if (cudaMemGetInfo(&available, &total) == cudaSuccess) gpu->cache_limit = total / 5;
    status = cudaMalloc(reinterpret_cast<void **>(&gpu->status_device), sizeof(int));
    if (status == cudaSuccess) status = cudaMemset(gpu->status_device, 0, sizeof(int));
    if (status != cudaSuccess) {
        delete gpu;
        return fail("cannot allocate the kernel status word", status);
    }
    gpu->profile_mark = h3b_now();
    const char *profile = getenv("H3_PROFILE");
    if (profile && atoi(profile) >= 2) gpu->op_profile = new (std::nothrow) h3b_op_profile();
    return gpu;
}

static void sparse_clear(h3_gpu *gpu) {
    for (uint32_t **list : {&gpu->sparse_cta_ptr, &gpu->sparse_steps, &gpu->sparse_block_ptr,
                            &gpu->sparse_block_steps}) {
        if (*list) cudaFree(*list);
        *list = nullptr;
    }
    gpu->sparse_rows = 0;
}

extern "C" void h3_gpu_free(h3_gpu *gpu) {
    if (!gpu) return;
    cudaSetDevice(gpu->device);
    cudaStreamSynchronize(gpu->stream);
    if (gpu->workspace) cudaFree(gpu->workspace);
    if (gpu->split_scratch) cudaFree(gpu->split_scratch);
    cache_evict_all(gpu);
    for (h3b_pinned_slot &slot : gpu->slots) {
        if (slot.host) cudaFreeHost(slot.host);
        if (slot.done) cudaEventDestroy(slot.done);
    }
    h3b_loader_free(gpu->loader);
    if (gpu->op_profile) {
        gpu->op_profile->print(gpu->profile_label[0] ? gpu->profile_label : "gpu", "since the last mark");
        delete gpu->op_profile;
    }
    if (gpu->status_device) cudaFree(gpu->status_device);
    sparse_clear(gpu);
    delete gpu;
}

extern "C" int h3_gpu_is_m5(const h3_gpu *) { return 0; }
extern "C" int h3_gpu_has_nax_mlp(const h3_gpu *) { return 0; }
extern "C" int h3_gpu_has_int8_mlp(const h3_gpu *) { return 0; }
extern "C" int h3_gpu_prefers_gpu_sampler(const h3_gpu *) { return 1; }

extern "C" int h3x_set_stream(h3_gpu *gpu, void *cuda_stream) {
    if (!gpu) return 0;
    if (gpu->active) return h3b_fail(gpu, "cannot change the stream inside a command");
    cudaStreamSynchronize(gpu->stream);
    gpu->stream = static_cast<cudaStream_t>(cuda_stream);
    return 1;
}

extern "C" int h3x_kernel_status(h3_gpu *gpu) {
    if (!gpu) return -1;
    int status = 0;
    if (!download(gpu, &status, gpu->status_device, sizeof(int))) return -1;
    return status;
}

extern "C" int h3x_set_wait_budget_cycles(h3_gpu *gpu, long long kernel_cycles,
                                          long long barrier_cycles) {
    if (!gpu) return 0;
    if (gpu->active) return h3b_fail(gpu, "cannot change the wait budget inside a command");
    if (kernel_cycles > 0) gpu->wait_cycles = kernel_cycles;
    if (barrier_cycles > 0) gpu->barrier_cycles = barrier_cycles;
    return 1;
}

extern "C" int h3_gpu_begin(h3_gpu *gpu) {
    if (!gpu || gpu->active) return 0;
    gpu->error[0] = '\0';
    gpu->active = 1;
    gpu->command_start = h3b_now();
    if (gpu->op_profile) h3b_profile_record(gpu, nullptr);
    return 1;
}

extern "C" int h3_gpu_continue(h3_gpu *gpu) {
    if (!gpu || !gpu->active) return 0;
    double now = h3b_now();
    gpu->stats.submissions++;
    gpu->stats.command_encode_seconds += now - gpu->command_start;
    gpu->command_start = now;
    return 1;
}

extern "C" int h3_gpu_submit(h3_gpu *gpu) {
    if (!gpu || !gpu->active) return 0;
    gpu->active = 0;
    double committed = h3b_now();
    int kernel_status = 0;
    /* one small read-back both waits for the stream and fetches the status word */
    cudaError_t status = cudaMemcpyAsync(&kernel_status, gpu->status_device, sizeof(int),
                                         cudaMemcpyDeviceToHost, gpu->stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(gpu->stream);
    double completed = h3b_now();
    gpu->stats.submissions++;
    gpu->stats.command_encode_seconds += committed - gpu->command_start;
    gpu->stats.command_wait_seconds += completed - committed;
    gpu->stats.gpu_seconds += completed - committed;
    if (status != cudaSuccess) return h3b_fail_cuda(gpu, "command execution", status);
    if (gpu->op_profile) gpu->op_profile->collect();
    if (kernel_status != H3B_STATUS_OK) {
        cudaMemsetAsync(gpu->status_device, 0, sizeof(int), gpu->stream);
        gpu->status_seen = kernel_status;
        gpu->split_counters_dirty = 1;      /* a GEMM that gave up may have left its counters half-way */
        if (kernel_status == H3B_STATUS_PEER_TIMEOUT)
            return h3b_fail(gpu, "a peer barrier gave up waiting for another rank (status %d)",
                            kernel_status);
        return h3b_fail(gpu, "a %s kernel gave up waiting on its pipeline (status %d)",
                        kernel_status == H3B_STATUS_GEMM_TIMEOUT ? "GEMM" : "attention",
                        kernel_status);
    }
    return 1;
}

extern "C" const char *h3_gpu_error(const h3_gpu *gpu) {
    if (!gpu || !gpu->error[0]) return "unknown CUDA error";
    return gpu->error;
}

extern "C" int h3_gpu_get_stats(const h3_gpu *gpu, h3_gpu_stats *stats) {
    if (!gpu || !stats) return 0;
    *stats = gpu->stats;
    return 1;
}

extern "C" void h3_gpu_profile_set_label(h3_gpu *gpu, const char *label) {
    if (!gpu || !label || !*label) return;
    snprintf(gpu->profile_label, sizeof(gpu->profile_label), "%s", label);
}

extern "C" void h3_gpu_profile_mark(h3_gpu *gpu, const char *phase) {
    if (!gpu || !phase || !*phase) return;
    const char *enabled = getenv("H3_PROFILE");
    if (!enabled || !*enabled || !strcmp(enabled, "0")) return;
    double now = h3b_now();
    fprintf(stderr, "h3b200: [%s] %s: %.3f s wall, %.3f s waiting, %llu kernels, %llu GEMMs, %llu attention\n",
            gpu->profile_label[0] ? gpu->profile_label : "gpu", phase, now - gpu->profile_mark,
            gpu->stats.command_wait_seconds,
            (unsigned long long)gpu->stats.direct_dispatches,
            (unsigned long long)gpu->stats.mps_linear_dispatches,
            (unsigned long long)gpu->stats.mps_sdpa_dispatches);
    if (gpu->op_profile) gpu->op_profile->print(gpu->profile_label[0] ? gpu->profile_label : "gpu", phase);
    gpu->profile_mark = now;
}


/* Register / clear the block-sparse mask (reference h3_cuda_attention.cu:1812-1857: same
 * validation, same "applies to calls whose row count equals rows"). The CSR over 64-key tiles
 * per 128-row query block is regrouped on the host into step lists over 128-key tiles (see
 * h3_gpu in h3b_common.cuh), ascending: one list per query block with a bit per 64-key half,
 * and, for the kernel with two query tiles per CTA, the union of the two blocks' lists with
 * the per-(query block, half) bits. A tile listed twice for a block counts once (the
 * reference kernel would visit it twice; its own mask builder lists each tile once). */
extern "C" int h3_gpu_sdpa_set_sparse(h3_gpu *gpu, const uint32_t *ptr, size_t ptr_count,
                                      const uint32_t *idx, size_t idx_count, uint32_t rows) {
    if (!gpu) return 0;
    cudaDeviceSynchronize();   /* no attention call may still read the lists being replaced */
    sparse_clear(gpu);
    if (!ptr) return 1;
    if (!idx || !ptr_count || !idx_count || !rows) return 0;
    const uint32_t key_tiles64 = (rows + 63) / 64, query_blocks = (rows + 127) / 128;
    if (ptr[0] != 0 || ptr[ptr_count - 1] != uint32_t(idx_count)) return 0;
    for (size_t i = 1; i < ptr_count; i++)
        if (ptr[i] < ptr[i - 1]) return 0;
    for (size_t i = 0; i < idx_count; i++)
        if (idx[i] >= key_tiles64) return 0;
    const uint32_t listed_blocks = uint32_t(ptr_count - 1);
    const uint32_t ctas = (query_blocks + 1) / 2, key_tiles128 = (rows + 127) / 128;
    std::vector<uint32_t> cta_ptr(ctas + 1, 0), steps;
    std::vector<uint8_t> bits(key_tiles128);
    for (uint32_t c = 0; c < ctas; c++) {
        std::fill(bits.begin(), bits.end(), uint8_t(0));
        for (uint32_t t = 0; t < 2; t++) {
            const uint32_t block = 2 * c + t;
            if (block >= listed_blocks) continue;
            for (uint32_t e = ptr[block]; e < ptr[block + 1]; e++)
                bits[idx[e] >> 1] |= uint8_t(1u << (2 * t + (idx[e] & 1u)));
        }
        for (uint32_t k = 0; k < key_tiles128; k++)
            if (bits[k]) steps.push_back(k | (uint32_t(bits[k]) << 28));
        if (steps.size() == cta_ptr[c]) steps.push_back(0);   /* nothing listed: one all-masked step */
        cta_ptr[c + 1] = uint32_t(steps.size());
    }
    /* the same per 128-row query block (one query tile per CTA): two bits per step */
    std::vector<uint32_t> block_ptr(query_blocks + 1, 0), block_steps;
    for (uint32_t block = 0; block < query_blocks; block++) {
        std::fill(bits.begin(), bits.end(), uint8_t(0));
        if (block < listed_blocks)
            for (uint32_t e = ptr[block]; e < ptr[block + 1]; e++)
                bits[idx[e] >> 1] |= uint8_t(1u << (idx[e] & 1u));
        for (uint32_t k = 0; k < key_tiles128; k++)
            if (bits[k]) block_steps.push_back(k | (uint32_t(bits[k]) << 28));
        if (block_steps.size() == block_ptr[block]) block_steps.push_back(0);   /* one all-masked step */
        block_ptr[block + 1] = uint32_t(block_steps.size());
    }
    auto upload = [](uint32_t **device, const std::vector<uint32_t> &host) {
        return cudaMalloc(reinterpret_cast<void **>(device), host.size() * 4) == cudaSuccess &&
               cudaMemcpy(*device, host.data(), host.size() * 4, cudaMemcpyHostToDevice) == cudaSuccess;
    };
    if (!upload(&gpu->sparse_cta_ptr, cta_ptr) || !upload(&gpu->sparse_steps, steps) ||
        !upload(&gpu->sparse_block_ptr, block_ptr) || !upload(&gpu->sparse_block_steps, block_steps)) {
        cudaGetLastError();
        sparse_clear(gpu);
        return h3b_fail(gpu, "cannot upload the block-sparse attention mask");
    }
    gpu->sparse_rows = rows;
    return 1;
}

/* -------------------------------------------------------------- tensors */

static h3_gpu_tensor *tensor_new(h3_gpu *gpu, const void *values, size_t elements,
                                 h3_gpu_dtype dtype) {
    size_t item = h3b_item_size(dtype);
    if (!gpu || elements > SIZE_MAX / item) return nullptr;
    size_t bytes = elements * item;
    h3_gpu_tensor *tensor = new (std::nothrow) h3_gpu_tensor();
    if (!tensor) {
        h3b_fail(gpu, "out of memory");
        return nullptr;
    }
    cudaSetDevice(gpu->device);
    /* round the block up so that vector loads past an odd tail stay inside it */
    size_t block = ((bytes ? bytes : 1) + 255) & ~size_t(255);
    cudaError_t status = cache_alloc(gpu, block, &tensor->data);
    if (status != cudaSuccess) {
        cudaGetLastError();
        h3b_fail_cuda(gpu, "tensor allocation", status);
        delete tensor;
        return nullptr;
    }
    tensor->elements = elements;
    tensor->bytes = bytes;
    tensor->dtype = dtype;
    tensor->owner = gpu;
    tensor->external = 0;
    tensor->keeps_half = values && dtype == H3_GPU_F32;
    if (values && bytes && !upload(gpu, tensor->data, values, bytes)) {
        h3b_fail(gpu, "tensor upload failed");
        cache_release(gpu, tensor->data, block);
        delete tensor;
        return nullptr;
    }
    gpu->stats.allocated_bytes += bytes;
    gpu->stats.live_bytes += bytes;
    if (gpu->stats.live_bytes > gpu->stats.peak_live_bytes)
        gpu->stats.peak_live_bytes = gpu->stats.live_bytes;
    gpu->stats.tensor_allocations++;
    return tensor;
}

extern "C" h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *gpu, size_t n) {
    return tensor_new(gpu, nullptr, n, H3_GPU_F32);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t n) {
    return tensor_new(gpu, nullptr, n, H3_GPU_BF16);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_i8(h3_gpu *gpu, size_t n) {
    return tensor_new(gpu, nullptr, n, H3_GPU_I8);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *gpu, const float *v, size_t n) {
    return tensor_new(gpu, v, n, H3_GPU_F32);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *gpu, const uint16_t *v, size_t n) {
    return tensor_new(gpu, v, n, H3_GPU_BF16);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *v, size_t n) {
    return tensor_new(gpu, v, n, H3_GPU_U32);
}

extern "C" h3_gpu_tensor *h3x_tensor_wrap(h3_gpu *gpu, void *device_pointer, size_t elements,
                                          h3_gpu_dtype dtype) {
    if (!gpu || (!device_pointer && elements)) return nullptr;
    h3_gpu_tensor *tensor = new (std::nothrow) h3_gpu_tensor();
    if (!tensor) return nullptr;
    tensor->data = device_pointer;
    tensor->elements = elements;
    tensor->bytes = elements * h3b_item_size(dtype);
    tensor->dtype = dtype;
    tensor->owner = gpu;
    tensor->external = 1;
    return tensor;
}

extern "C" void *h3x_tensor_device_pointer(const h3_gpu_tensor *tensor) {
    return tensor ? tensor->data : nullptr;
}

extern "C" void h3_gpu_tensor_free(h3_gpu_tensor *tensor) {
    if (!tensor) return;
    h3_gpu *owner = tensor->owner;
    h3b_written(tensor);
    if (!tensor->external) {
        if (owner)
            owner->stats.live_bytes =
                owner->stats.live_bytes >= tensor->bytes ? owner->stats.live_bytes - tensor->bytes : 0;
        if (tensor->data) {
            size_t block = ((tensor->bytes ? tensor->bytes : 1) + 255) & ~size_t(255);
            if (owner) cache_release(owner, tensor->data, block);
            else cudaFree(tensor->data);
        }
    }
    delete tensor;
}

extern "C" size_t h3_gpu_tensor_elements(const h3_gpu_tensor *t) { return t ? t->elements : 0; }
extern "C" h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *t) {
    return t ? t->dtype : H3_GPU_F32;
}

static int read_range(const h3_gpu_tensor *t, h3_gpu_dtype dtype, size_t offset, void *values,
                      size_t elements) {
    if (!t || !values || t->dtype != dtype || offset > t->elements ||
        elements > t->elements - offset)
        return 0;
    size_t item = h3b_item_size(dtype);
    return download(t->owner, values, static_cast<const unsigned char *>(t->data) + offset * item,
                    elements * item);
}

static int write_range(h3_gpu_tensor *t, h3_gpu_dtype dtype, size_t offset, const void *values,
                       size_t elements) {
    if (!t || !values || !t->owner || t->dtype != dtype || offset > t->elements ||
        elements > t->elements - offset)
        return 0;
    size_t item = h3b_item_size(dtype);
    h3b_written(t);
    return upload(t->owner, static_cast<unsigned char *>(t->data) + offset * item, values,
                  elements * item);
}

extern "C" int h3_gpu_tensor_read_f32(const h3_gpu_tensor *t, float *v, size_t n) {
    return read_range(t, H3_GPU_F32, 0, v, n);
}
extern "C" int h3_gpu_tensor_read_f32_range(const h3_gpu_tensor *t, size_t o, float *v, size_t n) {
    return read_range(t, H3_GPU_F32, o, v, n);
}
extern "C" int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *t, uint16_t *v, size_t n) {
    return read_range(t, H3_GPU_BF16, 0, v, n);
}
extern "C" int h3_gpu_tensor_write_f32(h3_gpu_tensor *t, const float *v, size_t n) {
    return write_range(t, H3_GPU_F32, 0, v, n);
}
extern "C" int h3_gpu_tensor_write_f32_range(h3_gpu_tensor *t, size_t o, const float *v, size_t n) {
    return write_range(t, H3_GPU_F32, o, v, n);
}
extern "C" int h3_gpu_tensor_write_bf16(h3_gpu_tensor *t, const uint16_t *v, size_t n) {
    return write_range(t, H3_GPU_BF16, 0, v, n);
}
extern "C" int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *t, size_t o, const uint16_t *v,
                                              size_t n) {
    return write_range(t, H3_GPU_BF16, o, v, n);
}

/* ------------------------------------------------------------ file loads */
/* A payload is cut into 16 MiB chunks on a 4 KiB-aligned grid of the file. Up to four reader
 * threads pread() chunks into a ring of pinned buffers that belongs to the context (allocated
 * on first use, kept), while the calling thread uploads finished chunks in order with
 * cudaMemcpyAsync on a private copy stream: the disk, the page-cache copy and the host->device
 * DMA overlap, and nothing is allocated per call. Reads go through O_DIRECT where the file
 * system takes it (the raw device rate instead of the page cache's; every chunk is an aligned
 * superset of its payload bytes), else through the page cache; H3B_DIRECT_IO=0 forces the
 * latter. Replaces the reference's loader (h3_gpu_cuda.cu:455-689: whole tensor into one pinned
 * staging buffer with up to 16 threads, then one synchronous copy).
 * A load may run on an I/O thread while the context's thread keeps issuing kernels on tensors
 * that are not being filled; loads of one context are serialised among themselves.
 * after_context: the first copy waits (on the device, through an event) for the work queued
 * on the context's stream at the time of the call, so kernels that still read the tensor's
 * previous contents finish first. The streaming entry point does not wait: its contract is a
 * target that is idle on the context's stream, so that the upload overlaps the running block. */

struct h3b_loader {
    static constexpr int kBuffers = 6;
    static constexpr size_t kChunk = size_t(16) << 20;
    static constexpr size_t kAlign = 4096;
    void *pinned[kBuffers] = {};
    cudaEvent_t uploaded[kBuffers] = {};
    cudaStream_t stream = nullptr;
    bool ready = false;
    std::mutex mutex;                       /* one load at a time per context */

    bool prepare() {
        if (ready) return true;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return false;
        for (int i = 0; i < kBuffers; i++)
            if (cudaMallocHost(&pinned[i], kChunk + 2 * kAlign) != cudaSuccess ||
                cudaEventCreateWithFlags(&uploaded[i], cudaEventDisableTiming) != cudaSuccess)
                return false;
        ready = true;
        return true;
    }
    void release() {
        for (int i = 0; i < kBuffers; i++) {
            if (pinned[i]) cudaFreeHost(pinned[i]);
            if (uploaded[i]) cudaEventDestroy(uploaded[i]);
            pinned[i] = nullptr;
            uploaded[i] = nullptr;
        }
        if (stream) cudaStreamDestroy(stream);
        stream = nullptr;
        ready = false;
    }
};

void h3b_loader_free(h3b_loader *loader) {
    if (!loader) return;
    loader->release();
    delete loader;
}

/* pread of [offset, offset + bytes): 0 on success, errno on error, -1 when the file ended
 * before `need` bytes (an O_DIRECT span is rounded up past the payload, so it may be cut). */
static int read_span(int fd, unsigned char *dst, uint64_t offset, size_t bytes, size_t need) {
    size_t got = 0;
    while (got < bytes) {
        ssize_t n = pread(fd, dst + got, bytes - got, off_t(offset + got));
        if (n < 0 && errno == EINTR) continue;
        if (n < 0) return errno;
        if (n == 0) return got >= need ? 0 : -1;
        got += size_t(n);
    }
    return 0;
}

static bool direct_io_wanted() {
    const char *v = getenv("H3B_DIRECT_IO");
    return !(v && *v && strcmp(v, "0") == 0);
}

static int fill_from_file(h3_gpu_tensor *tensor, const char *path, uint64_t file_offset,
                          size_t elements, h3_gpu_dtype dtype, char *error, size_t error_size,
                          bool after_context = false) {
    auto fail = [&](const char *what) {
        if (error && error_size) snprintf(error, error_size, "%s: %s", what, path ? path : "(null)");
        return 0;
    };
    if (!tensor || !path || tensor->dtype != dtype || elements > tensor->elements || !tensor->owner)
        return fail("invalid tensor file read");
    const size_t bytes = elements * h3b_item_size(dtype);
    if (!bytes) return 1;
    h3_gpu *gpu = tensor->owner;
    if (!gpu->loader) gpu->loader = new (std::nothrow) h3b_loader();
    h3b_loader *ld = gpu->loader;
    if (!ld) return fail("out of memory for the file loader of");
    std::lock_guard<std::mutex> serial(ld->mutex);
    cudaSetDevice(gpu->device);
    if (!ld->prepare()) {
        cudaGetLastError();
        return fail("cannot allocate staging memory for");
    }
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail("cannot open tensor file");
    int fd_direct = direct_io_wanted() ? open(path, O_RDONLY | O_CLOEXEC | O_DIRECT) : -1;

    int ok = 1;
    if (after_context) {
        cudaEvent_t queued = nullptr;
        if (cudaEventCreateWithFlags(&queued, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(queued, gpu->stream) != cudaSuccess ||
            cudaStreamWaitEvent(ld->stream, queued, 0) != cudaSuccess)
            ok = fail("cannot order the upload after the context's stream for");
        if (queued) cudaEventDestroy(queued);
    }

    /* chunk c = file bytes [grid0 + c * kChunk, grid0 + (c + 1) * kChunk) cut to the payload */
    constexpr size_t kChunk = h3b_loader::kChunk, kAlign = h3b_loader::kAlign;
    constexpr int kBuffers = h3b_loader::kBuffers;
    const uint64_t grid0 = file_offset & ~uint64_t(kAlign - 1);
    const uint64_t payload_end = file_offset + bytes;
    const size_t chunks = size_t((payload_end - grid0 + kChunk - 1) / kChunk);
    std::vector<int> state(chunks, 0);          /* 0 pending, 1 read, <0 failed */
    std::vector<size_t> skip(chunks, 0);        /* payload offset inside the chunk's buffer */
    std::mutex m;
    std::condition_variable cv;
    size_t uploads_issued = 0;                  /* chunks whose copy has been enqueued */
    bool abort_all = !ok;
    std::atomic<bool> direct_refused(false);

    auto reader = [&](size_t first, size_t stride) {
        for (size_t c = first; c < chunks; c += stride) {
            const int slot = int(c % kBuffers);
            {   /* the slot is free once the copy of chunk c - kBuffers has finished */
                std::unique_lock<std::mutex> lock(m);
                cv.wait(lock, [&] { return abort_all || c < size_t(kBuffers) || uploads_issued + kBuffers > c; });
                if (abort_all) return;
            }
            if (c >= size_t(kBuffers) && cudaEventSynchronize(ld->uploaded[slot]) != cudaSuccess) {
                std::lock_guard<std::mutex> lock(m);
                state[c] = -1; abort_all = true; cv.notify_all();
                return;
            }
            const uint64_t begin = grid0 + uint64_t(c) * kChunk;
            const uint64_t first_byte = begin > file_offset ? begin : file_offset;
            const uint64_t last_byte = begin + kChunk < payload_end ? begin + kChunk : payload_end;
            unsigned char *dst = static_cast<unsigned char *>(ld->pinned[slot]);
            int rc = EINVAL;
            if (fd_direct >= 0 && !direct_refused.load()) {
                const uint64_t span_end = (last_byte + kAlign - 1) & ~uint64_t(kAlign - 1);
                rc = read_span(fd_direct, dst, begin, size_t(span_end - begin), size_t(last_byte - begin));
                if (rc == EINVAL) direct_refused.store(true);     /* the file system refuses O_DIRECT */
                else skip[c] = size_t(first_byte - begin);
            }
            if (rc == EINVAL) {
                rc = read_span(fd, dst, first_byte, size_t(last_byte - first_byte), size_t(last_byte - first_byte));
                skip[c] = 0;
            }
            std::lock_guard<std::mutex> lock(m);
            state[c] = rc == 0 ? 1 : -1;
            if (rc != 0) abort_all = true;
            cv.notify_all();
            if (rc != 0) return;
        }
    };

    const size_t reader_count = chunks < 4 ? chunks : 4;
    std::vector<std::thread> readers;
    if (ok && chunks > 1)
        for (size_t t = 0; t < reader_count; t++) readers.emplace_back(reader, t, reader_count);
    for (size_t c = 0; ok && c < chunks; c++) {
        if (chunks == 1) reader(0, 1);          /* small payloads are read inline */
        {
            std::unique_lock<std::mutex> lock(m);
            cv.wait(lock, [&] { return state[c] != 0 || abort_all; });
            if (state[c] != 1) { ok = fail("short or failed read from"); break; }
        }
        const int slot = int(c % kBuffers);
        const uint64_t begin = grid0 + uint64_t(c) * kChunk;
        const uint64_t first_byte = begin > file_offset ? begin : file_offset;
        const uint64_t last_byte = begin + kChunk < payload_end ? begin + kChunk : payload_end;
        if (cudaMemcpyAsync(static_cast<char *>(tensor->data) + (first_byte - file_offset),
                            static_cast<unsigned char *>(ld->pinned[slot]) + skip[c],
                            size_t(last_byte - first_byte), cudaMemcpyHostToDevice, ld->stream) != cudaSuccess ||
            cudaEventRecord(ld->uploaded[slot], ld->stream) != cudaSuccess) {
            ok = fail("device upload failed for");
            break;
        }
        std::lock_guard<std::mutex> lock(m);
        uploads_issued = c + 1;
        cv.notify_all();
    }
    {
        std::lock_guard<std::mutex> lock(m);
        if (!ok) abort_all = true;
        cv.notify_all();
    }
    for (std::thread &t : readers) t.join();
    if (cudaStreamSynchronize(ld->stream) != cudaSuccess && ok) ok = fail("device upload failed for");
    if (fd_direct >= 0) close(fd_direct);
    close(fd);
    cudaGetLastError();
    return ok;
}

static h3_gpu_tensor *load_file(h3_gpu *gpu, const char *path, uint64_t offset, size_t elements,
                                h3_gpu_dtype dtype) {
    h3_gpu_tensor *tensor = tensor_new(gpu, nullptr, elements, dtype);
    if (!tensor) return nullptr;
    /* the block may have been recycled from a tensor whose last kernels are still queued */
    cudaStreamSynchronize(gpu->stream);
    char message[400];
    if (!fill_from_file(tensor, path, offset, elements, dtype, message, sizeof(message))) {
        h3b_fail(gpu, "%s", message);
        h3_gpu_tensor_free(tensor);
        return nullptr;
    }
    tensor->keeps_half = dtype == H3_GPU_F32;
    return tensor;
}

extern "C" h3_gpu_tensor *h3_gpu_tensor_load_bf16(h3_gpu *gpu, const char *path, uint64_t offset,
                                                  size_t elements) {
    return load_file(gpu, path, offset, elements, H3_GPU_BF16);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_load_f32(h3_gpu *gpu, const char *path, uint64_t offset,
                                                 size_t elements) {
    return load_file(gpu, path, offset, elements, H3_GPU_F32);
}
extern "C" int h3_gpu_tensor_read_file_bf16(h3_gpu_tensor *tensor, const char *path,
                                            uint64_t offset, size_t elements, char *error,
                                            size_t error_size) {
    return fill_from_file(tensor, path, offset, elements, H3_GPU_BF16, error, error_size, true);
}
extern "C" int h3_gpu_tensor_stream_file_bf16(h3_gpu_tensor *tensor, const char *path,
                                              uint64_t offset, size_t elements, char *error,
                                              size_t error_size) {
    return fill_from_file(tensor, path, offset, elements, H3_GPU_BF16, error, error_size);
}

/* ----------------------------------------------------- casts and copies */

__global__ void h3b_cast_f32_bf16(const float *in, uint16_t *out, size_t count) {
    size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    bool aligned = ((reinterpret_cast<uintptr_t>(in) & 15u) | (reinterpret_cast<uintptr_t>(out) & 7u)) == 0;
    if (aligned && i + 3 < count) {
        float4 v = *reinterpret_cast<const float4 *>(in + i);
        uint2 packed = {h3b_narrow2(v.x, v.y), h3b_narrow2(v.z, v.w)};
        *reinterpret_cast<uint2 *>(out + i) = packed;
    } else {
        for (size_t e = i + 4 < count ? i + 4 : count; i < e; i++) out[i] = h3b_narrow(in[i]);
    }
}

__global__ void h3b_cast_bf16_f32(const uint16_t *in, float *out, size_t count) {
    size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    bool aligned = ((reinterpret_cast<uintptr_t>(in) & 7u) | (reinterpret_cast<uintptr_t>(out) & 15u)) == 0;
    if (aligned && i + 3 < count) {
        uint2 packed = *reinterpret_cast<const uint2 *>(in + i);
        *reinterpret_cast<float4 *>(out + i) =
            make_float4(h3b_lo(packed.x), h3b_hi(packed.x), h3b_lo(packed.y), h3b_hi(packed.y));
    } else {
        for (size_t e = i + 4 < count ? i + 4 : count; i < e; i++) out[i] = h3b_widen(in[i]);
    }
}

extern "C" int h3_gpu_cast_f32_to_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                       const h3_gpu_tensor *input, uint32_t elements) {
    if (!h3b_need(gpu, input, H3_GPU_F32, elements, "cast input") ||
        !h3b_need(gpu, output, H3_GPU_BF16, elements, "cast output") || !h3b_need_command(gpu))
        return 0;
    if (elements) {
        unsigned blocks = unsigned((size_t(elements) + 1023) / 1024);
        h3b_cast_f32_bf16<<<blocks, 256, 0, gpu->stream>>>(h3b_ptr<float>(input),
                                                          h3b_ptr<uint16_t>(output), elements);
    }
    return h3b_launched(gpu, "cast_f32_to_bf16");
}

extern "C" int h3_gpu_cast_bf16_to_f32(h3_gpu *gpu, h3_gpu_tensor *output,
                                       const h3_gpu_tensor *input, uint32_t elements) {
    if (!h3b_need(gpu, input, H3_GPU_BF16, elements, "cast input") ||
        !h3b_need(gpu, output, H3_GPU_F32, elements, "cast output") || !h3b_need_command(gpu))
        return 0;
    h3b_written(output);
    if (elements) {
        unsigned blocks = unsigned((size_t(elements) + 1023) / 1024);
        h3b_cast_bf16_f32<<<blocks, 256, 0, gpu->stream>>>(h3b_ptr<uint16_t>(input),
                                                          h3b_ptr<float>(output), elements);
    }
    return h3b_launched(gpu, "cast_bf16_to_f32");
}

static int device_copy(h3_gpu *gpu, h3_gpu_tensor *dst, size_t dst_offset,
                       const h3_gpu_tensor *src, size_t src_offset, size_t elements,
                       h3_gpu_dtype dtype) {
    if (!dst || !src || dst->dtype != dtype || src->dtype != dtype)
        return h3b_fail(gpu, "copy tensor has the wrong dtype");
    if (dst_offset > dst->elements || elements > dst->elements - dst_offset ||
        src_offset > src->elements || elements > src->elements - src_offset)
        return h3b_fail(gpu, "copy range is out of bounds");
    if (!h3b_need_command(gpu)) return 0;
    size_t item = h3b_item_size(dtype);
    h3b_written(dst);
    if (elements) {
        cudaError_t status = cudaMemcpyAsync(
            static_cast<unsigned char *>(dst->data) + dst_offset * item,
            static_cast<const unsigned char *>(src->data) + src_offset * item, elements * item,
            cudaMemcpyDeviceToDevice, gpu->stream);
        if (status != cudaSuccess) return h3b_fail_cuda(gpu, "device copy", status);
        if (gpu->op_profile) h3b_profile_record(gpu, "copy");
    }
    gpu->stats.blit_copies++;
    return 1;
}

extern "C" int h3_gpu_copy_bf16(h3_gpu *gpu, h3_gpu_tensor *dst, size_t dst_offset,
                                const h3_gpu_tensor *src, size_t src_offset, size_t elements) {
    return device_copy(gpu, dst, dst_offset, src, src_offset, elements, H3_GPU_BF16);
}
extern "C" int h3_gpu_copy_f32(h3_gpu *gpu, h3_gpu_tensor *dst, size_t dst_offset,
                               const h3_gpu_tensor *src, size_t src_offset, size_t elements) {
    return device_copy(gpu, dst, dst_offset, src, src_offset, elements, H3_GPU_F32);
}

extern "C" int h3_cuda_probe(h3_device_info *info, char *error, size_t error_size) {
    if (!info) return 0;
    memset(info, 0, sizeof(*info));
    int count = 0;
    cudaError_t status = cudaGetDeviceCount(&count);
    if (status != cudaSuccess || count < 1) {
        if (error && error_size)
            snprintf(error, error_size, "no CUDA device available: %s", cudaGetErrorString(status));
        cudaGetLastError();
        return 0;
    }
    cudaDeviceProp prop;
    status = cudaGetDeviceProperties(&prop, g_device);
    if (status != cudaSuccess) {
        if (error && error_size)
            snprintf(error, error_size, "cannot query CUDA device: %s", cudaGetErrorString(status));
        cudaGetLastError();
        return 0;
    }
    snprintf(info->name, sizeof(info->name), "%.127s", prop.name);
    snprintf(info->architecture, sizeof(info->architecture), "sm_%d%d", prop.major, prop.minor);
    const long pages = sysconf(_SC_PHYS_PAGES), page_size = sysconf(_SC_PAGESIZE);
    if (pages > 0 && page_size > 0) info->physical_memory = uint64_t(pages) * uint64_t(page_size);
    info->recommended_working_set = prop.totalGlobalMem;
    info->max_buffer_length = prop.totalGlobalMem;
    return 1;
}

extern "C" int h3b200_probe(h3b200_device_info *info, char *error, size_t error_size) {
    if (!info) return 0;
    memset(info, 0, sizeof(*info));
    cudaDeviceProp prop;
    cudaError_t status = cudaGetDeviceProperties(&prop, g_device);
    if (status != cudaSuccess) {
        if (error && error_size)
            snprintf(error, error_size, "no CUDA device: %s", cudaGetErrorString(status));
        cudaGetLastError();
        return 0;
    }
    snprintf(info->name, sizeof(info->name), "%s", prop.name);
    info->total_memory = prop.totalGlobalMem;
    info->compute_major = prop.major;
    info->compute_minor = prop.minor;
    info->multiprocessors = prop.multiProcessorCount;
    return 1;
}
