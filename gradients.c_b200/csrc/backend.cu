// Backend lifecycle, buffers, stream scope, fences, transfers and the small memory
// primitives (fill / rand_uniform / accumulate / scale).
//
// Reference behaviour followed here: src/backends/metal/backend_metal.m:354-394 (ops
// outside a scope run to completion), :534-577 (flush = submit + wait), :836-897 (fences),
// src/backends/metal/primitives/memory/metal_memory.metal:8-57 and
// src/backends/metal/primitives/random/metal_random.metal:8-30 (kernel arithmetic).
//
// Execution model on CUDA: one in-order stream per backend. Every entry enqueues on it;
// gd_backend_flush and the synchronous transfers wait for it, so an op issued outside a
// begin/end scope is observed by the next read exactly as in the reference.
#include "common.cuh"

#include <atomic>

#include <stdlib.h>
#include <sys/mman.h>

namespace {

struct gdb_fence {
    cudaEvent_t event;
    int device;
};

size_t env_size(const char *name, size_t dflt)
{
    const char *s = getenv(name);
    if (s == NULL || *s == '\0') {
        return dflt;
    }
    char *end = NULL;
    unsigned long long v = strtoull(s, &end, 10);
    return end == s ? dflt : (size_t)v;
}

int pick_device(void)
{
    const char *s = getenv("GD_CUDA_DEVICE");
    if (s == NULL || *s == '\0') {
        s = getenv("LOCAL_RANK");
    }
    return (s != NULL && *s != '\0') ? atoi(s) : 0;
}

__global__ void fill_kernel(unsigned char *dst, size_t count, unsigned elem_size, unsigned pattern)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        if (elem_size == 4U) {
            reinterpret_cast<unsigned *>(dst)[i] = pattern;
        } else if (elem_size == 2U) {
            reinterpret_cast<unsigned short *>(dst)[i] = (unsigned short)(pattern & 0xffffU);
        } else {
            for (unsigned b = 0; b < elem_size; ++b) {
                dst[i * elem_size + b] = (unsigned char)((pattern >> (8U * b)) & 255U);
            }
        }
    }
}

template <typename T>
__global__ void rand_uniform_kernel(T *dst, size_t count, uint64_t seed, float low, float high)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const uint64_t r = gdb_splitmix64(seed + (uint64_t)i);
        const unsigned mant = (unsigned)((r >> 40) & 0xffffffULL);
        const float u = (float)mant * (1.0f / 16777216.0f);
        gdb_io<T>::st(dst, i, low + (high - low) * u);
    }
}

// dst[i] = round(dst[i] + src[i]): the 16-bit path rounds after every add, as the
// reference does (metal_memory.metal:31).
template <typename T>
__global__ void accumulate_kernel(T *dst, const T *src, size_t count)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        gdb_io<T>::st(dst, i, gdb_io<T>::ld(dst, i) + gdb_io<T>::ld(src, i));
    }
}
template <typename T>
__global__ void accumulate_vec8_kernel(uint4 *dst, const uint4 *src, size_t vecs)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        gdb_vec8<T> d, s;
        d.raw = dst[i];
        s.raw = src[i];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            d.set(e, d.get(e) + s.get(e));
        }
        dst[i] = d.raw;
    }
}

template <typename T>
__global__ void scale_kernel(T *dst, const T *src, size_t count, float scale)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        gdb_io<T>::st(dst, i, gdb_io<T>::ld(src, i) * scale);
    }
}

__global__ void l2_flush_kernel(uint4 *buf, size_t vecs, unsigned tag)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        buf[i] = make_uint4(tag, tag, tag, tag);
    }
}

}  // namespace

extern "C" {

gd_status gd_backend_create_default(gd_backend **out_backend)
{
    int count = 0;
    cudaDeviceProp prop;
    gd_backend *be;
    if (out_backend == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    *out_backend = NULL;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        return GD_ERR_UNSUPPORTED;  // no CUDA device: same answer as the null backend
    }
    be = (gd_backend *)calloc(1, sizeof(*be));
    if (be == NULL) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    be->device = pick_device();
    if (be->device < 0 || be->device >= count) {
        free(be);
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (cudaSetDevice(be->device) != cudaSuccess || cudaGetDeviceProperties(&prop, be->device) != cudaSuccess) {
        free(be);
        return GD_ERR_INTERNAL;
    }
    if (prop.major != 10) {
        // Kernels are built for sm_100a only; refuse loudly instead of failing at first launch.
        fprintf(stderr, "gd_backend_b200: device %d is sm_%d%d, this backend requires sm_100a\n",
                be->device, prop.major, prop.minor);
        free(be);
        return GD_ERR_UNSUPPORTED;
    }
    {
        // One device per process: the kernels' one-time set-up (dynamic shared memory limits, occupancy, cluster sizes)
        // is cached in process-wide flags, and CUDA function attributes are per device. A backend on a second device
        // would skip that set-up and fail at its first large launch, so it is refused here with a clear message
        // (data parallelism runs one process per GPU).
        static std::atomic<int> process_device(-1);
        int expected = -1;
        if (!process_device.compare_exchange_strong(expected, be->device) && expected != be->device) {
            fprintf(stderr, "gd_backend_b200: this process already runs a backend on device %d; device %d needs its own process\n",
                    expected, be->device);
            free(be);
            return GD_ERR_UNSUPPORTED;
        }
    }
    be->sm_count = prop.multiProcessorCount;
    be->ws_bytes = env_size("GD_CUDA_WORKSPACE_MB", 512U) << 20;
    be->l2_flush_bytes = (size_t)256U << 20;
    if (cudaStreamCreateWithFlags(&be->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc((void **)&be->ws, be->ws_bytes) != cudaSuccess ||
        cudaMalloc((void **)&be->err_flag, GDB_FLAG_BYTES) != cudaSuccess ||
        cudaMallocHost((void **)&be->err_flag_host, 256) != cudaSuccess ||
        cudaMemset(be->err_flag, 0, GDB_FLAG_BYTES) != cudaSuccess) {
        gd_backend_destroy(be);
        return GD_ERR_OUT_OF_MEMORY;
    }
    *out_backend = be;
    return GD_OK;
}

void gd_backend_destroy(gd_backend *be)
{
    if (be == NULL) {
        return;
    }
    cudaSetDevice(be->device);
    if (be->stream != NULL) {
        cudaStreamSynchronize(be->stream);
    }
    gdb_dp_destroy(be);
    gdb_tmap_cache_destroy(be);
    cudaFree(be->ws);
    cudaFree(be->err_flag);
    cudaFreeHost(be->err_flag_host);
    cudaFree(be->rope_table);
    cudaFree(be->l2_flush);
    if (be->stream != NULL) {
        cudaStreamDestroy(be->stream);
    }
    free(be);
}

gd_backend_kind gd_backend_kind_query(const gd_backend *backend)
{
    (void)backend;
    return (gd_backend_kind)2;
}

const char *gd_backend_name(const gd_backend *backend)
{
    (void)backend;
    return "cuda-b200";
}

// Buffers. The host runtime insists on a host-visible base pointer for every arena
// (reference src/core/memory.c:231-236) although only the data ring is ever written through
// it (src/dataset/dataloader.c:487-492: loader threads memcpy into host_ptr). Buffers up to
// GD_CUDA_MANAGED_MAX_MB (default 1024, which covers the data slots the reference's examples create:
// examples/gpt_lm/gpt_lm_shared.h:67 asks for 128 MiB or more per slot) are CUDA managed memory that
// prefers the device and is populated there when it is created, so kernels find it resident and a host
// write simply migrates the pages it touches. Larger buffers (the multi-GiB scratch slots) are plain
// device memory and report a reserved, inaccessible host address range that only satisfies the
// non-NULL / 256-byte alignment contract; nothing in the reference dereferences those.
gd_status gd_backend_buffer_create(gd_backend *be, size_t nbytes, gd_backend_buffer **out_buffer)
{
    gd_backend_buffer *buf;
    cudaError_t e;
    const size_t managed_max = env_size("GD_CUDA_MANAGED_MAX_MB", 1024U) << 20;
    if (out_buffer == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    *out_buffer = NULL;
    if (be == NULL || nbytes == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    buf = (gd_backend_buffer *)calloc(1, sizeof(*buf));
    if (buf == NULL) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    buf->backend = be;
    buf->nbytes = nbytes;
    if (nbytes <= managed_max) {
        e = cudaMallocManaged((void **)&buf->dptr, nbytes, cudaMemAttachGlobal);
        if (e != cudaSuccess) {
            free(buf);
            return gdb_fail(be, e, "cudaMallocManaged");
        }
        buf->kind = GDB_BUF_MANAGED;
        buf->hptr = buf->dptr;
        
        
        
        (void)cudaMemAdvise(buf->dptr, nbytes, cudaMemAdviseSetPreferredLocation, be->device);
        // keep the pages mapped into the GPU's page tables wherever they live: after a host write a kernel reads the
        // touched pages over the bus instead of taking a page fault per 64 KB block (0.47 ms per gpt_lm step measured)
        if (env_size("GD_CUDA_MANAGED_ACCESSED_BY", 1U) != 0U) {
            (void)cudaMemAdvise(buf->dptr, nbytes, cudaMemAdviseSetAccessedBy, be->device);
        }
        (void)cudaMemPrefetchAsync(buf->dptr, nbytes, be->device, be->stream);   // resident before the first kernel touches it
        (void)cudaGetLastError();
    } else {
        e = cudaMalloc((void **)&buf->dptr, nbytes);
        if (e != cudaSuccess) {
            free(buf);
            return gdb_fail(be, e, "cudaMalloc");
        }
        buf->kind = GDB_BUF_DEVICE;
        buf->reserve_bytes = (nbytes + 4095U) & ~(size_t)4095U;
        buf->hptr = mmap(NULL, buf->reserve_bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
        if (buf->hptr == MAP_FAILED) {
            cudaFree(buf->dptr);
            free(buf);
            return GD_ERR_OUT_OF_MEMORY;
        }
    }
    *out_buffer = buf;
    return GD_OK;
}

void gd_backend_buffer_destroy(gd_backend_buffer *buf)
{
    if (buf == NULL) {
        return;
    }
    if (buf->backend != NULL) {
        cudaSetDevice(buf->backend->device);
        cudaStreamSynchronize(buf->backend->stream);
    }
    cudaFree(buf->dptr);
    if (buf->kind == GDB_BUF_DEVICE && buf->hptr != NULL) {
        munmap(buf->hptr, buf->reserve_bytes);
    }
    free(buf);
}

size_t gd_backend_buffer_nbytes(const gd_backend_buffer *buf) { return buf != NULL ? buf->nbytes : 0U; }
void *gd_backend_buffer_host_ptr(gd_backend_buffer *buf) { return buf != NULL ? buf->hptr : NULL; }
bool gd_backend_buffer_is_host_visible(const gd_backend_buffer *buf) { return buf != NULL && buf->hptr != NULL; }

gd_status gd_backend_scope_begin(gd_backend *be)
{
    if (be == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    return GD_OK;
}

gd_status gd_backend_flush(gd_backend *be)
{
    cudaError_t e;
    if (be == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    e = cudaStreamSynchronize(be->stream);
    if (e != cudaSuccess) {
        return gdb_fail(be, e, "flush");
    }
    // kernels with bounded waits report a give-up through the device error word
    e = cudaMemcpy(be->err_flag_host, be->err_flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        return gdb_fail(be, e, "flush error word");
    }
    if (*be->err_flag_host != 0) {
        snprintf(be->last_error, sizeof(be->last_error), "device kernel gave up a bounded wait (code %d)", *be->err_flag_host);
        cudaMemset(be->err_flag, 0, sizeof(int));
        return GD_ERR_INTERNAL;
    }
    return GD_OK;
}

gd_status gd_backend_record_fence(gd_backend *be, gd_backend_fence *out_fence)
{
    gdb_fence *f;
    cudaError_t e;
    if (be == NULL || out_fence == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    out_fence->handle = NULL;
    cudaSetDevice(be->device);
    f = (gdb_fence *)malloc(sizeof(*f));
    if (f == NULL) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    f->device = be->device;
    e = cudaEventCreateWithFlags(&f->event, cudaEventDisableTiming);
    if (e == cudaSuccess) {
        e = cudaEventRecord(f->event, be->stream);
        if (e != cudaSuccess) {
            cudaEventDestroy(f->event);
        }
    }
    if (e != cudaSuccess) {
        free(f);
        return gdb_fail(be, e, "record_fence");
    }
    out_fence->handle = f;
    return GD_OK;
}

// Fence calls also arrive from dataloader worker threads (reference src/core/memory.c:516-569),
// so each sets the device for the calling thread and touches no backend state.
void gd_backend_fence_destroy(gd_backend_fence *fence)
{
    if (fence == NULL || fence->handle == NULL) {
        return;
    }
    gdb_fence *f = (gdb_fence *)fence->handle;
    cudaSetDevice(f->device);
    cudaEventDestroy(f->event);
    free(f);
    fence->handle = NULL;
}

bool gd_backend_fence_is_complete(gd_backend_fence *fence)
{
    if (fence == NULL || fence->handle == NULL) {
        return true;
    }
    gdb_fence *f = (gdb_fence *)fence->handle;
    cudaSetDevice(f->device);
    return cudaEventQuery(f->event) != cudaErrorNotReady;
}

gd_status gd_backend_fence_wait(gd_backend_fence *fence)
{
    if (fence == NULL || fence->handle == NULL) {
        return GD_OK;
    }
    gdb_fence *f = (gdb_fence *)fence->handle;
    cudaSetDevice(f->device);
    return cudaEventSynchronize(f->event) == cudaSuccess ? GD_OK : GD_ERR_INTERNAL;
}

gd_status gd_backend_upload(gd_backend *be, gd_backend_buffer *buffer, size_t offset, const void *src, size_t nbytes)
{
    cudaError_t e;
    if (be == NULL || (src == NULL && nbytes != 0U) || !gdb_range_ok(buffer, offset, nbytes)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (nbytes == 0U) {
        return GD_OK;
    }
    cudaSetDevice(be->device);
    e = cudaMemcpyAsync(buffer->dptr + offset, src, nbytes, cudaMemcpyHostToDevice, be->stream);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(be->stream);
    }
    return e == cudaSuccess ? GD_OK : gdb_fail(be, e, "upload");
}

gd_status gd_backend_download(gd_backend *be, gd_backend_buffer *buffer, size_t offset, void *dst, size_t nbytes)
{
    cudaError_t e;
    if (be == NULL || (dst == NULL && nbytes != 0U) || !gdb_range_ok(buffer, offset, nbytes)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (nbytes == 0U) {
        return GD_OK;
    }
    cudaSetDevice(be->device);
    e = cudaMemcpyAsync(dst, buffer->dptr + offset, nbytes, cudaMemcpyDeviceToHost, be->stream);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(be->stream);
    }
    return e == cudaSuccess ? GD_OK : gdb_fail(be, e, "download");
}

// Stream-ordered copies between page-locked host memory and a buffer: enqueued behind the work already
// submitted and not waited for, so the host can prepare step k + 1 while step k runs. This is the device half of
// the reference's data-slot ring, where loader threads fill the next slot's host span while the device still
// reads the previous one and a fence guards reuse (src/core/memory.c:1149-1208, src/dataset/dataloader.c:487-492).
// The host range must stay untouched (upload) or unread (download) until a fence recorded after the call completes.
gd_status gdb200_upload_async(gd_backend *be, gd_backend_buffer *buffer, size_t offset, const void *pinned_src, size_t nbytes)
{
    if (be == NULL || (pinned_src == NULL && nbytes != 0U) || !gdb_range_ok(buffer, offset, nbytes)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (nbytes == 0U) {
        return GD_OK;
    }
    cudaSetDevice(be->device);
    cudaError_t e = cudaMemcpyAsync(buffer->dptr + offset, pinned_src, nbytes, cudaMemcpyHostToDevice, be->stream);
    return e == cudaSuccess ? GD_OK : gdb_fail(be, e, "upload_async");
}

gd_status gdb200_download_async(gd_backend *be, gd_backend_buffer *buffer, size_t offset, void *pinned_dst, size_t nbytes)
{
    if (be == NULL || (pinned_dst == NULL && nbytes != 0U) || !gdb_range_ok(buffer, offset, nbytes)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (nbytes == 0U) {
        return GD_OK;
    }
    cudaSetDevice(be->device);
    cudaError_t e = cudaMemcpyAsync(pinned_dst, buffer->dptr + offset, nbytes, cudaMemcpyDeviceToHost, be->stream);
    return e == cudaSuccess ? GD_OK : gdb_fail(be, e, "download_async");
}

gd_status gd_backend_fill(gd_backend *be, gd_backend_buffer *buffer, size_t offset, size_t count, size_t elem_size, uint32_t pattern)
{
    if (be == NULL || elem_size == 0U || elem_size > 4U || count > SIZE_MAX / elem_size ||
        !gdb_range_ok(buffer, offset, count * elem_size)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    if ((elem_size == 4U || elem_size == 2U) && (offset % elem_size) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    unsigned char *dst = buffer->dptr + offset;
    const unsigned bytepat = pattern & 255U;
    bool uniform = true;
    for (size_t b = 1; b < elem_size; ++b) {
        uniform = uniform && (((pattern >> (8U * b)) & 255U) == bytepat);
    }
    // small fills go through the kernel: a memset node between two kernels gives up their programmatic launch overlap
    if (uniform && count * elem_size > (1U << 20)) {
        cudaError_t e = cudaMemsetAsync(dst, (int)bytepat, count * elem_size, be->stream);
        be->launches += 1U;
        return e == cudaSuccess ? GD_OK : gdb_fail(be, e, "fill");
    }
    gdb_launch(fill_kernel, gdb_grid_for(count, 256, be, 8), 256, 0, be->stream, dst, count, (unsigned)elem_size, pattern);
    return gdb_launched(be, "fill");
}

gd_status gd_backend_rand_uniform(gd_backend *be, gd_backend_buffer *buffer, size_t offset, size_t count, uint32_t dtype, uint64_t seed, float low, float high)
{
    const size_t es = gdb_dtype_size(dtype);
    if (be == NULL || !gdb_is_float_dtype(dtype) || count > SIZE_MAX / es || (offset % es) != 0U ||
        !gdb_range_ok(buffer, offset, count * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    void *dst = buffer->dptr + offset;
    const unsigned grid = gdb_grid_for(count, 256, be, 8);
    if (dtype == GDB_DTYPE_F16) {
        gdb_launch(rand_uniform_kernel<__half>, grid, 256, 0, be->stream, (__half *)dst, count, seed, low, high);
    } else if (dtype == GDB_DTYPE_BF16) {
        gdb_launch(rand_uniform_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (__nv_bfloat16 *)dst, count, seed, low, high);
    } else {
        gdb_launch(rand_uniform_kernel<float>, grid, 256, 0, be->stream, (float *)dst, count, seed, low, high);
    }
    return gdb_launched(be, "rand_uniform");
}

gd_status gd_backend_accumulate(gd_backend *be, gd_backend_buffer *dst_buffer, size_t dst_offset, gd_backend_buffer *src_buffer, size_t src_offset, size_t count, uint32_t dtype)
{
    const size_t es = gdb_dtype_size(dtype);
    if (be == NULL || !gdb_is_float_dtype(dtype) || count > SIZE_MAX / es ||
        (dst_offset % es) != 0U || (src_offset % es) != 0U ||
        !gdb_range_ok(dst_buffer, dst_offset, count * es) || !gdb_range_ok(src_buffer, src_offset, count * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    unsigned char *d = dst_buffer->dptr + dst_offset;
    const unsigned char *s = src_buffer->dptr + src_offset;
    const bool vec = es == 2U && (count % 8U) == 0U && ((uintptr_t)d % 16U) == 0U && ((uintptr_t)s % 16U) == 0U;
    if (vec) {
        const unsigned grid = gdb_grid_for(count / 8U, 256, be, 8);
        if (dtype == GDB_DTYPE_F16) {
            gdb_launch(accumulate_vec8_kernel<__half>, grid, 256, 0, be->stream, (uint4 *)d, (const uint4 *)s, count / 8U);
        } else {
            gdb_launch(accumulate_vec8_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (uint4 *)d, (const uint4 *)s, count / 8U);
        }
    } else {
        const unsigned grid = gdb_grid_for(count, 256, be, 8);
        if (dtype == GDB_DTYPE_F16) {
            gdb_launch(accumulate_kernel<__half>, grid, 256, 0, be->stream, (__half *)d, (const __half *)s, count);
        } else if (dtype == GDB_DTYPE_BF16) {
            gdb_launch(accumulate_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (__nv_bfloat16 *)d, (const __nv_bfloat16 *)s, count);
        } else {
            gdb_launch(accumulate_kernel<float>, grid, 256, 0, be->stream, (float *)d, (const float *)s, count);
        }
    }
    return gdb_launched(be, "accumulate");
}

gd_status gd_backend_scale(gd_backend *be, gd_backend_buffer *dst_buffer, size_t dst_offset, gd_backend_buffer *src_buffer, size_t src_offset, size_t count, uint32_t dtype, float scale)
{
    const size_t es = gdb_dtype_size(dtype);
    if (be == NULL || !gdb_is_float_dtype(dtype) || count > SIZE_MAX / es ||
        (dst_offset % es) != 0U || (src_offset % es) != 0U ||
        !gdb_range_ok(dst_buffer, dst_offset, count * es) || !gdb_range_ok(src_buffer, src_offset, count * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    unsigned char *d = dst_buffer->dptr + dst_offset;
    const unsigned char *s = src_buffer->dptr + src_offset;
    if (scale == 1.0f) {
        // scale == 1 is a bit copy in the reference (metal_memory.metal:51).
        cudaError_t e = d == s ? cudaSuccess : cudaMemcpyAsync(d, s, count * es, cudaMemcpyDeviceToDevice, be->stream);
        be->launches += 1U;
        return e == cudaSuccess ? GD_OK : gdb_fail(be, e, "scale copy");
    }
    const unsigned grid = gdb_grid_for(count, 256, be, 8);
    if (dtype == GDB_DTYPE_F16) {
        gdb_launch(scale_kernel<__half>, grid, 256, 0, be->stream, (__half *)d, (const __half *)s, count, scale);
    } else if (dtype == GDB_DTYPE_BF16) {
        gdb_launch(scale_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (__nv_bfloat16 *)d, (const __nv_bfloat16 *)s, count, scale);
    } else {
        gdb_launch(scale_kernel<float>, grid, 256, 0, be->stream, (float *)d, (const float *)s, count, scale);
    }
    return gdb_launched(be, "scale");
}

// ---- additive helpers ----
void *gdb200_buffer_device_ptr(gd_backend_buffer *buffer, size_t offset)
{
    return gdb_range_ok(buffer, offset, 0U) ? (void *)(buffer->dptr + offset) : NULL;
}
void *gdb200_stream(gd_backend *be) { return be != NULL ? (void *)be->stream : NULL; }
int gdb200_device(const gd_backend *be) { return be != NULL ? be->device : -1; }
uint64_t gdb200_launch_count(const gd_backend *be) { return be != NULL ? be->launches : 0U; }
const char *gdb200_last_error(const gd_backend *be) { return be != NULL ? be->last_error : ""; }
int gdb200_set_gemm_mode(gd_backend *be, int mode)
{
    if (be == NULL) {
        return -1;
    }
    const int old = be->gemm_mode;
    if (mode >= 0 && mode <= 3) {
        be->gemm_mode = mode;
    }
    return old;
}

int gdb200_set_attention_mode(gd_backend *be, int mode)
{
    if (be == NULL) {
        return -1;
    }
    const int old = be->attn_mode;
    if (mode == 0 || mode == 1) {
        be->attn_mode = mode;
    }
    return old;
}

void *gdb200_event_record(gd_backend *be)
{
    cudaEvent_t ev;
    if (be == NULL) {
        return NULL;
    }
    cudaSetDevice(be->device);
    if (cudaEventCreate(&ev) != cudaSuccess) {
        return NULL;
    }
    if (cudaEventRecord(ev, be->stream) != cudaSuccess) {
        cudaEventDestroy(ev);
        return NULL;
    }
    return (void *)ev;
}
float gdb200_event_elapsed_ms(void *start, void *stop)
{
    float ms = -1.0f;
    if (start == NULL || stop == NULL || cudaEventSynchronize((cudaEvent_t)stop) != cudaSuccess ||
        cudaEventElapsedTime(&ms, (cudaEvent_t)start, (cudaEvent_t)stop) != cudaSuccess) {
        return -1.0f;
    }
    return ms;
}
void gdb200_event_destroy(void *event)
{
    if (event != NULL) {
        cudaEventDestroy((cudaEvent_t)event);
    }
}

void *gdb200_pinned_alloc(size_t nbytes)
{
    void *p = NULL;
    return (nbytes != 0U && cudaMallocHost(&p, nbytes) == cudaSuccess) ? p : NULL;
}
void gdb200_pinned_free(void *p)
{
    if (p != NULL) {
        cudaFreeHost(p);
    }
}

gd_status gdb200_flush_l2(gd_backend *be)
{
    static unsigned tag = 0;
    if (be == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    if (be->l2_flush == NULL) {
        cudaError_t e = cudaMalloc((void **)&be->l2_flush, be->l2_flush_bytes);
        if (e != cudaSuccess) {
            return gdb_fail(be, e, "l2 flush buffer");
        }
    }
    gdb_launch(l2_flush_kernel, be->sm_count * 8, 256, 0, be->stream, (uint4 *)be->l2_flush, be->l2_flush_bytes / 16U, ++tag);
    return gdb_launched(be, "flush_l2");
}

}  // extern "C"
