// Embedding table gradient for callers that must not allocate device memory.
//
// gd_backend_embedding_backward needs an FP32 accumulation table [vocab, dim] and takes it from the
// caller. Some callers have nowhere to get one: a host runtime that handed every byte of device
// memory to its arenas when the context was created (so a later cudaMalloc can fail, and its heap
// guard forbids allocating while a step is being enqueued), or a foreign-function caller that only
// holds raw device pointers to its inputs and outputs. For them this file keeps the table in a
// file-scope device array of fixed size that is part of the loaded library image.
//
// Consequences of that choice, all visible to the caller:
//   * the array is resident on every GPU that loads the library until the process exits
//     (GDB200_STATIC_EMBEDDING_MAX_ELEMS floats = 4 MiB);
//   * vocab * dim beyond that maximum is refused with GD_ERR_INVALID_ARGUMENT and a message;
//   * all calls share the one array and it keeps the previous call's sums, so every call clears the
//     part it uses first; two calls whose kernels overlap on the GPU (different streams, or
//     different host threads) race on it - keep calls on one stream or order them yourself;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress);
//     make that first call outside of any stream capture.
// Nothing here calls cudaMalloc, cudaFree or any routine that allocates.
#include "common.cuh"

#define GDB200_STATIC_EMBEDDING_MAX_ELEMS (1024u * 1024u)

namespace {

static __device__ __align__(256) float g_static_table[GDB200_STATIC_EMBEDDING_MAX_ELEMS];

constexpr int MAX_DEVICES = 64;
// Device address of g_static_table, per device, filled on first use. Host threads may race on the first call for a
// device; every one of them obtains the same address from cudaGetSymbolAddress, so the duplicate stores are harmless.
float *g_table_addr[MAX_DEVICES];
thread_local char g_error[192];

template <typename T>
__global__ void static_scatter_kernel(const T *grad, const int *ids, float *acc, size_t n_ids, size_t vocab, size_t dim)
{
    gdb_pdl_sync();
    const size_t n = n_ids * dim, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t row = i / dim, c = i - row * dim;
        const int id = ids[row];
        if (id >= 0 && (size_t)id < vocab) {
            atomicAdd(&acc[(size_t)id * dim + c], gdb_io<T>::ld(grad, i));
        }
    }
}

template <typename T>
__global__ void static_cast_kernel(const float *acc, T *out, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        gdb_io<T>::st(out, i, acc[i]);
    }
}

gd_status fail(gd_status st, const char *msg)
{
    snprintf(g_error, sizeof(g_error), "%s", msg);
    return st;
}

// The array's name is only a host-side handle; kernels need the address that
// cudaGetSymbolAddress returns for the device that is current.
gd_status table_for_current_device(float **out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        return fail(GD_ERR_INTERNAL, "no current CUDA device");
    }
    if (g_table_addr[dev] == NULL) {
        void *p = NULL;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_table);
        if (e != cudaSuccess || p == NULL) {
            snprintf(g_error, sizeof(g_error), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return GD_ERR_INTERNAL;
        }
        g_table_addr[dev] = (float *)p;
    }
    *out = g_table_addr[dev];
    return GD_OK;
}

unsigned grid_for(size_t items)
{
    const size_t blocks = (items + 255U) / 256U;
    return (unsigned)(blocks > 148U * 16U ? 148U * 16U : (blocks == 0U ? 1U : blocks));
}

}  // namespace

extern "C" {

const char *gdb200_embedding_backward_static_error(void) { return g_error; }

uint64_t gdb200_embedding_backward_static_max_elems(void) { return GDB200_STATIC_EMBEDDING_MAX_ELEMS; }

// grad_table[v, :] = sum over i with ids[i] == v of grad_out[i, :], accumulated in FP32 and rounded
// once. All pointers are device pointers on the current device; `stream` is a cudaStream_t (NULL =
// default stream). dtype: 1 = F16, 2 = BF16, 3 = F32 (gd_dtype codes). Ids outside [0, vocab) are
// skipped.
gd_status gdb200_embedding_backward_static(void *stream, const void *grad_out, const int32_t *ids, void *grad_table,
                                           uint64_t ids_count, uint64_t vocab, uint64_t dim, uint32_t dtype)
{
    g_error[0] = '\0';
    if (grad_out == NULL || ids == NULL || grad_table == NULL || vocab == 0U || dim == 0U) {
        return fail(GD_ERR_INVALID_ARGUMENT, "null pointer or empty table");
    }
    if (dtype != GDB_DTYPE_F16 && dtype != GDB_DTYPE_BF16 && dtype != GDB_DTYPE_F32) {
        return fail(GD_ERR_UNSUPPORTED, "dtype must be F16, BF16 or F32");
    }
    if (vocab > GDB200_STATIC_EMBEDDING_MAX_ELEMS / dim) {
        snprintf(g_error, sizeof(g_error), "vocab * dim = %llu exceeds the static scratch of %u floats",
                 (unsigned long long)(vocab * dim), GDB200_STATIC_EMBEDDING_MAX_ELEMS);
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (ids_count > SIZE_MAX / dim) {
        return fail(GD_ERR_INVALID_ARGUMENT, "ids_count * dim overflows size_t");
    }
    float *table = NULL;
    gd_status st = table_for_current_device(&table);
    if (st != GD_OK) {
        return st;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)(vocab * dim);
    // the array still holds the previous call's sums
    cudaError_t e = cudaMemsetAsync(table, 0, total * sizeof(float), s);
    if (e != cudaSuccess) {
        return fail(GD_ERR_INTERNAL, cudaGetErrorString(e));
    }
    if (ids_count != 0U) {
        const size_t items = (size_t)(ids_count * dim);
        if (dtype == GDB_DTYPE_F16) {
            gdb_launch(static_scatter_kernel<__half>, grid_for(items), 256, 0, s, (const __half *)grad_out, ids, table, ids_count, vocab, dim);
        } else if (dtype == GDB_DTYPE_BF16) {
            gdb_launch(static_scatter_kernel<__nv_bfloat16>, grid_for(items), 256, 0, s, (const __nv_bfloat16 *)grad_out, ids, table, ids_count, vocab, dim);
        } else {
            gdb_launch(static_scatter_kernel<float>, grid_for(items), 256, 0, s, (const float *)grad_out, ids, table, ids_count, vocab, dim);
        }
    }
    if (dtype == GDB_DTYPE_F16) {
        gdb_launch(static_cast_kernel<__half>, grid_for(total), 256, 0, s, table, (__half *)grad_table, total);
    } else if (dtype == GDB_DTYPE_BF16) {
        gdb_launch(static_cast_kernel<__nv_bfloat16>, grid_for(total), 256, 0, s, table, (__nv_bfloat16 *)grad_table, total);
    } else {
        gdb_launch(static_cast_kernel<float>, grid_for(total), 256, 0, s, table, (float *)grad_table, total);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        return fail(GD_ERR_INTERNAL, cudaGetErrorString(e));
    }
    return GD_OK;
}

}  // extern "C"
