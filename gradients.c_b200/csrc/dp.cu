// Data-parallel gradient exchange over NCCL (one process per GPU). The reference has no
// collective of any kind; these additive entries give its optimizer step the one exchange a
// batch-sharded run needs: an in-place sum all-reduce of parameter gradients, issued on a
// separate stream so it overlaps the rest of the backward pass.
//
// NCCL is bound at run time with dlopen("libnccl.so.2") on the first call, not at link time:
// a process that has already loaded an NCCL (for instance through PyTorch) keeps using that
// one copy, and single-GPU users of the backend carry no NCCL dependency at all.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>
#include <sched.h>
#include <stdlib.h>
#include <time.h>

namespace {

struct nccl_api {
    void *handle;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    const char *(*GetErrorString)(ncclResult_t);
    ncclResult_t (*GroupStart)(void);
    ncclResult_t (*GroupEnd)(void);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *);   // optional
};

nccl_api *load_nccl(void)
{
    static nccl_api api;
    static bool tried = false;
    if (tried) {
        return api.handle != NULL ? &api : NULL;
    }
    tried = true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle != NULL) {
            break;
        }
    }
    if (api.handle == NULL) {
        return NULL;
    }
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
    api.CommInitRankConfig = (decltype(api.CommInitRankConfig))dlsym(api.handle, "ncclCommInitRankConfig");   // optional
    api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
    api.GroupStart = (decltype(api.GroupStart))dlsym(api.handle, "ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))dlsym(api.handle, "ncclGroupEnd");
    api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(api.handle, "ncclCommGetAsyncError");   // optional
    if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy || !api.GetErrorString ||
        !api.GroupStart || !api.GroupEnd) {
        api.handle = NULL;
        return NULL;
    }
    return &api;
}

}  // namespace

struct gdb_dp_state {
    ncclComm_t comm;
    cudaStream_t stream;
    cudaEvent_t ready;  // compute -> comm dependency
    cudaEvent_t done;   // comm -> compute dependency
    int rank, world;
};

void gdb_dp_destroy(gd_backend *be)
{
    if (be == NULL || be->dp == NULL) {
        return;
    }
    gdb_dp_state *dp = be->dp;
    nccl_api *api = load_nccl();
    cudaStreamSynchronize(dp->stream);
    if (api != NULL) {
        api->CommDestroy(dp->comm);
    }
    cudaEventDestroy(dp->ready);
    cudaEventDestroy(dp->done);
    cudaStreamDestroy(dp->stream);
    free(dp);
    be->dp = NULL;
}

extern "C" {

gd_status gdb200_dp_unique_id(void *id_bytes_128)
{
    ncclUniqueId id;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    nccl_api *api = load_nccl();
    if (api == NULL) {
        return GD_ERR_UNSUPPORTED;
    }
    if (id_bytes_128 == NULL || api->GetUniqueId(&id) != ncclSuccess) {
        return GD_ERR_INTERNAL;
    }
    memcpy(id_bytes_128, &id, sizeof(id));
    return GD_OK;
}

gd_status gdb200_dp_init(gd_backend *be, const void *id_bytes_128, int rank, int world)
{
    ncclUniqueId id;
    if (be == NULL || id_bytes_128 == NULL || world < 1 || rank < 0 || rank >= world || be->dp != NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    nccl_api *api = load_nccl();
    if (api == NULL) {
        snprintf(be->last_error, sizeof(be->last_error), "libnccl.so.2 could not be loaded: %s", dlerror());
        return GD_ERR_UNSUPPORTED;
    }
    cudaSetDevice(be->device);
    gdb_dp_state *dp = (gdb_dp_state *)calloc(1, sizeof(*dp));
    if (dp == NULL) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    memcpy(&id, id_bytes_128, sizeof(id));
    dp->rank = rank;
    dp->world = world;
    // the collective runs on a stream of the highest priority, so that its few CTAs are placed as soon as any
    // compute CTA retires instead of queueing behind the persistent kernels of the backward pass
    int prio_lo = 0, prio_hi = 0;
    cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
    if (cudaStreamCreateWithPriority(&dp->stream, cudaStreamNonBlocking, prio_hi) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->done, cudaEventDisableTiming) != cudaSuccess) {
        free(dp);
        return GD_ERR_INTERNAL;
    }
    // The exchange overlaps the backward pass, whose persistent GEMM and attention kernels want every SM;
    // GDB200_DP_MAX_CTAS > 0 caps the CTAs of the collective (default 0 = NCCL's own choice: at two ranks a cap
    // of 2 / 4 / 8 measured 4.68 / 4.48 / 4.40 ms per step against 4.35 ms uncapped).
    int max_ctas = 0;
    const char *env = getenv("GDB200_DP_MAX_CTAS");
    if (env != NULL && env[0] != '\0') {
        max_ctas = atoi(env);
    }
    ncclResult_t r;
    if (api->CommInitRankConfig != NULL && max_ctas > 0) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.minCTAs = 1;
        cfg.maxCTAs = max_ctas;
        r = api->CommInitRankConfig(&dp->comm, world, id, rank, &cfg);
    } else {
        r = api->CommInitRank(&dp->comm, world, id, rank);
    }
    if (r != ncclSuccess) {
        snprintf(be->last_error, sizeof(be->last_error), "ncclCommInitRank: %s", api->GetErrorString(r));
        cudaEventDestroy(dp->ready);
        cudaEventDestroy(dp->done);
        cudaStreamDestroy(dp->stream);
        free(dp);
        return GD_ERR_INTERNAL;
    }
    be->dp = dp;
    // GDB200_DP_RESERVE_SMS: SMs that the persistent GEMM / attention kernels leave free while a communicator exists,
    // so that a collective running beside the backward pass cannot push part of a persistent grid into a second wave
    const char *rs = getenv("GDB200_DP_RESERVE_SMS");
    be->sm_reserve = rs != NULL ? atoi(rs) : 0;
    if (be->sm_reserve < 0 || be->sm_reserve > be->sm_count / 2) be->sm_reserve = 0;
    return GD_OK;
}

gd_status gdb200_dp_all_reduce(gd_backend *be, gd_backend_buffer *buffer, size_t offset, size_t count, uint32_t dtype)
{
    if (be == NULL || be->dp == NULL) {
        return GD_ERR_BAD_STATE;
    }
    const size_t es = gdb_dtype_size(dtype);
    if (!gdb_is_float_dtype(dtype) || !gdb_range_ok(buffer, offset, count * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    gdb_dp_state *dp = be->dp;
    nccl_api *api = load_nccl();
    const ncclDataType_t nt = dtype == GDB_DTYPE_F16 ? ncclFloat16 : (dtype == GDB_DTYPE_BF16 ? ncclBfloat16 : ncclFloat32);
    void *p = buffer->dptr + offset;
    if (cudaEventRecord(dp->ready, be->stream) != cudaSuccess || cudaStreamWaitEvent(dp->stream, dp->ready, 0) != cudaSuccess) {
        return GD_ERR_INTERNAL;
    }
    ncclResult_t r = api->AllReduce(p, p, count, nt, ncclSum, dp->comm, dp->stream);
    be->launches += 1U;
    if (r != ncclSuccess) {
        snprintf(be->last_error, sizeof(be->last_error), "ncclAllReduce: %s", api->GetErrorString(r));
        return GD_ERR_INTERNAL;
    }
    return GD_OK;
}

// Host-side wait shared by gdb200_dp_join and its CPU test: polls `completed` (1 = the awaited work is done) and
// `failed` (non-zero = the communicator reports an asynchronous error) until one of them answers or timeout_ms runs out.
// Returns GD_OK, or GD_ERR_INTERNAL with *reason = 1 (error reported) / 2 (timeout). The callbacks carry no CUDA types,
// so the loop can be driven by stubs on a machine without a GPU.
gd_status gdb200_dp_wait_with(int (*completed)(void *), int (*failed)(void *), void *user, uint32_t timeout_ms, int32_t *reason)
{
    if (reason != NULL) *reason = 0;
    if (completed == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    struct timespec t0, t;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        if (failed != NULL && failed(user) != 0) {
            if (reason != NULL) *reason = 1;
            return GD_ERR_INTERNAL;
        }
        if (completed(user) != 0) {
            return GD_OK;
        }
        clock_gettime(CLOCK_MONOTONIC, &t);
        const double ms = (double)(t.tv_sec - t0.tv_sec) * 1.0e3 + (double)(t.tv_nsec - t0.tv_nsec) * 1.0e-6;
        if (ms >= (double)timeout_ms) {
            if (reason != NULL) *reason = 2;
            return GD_ERR_INTERNAL;
        }
        sched_yield();
    }
}

namespace {
int dp_done_query(void *user)
{
    gd_backend *be = (gd_backend *)user;
    return cudaEventQuery(be->dp->done) == cudaSuccess ? 1 : 0;
}
int dp_async_error(void *user)
{
    gd_backend *be = (gd_backend *)user;
    nccl_api *api = load_nccl();
    ncclResult_t async = ncclSuccess;
    if (api == NULL || api->CommGetAsyncError == NULL) return 0;
    if (api->CommGetAsyncError(be->dp->comm, &async) != ncclSuccess) return 1;
    return (async != ncclSuccess && async != ncclInProgress) ? 1 : 0;
}
}  // namespace

// Makes the compute stream wait for all outstanding all-reduces. The communicator's asynchronous error state is
// polled on every call (a failed or aborted collective then surfaces here as GD_ERR_INTERNAL instead of as a hang at the
// next synchronisation); with GDB200_DP_TIMEOUT_MS > 0 the host also waits, at most that long, for the collectives
// themselves, so that a peer that never joins ends this rank's step with an error.
gd_status gdb200_dp_join(gd_backend *be)
{
    if (be == NULL || be->dp == NULL) {
        return GD_ERR_BAD_STATE;
    }
    if (cudaEventRecord(be->dp->done, be->dp->stream) != cudaSuccess ||
        cudaStreamWaitEvent(be->stream, be->dp->done, 0) != cudaSuccess) {
        return GD_ERR_INTERNAL;
    }
    if (dp_async_error(be) != 0) {
        snprintf(be->last_error, sizeof(be->last_error), "NCCL communicator reports an asynchronous error");
        return GD_ERR_INTERNAL;
    }
    static int timeout_ms = -1;
    if (timeout_ms < 0) {
        const char *env = getenv("GDB200_DP_TIMEOUT_MS");
        timeout_ms = env != NULL ? atoi(env) : 0;
        if (timeout_ms < 0) timeout_ms = 0;
    }
    if (timeout_ms > 0) {
        int32_t reason = 0;
        const gd_status st = gdb200_dp_wait_with(dp_done_query, dp_async_error, be, (uint32_t)timeout_ms, &reason);
        if (st != GD_OK) {
            snprintf(be->last_error, sizeof(be->last_error), reason == 2 ? "data-parallel exchange did not complete within %d ms"
                                                                          : "NCCL communicator reports an asynchronous error (after %d ms limit armed)", timeout_ms);
            return st;
        }
    }
    return GD_OK;
}

void gdb200_dp_shutdown(gd_backend *be) { gdb_dp_destroy(be); }

}  // extern "C"
