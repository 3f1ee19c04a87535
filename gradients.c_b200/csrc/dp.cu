// Data-parallel gradient exchange over NCCL (one process per GPU). The reference has no
// collective of any kind; these additive entries give its optimizer step the one exchange a
// batch-sharded run needs: an in-place sum all-reduce of parameter gradients, issued on a
// separate stream so it overlaps the rest of the backward pass.
#include "common.cuh"

#include <nccl.h>
#include <stdlib.h>

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
    cudaStreamSynchronize(dp->stream);
    ncclCommDestroy(dp->comm);
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
    if (id_bytes_128 == NULL || ncclGetUniqueId(&id) != ncclSuccess) {
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
    cudaSetDevice(be->device);
    gdb_dp_state *dp = (gdb_dp_state *)calloc(1, sizeof(*dp));
    if (dp == NULL) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    memcpy(&id, id_bytes_128, sizeof(id));
    dp->rank = rank;
    dp->world = world;
    if (cudaStreamCreateWithFlags(&dp->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->done, cudaEventDisableTiming) != cudaSuccess) {
        free(dp);
        return GD_ERR_INTERNAL;
    }
    ncclResult_t r = ncclCommInitRank(&dp->comm, world, id, rank);
    if (r != ncclSuccess) {
        snprintf(be->last_error, sizeof(be->last_error), "ncclCommInitRank: %s", ncclGetErrorString(r));
        cudaEventDestroy(dp->ready);
        cudaEventDestroy(dp->done);
        cudaStreamDestroy(dp->stream);
        free(dp);
        return GD_ERR_INTERNAL;
    }
    be->dp = dp;
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
    const ncclDataType_t nt = dtype == GDB_DTYPE_F16 ? ncclFloat16 : (dtype == GDB_DTYPE_BF16 ? ncclBfloat16 : ncclFloat32);
    void *p = buffer->dptr + offset;
    if (cudaEventRecord(dp->ready, be->stream) != cudaSuccess || cudaStreamWaitEvent(dp->stream, dp->ready, 0) != cudaSuccess) {
        return GD_ERR_INTERNAL;
    }
    ncclResult_t r = ncclAllReduce(p, p, count, nt, ncclSum, dp->comm, dp->stream);
    be->launches += 1U;
    if (r != ncclSuccess) {
        snprintf(be->last_error, sizeof(be->last_error), "ncclAllReduce: %s", ncclGetErrorString(r));
        return GD_ERR_INTERNAL;
    }
    return GD_OK;
}

gd_status gdb200_dp_join(gd_backend *be)
{
    if (be == NULL || be->dp == NULL) {
        return GD_ERR_BAD_STATE;
    }
    if (cudaEventRecord(be->dp->done, be->dp->stream) != cudaSuccess ||
        cudaStreamWaitEvent(be->stream, be->dp->done, 0) != cudaSuccess) {
        return GD_ERR_INTERNAL;
    }
    return GD_OK;
}

void gdb200_dp_shutdown(gd_backend *be) { gdb_dp_destroy(be); }

}  // extern "C"
