// Failure-detection checks that fault nothing: the path by which a device-side give-up reaches the host.
//
// Every wait in the kernels of this backend (on an mbarrier, a ticket or a flag) is bounded; when the limit runs out the
// kernel stores a code in the backend's device error word and returns normally, and gd_backend_flush / fence_wait turn
// the word into GD_ERR_INTERNAL (the reference maps a failed Metal command buffer to GD_ERR_INTERNAL at flush in the same
// way, src/backends/metal/backend_metal.m:569-573). The two entries here let a test drive that path on purpose:
//   gdb200_inject_device_error     stores a code in the error word in stream order (a host-injected failure)
//   gdb200_selftest_bounded_wait   runs a one-warp kernel that waits, with a caller-chosen iteration limit, on an mbarrier
//                                  nobody ever arrives at, stores code 399 when the limit runs out and returns
// Neither traps, spins without bound or touches memory it does not own; the CUDA context stays usable.
#include "tcgen05.cuh"

namespace {

__global__ void inject_error_kernel(int *err_flag, int code)
{
    gdb_pdl_sync();
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(err_flag, code);
}

__global__ void bounded_wait_kernel(int *err_flag, unsigned max_iters, unsigned *iters_out)
{
    gdb_pdl_sync();
    __shared__ uint64_t bar;
    const uint32_t b = gdb_t5::smem_u32(&bar);
    if (threadIdx.x == 0) {
        gdb_t5::mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the same polling instruction as gdb_t5::mbar_wait, with the caller's limit instead of the production one
    unsigned it = 0;
    bool done = false;
    for (; it < max_iters && !done; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(b), "r"(0U)
            : "memory");
        done = ok != 0U;
    }
    if (threadIdx.x == 0) {
        if (!done) atomicExch(err_flag, 399);
        if (iters_out != nullptr) *iters_out = it;
    }
}

}  // namespace

extern "C" {

gd_status gdb200_inject_device_error(gd_backend *be, int32_t code)
{
    if (be == NULL || code == 0) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    gdb_launch(inject_error_kernel, 1, 32, 0, be->stream, be->err_flag, (int)code);
    return gdb_launched(be, "inject_device_error");
}

gd_status gdb200_selftest_bounded_wait(gd_backend *be, uint32_t max_iters)
{
    if (be == NULL || max_iters == 0U || max_iters > (1U << 20)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    gdb_launch(bounded_wait_kernel, 1, 32, 0, be->stream, be->err_flag, (unsigned)max_iters, (unsigned *)nullptr);
    return gdb_launched(be, "selftest_bounded_wait");
}

}  // extern "C"
