// Tensor-core flash attention for packed variable-length sequences (placeholder dispatch:
// every configuration is currently routed to the general kernels).
#include "attention.cuh"

gd_status gdb_flash_varlen_forward(gd_backend *be, const gdb_flash_args *a)
{
    (void)be;
    (void)a;
    return GD_ERR_UNSUPPORTED;
}

gd_status gdb_flash_varlen_backward(gd_backend *be, const gdb_flash_args *a, bool have_forward_stats)
{
    (void)be;
    (void)a;
    (void)have_forward_stats;
    return GD_ERR_UNSUPPORTED;
}
