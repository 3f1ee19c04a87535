// Internal interface between the attention entry points (attention.cu) and the tensor-core
// flash kernels (attention_flash.cu).
#pragma once
#include "common.cuh"

struct gdb_flash_args {
    const void *q, *k, *v, *grad_out;
    const int *cu;
    void *out_or_dq;   // forward: out; backward: dQ
    void *dk, *dv;     // backward only
    float *stats;      // [N, Hq, 3] (row max, exp-sum, D); may be NULL in forward
    int n_tokens, batch, hq, hkv, dh;
    int causal, window, prefix, max_seqlen;
    float scale;
    uint32_t dtype;
    int keep_dq32;     // single-pass backward: leave the query gradient unrounded in the FP32 accumulator, do not write dQ
};

// Both return GD_ERR_UNSUPPORTED when the configuration is outside the fast path; the caller
// then runs the general kernels.
gd_status gdb_flash_varlen_forward(gd_backend *be, const gdb_flash_args *a);
gd_status gdb_flash_varlen_backward(gd_backend *be, const gdb_flash_args *a, bool have_forward_stats);
// Single-pass backward when the forward output is available (attention_flash.cu); dq32: FP32 scratch [N, Hq, 64].
gd_status gdb_flash_varlen_backward_with_out(gd_backend *be, const gdb_flash_args *a, const void *out, float *dq32);
// tcgen05 / tensor-memory forward (attention_tcgen05.cu); GD_ERR_UNSUPPORTED outside its fast path.
gd_status gdb_attn5_forward(gd_backend *be, const gdb_flash_args *a);
// tcgen05 / tensor-memory key-stationary backward (attention_tcgen05_bwd.cu): dK, dV and the FP32 dQ accumulator dq32
// [N, Hq, 64] (zero on entry) from complete statistics (max, sum, D) and the mask bounds `meta` (int [N + ceil(N / 128)]:
// first allowed key per query row, query tiles per key tile; written by the preparation kernel in attention_flash.cu).
// GD_ERR_UNSUPPORTED outside its fast path.
gd_status gdb_attn5_backward(gd_backend *be, const gdb_flash_args *a, float *dq32, const int *meta);
