// Shared definitions of the B200 backend: the opaque backend/buffer structs, view -> device
// pointer resolution with byte-range checks (the CUDA counterpart of
// gd_metal_byte_range_valid, reference src/backends/metal/backend_metal.m:340-352), storage
// dtype conversion helpers and launch bookkeeping.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdio.h>
#ifdef __cplusplus
#include <utility>
#endif

#include "../../include/gd_backend_b200.h"

#define GDB_SM_COUNT_DEFAULT 148
// gd_backend::err_flag points at GDB_FLAG_BYTES of zeroed device words: word 0 is the error code of
// bounded waits; words 64.. are arrival tickets of multi-block reductions (each user leaves them zero).
#define GDB_FLAG_BYTES 16384
#define GDB_TICKET_WORDS ((GDB_FLAG_BYTES / 4) - 64)

struct gdb_tmap_cache;  // tcgen05 GEMM tensor-map cache (gemm_tcgen05.cu)
struct gdb_dp_state;    // NCCL state (dp.cu)

struct gd_backend {
    int device;
    int sm_count;
    cudaStream_t stream;
    uint64_t launches;
    int gemm_mode;            // 0 auto, 1 portable, 2 tcgen05 required, 3 auto without the CTA-pair kernel
    int attn_mode;            // 0 auto (tcgen05 attention when the shape allows), 1 mma.sync flash kernels only
    int sm_reserve;           // SMs the persistent kernels leave free (for a concurrent collective); 0 = none
    char last_error[256];
    // private workspace (split-K partials, reductions, attention scratch); created once at
    // create_default so no allocation happens while a step is being enqueued.
    unsigned char *ws;
    size_t ws_bytes;
    int *err_flag;            // device int: set by kernels whose bounded waits gave up
    int *err_flag_host;       // pinned mirror
    float *rope_table;        // cos/sin table [512][32][2] for head_dim 64, theta 10000
    unsigned char *l2_flush;  // >L2 scratch for gdb200_flush_l2
    size_t l2_flush_bytes;
    gdb_tmap_cache *tmaps;
    gdb_dp_state *dp;
    // scratch offsets of the parameter gradients of the last gdb200_gpt_train_step (valid until the arena is reused)
    int32_t last_grad_count;
    size_t last_grad_offset[GDB200_GPT_MAX_PARAMS];
};

enum { GDB_BUF_DEVICE = 0, GDB_BUF_MANAGED = 1 };

struct gd_backend_buffer {
    gd_backend *backend;
    unsigned char *dptr;   // device address (equals hptr for managed buffers)
    void *hptr;            // address reported by gd_backend_buffer_host_ptr
    size_t nbytes;
    size_t reserve_bytes;  // size of the host address reservation when kind == DEVICE
    int kind;
};

static inline unsigned *gdb_tickets(const struct gd_backend *be) { return (unsigned *)be->err_flag + 64; }

static inline gd_status gdb_fail(gd_backend *be, cudaError_t e, const char *what)
{
    if (be != NULL) {
        snprintf(be->last_error, sizeof(be->last_error), "%s: %s", what, cudaGetErrorString(e));
    }
    return e == cudaErrorMemoryAllocation ? GD_ERR_OUT_OF_MEMORY : GD_ERR_INTERNAL;
}

// Check the launch that was just issued; counts it.
static inline gd_status gdb_launched(gd_backend *be, const char *what)
{
    cudaError_t e = cudaGetLastError();
    be->launches += 1U;
    if (e != cudaSuccess) {
        return gdb_fail(be, e, what);
    }
    return GD_OK;
}

static inline size_t gdb_dtype_size(uint32_t dtype)
{
    switch (dtype) {
    case GDB_DTYPE_F16: case GDB_DTYPE_BF16: case GDB_DTYPE_U16: return 2U;
    case GDB_DTYPE_F32: case GDB_DTYPE_I32: return 4U;
    case GDB_DTYPE_U8: return 1U;
    default: return 0U;
    }
}

static inline bool gdb_range_ok(const gd_backend_buffer *b, size_t offset, size_t nbytes)
{
    return b != NULL && b->dptr != NULL && offset <= b->nbytes && nbytes <= b->nbytes - offset;
}

// Resolve a contiguous tensor view to a device pointer; NULL when the view is invalid.
static inline void *gdb_tv_ptr(const gd_backend_tensor_view *v, uint32_t dtype)
{
    size_t es;
    if (v == NULL || v->buffer == NULL || v->dtype != dtype) {
        return NULL;
    }
    es = gdb_dtype_size(dtype);
    if (es == 0U || v->count > SIZE_MAX / es || !gdb_range_ok(v->buffer, v->offset, v->count * es)) {
        return NULL;
    }
    if ((v->offset % es) != 0U) {
        return NULL;
    }
    return v->buffer->dptr + v->offset;
}

static inline void *gdb_raw_ptr(gd_backend_buffer *b, size_t offset, size_t nbytes)
{
    return gdb_range_ok(b, offset, nbytes) ? (void *)(b->dptr + offset) : NULL;
}

static inline bool gdb_same_shape(const gd_backend_tensor_view *a, const gd_backend_tensor_view *b)
{
    if (a->rank != b->rank || a->count != b->count || a->rank > 8U) {
        return false;
    }
    for (uint32_t i = 0; i < a->rank; ++i) {
        if (a->shape[i] != b->shape[i]) {
            return false;
        }
    }
    return true;
}

static inline bool gdb_is_float_dtype(uint32_t dt)
{
    return dt == GDB_DTYPE_F16 || dt == GDB_DTYPE_BF16 || dt == GDB_DTYPE_F32;
}

static inline unsigned gdb_grid_for(size_t work_items, unsigned threads, const gd_backend *be, unsigned waves)
{
    size_t blocks = (work_items + threads - 1U) / threads;
    size_t cap = (size_t)(be != NULL && be->sm_count > 0 ? be->sm_count : GDB_SM_COUNT_DEFAULT) * waves;
    if (blocks > cap) {
        blocks = cap;
    }
    return blocks == 0U ? 1U : (unsigned)blocks;
}

#ifdef __CUDACC__
// ---- programmatic dependent launch ----
// Every kernel of the backend is launched with programmatic stream serialization and starts with
// gdb_pdl_sync(): it waits until the preceding kernel of the stream has completed and its writes are
// visible, then allows the following kernel to be scheduled, so launch latency and block scheduling of
// kernel N + 1 overlap the execution of kernel N instead of following it. Stream order is unchanged.
__device__ __forceinline__ void gdb_pdl_sync()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static inline cudaError_t gdb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- storage <-> float conversion ----
// Sigmoid of the SwiGLU gate, one definition for the stand-alone kernels and the fused GEMM epilogue
// (stable form of src/ops/swiglu/metal_swiglu.metal: exp of a non-positive argument only).
__device__ __forceinline__ float gdb_swiglu_sigmoid(float x)
{
    const float e = __expf(-fabsf(x));
    const float inv = __fdividef(1.0f, 1.0f + e);   // 1 + e lies in [1, 2]: the approximate reciprocal is good to 1-2 ulp there
    return x >= 0.0f ? inv : e * inv;
}

template <typename T> struct gdb_io;
template <> struct gdb_io<__half> {
    static __device__ __forceinline__ float ld(const __half *p, size_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ void st(__half *p, size_t i, float v) { p[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float rnd(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ float up(unsigned short bits) { return __half2float(__ushort_as_half(bits)); }
    static __device__ __forceinline__ unsigned short down(float v) { return __half_as_ushort(__float2half_rn(v)); }
};
template <> struct gdb_io<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p, size_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void st(__nv_bfloat16 *p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ float up(unsigned short bits) { return __uint_as_float(((unsigned)bits) << 16); }
    static __device__ __forceinline__ unsigned short down(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
};
template <> struct gdb_io<float> {
    static __device__ __forceinline__ float ld(const float *p, size_t i) { return p[i]; }
    static __device__ __forceinline__ void st(float *p, size_t i, float v) { p[i] = v; }
    static __device__ __forceinline__ float rnd(float v) { return v; }
};

// 8 x 16-bit values held in one 16-byte vector.
template <typename T> struct gdb_vec8 {
    uint4 raw;
    __device__ __forceinline__ float get(int i) const
    {
        const unsigned w = (&raw.x)[i >> 1];
        return gdb_io<T>::up((unsigned short)((i & 1) ? (w >> 16) : (w & 0xffffU)));
    }
    __device__ __forceinline__ void set(int i, float v)
    {
        unsigned *w = &(&raw.x)[i >> 1];
        const unsigned b = gdb_io<T>::down(v);
        *w = (i & 1) ? ((*w & 0x0000ffffU) | (b << 16)) : ((*w & 0xffff0000U) | b);
    }
};

__device__ __forceinline__ float gdb_warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffU, v, o);
    }
    return v;
}
__device__ __forceinline__ float gdb_warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffU, v, o));
    }
    return v;
}
// Block-wide sum for blocks of up to 1024 threads; `sh` must hold 33 floats.
__device__ __forceinline__ float gdb_block_sum(float v, float *sh)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = gdb_warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? sh[lane] : 0.0f;
        t = gdb_warp_sum(t);
        if (lane == 0) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}
__device__ __forceinline__ float gdb_block_max(float v, float *sh)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = gdb_warp_max(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? sh[lane] : -3.402823466e38f;
        t = gdb_warp_max(t);
        if (lane == 0) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}

__device__ __forceinline__ uint64_t gdb_splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}

// Dropout decision of element `index` (src/ops/dropout/metal_dropout.metal: 24 bits of splitmix64(seed + index) against a
// threshold of ceil(p * 2^24)); one definition for the stand-alone kernels and the fused residual + norm kernel.
__device__ __forceinline__ bool gdb_dropout_keep(uint64_t seed, uint64_t index, unsigned threshold)
{
    const uint64_t r = gdb_splitmix64(seed + index);
    return (unsigned)((r >> 40) & 0xffffffULL) >= threshold;
}
static inline unsigned gdb_dropout_threshold(float p)
{
    const double t = ceil((double)p * 16777216.0);
    if (t <= 0.0) {
        return 0U;
    }
    if (t >= 16777216.0) {
        return 16777216U;
    }
    return (unsigned)t;
}
#endif  // __CUDACC__

// ---- entry points implemented in other translation units and shared internally ----
gd_status gdb_gemm_dispatch(gd_backend *be, int ta, int tb,
                            const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                            const gd_backend_vector_view *bias, const gd_backend_matrix_view *y, int bias_mode = 1);
// tcgen05 path: returns GD_ERR_UNSUPPORTED when the shape/alignment cannot use it.
gd_status gdb_gemm_tcgen05(gd_backend *be, int ta, int tb, uint32_t dtype,
                           const void *a, size_t lda_bytes, const void *b, size_t ldb_bytes,
                           void *c, size_t ldc_bytes, const void *bias, int bias_mode,
                           uint32_t M, uint32_t N, uint32_t K);
// `batch` equal-shaped contractions in one launch (byte pitches between batch elements; 0 broadcasts the operand).
gd_status gdb_gemm_tcgen05_batched(gd_backend *be, int ta, int tb, uint32_t dtype, const void *a, size_t lda_bytes, size_t a_batch_bytes,
                                   const void *b, size_t ldb_bytes, size_t b_batch_bytes, void *c, size_t ldc_bytes, size_t c_batch_bytes,
                                   uint32_t M, uint32_t N, uint32_t K, uint32_t batch);
// At most 64 output rows (decode): mma.sync kernel with K split over the warps of a CTA.
// sum = residual + dropout(x) (mask written), out = rms_norm(sum, weight), inv_rms saved: gd_backend_dropout_add_forward followed by
// gd_backend_rms_norm_forward_stats in one launch, same rounding points. GD_ERR_UNSUPPORTED when the vector path does not apply.
gd_status gdb_dropout_add_rms_norm(gd_backend *be, const gd_backend_tensor_view *residual, const gd_backend_tensor_view *x,
                                   const gd_backend_tensor_view *weight, const gd_backend_tensor_view *sum, const gd_backend_tensor_view *mask,
                                   const gd_backend_tensor_view *out, const gd_backend_tensor_view *inv, size_t rows, size_t cols, float eps,
                                   float p, uint64_t seed);
// sum = dropout(embedding(table, ids)) (mask written), out = rms_norm(sum, weight), inv_rms saved: gd_backend_embedding_forward,
// gd_backend_dropout_forward and gd_backend_rms_norm_forward_stats in one launch. GD_ERR_UNSUPPORTED when the vector path does not apply.
gd_status gdb_embedding_dropout_rms_norm(gd_backend *be, const gd_backend_tensor_view *table, const gd_backend_tensor_view *ids,
                                         const gd_backend_tensor_view *weight, const gd_backend_tensor_view *sum, const gd_backend_tensor_view *mask,
                                         const gd_backend_tensor_view *out, const gd_backend_tensor_view *inv, size_t rows, size_t cols, size_t vocab,
                                         float eps, float p, uint64_t seed);
// Loss normaliser of a data-parallel step: counts F32 [2] = {valid target rows of the global batch, of this rank's shard}.
// gdb_lm_ce_count_valid writes the local count into both; the caller sums element 0 over the ranks before
// gdb_lm_ce_reduce_normalize_global divides by it (the reference's kernel, src/ops/lm_cross_entropy/metal_lm_cross_entropy.metal:244-252,
// divides by the local count because it knows one device only).
gd_status gdb_lm_ce_count_valid(gd_backend *be, const gd_backend_tensor_view *targets, int32_t ignore_index, const gd_backend_tensor_view *counts);
gd_status gdb_lm_ce_reduce_normalize_global(gd_backend *be, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *counts,
                                            const gd_backend_tensor_view *loss, const gd_backend_tensor_view *inv_valid_count);
gd_status gdb_rms_norm_backward_with_weight(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                            const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                            const gd_backend_tensor_view *grad_x, bool add_to_dx, const gd_backend_tensor_view *grad_weight,
                                            const gd_backend_tensor_view *partial, const gd_backend_rms_norm_args *args,
                                            const gd_backend_tensor_view *mask, const gd_backend_tensor_view *masked, float mask_scale,
                                            const gd_backend_tensor_view *masked_colsum);
gd_status gdb_rms_norm_backward_accumulate(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                           const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                           const gd_backend_tensor_view *grad_accum, const gd_backend_rms_norm_args *args);
gd_status gdb_gemm_skinny_swiglu(gd_backend *be, uint32_t dtype, const void *a, size_t lda_bytes, const void *w, size_t ldw_bytes,
                                 const void *bias, void *c, size_t ldc_bytes, uint32_t M, uint32_t N, uint32_t K);
gd_status gdb_gemm_skinny(gd_backend *be, int tb, uint32_t dtype, const void *a, size_t lda_bytes, const void *b, size_t ldb_bytes,
                          void *c, size_t ldc_bytes, const void *bias, int bias_mode, uint32_t M, uint32_t N, uint32_t K);
// up / gate projection with the SwiGLU gate in the epilogue of the CTA-pair kernel: x12 [M, 2F] and act [M, F] from one contraction.
gd_status gdb_gemm_tcgen05_pair_swiglu(gd_backend *be, uint32_t dtype, const void *x, size_t ldx_bytes, const void *w, size_t ldw_bytes,
                                       const void *bias, void *x12, size_t ld12_bytes, void *act, size_t ldact_bytes, uint32_t M, uint32_t F,
                                       uint32_t K);
// input gradient of the down projection with the SwiGLU backward in the epilogue: d_x12 [M, 2F] from g [M, K], w [F, K], x12 [M, 2F]
gd_status gdb_gemm_tcgen05_pair_swiglu_bwd(gd_backend *be, uint32_t dtype, const void *g, size_t ldg_bytes, const void *w, size_t ldw_bytes,
                                           const void *x12, size_t ld12_bytes, void *d_x12, size_t ldd_bytes, uint32_t M, uint32_t F, uint32_t K);
// CTA-pair persistent variant; *splits_out > 1 means FP32 partials were left in the workspace.
gd_status gdb_gemm_tcgen05_pair(gd_backend *be, int ta, int tb, uint32_t dtype,
                                const void *a, size_t lda_bytes, const void *b, size_t ldb_bytes,
                                void *c, size_t ldc_bytes, const void *bias, int bias_mode,
                                uint32_t M, uint32_t N, uint32_t K, uint32_t *splits_out, float **colsum_partial_out = nullptr);
// C[M, N] = A^T B with A stored [K, M], B stored [K, N], and colsum[m] = sum_k A[k, m] from the same pass over A
// (weight gradient + bias gradient of a linear layer). GD_ERR_UNSUPPORTED when the CTA-pair kernel does not apply.
gd_status gdb_gemm_tcgen05_tn_colsum(gd_backend *be, uint32_t dtype, const void *a, size_t lda_bytes, const void *b, size_t ldb_bytes,
                                     void *c, size_t ldc_bytes, void *colsum, uint32_t M, uint32_t N, uint32_t K);
// Fusions used by the native decode driver (GD_ERR_UNSUPPORTED when their vector paths do not apply).
gd_status gdb_add_rms_norm(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *weight,
                           const gd_backend_tensor_view *sum, const gd_backend_tensor_view *out, size_t rows, size_t cols, float eps);
gd_status gdb_qkv_rope_append(gd_backend *be, const gd_backend_tensor_view *qkv, const gd_backend_tensor_view *pos_ids,
                              const gd_backend_tensor_view *q, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache,
                              uint32_t n_heads, uint32_t head_dim, uint32_t tmax, const gd_backend_rope_args *args);
void gdb_tmap_cache_destroy(gd_backend *be);
void gdb_dp_destroy(gd_backend *be);
