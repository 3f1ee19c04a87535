// Dense contraction entry points (matmul / matmul_nt / matmul_tn / linear / batched variants /
// reduce_rows) and the portable tiled kernel used for shapes the tcgen05 path cannot take
// (ragged sizes, strides that are not 16-byte multiples, F32 operands).
//
// Reference semantics: src/core/backend.h:187-223; F16 storage with FP32 accumulation and one
// rounding at the store; gd_backend_linear adds the bias in FP32 before that rounding
// (src/ops/_shared/gemm/metal_gemm_common.h:124-133); reduce_rows accumulates in FP32 and
// rounds once (src/ops/linear/metal_linear.metal:33-52).
#include "common.cuh"
#include "colreduce.cuh"

// Optional per-launch timing of the dense contractions (benchmark instrumentation): when enabled,
// every dispatch is bracketed by a CUDA event pair on the backend stream and its algorithmic
// FLOPs and bytes are accumulated; gdb200_gemm_profile_read sums the elapsed times.
struct gdb_gemm_profile {
    static constexpr int CAP = 8192;
    cudaEvent_t start[CAP], stop[CAP];
    int created, used;
    double flops, bytes;
    bool enabled;
};
static gdb_gemm_profile *g_profile = nullptr;

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

// C[m, n] = sum_k A(m, k) * B(k, n) (+ bias[n]); A(m,k) = a[m*sam + k*sak], B(k,n) = b[k*sbk + n*sbn]
// (element strides), C row-major with leading dimension ldc. 256 threads, 4x4 outputs each.
template <typename T>
__global__ void gemm_portable_kernel(const T *__restrict__ a, size_t sam, size_t sak,
                                     const T *__restrict__ b, size_t sbk, size_t sbn,
                                     T *__restrict__ c, size_t ldc, const T *__restrict__ bias,
                                     unsigned M, unsigned N, unsigned K,
                                     size_t batch_a, size_t batch_b, size_t batch_c, int bias_mode)
{
    gdb_pdl_sync();
    __shared__ float as[TK][TM + 4];
    __shared__ float bs[TK][TN + 4];
    a += (size_t)blockIdx.z * batch_a;
    b += (size_t)blockIdx.z * batch_b;
    c += (size_t)blockIdx.z * batch_c;
    const unsigned m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const unsigned tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (unsigned k0 = 0; k0 < K; k0 += TK) {
        // A tile: TM x TK = 1024 elements, 4 per thread. Pick the loop order that walks the
        // unit-stride dimension fastest across adjacent threads.
        for (unsigned e = threadIdx.x; e < TM * TK; e += 256) {
            unsigned mm, kk;
            if (sak == 1) {
                kk = e % TK;
                mm = e / TK;
            } else {
                mm = e % TM;
                kk = e / TM;
            }
            const unsigned gm = m0 + mm, gk = k0 + kk;
            as[kk][mm] = (gm < M && gk < K) ? gdb_io<T>::ld(a, (size_t)gm * sam + (size_t)gk * sak) : 0.0f;
        }
        for (unsigned e = threadIdx.x; e < TN * TK; e += 256) {
            unsigned nn, kk;
            if (sbk == 1) {
                kk = e % TK;
                nn = e / TK;
            } else {
                nn = e % TN;
                kk = e / TN;
            }
            const unsigned gn = n0 + nn, gk = k0 + kk;
            bs[kk][nn] = (gn < N && gk < K) ? gdb_io<T>::ld(b, (size_t)gk * sbk + (size_t)gn * sbn) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = as[kk][ty * 4 + i];
                bv[i] = bs[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned gm = m0 + ty * 4 + i;
        if (gm >= M) {
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned gn = n0 + tx * 4 + j;
            if (gn < N) {
                float val = acc[i][j];
                if (bias != nullptr) {
                    if (bias_mode == 2) val = gdb_io<T>::rnd(val);
                    val += gdb_io<T>::ld(bias, gn);
                }
                gdb_io<T>::st(c, (size_t)gm * ldc + gn, val);
            }
        }
    }
}

// reduce_rows stage 1: block (cb, rb) sums its row chunk for 256 columns into ws[rb, c].
template <typename T>
__global__ void reduce_rows_stage_kernel(const T *x, size_t ld, float *partial, size_t rows, size_t cols, size_t chunk)
{
    gdb_pdl_sync();
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t r0 = (size_t)blockIdx.y * chunk;
    size_t r1 = r0 + chunk;
    if (r1 > rows) {
        r1 = rows;
    }
    if (c >= cols) {
        return;
    }
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    size_t r = r0;
    for (; r + 4 <= r1; r += 4) {
        a0 += gdb_io<T>::ld(x, (r + 0) * ld + c);
        a1 += gdb_io<T>::ld(x, (r + 1) * ld + c);
        a2 += gdb_io<T>::ld(x, (r + 2) * ld + c);
        a3 += gdb_io<T>::ld(x, (r + 3) * ld + c);
    }
    for (; r < r1; ++r) {
        a0 += gdb_io<T>::ld(x, r * ld + c);
    }
    partial[(size_t)blockIdx.y * cols + c] = (a0 + a1) + (a2 + a3);
}
template <typename T>
__global__ void reduce_rows_final_kernel(const float *partial, T *y, size_t blocks, size_t cols)
{
    gdb_pdl_sync();
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) {
        return;
    }
    float s = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        s += partial[b * cols + c];
    }
    gdb_io<T>::st(y, c, s);
}

bool mv_ok(const gd_backend_matrix_view *v, size_t es)
{
    if (v == NULL || v->buffer == NULL || v->rows == 0U || v->cols == 0U || es == 0U) {
        return false;
    }
    if (v->row_bytes < (size_t)v->cols * es || (v->row_bytes % es) != 0U || (v->offset % es) != 0U) {
        return false;
    }
    const size_t span = (size_t)(v->rows - 1U) * v->row_bytes + (size_t)v->cols * es;
    return gdb_range_ok(v->buffer, v->offset, span);
}

template <typename T>
void launch_portable(gd_backend *be, int ta, int tb, const void *a, size_t lda, const void *b, size_t ldb,
                     void *c, size_t ldc, const void *bias, unsigned M, unsigned N, unsigned K,
                     unsigned batch, size_t ba, size_t bb, size_t bc, int bias_mode)
{
    // lda/ldb/ldc in elements. ta: A stored [K, M]; tb: B stored [N, K].
    const size_t sam = ta ? 1 : lda, sak = ta ? lda : 1;
    const size_t sbk = tb ? 1 : ldb, sbn = tb ? ldb : 1;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, batch);
    gdb_launch(gemm_portable_kernel<T>, grid, 256, 0, be->stream, (const T *)a, sam, sak, (const T *)b, sbk, sbn, (T *)c, ldc,
                                                           (const T *)bias, M, N, K, ba, bb, bc, bias_mode);
}

}  // namespace

namespace {
// Brackets one contraction with a pair of events when GEMM profiling is enabled (gdb200_gemm_profile_enable).
struct profile_scope {
    gd_backend *be;
    int slot;
    profile_scope(gd_backend *b, double flops, double bytes) : be(b), slot(-1)
    {
        gdb_gemm_profile *p = g_profile;
        if (p == nullptr || !p->enabled || p->used >= gdb_gemm_profile::CAP) {
            return;
        }
        if (p->used >= p->created) {
            if (cudaEventCreate(&p->start[p->created]) != cudaSuccess || cudaEventCreate(&p->stop[p->created]) != cudaSuccess) {
                return;
            }
            p->created += 1;
        }
        slot = p->used++;
        p->flops += flops;
        p->bytes += bytes;
        cudaEventRecord(p->start[slot], be->stream);
    }
    ~profile_scope()
    {
        if (slot >= 0) {
            cudaEventRecord(g_profile->stop[slot], be->stream);
        }
    }
};

}  // namespace

// x: [M, K] (or [K, M] when ta), w: [K, N] (or [N, K] when tb), y: [M, N].
gd_status gdb_gemm_dispatch(gd_backend *be, int ta, int tb, const gd_backend_matrix_view *x,
                            const gd_backend_matrix_view *w, const gd_backend_vector_view *bias,
                            const gd_backend_matrix_view *y, int bias_mode)
{
    if (be == NULL || x == NULL || w == NULL || y == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = y->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (x->dtype != dt || w->dtype != dt) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    if (!mv_ok(x, es) || !mv_ok(w, es) || !mv_ok(y, es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t M = y->rows, N = y->cols;
    const uint32_t K = ta ? x->rows : x->cols;
    if ((ta ? x->cols : x->rows) != M || (tb ? w->rows : w->cols) != N || (tb ? w->cols : w->rows) != K) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *bp = NULL;
    if (bias != NULL) {
        if (bias->buffer == NULL || bias->dtype != dt || bias->length != N || (bias->offset % es) != 0U ||
            !gdb_range_ok(bias->buffer, bias->offset, (size_t)N * es)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        bp = bias->buffer->dptr + bias->offset;
    }
    const void *ap = x->buffer->dptr + x->offset;
    const void *wp = w->buffer->dptr + w->offset;
    void *cp = y->buffer->dptr + y->offset;
    profile_scope scope(be, 2.0 * M * N * K, (double)es * ((double)M * K + (double)K * N + (double)M * N));
    if (be->gemm_mode != 1 && be->gemm_mode != 2 && !ta && M <= 64U) {
        gd_status st = gdb_gemm_skinny(be, tb, dt, ap, x->row_bytes, wp, w->row_bytes, cp, y->row_bytes, bp, bias_mode, M, N, K);
        if (st != GD_ERR_UNSUPPORTED) {
            return st;
        }
    }
    if (be->gemm_mode != 1 && dt != GDB_DTYPE_F32) {
        gd_status st = gdb_gemm_tcgen05(be, ta, tb, dt, ap, x->row_bytes, wp, w->row_bytes, cp, y->row_bytes, bp, bias_mode, M, N, K);
        if (st != GD_ERR_UNSUPPORTED) {
            return st;
        }
        if (be->gemm_mode == 2) {
            return GD_ERR_UNSUPPORTED;
        }
    } else if (be->gemm_mode == 2) {
        return GD_ERR_UNSUPPORTED;
    }
    if (dt == GDB_DTYPE_F16) {
        launch_portable<__half>(be, ta, tb, ap, x->row_bytes / es, wp, w->row_bytes / es, cp, y->row_bytes / es, bp, M, N, K, 1, 0, 0, 0, bias_mode);
    } else if (dt == GDB_DTYPE_BF16) {
        launch_portable<__nv_bfloat16>(be, ta, tb, ap, x->row_bytes / es, wp, w->row_bytes / es, cp, y->row_bytes / es, bp, M, N, K, 1, 0, 0, 0, bias_mode);
    } else {
        launch_portable<float>(be, ta, tb, ap, x->row_bytes / es, wp, w->row_bytes / es, cp, y->row_bytes / es, bp, M, N, K, 1, 0, 0, 0, bias_mode);
    }
    return gdb_launched(be, "gemm_portable");
}

namespace {

bool bv_ok(const gd_backend_batched_matrix_view *v, size_t es)
{
    if (v == NULL || v->buffer == NULL || v->rows == 0U || v->cols == 0U || v->batch_rank > GD_BACKEND_MAX_BATCH_DIMS ||
        v->row_bytes < (size_t)v->cols * es || (v->row_bytes % es) != 0U || (v->offset % es) != 0U) {
        return false;
    }
    size_t max_off = (size_t)(v->rows - 1U) * v->row_bytes + (size_t)v->cols * es;
    for (uint32_t d = 0; d < v->batch_rank; ++d) {
        if (v->batch_shape[d] == 0U || (v->batch_strides[d] % es) != 0U) {
            return false;
        }
        max_off += (size_t)(v->batch_shape[d] - 1U) * v->batch_strides[d];
    }
    return gdb_range_ok(v->buffer, v->offset, max_off);
}

// Batched contraction with numpy-style broadcast over the batch dims of the output view.
// batch_strides are byte strides; a stride of 0 broadcasts that operand.
gd_status batched_dispatch(gd_backend *be, int ta, int tb, const gd_backend_batched_matrix_view *x,
                           const gd_backend_batched_matrix_view *w, const gd_backend_batched_matrix_view *y)
{
    if (be == NULL || x == NULL || w == NULL || y == NULL || x->dtype != y->dtype || w->dtype != y->dtype) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = y->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (!gdb_is_float_dtype(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    if (!bv_ok(x, es) || !bv_ok(w, es) || !bv_ok(y, es) || x->batch_rank != y->batch_rank || w->batch_rank != y->batch_rank) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t M = y->rows, N = y->cols, K = ta ? x->rows : x->cols;
    if ((ta ? x->cols : x->rows) != M || (tb ? w->rows : w->cols) != N || (tb ? w->cols : w->rows) != K) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    size_t total = 1;
    for (uint32_t d = 0; d < y->batch_rank; ++d) {
        total *= y->batch_shape[d];
    }
    if (total == 0U || total != y->batch_count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    // The innermost batch dimension goes into ONE launch (third grid dimension / third tensor-map coordinate) wherever the
    // tensor-memory kernel takes the shape; when all batch dimensions are nested (each operand's pitch of a dimension is the
    // extent times the pitch of the next, or the operand is broadcast over all of them) they collapse into that one
    // dimension, otherwise the outer dimensions are walked on the host.
    if (y->batch_rank >= 1U && total > 1U) {
        const uint32_t r = y->batch_rank;
        auto eff = [&](const gd_backend_batched_matrix_view *v, uint32_t d) { return v->batch_shape[d] == 1U ? (size_t)0 : v->batch_strides[d]; };
        bool nested = true;
        for (const gd_backend_batched_matrix_view *v : {x, w, y}) {
            bool all_bcast = true, all_full = true;
            for (uint32_t d = 0; d < r; ++d) {
                all_bcast = all_bcast && (v->batch_shape[d] == 1U || y->batch_shape[d] == 1U);
                all_full = all_full && (v->batch_shape[d] == y->batch_shape[d]);
            }
            bool chain = all_full;
            for (uint32_t d = 0; chain && d + 1U < r; ++d) chain = v->batch_strides[d] == (size_t)y->batch_shape[d + 1U] * v->batch_strides[d + 1U];
            nested = nested && (all_bcast || chain);
        }
        const uint32_t inner = nested ? (uint32_t)total : y->batch_shape[r - 1U];
        const size_t outer = total / inner;
        if (inner > 1U && inner <= 65535U) {
            bool fast = true;
            for (size_t bo = 0; bo < outer && fast; ++bo) {
                size_t rem = bo, xo = 0, wo = 0, yo = 0;
                for (int d = (int)r - 2; d >= 0 && !nested; --d) {
                    const size_t idx = rem % y->batch_shape[d];
                    rem /= y->batch_shape[d];
                    xo += idx * eff(x, (uint32_t)d);
                    wo += idx * eff(w, (uint32_t)d);
                    yo += idx * y->batch_strides[d];
                }
                bool x_b = true, w_b = true;   // broadcast over everything that is batched inside the launch
                for (uint32_t d = nested ? 0U : r - 1U; d < r; ++d) {
                    x_b = x_b && eff(x, d) == 0U;
                    w_b = w_b && eff(w, d) == 0U;
                }
                const gd_status st = gdb_gemm_tcgen05_batched(be, ta, tb, dt, x->buffer->dptr + x->offset + xo, x->row_bytes, x_b ? 0U : x->batch_strides[r - 1U],
                                                              w->buffer->dptr + w->offset + wo, w->row_bytes, w_b ? 0U : w->batch_strides[r - 1U],
                                                              y->buffer->dptr + y->offset + yo, y->row_bytes, y->batch_strides[r - 1U], M, N, K, inner);
                if (st == GD_ERR_UNSUPPORTED && bo == 0U) {
                    fast = false;            // nothing launched yet: the loop below handles every element
                } else if (st != GD_OK) {
                    return st;
                }
            }
            if (fast) {
                return GD_OK;
            }
        }
    }
    for (size_t bi = 0; bi < total; ++bi) {
        size_t rem = bi, xo = 0, wo = 0, yo = 0;
        for (int d = (int)y->batch_rank - 1; d >= 0; --d) {
            const size_t idx = rem % y->batch_shape[d];
            rem /= y->batch_shape[d];
            xo += (x->batch_shape[d] == 1U ? 0U : idx) * x->batch_strides[d];
            wo += (w->batch_shape[d] == 1U ? 0U : idx) * w->batch_strides[d];
            yo += idx * y->batch_strides[d];
        }
        gd_backend_matrix_view xv = {x->buffer, x->offset + xo, x->rows, x->cols, x->row_bytes, dt};
        gd_backend_matrix_view wv = {w->buffer, w->offset + wo, w->rows, w->cols, w->row_bytes, dt};
        gd_backend_matrix_view yv = {y->buffer, y->offset + yo, y->rows, y->cols, y->row_bytes, dt};
        gd_status st = gdb_gemm_dispatch(be, ta, tb, &xv, &wv, NULL, &yv);
        if (st != GD_OK) {
            return st;
        }
    }
    return GD_OK;
}

}  // namespace

extern "C" {

void gdb200_gemm_profile_enable(gd_backend *be, int enable)
{
    (void)be;
    if (g_profile == nullptr) {
        g_profile = new gdb_gemm_profile();
        g_profile->created = 0;
    }
    g_profile->enabled = enable != 0;
    g_profile->used = 0;
    g_profile->flops = 0.0;
    g_profile->bytes = 0.0;
}

// Waits for the stream, then reports launches, summed device milliseconds, FLOPs and bytes since enable.
gd_status gdb200_gemm_profile_read(gd_backend *be, uint64_t *launches, double *total_ms, double *flops, double *bytes)
{
    if (be == NULL || g_profile == nullptr) {
        return GD_ERR_BAD_STATE;
    }
    if (cudaStreamSynchronize(be->stream) != cudaSuccess) {
        return GD_ERR_INTERNAL;
    }
    double ms = 0.0;
    for (int i = 0; i < g_profile->used; ++i) {
        float t = 0.0f;
        if (cudaEventElapsedTime(&t, g_profile->start[i], g_profile->stop[i]) == cudaSuccess) {
            ms += t;
        }
    }
    if (launches) *launches = (uint64_t)g_profile->used;
    if (total_ms) *total_ms = ms;
    if (flops) *flops = g_profile->flops;
    if (bytes) *bytes = g_profile->bytes;
    return GD_OK;
}

gd_status gd_backend_matmul(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w, const gd_backend_matrix_view *y)
{
    return gdb_gemm_dispatch(be, 0, 0, x, w, NULL, y);
}
gd_status gd_backend_matmul_nt(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w, const gd_backend_matrix_view *y)
{
    return gdb_gemm_dispatch(be, 0, 1, x, w, NULL, y);
}
gd_status gd_backend_matmul_tn(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w, const gd_backend_matrix_view *y)
{
    return gdb_gemm_dispatch(be, 1, 0, x, w, NULL, y);
}
gd_status gd_backend_linear(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w, const gd_backend_vector_view *bias, const gd_backend_matrix_view *y)
{
    return gdb_gemm_dispatch(be, 0, 0, x, w, bias, y);
}
// Additive: y = round(round(x w^T) + bias) in one pass, bit-identical to gd_backend_matmul_nt followed
// by gd_backend_add of the bias row (the sequence of the reference's linear_transposed_weight capsule,
// src/ops/linear_transposed_weight/core_linear_transposed_weight.c:51-79) without the extra
// write and read of the [M, N] product.
gd_status gdb200_matmul_nt_bias(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w, const gd_backend_vector_view *bias, const gd_backend_matrix_view *y)
{
    return gdb_gemm_dispatch(be, 0, 1, x, w, bias, y, 2);
}
// out[M, F] = swiglu_split(round(round(x w^T) + bias)) for w [2F, K], bias [2F]: the up / gate projection of the decode step
// (examples/gpt_lm/gpt_lm_shared.c:1032-1046) in one launch. Only the 64-row kernel has this epilogue: other shapes
// answer GD_ERR_UNSUPPORTED and the caller issues gdb200_matmul_nt_bias + gd_backend_swiglu_split_forward.
gd_status gdb200_matmul_nt_bias_swiglu(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                                       const gd_backend_vector_view *bias, const gd_backend_matrix_view *out)
{
    if (be == NULL || x == NULL || w == NULL || bias == NULL || out == NULL || bias->buffer == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = out->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (x->dtype != dt || w->dtype != dt || bias->dtype != dt || !mv_ok(x, es) || !mv_ok(w, es) || !mv_ok(out, es) || x->cols != w->cols ||
        w->rows != 2U * out->cols || out->rows != x->rows || bias->length != w->rows ||
        !gdb_range_ok(bias->buffer, bias->offset, (size_t)bias->length * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (be->gemm_mode == 1 || be->gemm_mode == 2) {
        return GD_ERR_UNSUPPORTED;
    }
    cudaSetDevice(be->device);
    return gdb_gemm_skinny_swiglu(be, dt, x->buffer->dptr + x->offset, x->row_bytes, w->buffer->dptr + w->offset, w->row_bytes,
                                  bias->buffer->dptr + bias->offset, out->buffer->dptr + out->offset, out->row_bytes, (uint32_t)x->rows,
                                  (uint32_t)out->cols, (uint32_t)x->cols);
}
// up_gate[M, 2F] = round(round(x w^T) + bias) AND act[M, F] = swiglu_split(up_gate) from one contraction (training path:
// the backward pass needs up_gate). Same bits as gdb200_matmul_nt_bias followed by gd_backend_swiglu_split_forward, which is
// also what runs when the fused kernel does not take the shape.
gd_status gdb200_matmul_nt_bias_swiglu_both(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                                            const gd_backend_vector_view *bias, const gd_backend_matrix_view *up_gate, const gd_backend_matrix_view *act)
{
    if (be == NULL || x == NULL || w == NULL || bias == NULL || up_gate == NULL || act == NULL || bias->buffer == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = act->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (x->dtype != dt || w->dtype != dt || bias->dtype != dt || up_gate->dtype != dt || !mv_ok(x, es) || !mv_ok(w, es) || !mv_ok(up_gate, es) ||
        !mv_ok(act, es) || x->cols != w->cols || w->rows != 2U * act->cols || up_gate->cols != w->rows || act->rows != x->rows ||
        up_gate->rows != x->rows || bias->length != w->rows || !gdb_range_ok(bias->buffer, bias->offset, (size_t)bias->length * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    static const bool unfused = getenv("GDB200_FUSE_SWIGLU_FWD") != NULL && getenv("GDB200_FUSE_SWIGLU_FWD")[0] == '0';   // A/B switch
    if (!unfused && (be->gemm_mode == 0 || be->gemm_mode == 2)) {
        // counted as the contraction it is (2 M (2F) K FLOP; x, w read, x12 and act written)
        profile_scope scope(be, 2.0 * x->rows * (double)w->rows * x->cols,
                            (double)es * ((double)x->rows * x->cols + (double)w->rows * w->cols + (double)x->rows * w->rows + (double)x->rows * act->cols));
        const gd_status st = gdb_gemm_tcgen05_pair_swiglu(be, dt, x->buffer->dptr + x->offset, x->row_bytes, w->buffer->dptr + w->offset, w->row_bytes,
                                                          bias->buffer->dptr + bias->offset, up_gate->buffer->dptr + up_gate->offset, up_gate->row_bytes,
                                                          act->buffer->dptr + act->offset, act->row_bytes, x->rows, act->cols, x->cols);
        if (st != GD_ERR_UNSUPPORTED) {
            return st;
        }
    }
    gd_status st = gdb200_matmul_nt_bias(be, x, w, bias, up_gate);
    if (st != GD_OK) {
        return st;
    }
    gd_backend_tensor_view uv, av;
    memset(&uv, 0, sizeof(uv));
    memset(&av, 0, sizeof(av));
    if (up_gate->row_bytes != (size_t)up_gate->cols * es || act->row_bytes != (size_t)act->cols * es) {
        return GD_ERR_UNSUPPORTED;   // the unfused pair of calls takes contiguous tensors
    }
    uv.buffer = up_gate->buffer; uv.offset = up_gate->offset; uv.count = (size_t)up_gate->rows * up_gate->cols; uv.dtype = dt; uv.rank = 2;
    uv.shape[0] = up_gate->rows; uv.shape[1] = up_gate->cols; uv.strides[0] = up_gate->cols; uv.strides[1] = 1;
    av.buffer = act->buffer; av.offset = act->offset; av.count = (size_t)act->rows * act->cols; av.dtype = dt; av.rank = 2;
    av.shape[0] = act->rows; av.shape[1] = act->cols; av.strides[0] = act->cols; av.strides[1] = 1;
    return gd_backend_swiglu_split_forward(be, &uv, &av);
}
// d_up_gate[M, 2F] = swiglu_split_backward(up_gate, round(g w^T)), w stored [F, K]: gd_backend_matmul_nt into a scratch dact followed
// by gd_backend_swiglu_split_backward, in one launch and without the scratch. GD_ERR_UNSUPPORTED when the fused kernel does
// not take the shape: the caller then makes the two calls (same bits).
gd_status gdb200_matmul_nt_swiglu_backward(gd_backend *be, const gd_backend_matrix_view *g, const gd_backend_matrix_view *w,
                                           const gd_backend_matrix_view *up_gate, const gd_backend_matrix_view *d_up_gate)
{
    if (be == NULL || g == NULL || w == NULL || up_gate == NULL || d_up_gate == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = d_up_gate->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (g->dtype != dt || w->dtype != dt || up_gate->dtype != dt || !mv_ok(g, es) || !mv_ok(w, es) || !mv_ok(up_gate, es) || !mv_ok(d_up_gate, es) ||
        g->cols != w->cols || up_gate->cols != 2U * w->rows || d_up_gate->cols != up_gate->cols || up_gate->rows != g->rows || d_up_gate->rows != g->rows) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (be->gemm_mode != 0 && be->gemm_mode != 2) {
        return GD_ERR_UNSUPPORTED;
    }
    cudaSetDevice(be->device);
    profile_scope scope(be, 2.0 * g->rows * (double)w->rows * g->cols,
                        (double)es * ((double)g->rows * g->cols + (double)w->rows * w->cols + 2.0 * (double)g->rows * up_gate->cols));
    return gdb_gemm_tcgen05_pair_swiglu_bwd(be, dt, g->buffer->dptr + g->offset, g->row_bytes, w->buffer->dptr + w->offset, w->row_bytes,
                                            up_gate->buffer->dptr + up_gate->offset, up_gate->row_bytes, d_up_gate->buffer->dptr + d_up_gate->offset,
                                            d_up_gate->row_bytes, g->rows, w->rows, g->cols);
}
gd_status gdb200_matmul_tn_colsum(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w, const gd_backend_matrix_view *y,
                                  const gd_backend_vector_view *colsum)
{
    if (be == NULL || x == NULL || w == NULL || y == NULL || colsum == NULL || colsum->buffer == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = y->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (x->dtype != dt || w->dtype != dt || colsum->dtype != dt || colsum->length != x->cols) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (gdb_is_float_dtype(dt) && mv_ok(x, es) && mv_ok(w, es) && mv_ok(y, es) && x->rows == w->rows && y->rows == x->cols && y->cols == w->cols &&
        gdb_range_ok(colsum->buffer, colsum->offset, (size_t)colsum->length * es)) {
        profile_scope scope(be, 2.0 * x->cols * w->cols * x->rows,
                            (double)es * ((double)x->rows * x->cols + (double)x->rows * w->cols + (double)x->cols * w->cols));
        const gd_status st = gdb_gemm_tcgen05_tn_colsum(be, dt, x->buffer->dptr + x->offset, x->row_bytes, w->buffer->dptr + w->offset, w->row_bytes,
                                                        y->buffer->dptr + y->offset, y->row_bytes, colsum->buffer->dptr + colsum->offset,
                                                        x->cols, w->cols, x->rows);
        if (st != GD_ERR_UNSUPPORTED) {
            return st;
        }
    }
    // shapes the fused kernel does not take: the two entries it stands for
    const gd_status st = gd_backend_matmul_tn(be, x, w, y);
    return st != GD_OK ? st : gd_backend_reduce_rows(be, x, colsum);
}
gd_status gd_backend_batched_matmul(gd_backend *be, const gd_backend_batched_matrix_view *x, const gd_backend_batched_matrix_view *w, const gd_backend_batched_matrix_view *y)
{
    return batched_dispatch(be, 0, 0, x, w, y);
}
gd_status gd_backend_batched_matmul_nt(gd_backend *be, const gd_backend_batched_matrix_view *x, const gd_backend_batched_matrix_view *w, const gd_backend_batched_matrix_view *y)
{
    return batched_dispatch(be, 0, 1, x, w, y);
}
gd_status gd_backend_batched_matmul_tn(gd_backend *be, const gd_backend_batched_matrix_view *x, const gd_backend_batched_matrix_view *w, const gd_backend_batched_matrix_view *y)
{
    return batched_dispatch(be, 1, 0, x, w, y);
}

gd_status gd_backend_reduce_rows(gd_backend *be, const gd_backend_matrix_view *x, const gd_backend_vector_view *y)
{
    if (be == NULL || x == NULL || y == NULL || y->buffer == NULL || x->dtype != y->dtype || y->length != x->cols) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = x->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (!gdb_is_float_dtype(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    if (!mv_ok(x, es) || (y->offset % es) != 0U || !gdb_range_ok(y->buffer, y->offset, (size_t)y->length * es)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t rows = x->rows, cols = x->cols, ld = x->row_bytes / es;
    if (es == 2U && gdb_colreduce::usable(x->buffer->dptr + x->offset, ld, NULL, 0, cols) && cols * sizeof(float) <= be->ws_bytes) {
        const size_t cap = be->ws_bytes / (cols * sizeof(float));
        const void *xa = x->buffer->dptr + x->offset;
        void *ya = y->buffer->dptr + y->offset;
        return dt == GDB_DTYPE_F16
                   ? gdb_colreduce::run<__half, false>(be, xa, ld, NULL, 0, NULL, (float *)be->ws, cap, ya, rows, cols)
                   : gdb_colreduce::run<__nv_bfloat16, false>(be, xa, ld, NULL, 0, NULL, (float *)be->ws, cap, ya, rows, cols);
    }
    const unsigned col_blocks = (unsigned)((cols + 255U) / 256U);
    size_t blocks = ((size_t)be->sm_count * 8U + col_blocks - 1U) / col_blocks;
    if (blocks > (rows + 31U) / 32U) {
        blocks = (rows + 31U) / 32U;
    }
    if (blocks * cols * sizeof(float) > be->ws_bytes) {
        blocks = be->ws_bytes / (cols * sizeof(float));
    }
    if (blocks == 0U) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    const size_t chunk = (rows + blocks - 1U) / blocks;
    blocks = (rows + chunk - 1U) / chunk;
    const void *xp = x->buffer->dptr + x->offset;
    void *yp = y->buffer->dptr + y->offset;
    float *ws = (float *)be->ws;
    dim3 grid(col_blocks, (unsigned)blocks);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(reduce_rows_stage_kernel<__half>, grid, 256, 0, be->stream, (const __half *)xp, ld, ws, rows, cols, chunk);
    } else if (dt == GDB_DTYPE_BF16) {
        gdb_launch(reduce_rows_stage_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, ld, ws, rows, cols, chunk);
    } else {
        gdb_launch(reduce_rows_stage_kernel<float>, grid, 256, 0, be->stream, (const float *)xp, ld, ws, rows, cols, chunk);
    }
    gd_status st = gdb_launched(be, "reduce_rows stage");
    if (st != GD_OK) {
        return st;
    }
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(reduce_rows_final_kernel<__half>, col_blocks, 256, 0, be->stream, ws, (__half *)yp, blocks, cols);
    } else if (dt == GDB_DTYPE_BF16) {
        gdb_launch(reduce_rows_final_kernel<__nv_bfloat16>, col_blocks, 256, 0, be->stream, ws, (__nv_bfloat16 *)yp, blocks, cols);
    } else {
        gdb_launch(reduce_rows_final_kernel<float>, col_blocks, 256, 0, be->stream, ws, (float *)yp, blocks, cols);
    }
    return gdb_launched(be, "reduce_rows final");
}

}  // extern "C"
