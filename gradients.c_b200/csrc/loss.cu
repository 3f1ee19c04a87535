// Fused LM-head cross-entropy helpers (chunked online softmax with soft-capping, ignore index)
// and the materialised-logits cross-entropy kernels. One block per row, 16-byte logits loads.
//
// Reference arithmetic: src/ops/lm_cross_entropy/metal_lm_cross_entropy.metal:13-311
//   raw    = f16(matmul_logit + bias)          (:121 - bias add re-rounded to storage precision)
//   logit  = cap * tanh(raw / cap) when cap > 0 (:13-31)
//   online (max, sum) merge per chunk           (:157-163)
//   loss   = log(sum) + max - target_logit      (:184-203), mean over valid rows (:244-252)
//   dlogit = (p - 1[target]) * max(0, 1 - (logit/cap)^2) * grad * scale * inv_valid (:294-310)
// and src/ops/cross_entropy/metal_cross_entropy.metal for the materialised path.
#include "common.cuh"

namespace {

constexpr float NEG_BIG = -3.402823466e38f;

__device__ __forceinline__ float softcap_tanh(float x)
{
    const float ax = fabsf(x);
    if (ax < 0.000244140625f) {
        return x;
    }
    const float e = __expf(-2.0f * ax);
    const float y = (1.0f - e) / (1.0f + e);
    return x < 0.0f ? -y : y;
}
__device__ __forceinline__ float apply_softcap(float logit, float cap, float inv_cap)
{
    return cap > 0.0f ? cap * softcap_tanh(logit * inv_cap) : logit;
}
template <typename T>
__device__ __forceinline__ float eff_logit(float matmul_logit, const T *bias, size_t c, float cap, float inv_cap)
{
    const float raw = bias != nullptr ? gdb_io<T>::rnd(matmul_logit + gdb_io<T>::ld(bias, c)) : matmul_logit;
    return apply_softcap(raw, cap, inv_cap);
}

// Row pass helper: calls f(c, effective_logit) for every class of the row chunk.
template <typename T, typename F>
__device__ __forceinline__ void for_each_logit(const T *row, const T *bias, size_t classes, float cap, float inv_cap, F f)
{
    if (sizeof(T) == 2 && (classes % 8U) == 0U && ((uintptr_t)row % 16U) == 0U) {
        const uint4 *rv = reinterpret_cast<const uint4 *>(row);
        for (size_t v = threadIdx.x; v < classes / 8U; v += blockDim.x) {
            gdb_vec8<T> a;
            a.raw = rv[v];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const size_t c = v * 8U + (size_t)e;
                f(c, eff_logit<T>(a.get(e), bias, c, cap, inv_cap));
            }
        }
    } else {
        for (size_t c = threadIdx.x; c < classes; c += blockDim.x) {
            f(c, eff_logit<T>(gdb_io<T>::ld(row, c), bias, c, cap, inv_cap));
        }
    }
}

// One warp per row, one pass: every lane keeps a running (max, sum) over its classes, the lanes
// are merged with shuffles. No block-level synchronisation.
template <typename T>
__global__ void lmce_online_update_kernel(const T *logits, const T *bias, const int *targets, float *target_logit,
                                          float *row_max, float *row_sum, size_t rows, size_t classes, uint64_t class_start,
                                          uint64_t total_classes, float cap, float inv_cap)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    const T *lr = logits + row * classes;
    float m = NEG_BIG, s = 0.0f;
    if (sizeof(T) == 2 && (classes % 8U) == 0U && ((uintptr_t)lr % 16U) == 0U) {
        const uint4 *rv = reinterpret_cast<const uint4 *>(lr);
        for (size_t v = lane; v < classes / 8U; v += 32) {
            gdb_vec8<T> a;
            a.raw = rv[v];
            float x[8], vm = NEG_BIG;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x[e] = eff_logit<T>(a.get(e), bias, v * 8U + (size_t)e, cap, inv_cap);
                vm = fmaxf(vm, x[e]);
            }
            const float nm = fmaxf(m, vm);
            float add = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) add += __expf(x[e] - nm);
            s = s * __expf(m - nm) + add;
            m = nm;
        }
    } else {
        for (size_t c = lane; c < classes; c += 32) {
            const float x = eff_logit<T>(gdb_io<T>::ld(lr, c), bias, c, cap, inv_cap);
            const float nm = fmaxf(m, x);
            s = s * __expf(m - nm) + __expf(x - nm);
            m = nm;
        }
    }
    const float cmax = gdb_warp_max(m);
    const float csum = gdb_warp_sum(s * __expf(m - cmax));
    if (lane == 0) {
        const int t = targets[row];
        if (t >= 0) {
            const uint64_t tu = (uint64_t)t;
            if (tu >= class_start && tu < class_start + classes && tu < total_classes) {
                const size_t c = (size_t)(tu - class_start);
                target_logit[row] = eff_logit<T>(gdb_io<T>::ld(lr, c), bias, c, cap, inv_cap);
            }
        }
        const float om = row_max[row], os = row_sum[row];
        const float nm = fmaxf(om, cmax);
        row_max[row] = nm;
        row_sum[row] = os * __expf(om - nm) + csum * __expf(cmax - nm);
    }
}

__global__ void lmce_finalize_kernel(const int *targets, float *row_loss, float *row_max, float *row_inv_sum,
                                     float *row_valid, size_t rows, uint64_t total_classes, int ignore_index)
{
    gdb_pdl_sync();
    const size_t row = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) {
        return;
    }
    const int t = targets[row];
    if (t < 0 || t == ignore_index) {
        row_loss[row] = 0.0f;
        row_max[row] = 0.0f;
        row_inv_sum[row] = 0.0f;
        row_valid[row] = 0.0f;
        return;
    }
    if ((uint64_t)t >= total_classes) {
        row_loss[row] = __int_as_float(0x7fc00000);
        row_max[row] = 0.0f;
        row_inv_sum[row] = 0.0f;
        row_valid[row] = 1.0f;
        return;
    }
    row_valid[row] = 1.0f;
    const float sum = row_inv_sum[row];
    row_loss[row] = logf(sum) + row_max[row] - row_loss[row];
    row_inv_sum[row] = 1.0f / sum;
}

__global__ void lmce_reduce_normalize_kernel(const float *row_loss, const float *row_valid, float *loss,
                                             float *inv_valid_count, size_t rows)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    float ll = 0.0f, lv = 0.0f;
    for (size_t i = threadIdx.x; i < rows; i += blockDim.x) {
        ll += row_loss[i];
        lv += row_valid[i];
    }
    const float loss_sum = gdb_block_sum(ll, sh);
    const float valid = gdb_block_sum(lv, sh);
    if (threadIdx.x == 0) {
        if (valid > 0.0f) {
            const float inv = 1.0f / valid;
            inv_valid_count[0] = inv;
            loss[0] = loss_sum * inv;
        } else {
            inv_valid_count[0] = 0.0f;
            loss[0] = __int_as_float(0x7fc00000);
        }
    }
}

// Data-parallel form of the normaliser: counts[0] holds the number of valid target rows of the GLOBAL batch
// (all ranks), so loss[0] becomes this rank's share of the global mean (the shares add up to it) and the
// backward pass divides by the global count instead of the local one.
__global__ void lmce_reduce_normalize_global_kernel(const float *row_loss, const float *counts, float *loss,
                                                    float *inv_valid_count, size_t rows)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    float ll = 0.0f;
    for (size_t i = threadIdx.x; i < rows; i += blockDim.x) {
        ll += row_loss[i];
    }
    const float loss_sum = gdb_block_sum(ll, sh);
    if (threadIdx.x == 0) {
        const float global = counts[0];
        if (global > 0.0f) {
            const float inv = 1.0f / global;
            inv_valid_count[0] = inv;
            loss[0] = loss_sum * inv;
        } else {
            inv_valid_count[0] = 0.0f;
            loss[0] = __int_as_float(0x7fc00000);
        }
    }
}

// counts[0] = counts[1] = number of rows whose target takes part in the loss (same rule as lmce_finalize_kernel).
__global__ void lmce_count_valid_kernel(const int *targets, size_t rows, int ignore_index, float *counts)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    float n = 0.0f;
    for (size_t i = threadIdx.x; i < rows; i += blockDim.x) {
        const int t = targets[i];
        n += (t >= 0 && t != ignore_index) ? 1.0f : 0.0f;   // out-of-range ids count (their loss is NaN), as in finalize
    }
    const float total = gdb_block_sum(n, sh);
    if (threadIdx.x == 0) {
        counts[0] = total;
        counts[1] = total;
    }
}

template <typename T>
__global__ void lmce_backward_chunk_kernel(const T *logits, const T *bias, const int *targets, const float *row_max,
                                           const float *row_inv_sum, const float *grad_loss, const float *inv_valid,
                                           T *dlogits, size_t classes, uint64_t class_start, uint64_t total_classes,
                                           float scale, float cap, float inv_cap, int ignore_index)
{
    gdb_pdl_sync();
    const size_t row = blockIdx.x;
    const T *lr = logits + row * classes;
    T *dr = dlogits + row * classes;
    const int t = targets[row];
    const bool vec = sizeof(T) == 2 && (classes % 8U) == 0U && (((uintptr_t)lr | (uintptr_t)dr) % 16U) == 0U;
    if (t < 0 || t == ignore_index || (uint64_t)t >= total_classes) {
        if (vec) {
            for (size_t v = threadIdx.x; v < classes / 8U; v += blockDim.x) {
                reinterpret_cast<uint4 *>(dr)[v] = make_uint4(0U, 0U, 0U, 0U);
            }
        } else {
            for (size_t c = threadIdx.x; c < classes; c += blockDim.x) {
                gdb_io<T>::st(dr, c, 0.0f);
            }
        }
        return;
    }
    const float seed = grad_loss[0] * scale * inv_valid[0];
    const float rm = row_max[row], inv_sum = row_inv_sum[row];
    const uint64_t tu = (uint64_t)t;
    auto grad_of = [&](size_t c, float soft) {
        float p = __expf(soft - rm) * inv_sum;
        if (class_start + c == tu) {
            p -= 1.0f;
        }
        if (cap > 0.0f) {
            const float y = soft * inv_cap;
            p *= fmaxf(0.0f, 1.0f - y * y);
        }
        return p * seed;
    };
    if (vec) {
        const uint4 *rv = reinterpret_cast<const uint4 *>(lr);
        uint4 *dv = reinterpret_cast<uint4 *>(dr);
        for (size_t v = threadIdx.x; v < classes / 8U; v += blockDim.x) {
            gdb_vec8<T> a;
            a.raw = rv[v];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const size_t c = v * 8U + (size_t)e;
                a.set(e, grad_of(c, eff_logit<T>(a.get(e), bias, c, cap, inv_cap)));
            }
            dv[v] = a.raw;
        }
    } else {
        for (size_t c = threadIdx.x; c < classes; c += blockDim.x) {
            gdb_io<T>::st(dr, c, grad_of(c, eff_logit<T>(gdb_io<T>::ld(lr, c), bias, c, cap, inv_cap)));
        }
    }
}

// Materialised cross entropy: row_loss[n] = logsumexp(logits[n,:]) - logits[n, target[n]].
template <typename T, bool STATS>
__global__ void ce_loss_kernel(const T *logits, const int *targets, float *row_loss, float *row_max, float *row_inv_sum, size_t classes)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    const size_t row = blockIdx.x;
    const T *lr = logits + row * classes;
    float lmax = NEG_BIG;
    for_each_logit<T>(lr, (const T *)nullptr, classes, 0.0f, 0.0f, [&](size_t, float v) { lmax = fmaxf(lmax, v); });
    const float m = gdb_block_max(lmax, sh);
    float lsum = 0.0f;
    for_each_logit<T>(lr, (const T *)nullptr, classes, 0.0f, 0.0f, [&](size_t, float v) { lsum += __expf(v - m); });
    const float s = gdb_block_sum(lsum, sh);
    if (threadIdx.x == 0) {
        const int t = targets[row];
        if (t < 0 || (size_t)t >= classes) {
            row_loss[row] = __int_as_float(0x7fc00000);
        } else {
            row_loss[row] = logf(s) + m - gdb_io<T>::ld(lr, (size_t)t);
        }
        if (STATS) {
            row_max[row] = m;
            row_inv_sum[row] = 1.0f / s;
        }
    }
}

// grad_logits[n, c] = (softmax - onehot) * g * scale; g = grad_loss[0] (scalar) or grad_loss[n].
template <typename T, bool STATS>
__global__ void ce_backward_kernel(const T *logits, const int *targets, const float *row_max, const float *row_inv_sum,
                                   const float *grad_loss, size_t grad_count, T *dlogits, size_t classes, float scale)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    const size_t row = blockIdx.x;
    const T *lr = logits + row * classes;
    T *dr = dlogits + row * classes;
    float m, inv_sum;
    if (STATS) {
        m = row_max[row];
        inv_sum = row_inv_sum[row];
    } else {
        float lmax = NEG_BIG;
        for_each_logit<T>(lr, (const T *)nullptr, classes, 0.0f, 0.0f, [&](size_t, float v) { lmax = fmaxf(lmax, v); });
        m = gdb_block_max(lmax, sh);
        float lsum = 0.0f;
        for_each_logit<T>(lr, (const T *)nullptr, classes, 0.0f, 0.0f, [&](size_t, float v) { lsum += __expf(v - m); });
        inv_sum = 1.0f / gdb_block_sum(lsum, sh);
    }
    const int t = targets[row];
    const float g = grad_loss[grad_count > 1U ? row : 0U] * scale;
    for (size_t c = threadIdx.x; c < classes; c += blockDim.x) {
        float p = __expf(gdb_io<T>::ld(lr, c) - m) * inv_sum;
        if (t >= 0 && (size_t)t == c) {
            p -= 1.0f;
        }
        gdb_io<T>::st(dr, c, p * g);
    }
}

bool half_dt(uint32_t dt) { return dt == GDB_DTYPE_F16 || dt == GDB_DTYPE_BF16; }

unsigned row_threads(size_t classes)
{
    const size_t per = (classes + 7U) / 8U;
    unsigned t = 32;
    while (t < 256 && t < per) {
        t <<= 1;
    }
    return t;
}

struct chunk_shape {
    size_t rows, classes;
};
bool chunk_dims(const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, chunk_shape *o)
{
    if (logits->rank < 1U || logits->rank > 8U || targets->count == 0U) {
        return false;
    }
    o->classes = (size_t)logits->shape[logits->rank - 1U];
    o->rows = targets->count;
    return o->classes > 0U && logits->count == o->rows * o->classes;
}

}  // namespace

extern "C" {

gd_status gd_backend_lm_cross_entropy_online_update(gd_backend *be, const gd_backend_tensor_view *logits_chunk, const gd_backend_tensor_view *bias_chunk, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum, uint64_t class_start, uint64_t total_classes, float logits_softcap)
{
    chunk_shape cs;
    if (be == NULL || logits_chunk == NULL || targets == NULL || row_loss == NULL || row_max == NULL ||
        row_inv_sum == NULL || !(logits_softcap >= 0.0f) || !chunk_dims(logits_chunk, targets, &cs) ||
        row_loss->count != cs.rows || row_max->count != cs.rows || row_inv_sum->count != cs.rows ||
        class_start + cs.classes > total_classes) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = logits_chunk->dtype;
    if (!half_dt(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *lp = gdb_tv_ptr(logits_chunk, dt);
    const void *bp = NULL;
    if (bias_chunk != NULL) {
        if (bias_chunk->count != cs.classes || (bp = gdb_tv_ptr(bias_chunk, dt)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    float *rl = (float *)gdb_tv_ptr(row_loss, GDB_DTYPE_F32), *rm = (float *)gdb_tv_ptr(row_max, GDB_DTYPE_F32);
    float *rs = (float *)gdb_tv_ptr(row_inv_sum, GDB_DTYPE_F32);
    if (lp == NULL || tp == NULL || rl == NULL || rm == NULL || rs == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const float inv_cap = logits_softcap > 0.0f ? 1.0f / logits_softcap : 0.0f;
    const unsigned grid = (unsigned)((cs.rows + 3U) / 4U);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(lmce_online_update_kernel<__half>, grid, 128, 0, be->stream, (const __half *)lp, (const __half *)bp, tp, rl, rm, rs, cs.rows, cs.classes, class_start, total_classes, logits_softcap, inv_cap);
    } else {
        gdb_launch(lmce_online_update_kernel<__nv_bfloat16>, grid, 128, 0, be->stream, (const __nv_bfloat16 *)lp, (const __nv_bfloat16 *)bp, tp, rl, rm, rs, cs.rows, cs.classes, class_start, total_classes, logits_softcap, inv_cap);
    }
    return gdb_launched(be, "lm_cross_entropy_online_update");
}

gd_status gd_backend_lm_cross_entropy_finalize(gd_backend *be, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum, const gd_backend_tensor_view *row_valid, uint64_t total_classes, int32_t ignore_index)
{
    if (be == NULL || targets == NULL || row_loss == NULL || row_max == NULL || row_inv_sum == NULL || row_valid == NULL ||
        targets->count == 0U || row_loss->count != targets->count || row_max->count != targets->count ||
        row_inv_sum->count != targets->count || row_valid->count != targets->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    float *rl = (float *)gdb_tv_ptr(row_loss, GDB_DTYPE_F32), *rm = (float *)gdb_tv_ptr(row_max, GDB_DTYPE_F32);
    float *rs = (float *)gdb_tv_ptr(row_inv_sum, GDB_DTYPE_F32), *rv = (float *)gdb_tv_ptr(row_valid, GDB_DTYPE_F32);
    if (tp == NULL || rl == NULL || rm == NULL || rs == NULL || rv == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t rows = targets->count;
    gdb_launch(lmce_finalize_kernel, (unsigned)((rows + 255U) / 256U), 256, 0, be->stream, tp, rl, rm, rs, rv, rows, total_classes, ignore_index);
    return gdb_launched(be, "lm_cross_entropy_finalize");
}

gd_status gd_backend_lm_cross_entropy_reduce_normalize(gd_backend *be, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *row_valid, const gd_backend_tensor_view *loss, const gd_backend_tensor_view *inv_valid_count)
{
    if (be == NULL || row_loss == NULL || row_valid == NULL || loss == NULL || inv_valid_count == NULL ||
        row_loss->count == 0U || row_valid->count != row_loss->count || loss->count != 1U || inv_valid_count->count != 1U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const float *rl = (const float *)gdb_tv_ptr(row_loss, GDB_DTYPE_F32), *rv = (const float *)gdb_tv_ptr(row_valid, GDB_DTYPE_F32);
    float *lp = (float *)gdb_tv_ptr(loss, GDB_DTYPE_F32), *ip = (float *)gdb_tv_ptr(inv_valid_count, GDB_DTYPE_F32);
    if (rl == NULL || rv == NULL || lp == NULL || ip == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gdb_launch(lmce_reduce_normalize_kernel, 1, 1024, 0, be->stream, rl, rv, lp, ip, row_loss->count);
    return gdb_launched(be, "lm_cross_entropy_reduce_normalize");
}

gd_status gd_backend_lm_cross_entropy_backward_chunk(gd_backend *be, const gd_backend_tensor_view *logits_chunk, const gd_backend_tensor_view *bias_chunk, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum, const gd_backend_tensor_view *grad_loss, const gd_backend_tensor_view *inv_valid_count, const gd_backend_tensor_view *grad_logits_chunk, uint64_t class_start, uint64_t total_classes, float scale, float logits_softcap, int32_t ignore_index)
{
    chunk_shape cs;
    if (be == NULL || logits_chunk == NULL || targets == NULL || row_max == NULL || row_inv_sum == NULL ||
        grad_loss == NULL || inv_valid_count == NULL || grad_logits_chunk == NULL || !(logits_softcap >= 0.0f) ||
        !chunk_dims(logits_chunk, targets, &cs) || grad_logits_chunk->count != logits_chunk->count ||
        grad_logits_chunk->dtype != logits_chunk->dtype || row_max->count != cs.rows || row_inv_sum->count != cs.rows ||
        grad_loss->count != 1U || inv_valid_count->count != 1U || class_start + cs.classes > total_classes) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = logits_chunk->dtype;
    if (!half_dt(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *lp = gdb_tv_ptr(logits_chunk, dt);
    void *dp = gdb_tv_ptr(grad_logits_chunk, dt);
    const void *bp = NULL;
    if (bias_chunk != NULL) {
        if (bias_chunk->count != cs.classes || (bp = gdb_tv_ptr(bias_chunk, dt)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    const float *rm = (const float *)gdb_tv_ptr(row_max, GDB_DTYPE_F32), *rs = (const float *)gdb_tv_ptr(row_inv_sum, GDB_DTYPE_F32);
    const float *gl = (const float *)gdb_tv_ptr(grad_loss, GDB_DTYPE_F32), *iv = (const float *)gdb_tv_ptr(inv_valid_count, GDB_DTYPE_F32);
    if (lp == NULL || dp == NULL || tp == NULL || rm == NULL || rs == NULL || gl == NULL || iv == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const float inv_cap = logits_softcap > 0.0f ? 1.0f / logits_softcap : 0.0f;
    const unsigned threads = row_threads(cs.classes);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(lmce_backward_chunk_kernel<__half>, (unsigned)cs.rows, threads, 0, be->stream, (const __half *)lp, (const __half *)bp, tp, rm, rs, gl, iv, (__half *)dp, cs.classes, class_start, total_classes, scale, logits_softcap, inv_cap, ignore_index);
    } else {
        gdb_launch(lmce_backward_chunk_kernel<__nv_bfloat16>, (unsigned)cs.rows, threads, 0, be->stream, (const __nv_bfloat16 *)lp, (const __nv_bfloat16 *)bp, tp, rm, rs, gl, iv, (__nv_bfloat16 *)dp, cs.classes, class_start, total_classes, scale, logits_softcap, inv_cap, ignore_index);
    }
    return gdb_launched(be, "lm_cross_entropy_backward_chunk");
}

static gd_status ce_loss_common(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum, bool stats)
{
    chunk_shape cs;
    if (be == NULL || logits == NULL || targets == NULL || row_loss == NULL || !chunk_dims(logits, targets, &cs) ||
        row_loss->count != cs.rows || (stats && (row_max == NULL || row_inv_sum == NULL || row_max->count != cs.rows || row_inv_sum->count != cs.rows))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = logits->dtype;
    if (!half_dt(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *lp = gdb_tv_ptr(logits, dt);
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    float *rl = (float *)gdb_tv_ptr(row_loss, GDB_DTYPE_F32);
    float *rm = stats ? (float *)gdb_tv_ptr(row_max, GDB_DTYPE_F32) : NULL;
    float *rs = stats ? (float *)gdb_tv_ptr(row_inv_sum, GDB_DTYPE_F32) : NULL;
    if (lp == NULL || tp == NULL || rl == NULL || (stats && (rm == NULL || rs == NULL))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned threads = row_threads(cs.classes);
    if (dt == GDB_DTYPE_F16) {
        if (stats) gdb_launch(ce_loss_kernel<__half, true>, (unsigned)cs.rows, threads, 0, be->stream, (const __half *)lp, tp, rl, rm, rs, cs.classes);
        else gdb_launch(ce_loss_kernel<__half, false>, (unsigned)cs.rows, threads, 0, be->stream, (const __half *)lp, tp, rl, rm, rs, cs.classes);
    } else {
        if (stats) gdb_launch(ce_loss_kernel<__nv_bfloat16, true>, (unsigned)cs.rows, threads, 0, be->stream, (const __nv_bfloat16 *)lp, tp, rl, rm, rs, cs.classes);
        else gdb_launch(ce_loss_kernel<__nv_bfloat16, false>, (unsigned)cs.rows, threads, 0, be->stream, (const __nv_bfloat16 *)lp, tp, rl, rm, rs, cs.classes);
    }
    return gdb_launched(be, "cross_entropy_loss");
}

gd_status gd_backend_cross_entropy_loss(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_loss)
{
    return ce_loss_common(be, logits, targets, row_loss, NULL, NULL, false);
}
gd_status gd_backend_cross_entropy_loss_stats(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum)
{
    return ce_loss_common(be, logits, targets, row_loss, row_max, row_inv_sum, true);
}

static gd_status ce_bwd_common(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum, const gd_backend_tensor_view *grad_loss, const gd_backend_tensor_view *grad_logits, float scale, bool stats)
{
    chunk_shape cs;
    if (be == NULL || logits == NULL || targets == NULL || grad_loss == NULL || grad_logits == NULL ||
        !chunk_dims(logits, targets, &cs) || grad_logits->count != logits->count || grad_logits->dtype != logits->dtype ||
        (grad_loss->count != 1U && grad_loss->count != cs.rows) ||
        (stats && (row_max == NULL || row_inv_sum == NULL || row_max->count != cs.rows || row_inv_sum->count != cs.rows))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = logits->dtype;
    if (!half_dt(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *lp = gdb_tv_ptr(logits, dt);
    void *dp = gdb_tv_ptr(grad_logits, dt);
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    const float *gl = (const float *)gdb_tv_ptr(grad_loss, GDB_DTYPE_F32);
    const float *rm = stats ? (const float *)gdb_tv_ptr(row_max, GDB_DTYPE_F32) : NULL;
    const float *rs = stats ? (const float *)gdb_tv_ptr(row_inv_sum, GDB_DTYPE_F32) : NULL;
    if (lp == NULL || dp == NULL || tp == NULL || gl == NULL || (stats && (rm == NULL || rs == NULL))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned threads = row_threads(cs.classes);
    if (dt == GDB_DTYPE_F16) {
        if (stats) gdb_launch(ce_backward_kernel<__half, true>, (unsigned)cs.rows, threads, 0, be->stream, (const __half *)lp, tp, rm, rs, gl, grad_loss->count, (__half *)dp, cs.classes, scale);
        else gdb_launch(ce_backward_kernel<__half, false>, (unsigned)cs.rows, threads, 0, be->stream, (const __half *)lp, tp, rm, rs, gl, grad_loss->count, (__half *)dp, cs.classes, scale);
    } else {
        if (stats) gdb_launch(ce_backward_kernel<__nv_bfloat16, true>, (unsigned)cs.rows, threads, 0, be->stream, (const __nv_bfloat16 *)lp, tp, rm, rs, gl, grad_loss->count, (__nv_bfloat16 *)dp, cs.classes, scale);
        else gdb_launch(ce_backward_kernel<__nv_bfloat16, false>, (unsigned)cs.rows, threads, 0, be->stream, (const __nv_bfloat16 *)lp, tp, rm, rs, gl, grad_loss->count, (__nv_bfloat16 *)dp, cs.classes, scale);
    }
    return gdb_launched(be, "cross_entropy_backward");
}

gd_status gd_backend_cross_entropy_backward(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *grad_loss, const gd_backend_tensor_view *grad_logits, float scale)
{
    return ce_bwd_common(be, logits, targets, NULL, NULL, grad_loss, grad_logits, scale, false);
}
gd_status gd_backend_cross_entropy_backward_stats(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *targets, const gd_backend_tensor_view *row_max, const gd_backend_tensor_view *row_inv_sum, const gd_backend_tensor_view *grad_loss, const gd_backend_tensor_view *grad_logits, float scale)
{
    return ce_bwd_common(be, logits, targets, row_max, row_inv_sum, grad_loss, grad_logits, scale, true);
}

}  // extern "C"

gd_status gdb_lm_ce_count_valid(gd_backend *be, const gd_backend_tensor_view *targets, int32_t ignore_index, const gd_backend_tensor_view *counts)
{
    if (be == NULL || targets == NULL || counts == NULL || targets->count == 0U || counts->count != 2U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    float *cp = (float *)gdb_tv_ptr(counts, GDB_DTYPE_F32);
    if (tp == NULL || cp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gdb_launch(lmce_count_valid_kernel, 1, 1024, 0, be->stream, tp, (size_t)targets->count, (int)ignore_index, cp);
    return gdb_launched(be, "lm_cross_entropy_count_valid");
}

gd_status gdb_lm_ce_reduce_normalize_global(gd_backend *be, const gd_backend_tensor_view *row_loss, const gd_backend_tensor_view *counts,
                                            const gd_backend_tensor_view *loss, const gd_backend_tensor_view *inv_valid_count)
{
    if (be == NULL || row_loss == NULL || counts == NULL || loss == NULL || inv_valid_count == NULL || row_loss->count == 0U ||
        counts->count != 2U || loss->count != 1U || inv_valid_count->count != 1U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const float *rl = (const float *)gdb_tv_ptr(row_loss, GDB_DTYPE_F32), *cp = (const float *)gdb_tv_ptr(counts, GDB_DTYPE_F32);
    float *lp = (float *)gdb_tv_ptr(loss, GDB_DTYPE_F32), *ip = (float *)gdb_tv_ptr(inv_valid_count, GDB_DTYPE_F32);
    if (rl == NULL || cp == NULL || lp == NULL || ip == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gdb_launch(lmce_reduce_normalize_global_kernel, 1, 1024, 0, be->stream, rl, cp, lp, ip, (size_t)row_loss->count);
    return gdb_launched(be, "lm_cross_entropy_reduce_normalize(global)");
}
