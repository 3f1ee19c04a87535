// Packed variable-length attention (forward + backward), KV-cache decode attention and
// KV-cache append: entry points, argument validation and the general-shape kernels.
// The tensor-core flash kernels for the hot configuration (16-bit storage, head_dim 64 or
// 128, no prefix) live in attention_flash.cu and are tried first.
//
// Reference semantics: src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55 (mask rule),
// :137-228 (forward, online softmax in FP32, rows without an allowed key give zeros),
// :230-533 (backward: D = sum_j P_ij dP_ij, dS = P (dP - D), dQ = scale dS K,
// dK = scale dS^T Q, dV = P^T dO); src/ops/sdpa_decode/metal_sdpa_decode.metal:31-281;
// src/ops/kv_cache_append/metal_kv_cache_append.metal:30-122 (rows that would cross the
// cache capacity are dropped).
// stats layout [N, Hq, 3] F32 = (row max of scaled scores, sum of exp, D).
#include "common.cuh"
#include "decode_parts.cuh"
#include "attention.cuh"

#include <stdlib.h>

#include <math.h>

namespace {

using gdb_dec::mask_allowed;

// Find the segment that holds packed row `row` (cu[0] == 0, cu non-decreasing).
__device__ __forceinline__ int find_segment(const int *cu, int batch, int row)
{
    int lo = 0, hi = batch;
    while (lo + 1 < hi) {
        const int mid = (lo + hi) >> 1;
        if (cu[mid] <= row) lo = mid; else hi = mid;
    }
    return lo;
}

constexpr int MAX_DPL = 8;  // head dims per lane: head_dim <= 256

struct varlen_params {
    int n_tokens, batch, hq, hkv, dh;
    int causal, window, prefix;
    float scale;
};

// MODE 0: forward (out, optional stats). MODE 1: backward stats (m, l, D).
// MODE 2: dQ from saved stats. One warp per (packed row, q head); lanes split head_dim.
template <typename T, int MODE>
__global__ void varlen_row_kernel(const T *q, const T *k, const T *v, const T *go, const int *cu, T *out_or_dq,
                                  float *stats, varlen_params p)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)p.n_tokens * p.hq) {
        return;
    }
    const int row = (int)(w / p.hq), h = (int)(w % p.hq);
    const int hk = h / (p.hq / p.hkv);
    if (row >= cu[p.batch]) {
        return;
    }
    const int b = find_segment(cu, p.batch, row);
    const int start = cu[b], T_seg = cu[b + 1] - start, i = row - start;
    const int dpl = (p.dh + 31) / 32;
    float qr[MAX_DPL], gr[MAX_DPL], acc[MAX_DPL];
    const size_t qbase = ((size_t)row * p.hq + h) * p.dh;
#pragma unroll
    for (int d = 0; d < MAX_DPL; ++d) {
        const int c = lane + 32 * d;
        const bool ok = d < dpl && c < p.dh;
        qr[d] = ok ? gdb_io<T>::ld(q, qbase + c) : 0.0f;
        gr[d] = (ok && MODE != 0) ? gdb_io<T>::ld(go, qbase + c) : 0.0f;
        acc[d] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f, raw = 0.0f, dterm = 0.0f;
    if (MODE == 2) {
        const size_t sb = ((size_t)row * p.hq + h) * 3U;
        m = stats[sb];
        l = stats[sb + 1];
        dterm = stats[sb + 2];
    }
    int j_hi = T_seg;
    if (p.causal && (p.prefix <= 0 || i >= p.prefix)) {
        j_hi = i + 1;
    } else if (p.causal) {
        j_hi = p.prefix < T_seg ? p.prefix : T_seg;
    }
    if (!(MODE == 2 && !(l > 0.0f))) {
        for (int j = 0; j < j_hi; ++j) {
            if (!mask_allowed(i, j, p.causal, p.window, p.prefix)) {
                // skip straight to the window start when there is no prefix region
                if (p.prefix <= 0 && p.window > 0 && i - j >= p.window) {
                    j = i - p.window;
                }
                continue;
            }
            const size_t kb = ((size_t)(start + j) * p.hkv + hk) * p.dh;
            float s = 0.0f, dp = 0.0f;
#pragma unroll
            for (int d = 0; d < MAX_DPL; ++d) {
                const int c = lane + 32 * d;
                if (d < dpl && c < p.dh) {
                    s += qr[d] * gdb_io<T>::ld(k, kb + c);
                    if (MODE != 0) dp += gr[d] * gdb_io<T>::ld(v, kb + c);
                }
            }
            s = gdb_warp_sum(s) * p.scale;
            if (MODE != 0) dp = gdb_warp_sum(dp);
            if (MODE == 2) {
                const float prob = expf(s - m) / l;
                const float ds = prob * (dp - dterm) * p.scale;
#pragma unroll
                for (int d = 0; d < MAX_DPL; ++d) {
                    const int c = lane + 32 * d;
                    if (d < dpl && c < p.dh) acc[d] += ds * gdb_io<T>::ld(k, kb + c);
                }
            } else {
                const float mnew = fmaxf(s, m);
                const float corr = expf(m - mnew), e = expf(s - mnew);
                l = l * corr + e;
                if (MODE == 1) {
                    raw = raw * corr + e * dp;
                } else {
#pragma unroll
                    for (int d = 0; d < MAX_DPL; ++d) {
                        const int c = lane + 32 * d;
                        if (d < dpl && c < p.dh) acc[d] = acc[d] * corr + e * gdb_io<T>::ld(v, kb + c);
                    }
                }
                m = mnew;
            }
        }
    }
    if (MODE == 1) {
        if (lane == 0) {
            const size_t sb = ((size_t)row * p.hq + h) * 3U;
            stats[sb] = m;
            stats[sb + 1] = l;
            stats[sb + 2] = l > 0.0f ? raw / l : 0.0f;
        }
        return;
    }
    const float inv_l = (MODE == 0) ? (l > 0.0f ? 1.0f / l : 0.0f) : 1.0f;
#pragma unroll
    for (int d = 0; d < MAX_DPL; ++d) {
        const int c = lane + 32 * d;
        if (d < dpl && c < p.dh) gdb_io<T>::st(out_or_dq, qbase + c, acc[d] * inv_l);
    }
    if (MODE == 0 && stats != nullptr && lane == 0) {
        const size_t sb = ((size_t)row * p.hq + h) * 3U;
        stats[sb] = m;
        stats[sb + 1] = l;
        stats[sb + 2] = 0.0f;
    }
}

// dK, dV: one warp per (packed key row, kv head); loops the q heads of the group and the
// query rows that may attend this key.
template <typename T>
__global__ void varlen_dkv_kernel(const T *q, const T *k, const T *v, const T *go, const int *cu, const float *stats,
                                  T *dk, T *dv, varlen_params p)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)p.n_tokens * p.hkv) {
        return;
    }
    const int row = (int)(w / p.hkv), hk = (int)(w % p.hkv);
    const int group = p.hq / p.hkv, dpl = (p.dh + 31) / 32;
    const size_t kbase = ((size_t)row * p.hkv + hk) * p.dh;
    if (row >= cu[p.batch]) {
        // rows beyond the last segment receive zero gradients
#pragma unroll
        for (int d = 0; d < MAX_DPL; ++d) {
            const int c = lane + 32 * d;
            if (d < dpl && c < p.dh) {
                gdb_io<T>::st(dk, kbase + c, 0.0f);
                gdb_io<T>::st(dv, kbase + c, 0.0f);
            }
        }
        return;
    }
    const int b = find_segment(cu, p.batch, row);
    const int start = cu[b], T_seg = cu[b + 1] - start, j = row - start;
    float kr[MAX_DPL], vr[MAX_DPL], ak[MAX_DPL], av[MAX_DPL];
#pragma unroll
    for (int d = 0; d < MAX_DPL; ++d) {
        const int c = lane + 32 * d;
        const bool ok = d < dpl && c < p.dh;
        kr[d] = ok ? gdb_io<T>::ld(k, kbase + c) : 0.0f;
        vr[d] = ok ? gdb_io<T>::ld(v, kbase + c) : 0.0f;
        ak[d] = av[d] = 0.0f;
    }
    int i_lo = 0, i_hi = T_seg;
    if (p.causal && p.prefix <= 0) {
        i_lo = j;
    }
    if (p.window > 0 && p.prefix <= 0 && j + p.window < i_hi) {
        i_hi = j + p.window;
    }
    for (int hh = 0; hh < group; ++hh) {
        const int h = hk * group + hh;
        for (int i = i_lo; i < i_hi; ++i) {
            if (!mask_allowed(i, j, p.causal, p.window, p.prefix)) {
                continue;
            }
            const size_t sb = ((size_t)(start + i) * p.hq + h) * 3U;
            const float l = stats[sb + 1];
            if (!(l > 0.0f)) {
                continue;
            }
            const size_t qb = ((size_t)(start + i) * p.hq + h) * p.dh;
            float s = 0.0f, dp = 0.0f, qv[MAX_DPL], gv[MAX_DPL];
#pragma unroll
            for (int d = 0; d < MAX_DPL; ++d) {
                const int c = lane + 32 * d;
                const bool ok = d < dpl && c < p.dh;
                qv[d] = ok ? gdb_io<T>::ld(q, qb + c) : 0.0f;
                gv[d] = ok ? gdb_io<T>::ld(go, qb + c) : 0.0f;
                s += qv[d] * kr[d];
                dp += gv[d] * vr[d];
            }
            s = gdb_warp_sum(s) * p.scale;
            dp = gdb_warp_sum(dp);
            const float prob = expf(s - stats[sb]) / l;
            const float ds = prob * (dp - stats[sb + 2]) * p.scale;
#pragma unroll
            for (int d = 0; d < MAX_DPL; ++d) {
                av[d] += prob * gv[d];
                ak[d] += ds * qv[d];
            }
        }
    }
#pragma unroll
    for (int d = 0; d < MAX_DPL; ++d) {
        const int c = lane + 32 * d;
        if (d < dpl && c < p.dh) {
            gdb_io<T>::st(dk, kbase + c, ak[d]);
            gdb_io<T>::st(dv, kbase + c, av[d]);
        }
    }
}

// ------------------------------------------------------------------ decode
using gdb_dec::decode_params;
using gdb_dec::decode_allowed;
using gdb_dec::decode_combine_query;

// Split-K decode: grid (ceil(queries / warps), splits). Each warp owns one (b, t, hq) query and the keys
// [split*chunk, split*chunk+chunk) of its live range (gdb_dec::decode_split_item); partial (m, l, acc) per split
// go to the workspace and are merged by decode_combine_query.
// `tickets` != NULL: the block that arrives last for its group of queries (over the splits) merges the
// partials and writes `out`, so no combine launch follows.
template <typename T, int DH>
__global__ void decode_split_kernel(const T *q, const T *kc, const T *vc, const int *pos_buf, float *part_ml,
                                    float *part_acc, decode_params p, int splits, T *out, unsigned *tickets)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long total = (long long)p.batch * p.tq * p.hq;
    const bool active = w < total;
    if (active) {
        const size_t item = (size_t)w * splits + blockIdx.y;
        gdb_dec::decode_split_item<T, DH, false>(q, kc, vc, pos_buf, part_ml + item * 2U, part_acc + item * DH, p, splits, w, (int)blockIdx.y, lane);
    }   // active
    if (tickets == nullptr) {
        return;
    }
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        last = atomicAdd(&tickets[blockIdx.x], 1U) == gridDim.y - 1U;
    }
    __syncthreads();
    if (last) {
        __threadfence();
        if (active) decode_combine_query<T, true>(part_ml + (size_t)w * splits * 2U, part_acc + (size_t)w * splits * DH, out + (size_t)w * DH, DH, splits, lane);
        if (threadIdx.x == 0) tickets[blockIdx.x] = 0U;
    }
}

template <typename T>
__global__ void decode_combine_kernel(const float *part_ml, const float *part_acc, T *out, long long total, int dh, int splits)
{
    gdb_pdl_sync();
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= total) {
        return;
    }
    decode_combine_query<T, true>(part_ml + (size_t)w * splits * 2U, part_acc + (size_t)w * splits * dh, out + (size_t)w * dh, dh, splits, lane);
}

// General head_dim decode: one warp per query, lanes split head_dim.
template <typename T>
__global__ void decode_generic_kernel(const T *q, const T *kc, const T *vc, const int *pos_buf, T *out, decode_params p)
{
    gdb_pdl_sync();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)p.batch * p.tq * p.hq) {
        return;
    }
    const int h = (int)(w % p.hq);
    const int t = (int)((w / p.hq) % p.tq);
    const int b = (int)(w / ((long long)p.hq * p.tq));
    const int hk = h / (p.hq / p.hkv);
    const int pos = p.pos_mode == 0 ? p.cache_pos : pos_buf[p.pos_mode == 2 ? b : 0];
    if (pos < 0) {
        return;
    }
    int live = pos + p.tq;
    if (live > p.tmax) live = p.tmax;
    const int qpos = pos + t;
    const int dpl = (p.dh + 31) / 32;
    const size_t qb = (size_t)w * p.dh;
    float qr[MAX_DPL], acc[MAX_DPL];
#pragma unroll
    for (int d = 0; d < MAX_DPL; ++d) {
        const int c = lane + 32 * d;
        qr[d] = (d < dpl && c < p.dh) ? gdb_io<T>::ld(q, qb + c) : 0.0f;
        acc[d] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    int j_hi = qpos + 1;
    if (p.prefix > 0 && qpos < p.prefix) j_hi = p.prefix;
    if (j_hi > live) j_hi = live;
    for (int j = 0; j < j_hi; ++j) {
        if (!decode_allowed(qpos, j, p.window, p.prefix)) continue;
        const size_t kb = (((size_t)b * p.tmax + j) * p.hkv + hk) * p.dh;
        float s = 0.0f;
#pragma unroll
        for (int d = 0; d < MAX_DPL; ++d) {
            const int c = lane + 32 * d;
            if (d < dpl && c < p.dh) s += qr[d] * gdb_io<T>::ld(kc, kb + c);
        }
        s = gdb_warp_sum(s) * p.scale;
        const float mnew = fmaxf(s, m);
        const float corr = expf(m - mnew), e = expf(s - mnew);
        l = l * corr + e;
#pragma unroll
        for (int d = 0; d < MAX_DPL; ++d) {
            const int c = lane + 32 * d;
            if (d < dpl && c < p.dh) acc[d] = acc[d] * corr + e * gdb_io<T>::ld(vc, kb + c);
        }
        m = mnew;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int d = 0; d < MAX_DPL; ++d) {
        const int c = lane + 32 * d;
        if (d < dpl && c < p.dh) gdb_io<T>::st(out, qb + c, acc[d] * inv);
    }
}

// ------------------------------------------------------------------ KV append
struct append_params {
    size_t total_units;
    unsigned unit, row_bytes, batch, tnew, tmax;
    int pos_mode;  // 0 scalar, 2 per-batch vector
    int cache_pos;
};
__device__ __forceinline__ void copy_unit(unsigned char *dst, const unsigned char *src, unsigned unit)
{
    if (unit == 16U) {
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
    } else if (unit == 4U) {
        *reinterpret_cast<unsigned *>(dst) = *reinterpret_cast<const unsigned *>(src);
    } else {
        *dst = *src;
    }
}
__global__ void kv_append_kernel(unsigned char *kc, unsigned char *vc, const unsigned char *kn, const unsigned char *vn,
                                 const int *pos_buf, append_params p)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < p.total_units; g += stride) {
        const size_t src = g * p.unit;
        const size_t row = src / p.row_bytes, within = src - row * p.row_bytes;
        const size_t b = row / p.tnew, t = row - b * p.tnew;
        if (b >= p.batch) continue;
        const int pos = p.pos_mode == 2 ? pos_buf[b] : p.cache_pos;
        if (pos < 0 || pos + (int)p.tnew > (int)p.tmax) continue;
        const size_t dst = ((b * p.tmax + (size_t)pos + t) * p.row_bytes) + within;
        copy_unit(kc + dst, kn + src, p.unit);
        copy_unit(vc + dst, vn + src, p.unit);
    }
}
__global__ void kv_append_packed_kernel(unsigned char *kc, unsigned char *vc, const unsigned char *kn,
                                        const unsigned char *vn, const int *pos_buf, const int *cu, append_params p)
{
    gdb_pdl_sync();
    const unsigned units_per_row = p.row_bytes / p.unit;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < p.total_units; g += stride) {
        const unsigned row = (unsigned)(g / units_per_row);
        const size_t within = (g - (size_t)row * units_per_row) * p.unit;
        if (cu[0] != 0 || (int)row >= cu[p.batch]) continue;
        const int b = find_segment(cu, (int)p.batch, (int)row);
        const int s0 = cu[b], s1 = cu[b + 1], t = (int)row - s0, pos = pos_buf[b];
        if (s0 < 0 || s1 < s0 || t < 0 || pos < 0 || pos + (s1 - s0) > (int)p.tmax) continue;
        const size_t src = (size_t)row * p.row_bytes + within;
        const size_t dst = (((size_t)b * p.tmax + (size_t)(pos + t)) * p.row_bytes) + within;
        copy_unit(kc + dst, kn + src, p.unit);
        copy_unit(vc + dst, vn + src, p.unit);
    }
}

// ------------------------------------------------------------------ host-side checks
bool attn_dtype(uint32_t dt) { return gdb_is_float_dtype(dt); }

gd_status varlen_check(const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v,
                       const gd_backend_tensor_view *cu, const gd_backend_sdpa_varlen_args *a, varlen_params *p)
{
    if (q == NULL || k == NULL || v == NULL || cu == NULL || a == NULL || q->rank != 3U || k->rank != 3U || v->rank != 3U ||
        k->dtype != q->dtype || v->dtype != q->dtype || cu->count < 2U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!attn_dtype(q->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const int64_t n = q->shape[0], hq = q->shape[1], dh = q->shape[2], hkv = k->shape[1];
    if (n <= 0 || hq <= 0 || dh <= 0 || hkv <= 0 || (hq % hkv) != 0 || k->shape[0] != n || v->shape[0] != n ||
        k->shape[2] != dh || v->shape[1] != hkv || v->shape[2] != dh || n > INT32_MAX ||
        q->count != (size_t)(n * hq * dh) || k->count != (size_t)(n * hkv * dh) || v->count != k->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (dh > 32 * MAX_DPL) {
        return GD_ERR_UNSUPPORTED;
    }
    p->n_tokens = (int)n;
    p->batch = (int)cu->count - 1;
    p->hq = (int)hq;
    p->hkv = (int)hkv;
    p->dh = (int)dh;
    p->causal = a->causal != 0U;
    p->window = (int)a->sliding_window;
    p->prefix = (int)a->prefix_len;
    p->scale = a->scale > 0.0f ? a->scale : (float)(1.0 / sqrt((double)dh));
    return GD_OK;
}

template <typename T>
gd_status varlen_fwd_generic(gd_backend *be, const void *q, const void *k, const void *v, const int *cu, void *out,
                             float *stats, const varlen_params &p)
{
    const long long warps = (long long)p.n_tokens * p.hq;
    gdb_launch(varlen_row_kernel<T, 0>, (unsigned)((warps + 3) / 4), 128, 0, be->stream, (const T *)q, (const T *)k, (const T *)v, nullptr, cu, (T *)out, stats, p);
    return gdb_launched(be, "sdpa_varlen generic");
}

template <typename T>
gd_status varlen_bwd_generic(gd_backend *be, const void *go, const void *q, const void *k, const void *v, const int *cu,
                             void *dq, void *dk, void *dv, float *stats, const varlen_params &p)
{
    const long long warps = (long long)p.n_tokens * p.hq;
    gdb_launch(varlen_row_kernel<T, 1>, (unsigned)((warps + 3) / 4), 128, 0, be->stream, (const T *)q, (const T *)k, (const T *)v, (const T *)go, cu, nullptr, stats, p);
    gd_status st = gdb_launched(be, "sdpa_varlen bwd stats");
    if (st != GD_OK) return st;
    gdb_launch(varlen_row_kernel<T, 2>, (unsigned)((warps + 3) / 4), 128, 0, be->stream, (const T *)q, (const T *)k, (const T *)v, (const T *)go, cu, (T *)dq, stats, p);
    st = gdb_launched(be, "sdpa_varlen bwd dq");
    if (st != GD_OK) return st;
    const long long kw = (long long)p.n_tokens * p.hkv;
    gdb_launch(varlen_dkv_kernel<T>, (unsigned)((kw + 3) / 4), 128, 0, be->stream, (const T *)q, (const T *)k, (const T *)v, (const T *)go, cu, stats, (T *)dk, (T *)dv, p);
    return gdb_launched(be, "sdpa_varlen bwd dkv");
}

gd_status decode_common(gd_backend *be, const gd_backend_tensor_view *q, const gd_backend_tensor_view *kc,
                        const gd_backend_tensor_view *vc, const gd_backend_tensor_view *cache_pos,
                        const gd_backend_tensor_view *out, const gd_backend_sdpa_decode_args *a, int pos_mode)
{
    if (be == NULL || q == NULL || kc == NULL || vc == NULL || out == NULL || a == NULL || q->rank != 4U ||
        kc->rank != 4U || vc->rank != 4U || kc->dtype != q->dtype || vc->dtype != q->dtype || out->dtype != q->dtype ||
        out->count != q->count || (pos_mode != 0 && cache_pos == NULL)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = q->dtype;
    if (!attn_dtype(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    decode_params p;
    p.batch = (int)q->shape[0];
    p.tq = (int)q->shape[1];
    p.hq = (int)q->shape[2];
    p.dh = (int)q->shape[3];
    p.tmax = (int)kc->shape[1];
    p.hkv = (int)kc->shape[2];
    if (p.batch <= 0 || p.tq <= 0 || p.hq <= 0 || p.dh <= 0 || p.tmax <= 0 || p.hkv <= 0 || (p.hq % p.hkv) != 0 ||
        kc->shape[0] != q->shape[0] || kc->shape[3] != q->shape[3] || kc->count != vc->count ||
        q->count != (size_t)p.batch * p.tq * p.hq * p.dh || kc->count != (size_t)p.batch * p.tmax * p.hkv * p.dh) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (p.dh > 32 * MAX_DPL) {
        return GD_ERR_UNSUPPORTED;
    }
    p.window = (int)a->sliding_window;
    p.prefix = (int)a->prefix_len;
    p.pos_mode = pos_mode;
    p.cache_pos = a->cache_pos;
    p.scale = a->scale > 0.0f ? a->scale : (float)(1.0 / sqrt((double)p.dh));
    const int *pp = NULL;
    if (pos_mode != 0) {
        if (cache_pos->count < (size_t)(pos_mode == 2 ? p.batch : 1)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        pp = (const int *)gdb_tv_ptr(cache_pos, GDB_DTYPE_I32);
        if (pp == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const void *qp = gdb_tv_ptr(q, dt), *kp = gdb_tv_ptr(kc, dt), *vp = gdb_tv_ptr(vc, dt);
    void *op = gdb_tv_ptr(out, dt);
    if (qp == NULL || kp == NULL || vp == NULL || op == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const long long total = (long long)p.batch * p.tq * p.hq;
    const bool al16 = (((uintptr_t)kp | (uintptr_t)vp) % 16U) == 0U;
    if ((p.dh == 64 || p.dh == 128) && dt != GDB_DTYPE_F32 && al16) {
        // choose splits so that about `wps` warps per SM are in flight (GDB200_DECODE_WARPS_PER_SM, default 32)
        static int wps = 0;
        if (wps == 0) {
            const char *env = getenv("GDB200_DECODE_WARPS_PER_SM");
            wps = env != NULL && atoi(env) > 0 ? atoi(env) : 32;
        }
        const int splits = gdb_dec::decode_choose_splits(be->sm_count, p.batch, p.tq, p.hq, p.dh, p.tmax, wps);
        const size_t need = (size_t)total * splits * (2U + (size_t)p.dh) * sizeof(float);
        if (need <= be->ws_bytes) {
            float *ml = (float *)be->ws;
            float *pa = ml + (size_t)total * splits * 2U;
            dim3 grid((unsigned)((total + 3) / 4), (unsigned)splits);
            const bool fused = grid.x <= (unsigned)GDB_TICKET_WORDS;
#define GDB_DECODE(T, DH) gdb_launch(decode_split_kernel<T, DH>, grid, 128, 0, be->stream, (const T *)qp, (const T *)kp, (const T *)vp, pp, ml, pa, p, splits, (T *)op, fused ? gdb_tickets(be) : (unsigned *)nullptr)
            if (dt == GDB_DTYPE_F16) {
                if (p.dh == 64) GDB_DECODE(__half, 64); else GDB_DECODE(__half, 128);
            } else {
                if (p.dh == 64) GDB_DECODE(__nv_bfloat16, 64); else GDB_DECODE(__nv_bfloat16, 128);
            }
#undef GDB_DECODE
            gd_status st = gdb_launched(be, "sdpa_decode split");
            if (st != GD_OK || fused) return st;
            if (dt == GDB_DTYPE_F16) {
                gdb_launch(decode_combine_kernel<__half>, (unsigned)((total + 3) / 4), 128, 0, be->stream, ml, pa, (__half *)op, total, p.dh, splits);
            } else {
                gdb_launch(decode_combine_kernel<__nv_bfloat16>, (unsigned)((total + 3) / 4), 128, 0, be->stream, ml, pa, (__nv_bfloat16 *)op, total, p.dh, splits);
            }
            return gdb_launched(be, "sdpa_decode combine");
        }
    }
    const unsigned grid = (unsigned)((total + 3) / 4);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(decode_generic_kernel<__half>, grid, 128, 0, be->stream, (const __half *)qp, (const __half *)kp, (const __half *)vp, pp, (__half *)op, p);
    } else if (dt == GDB_DTYPE_BF16) {
        gdb_launch(decode_generic_kernel<__nv_bfloat16>, grid, 128, 0, be->stream, (const __nv_bfloat16 *)qp, (const __nv_bfloat16 *)kp, (const __nv_bfloat16 *)vp, pp, (__nv_bfloat16 *)op, p);
    } else {
        gdb_launch(decode_generic_kernel<float>, grid, 128, 0, be->stream, (const float *)qp, (const float *)kp, (const float *)vp, pp, (float *)op, p);
    }
    return gdb_launched(be, "sdpa_decode generic");
}

gd_status append_common(gd_backend *be, const gd_backend_tensor_view *kc, const gd_backend_tensor_view *vc,
                        const gd_backend_tensor_view *cache_pos, const gd_backend_tensor_view *cu,
                        const gd_backend_tensor_view *kn, const gd_backend_tensor_view *vn,
                        const gd_backend_kv_cache_append_args *a, int mode)
{
    // mode 0: scalar position, new [B, Tnew, H, Dh]; mode 2: per-batch positions; mode 3: packed [N, H, Dh] + cu
    if (be == NULL || kc == NULL || vc == NULL || kn == NULL || vn == NULL || kc->rank != 4U || vc->rank != 4U ||
        kc->dtype != vc->dtype || kn->dtype != kc->dtype || vn->dtype != kc->dtype || kc->count != vc->count ||
        kn->count != vn->count || (mode == 0 && a == NULL) || (mode >= 2 && cache_pos == NULL) || (mode == 3 && cu == NULL)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = kc->dtype;
    const size_t es = gdb_dtype_size(dt);
    if (es == 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    append_params p;
    memset(&p, 0, sizeof(p));
    p.batch = (unsigned)kc->shape[0];
    p.tmax = (unsigned)kc->shape[1];
    const size_t row_elems = (size_t)kc->shape[2] * (size_t)kc->shape[3];
    p.row_bytes = (unsigned)(row_elems * es);
    if (p.batch == 0U || p.tmax == 0U || row_elems == 0U || kc->count != (size_t)p.batch * p.tmax * row_elems) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    size_t new_rows;
    if (mode == 3) {
        if (kn->rank != 3U || (size_t)kn->shape[1] * (size_t)kn->shape[2] != row_elems || cu->count != (size_t)p.batch + 1U ||
            cache_pos->count < p.batch) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        new_rows = (size_t)kn->shape[0];
    } else {
        if (kn->rank != 4U || (unsigned)kn->shape[0] != p.batch || (size_t)kn->shape[2] * (size_t)kn->shape[3] != row_elems ||
            kn->shape[1] <= 0 || (mode == 2 && cache_pos->count < p.batch)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        p.tnew = (unsigned)kn->shape[1];
        new_rows = (size_t)p.batch * p.tnew;
    }
    if (kn->count != new_rows * row_elems) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    unsigned char *kcp = (unsigned char *)gdb_tv_ptr(kc, dt), *vcp = (unsigned char *)gdb_tv_ptr(vc, dt);
    const unsigned char *knp = (const unsigned char *)gdb_tv_ptr(kn, dt), *vnp = (const unsigned char *)gdb_tv_ptr(vn, dt);
    const int *pp = mode >= 2 ? (const int *)gdb_tv_ptr(cache_pos, GDB_DTYPE_I32) : NULL;
    const int *cup = mode == 3 ? (const int *)gdb_tv_ptr(cu, GDB_DTYPE_I32) : NULL;
    if (kcp == NULL || vcp == NULL || knp == NULL || vnp == NULL || (mode >= 2 && pp == NULL) || (mode == 3 && cup == NULL)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (new_rows == 0U) {
        return GD_OK;
    }
    const uintptr_t al = (uintptr_t)kcp | (uintptr_t)vcp | (uintptr_t)knp | (uintptr_t)vnp | p.row_bytes;
    p.unit = (al % 16U) == 0U ? 16U : ((al % 4U) == 0U ? 4U : 1U);
    p.total_units = new_rows * (p.row_bytes / p.unit);
    p.pos_mode = mode == 0 ? 0 : 2;
    p.cache_pos = a != NULL ? a->cache_pos : 0;
    const unsigned grid = gdb_grid_for(p.total_units, 256, be, 16);
    if (mode == 3) {
        gdb_launch(kv_append_packed_kernel, grid, 256, 0, be->stream, kcp, vcp, knp, vnp, pp, cup, p);
    } else {
        gdb_launch(kv_append_kernel, grid, 256, 0, be->stream, kcp, vcp, knp, vnp, pp, p);
    }
    return gdb_launched(be, "kv_cache_append");
}

}  // namespace

extern "C" {

gd_status gd_backend_sdpa_varlen(gd_backend *be, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v, const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *out, const gd_backend_tensor_view *stats, const gd_backend_sdpa_varlen_args *args)
{
    varlen_params p;
    if (be == NULL || out == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gd_status st = varlen_check(q, k, v, cu_seqlens, args, &p);
    if (st != GD_OK) {
        return st;
    }
    const uint32_t dt = q->dtype;
    if (out->dtype != dt || out->count != q->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *qp = gdb_tv_ptr(q, dt), *kp = gdb_tv_ptr(k, dt), *vp = gdb_tv_ptr(v, dt);
    const int *cu = (const int *)gdb_tv_ptr(cu_seqlens, GDB_DTYPE_I32);
    void *op = gdb_tv_ptr(out, dt);
    float *sp = NULL;
    if (stats != NULL) {
        if (stats->count != (size_t)p.n_tokens * p.hq * 3U || (sp = (float *)gdb_tv_ptr(stats, GDB_DTYPE_F32)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    if (qp == NULL || kp == NULL || vp == NULL || cu == NULL || op == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gdb_flash_args fa = {qp, kp, vp, NULL, cu, op, NULL, NULL, sp, p.n_tokens, p.batch, p.hq, p.hkv, p.dh,
                         p.causal, p.window, p.prefix, (int)args->max_seqlen, p.scale, dt};
    st = gdb_flash_varlen_forward(be, &fa);
    if (st != GD_ERR_UNSUPPORTED) {
        return st;
    }
    if (dt == GDB_DTYPE_F16) return varlen_fwd_generic<__half>(be, qp, kp, vp, cu, op, sp, p);
    if (dt == GDB_DTYPE_BF16) return varlen_fwd_generic<__nv_bfloat16>(be, qp, kp, vp, cu, op, sp, p);
    return varlen_fwd_generic<float>(be, qp, kp, vp, cu, op, sp, p);
}

// `out` (the forward output) and `dq_accum` (FP32 scratch of q's element count) are optional: with both, forward
// statistics and head_dim 64 the backward runs as one attention pass.
static gd_status sdpa_varlen_backward_impl(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v, const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k, const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *stats, const gd_backend_sdpa_varlen_args *args, const gd_backend_tensor_view *out, const gd_backend_tensor_view *dq_accum,
                                           int32_t *query_grad_in_accum = NULL)
{
    varlen_params p;
    if (be == NULL || grad_out == NULL || grad_q == NULL || grad_k == NULL || grad_v == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (query_grad_in_accum != NULL) {
        *query_grad_in_accum = 0;
    }
    gd_status st = varlen_check(q, k, v, cu_seqlens, args, &p);
    if (st != GD_OK) {
        return st;
    }
    const uint32_t dt = q->dtype;
    if (grad_out->dtype != dt || grad_q->dtype != dt || grad_k->dtype != dt || grad_v->dtype != dt ||
        grad_out->count != q->count || grad_q->count != q->count || grad_k->count != k->count || grad_v->count != v->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *gp = gdb_tv_ptr(grad_out, dt), *qp = gdb_tv_ptr(q, dt), *kp = gdb_tv_ptr(k, dt), *vp = gdb_tv_ptr(v, dt);
    const int *cu = (const int *)gdb_tv_ptr(cu_seqlens, GDB_DTYPE_I32);
    void *dq = gdb_tv_ptr(grad_q, dt), *dk = gdb_tv_ptr(grad_k, dt), *dv = gdb_tv_ptr(grad_v, dt);
    if (gp == NULL || qp == NULL || kp == NULL || vp == NULL || cu == NULL || dq == NULL || dk == NULL || dv == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t stats_count = (size_t)p.n_tokens * p.hq * 3U;
    float *sp;
    bool have_fwd_stats = false;
    if (stats != NULL) {
        if (stats->count != stats_count || (sp = (float *)gdb_tv_ptr(stats, GDB_DTYPE_F32)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        have_fwd_stats = args->use_forward_stats != 0U;
    } else {
        // private stats: tail of the workspace (the flash kernels use its head)
        if (stats_count * sizeof(float) > be->ws_bytes / 4U) {
            return GD_ERR_OUT_OF_MEMORY;
        }
        sp = (float *)(be->ws + be->ws_bytes - ((stats_count * sizeof(float) + 255U) & ~(size_t)255U));
    }
    gdb_flash_args fa = {qp, kp, vp, gp, cu, dq, dk, dv, sp, p.n_tokens, p.batch, p.hq, p.hkv, p.dh,
                         p.causal, p.window, p.prefix, (int)args->max_seqlen, p.scale, dt};
    if (out != NULL && dq_accum != NULL && have_fwd_stats) {
        if (out->dtype != dt || out->count != q->count || dq_accum->count != q->count) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        const void *op = gdb_tv_ptr(out, dt);
        float *acc = (float *)gdb_tv_ptr(dq_accum, GDB_DTYPE_F32);
        if (op == NULL || acc == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        fa.keep_dq32 = query_grad_in_accum != NULL ? 1 : 0;
        st = gdb_flash_varlen_backward_with_out(be, &fa, op, acc);
        if (st != GD_ERR_UNSUPPORTED) {
            if (st == GD_OK && query_grad_in_accum != NULL) {
                *query_grad_in_accum = 1;
            }
            return st;
        }
        fa.keep_dq32 = 0;
    }
    st = gdb_flash_varlen_backward(be, &fa, have_fwd_stats);
    if (st != GD_ERR_UNSUPPORTED) {
        return st;
    }
    if (dt == GDB_DTYPE_F16) return varlen_bwd_generic<__half>(be, gp, qp, kp, vp, cu, dq, dk, dv, sp, p);
    if (dt == GDB_DTYPE_BF16) return varlen_bwd_generic<__nv_bfloat16>(be, gp, qp, kp, vp, cu, dq, dk, dv, sp, p);
    return varlen_bwd_generic<float>(be, gp, qp, kp, vp, cu, dq, dk, dv, sp, p);
}

gd_status gd_backend_sdpa_varlen_backward(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v, const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k, const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *stats, const gd_backend_sdpa_varlen_args *args)
{
    return sdpa_varlen_backward_impl(be, grad_out, q, k, v, cu_seqlens, grad_q, grad_k, grad_v, stats, args, NULL, NULL);
}

gd_status gdb200_sdpa_varlen_backward_with_output(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v, const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *out, const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k, const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *stats, const gd_backend_tensor_view *dq_accum, const gd_backend_sdpa_varlen_args *args)
{
    if (out == NULL || dq_accum == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return sdpa_varlen_backward_impl(be, grad_out, q, k, v, cu_seqlens, grad_q, grad_k, grad_v, stats, args, out, dq_accum);
}

gd_status gdb200_sdpa_varlen_backward_with_output_q32(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v, const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *out, const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k, const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *stats, const gd_backend_tensor_view *dq_accum, const gd_backend_sdpa_varlen_args *args, int32_t *query_grad_in_accum)
{
    if (out == NULL || dq_accum == NULL || query_grad_in_accum == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return sdpa_varlen_backward_impl(be, grad_out, q, k, v, cu_seqlens, grad_q, grad_k, grad_v, stats, args, out, dq_accum, query_grad_in_accum);
}

gd_status gd_backend_sdpa_decode(gd_backend *be, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache, const gd_backend_tensor_view *cache_pos, const gd_backend_tensor_view *out, const gd_backend_sdpa_decode_args *args)
{
    return decode_common(be, q, k_cache, v_cache, cache_pos, out, args, 1);
}
gd_status gd_backend_sdpa_decode_at(gd_backend *be, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache, const gd_backend_tensor_view *out, const gd_backend_sdpa_decode_args *args)
{
    return decode_common(be, q, k_cache, v_cache, NULL, out, args, 0);
}
gd_status gd_backend_sdpa_decode_positions(gd_backend *be, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache, const gd_backend_tensor_view *cache_pos, const gd_backend_tensor_view *out, const gd_backend_sdpa_decode_args *args)
{
    return decode_common(be, q, k_cache, v_cache, cache_pos, out, args, 2);
}
gd_status gd_backend_kv_cache_append_at(gd_backend *be, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache, const gd_backend_tensor_view *k_new, const gd_backend_tensor_view *v_new, const gd_backend_kv_cache_append_args *args)
{
    return append_common(be, k_cache, v_cache, NULL, NULL, k_new, v_new, args, 0);
}
gd_status gd_backend_kv_cache_append_positions(gd_backend *be, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache, const gd_backend_tensor_view *cache_pos, const gd_backend_tensor_view *k_new, const gd_backend_tensor_view *v_new, const gd_backend_kv_cache_append_args *args)
{
    return append_common(be, k_cache, v_cache, cache_pos, NULL, k_new, v_new, args, 2);
}
gd_status gd_backend_kv_cache_append_packed(gd_backend *be, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache, const gd_backend_tensor_view *cache_pos, const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *k_new, const gd_backend_tensor_view *v_new, const gd_backend_kv_cache_append_args *args)
{
    return append_common(be, k_cache, v_cache, cache_pos, cu_seqlens, k_new, v_new, args, 3);
}

}  // extern "C"
