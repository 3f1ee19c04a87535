// Embedding gather / scatter-add and rotary position embedding kernels.
//
// Reference arithmetic:
//   embedding: src/ops/embedding/metal_embedding.metal:11-179 (invalid id -> NaN row forward,
//              skipped backward; backward = zero F32 scratch, atomic scatter-add, cast).
//   qkv_split_rope: src/ops/qkv_split_rope/metal_qkv_split_rope.metal:6-253 and
//              metal_qkv_split_rope.m:40-64,228 (angle = pos * 2^(pair * -2*log2(theta)/n_dims),
//              cos/sin table for head_dim 64, theta 10000, positions < 512).
//   rope: same rotation applied to one tensor [..., heads, head_dim] (src/ops/rope/).
#include "common.cuh"
#include "decode_parts.cuh"

#include <math.h>
#include <stdlib.h>

namespace {

using namespace gdb_dec;   // rope_params, rope_cos_sin, rope_lo / rope_hi, the cos / sin table constants

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_fwd_kernel(const T *table, const int *ids, T *out, size_t n_ids, size_t vocab, size_t dim)
{
    gdb_pdl_sync();
    const size_t n = n_ids * dim, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t row = i / dim, c = i - row * dim;
        const int id = ids[row];
        if (id < 0 || (size_t)id >= vocab) {
            gdb_io<T>::st(out, i, __int_as_float(0x7fc00000));
        } else {
            out[i] = table[(size_t)id * dim + c];
        }
    }
}
// 16-byte units; nan_word is the 32-bit pattern of a NaN pair (F16 0x7e007e00, BF16 0x7fc07fc0) or one F32 NaN.
__global__ void embedding_fwd_vec_kernel(const uint4 *table, const int *ids, uint4 *out, size_t n_ids, size_t vocab,
                                         size_t row_vecs, unsigned nan_word)
{
    gdb_pdl_sync();
    const size_t n = n_ids * row_vecs, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t row = i / row_vecs, v = i - row * row_vecs;
        const int id = __ldg(&ids[row]);
        if (id < 0 || (size_t)id >= vocab) {
            out[i] = make_uint4(nan_word, nan_word, nan_word, nan_word);
        } else {
            out[i] = __ldg(&table[(size_t)id * row_vecs + v]);
        }
    }
}

template <typename T>
__global__ void embedding_scatter_kernel(const T *grad, const int *ids, float *acc, size_t n_ids, size_t vocab, size_t dim)
{
    gdb_pdl_sync();
    const size_t n = n_ids * dim, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t row = i / dim, c = i - row * dim;
        const int id = __ldg(&ids[row]);
        if (id >= 0 && (size_t)id < vocab) {
            atomicAdd(&acc[(size_t)id * dim + c], gdb_io<T>::ld(grad, i));
        }
    }
}
template <typename T>
__global__ void cast_from_f32_kernel(const float *src, T *dst, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        gdb_io<T>::st(dst, i, src[i]);
    }
}

// ------------------------------------------------------------------ rope
// One thread per (token, head, pair). FWD: src = qkv [N, 3*H*Dh] -> q,k,v [N,H,Dh].
// BWD: (gq, gk, gv) -> dqkv with sin_sign = -1.
template <typename T, bool FWD>
__global__ void qkv_split_rope_kernel(const T *a0, const T *a1, const T *a2, const int *pos_ids, T *o0, T *o1, T *o2,
                                      rope_params p, const float *table)
{
    gdb_pdl_sync();
    const unsigned half_dims = p.n_dims >> 1;
    const size_t area = (size_t)p.heads * p.head_dim;
    const size_t n = p.tokens * p.heads * half_dims, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned pair = (unsigned)(i % half_dims);
        const size_t th = i / half_dims;
        const unsigned h = (unsigned)(th % p.heads);
        const size_t token = th / p.heads;
        const unsigned ia = p.interleaved ? (pair << 1) : pair;
        const unsigned ib = p.interleaved ? (ia + 1U) : (pair + half_dims);
        float c, s;
        rope_cos_sin(p, table, pair, __ldg(&pos_ids[token]), &c, &s);
        const size_t packed = token * area * 3U + (size_t)h * p.head_dim;
        const size_t split = token * area + (size_t)h * p.head_dim;
        if (FWD) {
            const float q0 = gdb_io<T>::ld(a0, packed + ia), q1 = gdb_io<T>::ld(a0, packed + ib);
            const float k0 = gdb_io<T>::ld(a0, packed + area + ia), k1 = gdb_io<T>::ld(a0, packed + area + ib);
            gdb_io<T>::st(o0, split + ia, q0 * c - q1 * s);
            gdb_io<T>::st(o0, split + ib, q0 * s + q1 * c);
            gdb_io<T>::st(o1, split + ia, k0 * c - k1 * s);
            gdb_io<T>::st(o1, split + ib, k0 * s + k1 * c);
            o2[split + ia] = a0[packed + 2U * area + ia];
            o2[split + ib] = a0[packed + 2U * area + ib];
        } else {
            const float q0 = gdb_io<T>::ld(a0, split + ia), q1 = gdb_io<T>::ld(a0, split + ib);
            const float k0 = gdb_io<T>::ld(a1, split + ia), k1 = gdb_io<T>::ld(a1, split + ib);
            gdb_io<T>::st(o0, packed + ia, q0 * c - q1 * s);
            gdb_io<T>::st(o0, packed + ib, q0 * s + q1 * c);
            gdb_io<T>::st(o0, packed + area + ia, k0 * c - k1 * s);
            gdb_io<T>::st(o0, packed + area + ib, k0 * s + k1 * c);
            o0[packed + 2U * area + ia] = a2[split + ia];
            o0[packed + 2U * area + ib] = a2[split + ib];
        }
    }
}

// Fast path: NeoX half-split, n_dims == head_dim, head_dim % 16 == 0, 16-byte aligned tensors.
// One thread handles 8 consecutive pairs of one (token, head): two 16-byte loads per source.
// tmax > 0 (forward only): o1 / o2 are K / V caches [tokens, tmax, heads, head_dim] and the rotated key and the value of
// token t go to cache slot pos_ids[t] (one new token per cache row: the decode step), skipped when the slot is out of range.
template <typename T, bool FWD>
__global__ void qkv_split_rope_vec8_kernel(const T *a0, const T *a1, const T *a2, const int *pos_ids, T *o0, T *o1, T *o2,
                                           rope_params p, const float *table, unsigned tmax = 0, const float *q32 = nullptr)
{
    // q32 != nullptr (backward only): the query gradient comes unrounded from an FP32 accumulator [tokens, heads, head_dim]
    // and is rounded to T on load, which is what a separate conversion pass would have stored in a0.
    gdb_pdl_sync();
    const unsigned half_dims = p.head_dim >> 1, groups = half_dims >> 3;
    const size_t area = (size_t)p.heads * p.head_dim;
    const size_t n = p.tokens * p.heads * groups, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        unsigned grp, h;
        size_t token;
        if (n <= 0xffffffffULL) {   // 32-bit divisions (a 64-bit one costs tens of instructions per vector)
            const unsigned iu = (unsigned)i, th = iu / groups;
            grp = iu - th * groups;
            const unsigned tk = th / (unsigned)p.heads;
            h = th - tk * (unsigned)p.heads;
            token = tk;
        } else {
            grp = (unsigned)(i % groups);
            const size_t th = i / groups;
            h = (unsigned)(th % p.heads);
            token = th / p.heads;
        }
        const int pos = __ldg(&pos_ids[token]);
        const size_t packed = token * area * 3U + (size_t)h * p.head_dim + grp * 8U;
        const size_t split = token * area + (size_t)h * p.head_dim + grp * 8U;
        gdb_vec8<T> qa, qb, ka, kb, va, vb;
        if (FWD) {
            qa.raw = *reinterpret_cast<const uint4 *>(a0 + packed);
            qb.raw = *reinterpret_cast<const uint4 *>(a0 + packed + half_dims);
            ka.raw = *reinterpret_cast<const uint4 *>(a0 + packed + area);
            kb.raw = *reinterpret_cast<const uint4 *>(a0 + packed + area + half_dims);
            va.raw = *reinterpret_cast<const uint4 *>(a0 + packed + 2U * area);
            vb.raw = *reinterpret_cast<const uint4 *>(a0 + packed + 2U * area + half_dims);
        } else {
            if (q32 != nullptr) {
                const float4 l0 = *reinterpret_cast<const float4 *>(q32 + split), l1 = *reinterpret_cast<const float4 *>(q32 + split + 4U);
                const float4 h0 = *reinterpret_cast<const float4 *>(q32 + split + half_dims), h1 = *reinterpret_cast<const float4 *>(q32 + split + half_dims + 4U);
                const float lo[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w}, hi[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    qa.set(e, lo[e]);
                    qb.set(e, hi[e]);
                }
            } else {
                qa.raw = *reinterpret_cast<const uint4 *>(a0 + split);
                qb.raw = *reinterpret_cast<const uint4 *>(a0 + split + half_dims);
            }
            ka.raw = *reinterpret_cast<const uint4 *>(a1 + split);
            kb.raw = *reinterpret_cast<const uint4 *>(a1 + split + half_dims);
            va.raw = *reinterpret_cast<const uint4 *>(a2 + split);
            vb.raw = *reinterpret_cast<const uint4 *>(a2 + split + half_dims);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float c, s;
            rope_cos_sin(p, table, grp * 8U + (unsigned)e, pos, &c, &s);
            const float q0 = qa.get(e), q1 = qb.get(e), k0 = ka.get(e), k1 = kb.get(e);
            qa.set(e, rope_lo(q0, q1, c, s));
            qb.set(e, rope_hi(q0, q1, c, s));
            ka.set(e, rope_lo(k0, k1, c, s));
            kb.set(e, rope_hi(k0, k1, c, s));
        }
        if (FWD) {
            *reinterpret_cast<uint4 *>(o0 + split) = qa.raw;
            *reinterpret_cast<uint4 *>(o0 + split + half_dims) = qb.raw;
            size_t kv = split;
            if (tmax != 0U) {
                if (pos < 0 || (unsigned)pos >= tmax) continue;
                kv = (token * tmax + (size_t)pos) * area + (size_t)h * p.head_dim + grp * 8U;
            }
            *reinterpret_cast<uint4 *>(o1 + kv) = ka.raw;
            *reinterpret_cast<uint4 *>(o1 + kv + half_dims) = kb.raw;
            *reinterpret_cast<uint4 *>(o2 + kv) = va.raw;
            *reinterpret_cast<uint4 *>(o2 + kv + half_dims) = vb.raw;
        } else {
            *reinterpret_cast<uint4 *>(o0 + packed) = qa.raw;
            *reinterpret_cast<uint4 *>(o0 + packed + half_dims) = qb.raw;
            *reinterpret_cast<uint4 *>(o0 + packed + area) = ka.raw;
            *reinterpret_cast<uint4 *>(o0 + packed + area + half_dims) = kb.raw;
            *reinterpret_cast<uint4 *>(o0 + packed + 2U * area) = va.raw;
            *reinterpret_cast<uint4 *>(o0 + packed + 2U * area + half_dims) = vb.raw;
        }
    }
}

// Plain rope on x [tokens, heads, head_dim]; dims >= n_dims are copied through.
template <typename T>
__global__ void rope_kernel(const T *x, const int *pos_ids, T *out, rope_params p)
{
    gdb_pdl_sync();
    const size_t n = p.tokens * p.heads * p.head_dim, stride = (size_t)gridDim.x * blockDim.x;
    const unsigned half_dims = p.n_dims >> 1;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned d = (unsigned)(i % p.head_dim);
        const size_t th = i / p.head_dim;
        const size_t token = th / p.heads;
        if (d >= p.n_dims) {
            out[i] = x[i];
            continue;
        }
        unsigned pair, other;
        bool first;
        if (p.interleaved) {
            pair = d >> 1;
            first = (d & 1U) == 0U;
            other = first ? d + 1U : d - 1U;
        } else {
            first = d < half_dims;
            pair = first ? d : d - half_dims;
            other = first ? d + half_dims : d - half_dims;
        }
        float c, s;
        rope_cos_sin(p, nullptr, pair, __ldg(&pos_ids[token]), &c, &s);
        const float self = gdb_io<T>::ld(x, i), oth = gdb_io<T>::ld(x, th * p.head_dim + other);
        gdb_io<T>::st(out, i, first ? self * c - oth * s : oth * s + self * c);
    }
}

gd_status ensure_rope_table(gd_backend *be)
{
    if (be->rope_table != NULL) {
        return GD_OK;
    }
    const size_t n = (size_t)TABLE_POSITIONS * TABLE_PAIRS * 2U;
    float *host = (float *)malloc(n * sizeof(float));
    if (host == NULL) {
        return GD_ERR_OUT_OF_MEMORY;
    }
    const float freq_scale = -2.0f * log2f(TABLE_THETA) / (float)TABLE_HEAD_DIM;
    for (unsigned pos = 0; pos < TABLE_POSITIONS; ++pos) {
        for (unsigned pair = 0; pair < TABLE_PAIRS; ++pair) {
            const float angle = (float)pos * exp2f((float)pair * freq_scale);
            host[((size_t)pos * TABLE_PAIRS + pair) * 2U] = cosf(angle);
            host[((size_t)pos * TABLE_PAIRS + pair) * 2U + 1U] = sinf(angle);
        }
    }
    cudaError_t e = cudaMalloc((void **)&be->rope_table, n * sizeof(float));
    if (e == cudaSuccess) {
        e = cudaMemcpyAsync(be->rope_table, host, n * sizeof(float), cudaMemcpyHostToDevice, be->stream);
        if (e == cudaSuccess) {
            e = cudaStreamSynchronize(be->stream);
        }
    }
    free(host);
    if (e != cudaSuccess) {
        cudaFree(be->rope_table);
        be->rope_table = NULL;
        return gdb_fail(be, e, "rope table");
    }
    return GD_OK;
}

bool rope_args_ok(const gd_backend_rope_args *a, uint32_t head_dim)
{
    return a != NULL && isfinite(a->theta) && a->theta > 0.0f && a->n_dims > 0U && (a->n_dims & 1U) == 0U &&
           a->n_dims <= head_dim;
}

template <bool FWD>
gd_status qkv_dispatch(gd_backend *be, const gd_backend_tensor_view *s0, const gd_backend_tensor_view *s1,
                       const gd_backend_tensor_view *s2, const gd_backend_tensor_view *pos_ids,
                       const gd_backend_tensor_view *d0, const gd_backend_tensor_view *d1,
                       const gd_backend_tensor_view *d2, uint32_t n_heads, uint32_t head_dim,
                       const gd_backend_rope_args *args, uint32_t cache_tmax = 0, const gd_backend_tensor_view *sq32 = NULL)
{
    // FWD: s0 = qkv, d0..d2 = q,k,v. BWD: s0..s2 = gq,gk,gv, d0 = dqkv; with sq32 the query gradient is that FP32 tensor and s0 is unused.
    const gd_backend_tensor_view *packed = FWD ? s0 : d0;
    const gd_backend_tensor_view *sq = FWD ? d0 : (sq32 != NULL ? s1 : s0), *sk = FWD ? d1 : s1, *sv = FWD ? d2 : s2;
    if (sq32 != NULL && FWD) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (be == NULL || packed == NULL || sq == NULL || sk == NULL || sv == NULL || pos_ids == NULL || n_heads == 0U ||
        head_dim == 0U || (head_dim & 1U) != 0U || !rope_args_ok(args, head_dim)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = packed->dtype;
    if (dt != GDB_DTYPE_F16 && dt != GDB_DTYPE_BF16) {
        return GD_ERR_UNSUPPORTED;
    }
    if (args->n_dims != head_dim) {
        return GD_ERR_UNSUPPORTED;  // the reference kernel rotates the full head only
    }
    const size_t area = (size_t)n_heads * head_dim;
    if (packed->rank != 2U || (size_t)packed->shape[1] != area * 3U || packed->shape[0] <= 0) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t tokens = (size_t)packed->shape[0];
    const size_t kv_rows = cache_tmax != 0U ? tokens * cache_tmax : tokens;   // K / V destinations are caches when cache_tmax > 0
    if (packed->count != tokens * area * 3U || sq->count != tokens * area || sk->count != kv_rows * area ||
        sv->count != kv_rows * area || pos_ids->count != tokens || (cache_tmax != 0U && !FWD)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    void *pp = gdb_tv_ptr(packed, dt), *qp = gdb_tv_ptr(sq, dt), *kp = gdb_tv_ptr(sk, dt), *vp = gdb_tv_ptr(sv, dt);
    const int *ip = (const int *)gdb_tv_ptr(pos_ids, GDB_DTYPE_I32);
    if (pp == NULL || qp == NULL || kp == NULL || vp == NULL || ip == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    rope_params p;
    p.tokens = tokens;
    p.heads = n_heads;
    p.head_dim = head_dim;
    p.n_dims = args->n_dims;
    p.interleaved = args->interleaved;
    p.freq_scale = -2.0f * log2f(args->theta) / (float)args->n_dims;
    p.sin_sign = FWD ? 1.0f : -1.0f;
    p.use_table = (head_dim == TABLE_HEAD_DIM && args->n_dims == TABLE_HEAD_DIM && args->interleaved == 0U &&
                   fabsf(args->theta - TABLE_THETA) <= 1.0e-3f && getenv("GD_QKV_SPLIT_ROPE_NO_TABLE") == NULL) ? 1 : 0;
    if (p.use_table) {
        gd_status st = ensure_rope_table(be);
        if (st != GD_OK) {
            return st;
        }
    }
    const float *q32p = NULL;
    if (sq32 != NULL) {
        if (sq32->count != tokens * area || (q32p = (const float *)gdb_tv_ptr(sq32, GDB_DTYPE_F32)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const bool vec = args->interleaved == 0U && (head_dim % 16U) == 0U &&
                     (((uintptr_t)pp | (uintptr_t)qp | (uintptr_t)kp | (uintptr_t)vp | (uintptr_t)q32p) % 16U) == 0U;
    if ((cache_tmax != 0U || q32p != NULL) && !vec) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *a0 = FWD ? pp : qp, *a1 = FWD ? NULL : kp, *a2 = FWD ? NULL : vp;
    void *o0 = FWD ? qp : pp, *o1 = FWD ? kp : NULL, *o2 = FWD ? vp : NULL;
    const size_t items = vec ? tokens * n_heads * (head_dim / 16U) : tokens * n_heads * (head_dim / 2U);
    const unsigned grid = gdb_grid_for(items, 256, be, 16);
#define GDB_ROPE_LAUNCH(T)                                                                                          \
    do {                                                                                                            \
        if (vec) {                                                                                                  \
            gdb_launch(qkv_split_rope_vec8_kernel<T, FWD>, grid, 256, 0, be->stream, (const T *)a0, (const T *)a1, (const T *)a2, ip, (T *)o0, (T *)o1, (T *)o2, p, be->rope_table, (unsigned)cache_tmax, q32p); \
        } else {                                                                                                    \
            gdb_launch(qkv_split_rope_kernel<T, FWD>, grid, 256, 0, be->stream, (const T *)a0, (const T *)a1, (const T *)a2, ip, (T *)o0, (T *)o1, (T *)o2, p, be->rope_table); \
        }                                                                                                           \
    } while (0)
    if (dt == GDB_DTYPE_F16) {
        GDB_ROPE_LAUNCH(__half);
    } else {
        GDB_ROPE_LAUNCH(__nv_bfloat16);
    }
#undef GDB_ROPE_LAUNCH
    return gdb_launched(be, "qkv_split_rope");
}

}  // namespace

// Rotation parameters exactly as gdb_qkv_rope_append would use them (cos / sin table included), for a caller that
// applies the rotation inside its own kernel. GD_ERR_UNSUPPORTED where that entry would not take its vector path.
gd_status gdb_rope_params_for_decode(gd_backend *be, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args, size_t tokens,
                                     gdb_dec::rope_params *out)
{
    if (be == NULL || out == NULL || n_heads == 0U || head_dim == 0U || (head_dim & 1U) != 0U || !rope_args_ok(args, head_dim)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (args->n_dims != head_dim || args->interleaved != 0U || (head_dim % 16U) != 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    rope_params p;
    p.tokens = tokens;
    p.heads = n_heads;
    p.head_dim = head_dim;
    p.n_dims = args->n_dims;
    p.interleaved = args->interleaved;
    p.freq_scale = -2.0f * log2f(args->theta) / (float)args->n_dims;
    p.sin_sign = 1.0f;
    p.use_table = (head_dim == TABLE_HEAD_DIM && args->n_dims == TABLE_HEAD_DIM && fabsf(args->theta - TABLE_THETA) <= 1.0e-3f &&
                   getenv("GD_QKV_SPLIT_ROPE_NO_TABLE") == NULL) ? 1 : 0;
    if (p.use_table) {
        gd_status st = ensure_rope_table(be);
        if (st != GD_OK) {
            return st;
        }
    }
    *out = p;
    return GD_OK;
}

// Decode step: q = rope(split(qkv)) to `q`, and the rotated key / the value of row b straight into slot pos_ids[b] of
// the caches [rows, tmax, heads, head_dim] (qkv_split_rope_forward + kv_cache_append_positions in one launch).
gd_status gdb_qkv_rope_append(gd_backend *be, const gd_backend_tensor_view *qkv, const gd_backend_tensor_view *pos_ids,
                              const gd_backend_tensor_view *q, const gd_backend_tensor_view *k_cache, const gd_backend_tensor_view *v_cache,
                              uint32_t n_heads, uint32_t head_dim, uint32_t tmax, const gd_backend_rope_args *args)
{
    if (tmax == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return qkv_dispatch<true>(be, qkv, NULL, NULL, pos_ids, q, k_cache, v_cache, n_heads, head_dim, args, tmax);
}

namespace {

gd_status rope_dispatch(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *pos_ids,
                        const gd_backend_tensor_view *out, const gd_backend_rope_args *args, float sin_sign)
{
    if (be == NULL || x == NULL || pos_ids == NULL || out == NULL || x->rank < 2U || x->rank > 8U ||
        x->dtype != out->dtype || x->count != out->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const uint32_t head_dim = (uint32_t)x->shape[x->rank - 1U], heads = (uint32_t)x->shape[x->rank - 2U];
    if (head_dim == 0U || heads == 0U || !rope_args_ok(args, head_dim) || (x->count % ((size_t)heads * head_dim)) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t tokens = x->count / ((size_t)heads * head_dim);
    if (pos_ids->count != tokens) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype);
    void *op = gdb_tv_ptr(out, x->dtype);
    const int *ip = (const int *)gdb_tv_ptr(pos_ids, GDB_DTYPE_I32);
    if (xp == NULL || op == NULL || ip == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    rope_params p;
    p.tokens = tokens;
    p.heads = heads;
    p.head_dim = head_dim;
    p.n_dims = args->n_dims;
    p.interleaved = args->interleaved;
    p.freq_scale = -2.0f * log2f(args->theta) / (float)args->n_dims;
    p.sin_sign = sin_sign;
    p.use_table = 0;
    const unsigned grid = gdb_grid_for(x->count, 256, be, 16);
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(rope_kernel<__half>, grid, 256, 0, be->stream, (const __half *)xp, ip, (__half *)op, p);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(rope_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, ip, (__nv_bfloat16 *)op, p);
    } else {
        gdb_launch(rope_kernel<float>, grid, 256, 0, be->stream, (const float *)xp, ip, (float *)op, p);
    }
    return gdb_launched(be, "rope");
}

}  // namespace

extern "C" {

gd_status gd_backend_embedding_forward(gd_backend *be, const gd_backend_tensor_view *table, const gd_backend_tensor_view *ids, const gd_backend_tensor_view *out, const gd_backend_embedding_args *a)
{
    if (be == NULL || table == NULL || ids == NULL || out == NULL || a == NULL || a->vocab == 0U || a->dim == 0U ||
        table->dtype != out->dtype || table->count != a->vocab * a->dim || ids->count != a->ids_count ||
        out->count != a->ids_count * a->dim) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(table->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *tp = gdb_tv_ptr(table, table->dtype);
    const int *ip = (const int *)gdb_tv_ptr(ids, GDB_DTYPE_I32);
    void *op = gdb_tv_ptr(out, out->dtype);
    if (tp == NULL || ip == NULL || op == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (a->ids_count == 0U) {
        return GD_OK;
    }
    const size_t row_bytes = a->dim * gdb_dtype_size(table->dtype);
    if ((row_bytes % 16U) == 0U && (((uintptr_t)tp | (uintptr_t)op) % 16U) == 0U && table->dtype != GDB_DTYPE_BF16) {
        const unsigned nan_word = table->dtype == GDB_DTYPE_F16 ? 0x7e007e00U : (table->dtype == GDB_DTYPE_BF16 ? 0x7fc07fc0U : 0x7fc00000U);
        gdb_launch(embedding_fwd_vec_kernel, gdb_grid_for(a->ids_count * (row_bytes / 16U), 256, be, 16), 256, 0, be->stream, (const uint4 *)tp, ip, (uint4 *)op, a->ids_count, a->vocab, row_bytes / 16U, nan_word);
    } else if (table->dtype == GDB_DTYPE_F16) {
        gdb_launch(embedding_fwd_kernel<__half>, gdb_grid_for(out->count, 256, be, 16), 256, 0, be->stream, (const __half *)tp, ip, (__half *)op, a->ids_count, a->vocab, a->dim);
    } else if (table->dtype == GDB_DTYPE_BF16) {
        gdb_launch(embedding_fwd_kernel<__nv_bfloat16>, gdb_grid_for(out->count, 256, be, 16), 256, 0, be->stream, (const __nv_bfloat16 *)tp, ip, (__nv_bfloat16 *)op, a->ids_count, a->vocab, a->dim);
    } else {
        gdb_launch(embedding_fwd_kernel<float>, gdb_grid_for(out->count, 256, be, 16), 256, 0, be->stream, (const float *)tp, ip, (float *)op, a->ids_count, a->vocab, a->dim);
    }
    return gdb_launched(be, "embedding_forward");
}

// grad_table (16-bit) needs a caller-provided contiguous F32 scratch table [vocab, dim]; an F32
// grad_table is accumulated in place after being zeroed.
gd_status gd_backend_embedding_backward(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *ids, const gd_backend_tensor_view *grad_table, const gd_backend_tensor_view *scratch, const gd_backend_embedding_args *a)
{
    if (be == NULL || grad_out == NULL || ids == NULL || grad_table == NULL || a == NULL || a->vocab == 0U ||
        a->dim == 0U || grad_out->dtype != grad_table->dtype || grad_table->count != a->vocab * a->dim ||
        ids->count != a->ids_count || grad_out->count != a->ids_count * a->dim) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = grad_out->dtype;
    if (!gdb_is_float_dtype(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *gp = gdb_tv_ptr(grad_out, dt);
    const int *ip = (const int *)gdb_tv_ptr(ids, GDB_DTYPE_I32);
    void *tp = gdb_tv_ptr(grad_table, dt);
    float *acc;
    if (gp == NULL || ip == NULL || tp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (dt == GDB_DTYPE_F32) {
        acc = (float *)tp;
    } else {
        if (scratch == NULL || scratch->count != grad_table->count) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        acc = (float *)gdb_tv_ptr(scratch, GDB_DTYPE_F32);
        if (acc == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const size_t total = a->vocab * a->dim;
    cudaError_t e = cudaMemsetAsync(acc, 0, total * sizeof(float), be->stream);
    be->launches += 1U;
    if (e != cudaSuccess) {
        return gdb_fail(be, e, "embedding_backward zero");
    }
    if (a->ids_count != 0U) {
        const unsigned grid = gdb_grid_for(grad_out->count, 256, be, 16);
        if (dt == GDB_DTYPE_F16) {
            gdb_launch(embedding_scatter_kernel<__half>, grid, 256, 0, be->stream, (const __half *)gp, ip, acc, a->ids_count, a->vocab, a->dim);
        } else if (dt == GDB_DTYPE_BF16) {
            gdb_launch(embedding_scatter_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)gp, ip, acc, a->ids_count, a->vocab, a->dim);
        } else {
            gdb_launch(embedding_scatter_kernel<float>, grid, 256, 0, be->stream, (const float *)gp, ip, acc, a->ids_count, a->vocab, a->dim);
        }
        gd_status st = gdb_launched(be, "embedding_backward scatter");
        if (st != GD_OK) {
            return st;
        }
    }
    if (dt == GDB_DTYPE_F32) {
        return GD_OK;
    }
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(cast_from_f32_kernel<__half>, gdb_grid_for(total, 256, be, 8), 256, 0, be->stream, acc, (__half *)tp, total);
    } else {
        gdb_launch(cast_from_f32_kernel<__nv_bfloat16>, gdb_grid_for(total, 256, be, 8), 256, 0, be->stream, acc, (__nv_bfloat16 *)tp, total);
    }
    return gdb_launched(be, "embedding_backward cast");
}

gd_status gd_backend_rope(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *pos_ids, const gd_backend_tensor_view *out, const gd_backend_rope_args *args)
{
    return rope_dispatch(be, x, pos_ids, out, args, 1.0f);
}

gd_status gd_backend_rope_backward(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *pos_ids, const gd_backend_tensor_view *grad_x, const gd_backend_rope_args *args)
{
    return rope_dispatch(be, grad_out, pos_ids, grad_x, args, -1.0f);
}

gd_status gd_backend_qkv_split_rope_forward(gd_backend *be, const gd_backend_tensor_view *qkv, const gd_backend_tensor_view *pos_ids, const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *v, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args)
{
    return qkv_dispatch<true>(be, qkv, NULL, NULL, pos_ids, q, k, v, n_heads, head_dim, args);
}

gd_status gd_backend_qkv_split_rope_backward(gd_backend *be, const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k, const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *pos_ids, const gd_backend_tensor_view *grad_qkv, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args)
{
    return qkv_dispatch<false>(be, grad_q, grad_k, grad_v, pos_ids, grad_qkv, NULL, NULL, n_heads, head_dim, args);
}

gd_status gdb200_qkv_split_rope_backward_q32(gd_backend *be, const gd_backend_tensor_view *grad_q_f32, const gd_backend_tensor_view *grad_k, const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *pos_ids, const gd_backend_tensor_view *grad_qkv, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args)
{
    if (grad_q_f32 == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return qkv_dispatch<false>(be, NULL, grad_k, grad_v, pos_ids, grad_qkv, NULL, NULL, n_heads, head_dim, args, 0, grad_q_f32);
}

}  // extern "C"
