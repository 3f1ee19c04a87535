// MiniMax-M3 block-sparse attention: block selection (index top-k), forward and backward.
//
// Semantics follow the reference's Metal kernels (src/ops/minimax_m3_index_topk/metal_minimax_m3_index_topk.metal,
// src/ops/minimax_m3_sparse_attention/metal_minimax_m3_sparse_attention.metal): packed sequences given by
// cu_seqlens, query i of a sequence may attend keys j <= i that lie in one of its `topk` selected blocks of
// `block_size` keys; the selection scores a block by the largest index-head dot product q_i . k_j over the block's
// causal keys and always keeps the first `init_blocks` and the last `local_blocks` causal blocks.
//
// This op is not on the gpt_lm path. The kernels are one thread per query (or key) row with the row in registers,
// head_dim <= 64, and keep the reference's order of additions, which makes the selected block indices reproducible
// (the selection compares FP32 scores); they are functional rather than tuned: the gathered K / V rows are read
// through L1 / L2, nothing is staged with TMA.
#include "common.cuh"

namespace {

constexpr int M3_THREADS = 64;      // rows per block (the reference's row tile)
constexpr int M3_MAX_DH = 64;
constexpr int M3_MAX_TOPK = 16;
constexpr int M3_MAX_BLOCK = 128;
constexpr int M3_KTILE = 16;        // key / query rows staged per shared-memory tile

struct m3_params {
    long long total_tokens;
    int batch, hq, hkv, dh, block_size, topk, init_blocks, local_blocks;
    float scale;
};

// Plain multiply and add (no contraction into an FMA), so that scores compare like a scalar FP32 loop.
__device__ __forceinline__ float m3_mac(float acc, float a, float b) { return __fadd_rn(acc, __fmul_rn(a, b)); }

// topk[h, qg, t] = t-th selected block of query qg (sequence-local block index), -1 when fewer blocks are causal.
template <typename T>
__global__ void __launch_bounds__(M3_THREADS)
m3_index_topk_kernel(const T *__restrict__ q, const T *__restrict__ k, const int *__restrict__ cu, int *__restrict__ topk, m3_params p)
{
    gdb_pdl_sync();
    __shared__ float ksh[M3_KTILE * M3_MAX_DH];
    const int q0 = blockIdx.x * M3_THREADS, h = blockIdx.y, b = blockIdx.z;
    const int start = cu[b], T_len = cu[b + 1] - start;
    if (q0 >= T_len) {
        return;
    }
    const int i = q0 + (int)threadIdx.x;
    const bool active = i < T_len;
    const int qg = start + i;
    const int valid_blocks = active ? (i + p.block_size) / p.block_size : 0;
    const int max_i = min(q0 + M3_THREADS - 1, T_len - 1);
    const int max_valid_blocks = (max_i + p.block_size) / p.block_size;
    const int local_start = max(0, valid_blocks - p.local_blocks);
    float qreg[M3_MAX_DH];
#pragma unroll
    for (int c = 0; c < M3_MAX_DH; ++c) {
        qreg[c] = (active && c < p.dh) ? gdb_io<T>::ld(q, ((size_t)qg * p.hkv + h) * p.dh + c) : 0.0f;
    }
    int sel_idx[M3_MAX_TOPK];
    float sel_score[M3_MAX_TOPK];
#pragma unroll
    for (int t = 0; t < M3_MAX_TOPK; ++t) {
        sel_idx[t] = -1;
        sel_score[t] = -INFINITY;
    }
    for (int blk = 0; blk < max_valid_blocks; ++blk) {
        float block_score = -INFINITY;
        const int k_begin = blk * p.block_size, k_end = min(k_begin + p.block_size, T_len);
        for (int kb = k_begin; kb < k_end; kb += M3_KTILE) {
            const int tile = min(M3_KTILE, k_end - kb);
            for (int idx = threadIdx.x; idx < tile * p.dh; idx += M3_THREADS) {
                const int jj = idx / p.dh, c = idx - jj * p.dh;
                ksh[jj * M3_MAX_DH + c] = gdb_io<T>::ld(k, ((size_t)(start + kb + jj) * p.hkv + h) * p.dh + c);
            }
            __syncthreads();
            if (active && blk < valid_blocks) {
                for (int jj = 0; jj < tile; ++jj) {
                    if (kb + jj <= i) {
                        float s = 0.0f;
#pragma unroll
                        for (int c = 0; c < M3_MAX_DH; ++c) {
                            if (c < p.dh) s = m3_mac(s, qreg[c], ksh[jj * M3_MAX_DH + c]);
                        }
                        block_score = s > block_score ? s : block_score;
                    }
                }
            }
            __syncthreads();
        }
        if (active && blk < valid_blocks) {
            if (!(block_score == block_score)) block_score = -INFINITY;
            // priority of the reference: the first blocks highest, the local blocks next, index scores for the rest
            if (blk < p.init_blocks) block_score = 1.0e30f;
            if (blk >= local_start && p.local_blocks > 0) block_score = 1.0e29f;
            // insertion into the sorted list; a later block never displaces an equal score
#pragma unroll
            for (int slot = 0; slot < M3_MAX_TOPK; ++slot) {
                if (slot < p.topk && block_score > sel_score[slot]) {
#pragma unroll
                    for (int mv = M3_MAX_TOPK - 1; mv > 0; --mv) {
                        if (mv > slot && mv < p.topk) {
                            sel_score[mv] = sel_score[mv - 1];
                            sel_idx[mv] = sel_idx[mv - 1];
                        }
                    }
                    sel_score[slot] = block_score;
                    sel_idx[slot] = blk;
                    break;
                }
            }
        }
    }
    if (active) {
        int *out = topk + ((size_t)h * p.total_tokens + qg) * p.topk;
#pragma unroll
        for (int t = 0; t < M3_MAX_TOPK; ++t) {
            if (t < p.topk) out[t] = t < valid_blocks ? sel_idx[t] : -1;
        }
    }
}

// One thread per (query, head): online softmax over the causal keys of the selected blocks, in list order.
// MODE 0: out = softmax(s) V. MODE 1 (backward, query side): dQ and stats = (max, sum of exp, D = sum_j p_j dp_j).
template <typename T, int MODE>
__global__ void __launch_bounds__(M3_THREADS)
m3_query_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ go, const int *__restrict__ cu,
                const int *__restrict__ topk, T *__restrict__ out, float *__restrict__ stats, m3_params p)
{
    gdb_pdl_sync();
    const int hq = blockIdx.y, b = blockIdx.z;
    const int start = cu[b], T_len = cu[b + 1] - start;
    const int i = blockIdx.x * M3_THREADS + (int)threadIdx.x;
    if (i >= T_len) {
        return;
    }
    const int hkv = hq / (p.hq / p.hkv);
    const int qg = start + i;
    const size_t qbase = ((size_t)qg * p.hq + hq) * p.dh;
    float qreg[M3_MAX_DH], acc[M3_MAX_DH];
    float goreg[MODE == 1 ? M3_MAX_DH : 1], ksum[MODE == 1 ? M3_MAX_DH : 1];
#pragma unroll
    for (int c = 0; c < M3_MAX_DH; ++c) {
        qreg[c] = c < p.dh ? gdb_io<T>::ld(q, qbase + c) : 0.0f;
        acc[c] = 0.0f;
        if (MODE == 1) {
            goreg[c] = c < p.dh ? gdb_io<T>::ld(go, qbase + c) : 0.0f;
            ksum[c] = 0.0f;
        }
    }
    float m = -INFINITY, l = 0.0f, raw = 0.0f;
    const int *sel = topk + ((size_t)hkv * p.total_tokens + qg) * p.topk;
    for (int t = 0; t < p.topk; ++t) {
        const int blk = sel[t];
        if (blk < 0) {
            continue;
        }
        const int k_begin = blk * p.block_size, k_end = min(k_begin + p.block_size, T_len);
        for (int j = k_begin; j < k_end && j <= i; ++j) {
            const size_t kvbase = ((size_t)(start + j) * p.hkv + hkv) * p.dh;
            float kr[M3_MAX_DH];
            float dot = 0.0f, dp = 0.0f;
#pragma unroll
            for (int c = 0; c < M3_MAX_DH; ++c) {
                if (c < p.dh) {
                    kr[c] = gdb_io<T>::ld(k, kvbase + c);
                    dot += qreg[c] * kr[c];
                    if (MODE == 1) dp += goreg[c] * gdb_io<T>::ld(v, kvbase + c);
                }
            }
            const float s = dot * p.scale;
            const float mnew = s > m ? s : m;
            const float corr = expf(m - mnew), e = expf(s - mnew);
            l = l * corr + e;
            if (MODE == 1) raw = raw * corr + e * dp;
#pragma unroll
            for (int c = 0; c < M3_MAX_DH; ++c) {
                if (c < p.dh) {
                    if (MODE == 0) {
                        acc[c] = acc[c] * corr + e * gdb_io<T>::ld(v, kvbase + c);
                    } else {
                        acc[c] = acc[c] * corr + e * dp * kr[c];
                        ksum[c] = ksum[c] * corr + e * kr[c];
                    }
                }
            }
            m = mnew;
        }
    }
    const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
    if (MODE == 0) {
#pragma unroll
        for (int c = 0; c < M3_MAX_DH; ++c) {
            if (c < p.dh) gdb_io<T>::st(out, qbase + c, acc[c] * inv_l);
        }
    } else {
        const float D = l > 0.0f ? raw / l : 0.0f;
        float *st = stats + ((size_t)qg * p.hq + hq) * 3U;
        st[0] = m;
        st[1] = l;
        st[2] = D;
#pragma unroll
        for (int c = 0; c < M3_MAX_DH; ++c) {
            if (c < p.dh) gdb_io<T>::st(out, qbase + c, p.scale * (acc[c] - D * ksum[c]) * inv_l);
        }
    }
}

// One thread per key row of one KV head: walks the later queries of the sequence (all query heads of the group)
// whose selection contains the key's block; p_j from the saved statistics.
template <typename T>
__global__ void __launch_bounds__(M3_THREADS)
m3_dkv_kernel(const T *__restrict__ go, const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const int *__restrict__ cu,
              const int *__restrict__ topk, T *__restrict__ dk, T *__restrict__ dv, const float *__restrict__ stats, m3_params p)
{
    gdb_pdl_sync();
    __shared__ float qsh[M3_KTILE * M3_MAX_DH], gsh[M3_KTILE * M3_MAX_DH];
    __shared__ float msh[M3_KTILE], lsh[M3_KTILE], dsh[M3_KTILE];
    const int k0 = blockIdx.x * M3_THREADS, hkv = blockIdx.y, b = blockIdx.z;
    const int start = cu[b], T_len = cu[b + 1] - start;
    if (k0 >= T_len) {
        return;
    }
    const int j = k0 + (int)threadIdx.x;
    const bool active = j < T_len;
    const int block_id = j / p.block_size, group = p.hq / p.hkv;
    const size_t kvbase = active ? ((size_t)(start + j) * p.hkv + hkv) * p.dh : 0;
    float kreg[M3_MAX_DH], vreg[M3_MAX_DH], dkacc[M3_MAX_DH], dvacc[M3_MAX_DH];
#pragma unroll
    for (int c = 0; c < M3_MAX_DH; ++c) {
        kreg[c] = (active && c < p.dh) ? gdb_io<T>::ld(k, kvbase + c) : 0.0f;
        vreg[c] = (active && c < p.dh) ? gdb_io<T>::ld(v, kvbase + c) : 0.0f;
        dkacc[c] = 0.0f;
        dvacc[c] = 0.0f;
    }
    const int q_start = (k0 / M3_KTILE) * M3_KTILE;
    for (int g = 0; g < group; ++g) {
        const int hq = hkv * group + g;
        for (int qb = q_start; qb < T_len; qb += M3_KTILE) {
            const int tile = min(M3_KTILE, T_len - qb);
            for (int idx = threadIdx.x; idx < tile * p.dh; idx += M3_THREADS) {
                const int ii = idx / p.dh, c = idx - ii * p.dh;
                const size_t qbase = ((size_t)(start + qb + ii) * p.hq + hq) * p.dh;
                qsh[ii * M3_MAX_DH + c] = gdb_io<T>::ld(q, qbase + c);
                gsh[ii * M3_MAX_DH + c] = gdb_io<T>::ld(go, qbase + c);
            }
            for (int ii = threadIdx.x; ii < tile; ii += M3_THREADS) {
                const float *st = stats + ((size_t)(start + qb + ii) * p.hq + hq) * 3U;
                msh[ii] = st[0];
                lsh[ii] = st[1];
                dsh[ii] = st[2];
            }
            __syncthreads();
            if (active) {
                for (int ii = 0; ii < tile; ++ii) {
                    const int i = qb + ii;
                    if (i < j || lsh[ii] <= 0.0f) {
                        continue;
                    }
                    const int *sel = topk + ((size_t)hkv * p.total_tokens + (start + i)) * p.topk;
                    bool hit = false;
                    for (int t = 0; t < p.topk; ++t) hit = hit || sel[t] == block_id;
                    if (!hit) {
                        continue;
                    }
                    float dot = 0.0f, dp = 0.0f;
#pragma unroll
                    for (int c = 0; c < M3_MAX_DH; ++c) {
                        if (c < p.dh) {
                            dot += qsh[ii * M3_MAX_DH + c] * kreg[c];
                            dp += gsh[ii * M3_MAX_DH + c] * vreg[c];
                        }
                    }
                    const float pj = expf(dot * p.scale - msh[ii]) / lsh[ii];
                    const float ds = pj * (dp - dsh[ii]);
#pragma unroll
                    for (int c = 0; c < M3_MAX_DH; ++c) {
                        if (c < p.dh) {
                            dvacc[c] += pj * gsh[ii * M3_MAX_DH + c];
                            dkacc[c] += p.scale * ds * qsh[ii * M3_MAX_DH + c];
                        }
                    }
                }
            }
            __syncthreads();
        }
    }
    if (active) {
#pragma unroll
        for (int c = 0; c < M3_MAX_DH; ++c) {
            if (c < p.dh) {
                gdb_io<T>::st(dk, kvbase + c, dkacc[c]);
                gdb_io<T>::st(dv, kvbase + c, dvacc[c]);
            }
        }
    }
}

}  // namespace

namespace {

bool m3_contiguous(const gd_backend_tensor_view *v)
{
    int64_t stride = 1;
    if (v == NULL || v->buffer == NULL || v->rank > 8U) {
        return false;
    }
    for (int d = (int)v->rank - 1; d >= 0; --d) {
        if (v->shape[d] <= 0 || v->strides[d] != stride) {
            return false;
        }
        stride *= v->shape[d];
    }
    return gdb_tv_ptr(v, v->dtype) != NULL;
}

bool m3_same3(const gd_backend_tensor_view *a, const gd_backend_tensor_view *b)
{
    return a->rank == 3U && b->rank == 3U && a->dtype == b->dtype && a->shape[0] == b->shape[0] && a->shape[1] == b->shape[1] &&
           a->shape[2] == b->shape[2];
}

bool m3_half(uint32_t dt) { return dt == GDB_DTYPE_F16 || dt == GDB_DTYPE_BF16; }

// Shape rules shared by the three entries (src/ops/minimax_m3_sparse_attention/metal_minimax_m3_sparse_attention.m:95-126,
// src/ops/minimax_m3_index_topk/metal_minimax_m3_index_topk.m:75-101); q [N, Hq, Dh], k [N, Hkv, Dh], topk [Hkv, N, topk].
bool m3_common_ok(const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *cu,
                  const gd_backend_tensor_view *topk, const gd_backend_minimax_m3_sparse_args *a)
{
    if (!m3_contiguous(q) || !m3_contiguous(k) || !m3_contiguous(cu) || !m3_contiguous(topk) || a == NULL) {
        return false;
    }
    return m3_half(q->dtype) && k->dtype == q->dtype && cu->dtype == GDB_DTYPE_I32 && topk->dtype == GDB_DTYPE_I32 && q->rank == 3U &&
           k->rank == 3U && cu->rank == 1U && topk->rank == 3U && cu->shape[0] >= 2 && k->shape[0] == q->shape[0] && k->shape[2] == q->shape[2] &&
           (q->shape[1] % k->shape[1]) == 0 && q->shape[2] <= M3_MAX_DH && topk->shape[0] == k->shape[1] && topk->shape[1] == q->shape[0] &&
           topk->shape[2] == (int64_t)a->topk && a->topk != 0U && a->topk <= (uint32_t)M3_MAX_TOPK && a->block_size != 0U &&
           a->block_size <= (uint32_t)M3_MAX_BLOCK && a->max_seqlen != 0U && q->shape[0] <= 0x7fffffffLL && cu->shape[0] - 1 <= 65535;
}

m3_params m3_fill(const gd_backend_tensor_view *q, const gd_backend_tensor_view *k, const gd_backend_tensor_view *cu,
                  const gd_backend_minimax_m3_sparse_args *a)
{
    m3_params p;
    p.total_tokens = q->shape[0];
    p.batch = (int)(cu->shape[0] - 1);
    p.hq = (int)q->shape[1];
    p.hkv = (int)k->shape[1];
    p.dh = (int)q->shape[2];
    p.block_size = (int)a->block_size;
    p.topk = (int)a->topk;
    p.init_blocks = (int)a->init_blocks;
    p.local_blocks = (int)a->local_blocks;
    p.scale = a->scale;
    return p;
}

// rows of a sequence beyond max_seqlen are not visited, as in the reference's launch geometry
dim3 m3_grid(const gd_backend_minimax_m3_sparse_args *a, int heads, int batch)
{
    return dim3((a->max_seqlen + M3_THREADS - 1U) / M3_THREADS, (unsigned)heads, (unsigned)batch);
}

}  // namespace

extern "C" {

typedef const gd_backend_tensor_view *TV;

gd_status gd_backend_minimax_m3_index_topk(gd_backend *be, TV index_q, TV index_k, TV cu_seqlens, TV topk_idx, const gd_backend_minimax_m3_sparse_args *args)
{
    if (be == NULL || !m3_common_ok(index_q, index_k, cu_seqlens, topk_idx, args) || index_k->shape[1] != index_q->shape[1]) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const m3_params p = m3_fill(index_q, index_k, cu_seqlens, args);
    const dim3 grid = m3_grid(args, p.hkv, p.batch);
    const int *cu = (const int *)gdb_tv_ptr(cu_seqlens, GDB_DTYPE_I32);
    int *tk = (int *)gdb_tv_ptr(topk_idx, GDB_DTYPE_I32);
    if (index_q->dtype == GDB_DTYPE_F16) {
        gdb_launch(m3_index_topk_kernel<__half>, grid, M3_THREADS, 0, be->stream, (const __half *)gdb_tv_ptr(index_q, GDB_DTYPE_F16),
                   (const __half *)gdb_tv_ptr(index_k, GDB_DTYPE_F16), cu, tk, p);
    } else {
        gdb_launch(m3_index_topk_kernel<__nv_bfloat16>, grid, M3_THREADS, 0, be->stream, (const __nv_bfloat16 *)gdb_tv_ptr(index_q, GDB_DTYPE_BF16),
                   (const __nv_bfloat16 *)gdb_tv_ptr(index_k, GDB_DTYPE_BF16), cu, tk, p);
    }
    return gdb_launched(be, "minimax_m3_index_topk");
}

gd_status gd_backend_minimax_m3_sparse_attention(gd_backend *be, TV q, TV k, TV v, TV cu_seqlens, TV topk_idx, TV out,
                                                 const gd_backend_minimax_m3_sparse_args *args)
{
    if (be == NULL || !m3_common_ok(q, k, cu_seqlens, topk_idx, args) || !m3_contiguous(v) || !m3_contiguous(out) || !m3_same3(k, v) ||
        !m3_same3(q, out)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const m3_params p = m3_fill(q, k, cu_seqlens, args);
    const dim3 grid = m3_grid(args, p.hq, p.batch);
    const int *cu = (const int *)gdb_tv_ptr(cu_seqlens, GDB_DTYPE_I32), *tk = (const int *)gdb_tv_ptr(topk_idx, GDB_DTYPE_I32);
    const uint32_t dt = q->dtype;
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(m3_query_kernel<__half, 0>, grid, M3_THREADS, 0, be->stream, (const __half *)gdb_tv_ptr(q, dt), (const __half *)gdb_tv_ptr(k, dt),
                   (const __half *)gdb_tv_ptr(v, dt), (const __half *)nullptr, cu, tk, (__half *)gdb_tv_ptr(out, dt), (float *)nullptr, p);
    } else {
        gdb_launch(m3_query_kernel<__nv_bfloat16, 0>, grid, M3_THREADS, 0, be->stream, (const __nv_bfloat16 *)gdb_tv_ptr(q, dt),
                   (const __nv_bfloat16 *)gdb_tv_ptr(k, dt), (const __nv_bfloat16 *)gdb_tv_ptr(v, dt), (const __nv_bfloat16 *)nullptr, cu, tk,
                   (__nv_bfloat16 *)gdb_tv_ptr(out, dt), (float *)nullptr, p);
    }
    return gdb_launched(be, "minimax_m3_sparse_attention");
}

gd_status gd_backend_minimax_m3_sparse_attention_backward(gd_backend *be, TV grad_out, TV q, TV k, TV v, TV cu_seqlens, TV topk_idx, TV grad_q,
                                                          TV grad_k, TV grad_v, TV stats, const gd_backend_minimax_m3_sparse_args *args)
{
    if (be == NULL || !m3_common_ok(q, k, cu_seqlens, topk_idx, args) || !m3_contiguous(v) || !m3_contiguous(grad_out) || !m3_contiguous(grad_q) ||
        !m3_contiguous(grad_k) || !m3_contiguous(grad_v) || !m3_contiguous(stats) || !m3_same3(k, v) || !m3_same3(q, grad_out) ||
        !m3_same3(q, grad_q) || !m3_same3(k, grad_k) || !m3_same3(v, grad_v) || stats->dtype != GDB_DTYPE_F32 || stats->rank != 3U ||
        stats->shape[0] != q->shape[0] || stats->shape[1] != q->shape[1] || stats->shape[2] != 3) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const m3_params p = m3_fill(q, k, cu_seqlens, args);
    const int *cu = (const int *)gdb_tv_ptr(cu_seqlens, GDB_DTYPE_I32), *tk = (const int *)gdb_tv_ptr(topk_idx, GDB_DTYPE_I32);
    float *st = (float *)gdb_tv_ptr(stats, GDB_DTYPE_F32);
    const uint32_t dt = q->dtype;
    const dim3 gq = m3_grid(args, p.hq, p.batch), gk = m3_grid(args, p.hkv, p.batch);
    if (dt == GDB_DTYPE_F16) {
        typedef __half H;
        gdb_launch(m3_query_kernel<H, 1>, gq, M3_THREADS, 0, be->stream, (const H *)gdb_tv_ptr(q, dt), (const H *)gdb_tv_ptr(k, dt),
                   (const H *)gdb_tv_ptr(v, dt), (const H *)gdb_tv_ptr(grad_out, dt), cu, tk, (H *)gdb_tv_ptr(grad_q, dt), st, p);
        gd_status s1 = gdb_launched(be, "minimax_m3_sparse_attention_backward dq");
        if (s1 != GD_OK) return s1;
        gdb_launch(m3_dkv_kernel<H>, gk, M3_THREADS, 0, be->stream, (const H *)gdb_tv_ptr(grad_out, dt), (const H *)gdb_tv_ptr(q, dt),
                   (const H *)gdb_tv_ptr(k, dt), (const H *)gdb_tv_ptr(v, dt), cu, tk, (H *)gdb_tv_ptr(grad_k, dt), (H *)gdb_tv_ptr(grad_v, dt),
                   (const float *)st, p);
    } else {
        typedef __nv_bfloat16 H;
        gdb_launch(m3_query_kernel<H, 1>, gq, M3_THREADS, 0, be->stream, (const H *)gdb_tv_ptr(q, dt), (const H *)gdb_tv_ptr(k, dt),
                   (const H *)gdb_tv_ptr(v, dt), (const H *)gdb_tv_ptr(grad_out, dt), cu, tk, (H *)gdb_tv_ptr(grad_q, dt), st, p);
        gd_status s1 = gdb_launched(be, "minimax_m3_sparse_attention_backward dq");
        if (s1 != GD_OK) return s1;
        gdb_launch(m3_dkv_kernel<H>, gk, M3_THREADS, 0, be->stream, (const H *)gdb_tv_ptr(grad_out, dt), (const H *)gdb_tv_ptr(q, dt),
                   (const H *)gdb_tv_ptr(k, dt), (const H *)gdb_tv_ptr(v, dt), cu, tk, (H *)gdb_tv_ptr(grad_k, dt), (H *)gdb_tv_ptr(grad_v, dt),
                   (const float *)st, p);
    }
    return gdb_launched(be, "minimax_m3_sparse_attention_backward dkv");
}

}  // extern "C"
