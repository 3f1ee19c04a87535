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
#include "decode_parts.cuh"

namespace {

using gdb_dec::pack2;
using gdb_dec::unpack8;

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

// raw[e] = storage-precision (matmul_logit + bias) of the 8 classes of one 16-byte vector. The packed add rounds the exact sum
// once to the storage type; the FP32 sum of two 16-bit floats rounded to 16 bits gives the same bits (24 >= 2 * 11 + 2
// significand bits, so the intermediate rounding cannot change the result), which is what eff_logit computes per element.
template <typename T>
__device__ __forceinline__ void raw8(uint4 a, const uint4 *bias_vec, size_t v, float (&raw)[8])
{
    if (bias_vec != nullptr) {
        const uint4 b = bias_vec[v];
        a.x = pack2<T>::add(a.x, b.x);
        a.y = pack2<T>::add(a.y, b.y);
        a.z = pack2<T>::add(a.z, b.z);
        a.w = pack2<T>::add(a.w, b.w);
    }
    unpack8<T>(a, raw);
}

// Row pass helper: calls f(c, effective_logit) for every class of the row chunk.
template <typename T, typename F>
__device__ __forceinline__ void for_each_logit(const T *row, const T *bias, size_t classes, float cap, float inv_cap, F f)
{
    if (sizeof(T) == 2 && (classes % 8U) == 0U && (((uintptr_t)row | (uintptr_t)bias) % 16U) == 0U) {
        const uint4 *rv = reinterpret_cast<const uint4 *>(row), *bv = reinterpret_cast<const uint4 *>(bias);
        for (size_t v = threadIdx.x; v < classes / 8U; v += blockDim.x) {
            float raw[8];
            raw8<T>(rv[v], bv, v, raw);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                f(v * 8U + (size_t)e, apply_softcap(raw[e], cap, inv_cap));
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
    if (sizeof(T) == 2 && (classes % 8U) == 0U && (((uintptr_t)lr | (uintptr_t)bias) % 16U) == 0U) {
        const uint4 *rv = reinterpret_cast<const uint4 *>(lr), *bv = reinterpret_cast<const uint4 *>(bias);
        for (size_t v = lane; v < classes / 8U; v += 32) {
            float x[8], vm = NEG_BIG;
            raw8<T>(rv[v], bv, v, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x[e] = apply_softcap(x[e], cap, inv_cap);
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

// Sum of p[threadIdx.x], p[threadIdx.x + blockDim.x], ... in that order, eight loads in flight at a time (a single block
// walks over the rows here, so the latency of one load per step would be the whole run time).
template <typename F>
__device__ __forceinline__ float strided_sum(size_t n, F value)
{
    const size_t step = blockDim.x;
    float acc = 0.0f;
    size_t i = threadIdx.x;
    for (; i + 7U * step < n; i += 8U * step) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = value(i + (size_t)k * step);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc += v[k];
    }
    for (; i < n; i += step) acc += value(i);
    return acc;
}

__global__ void lmce_reduce_normalize_kernel(const float *row_loss, const float *row_valid, float *loss,
                                             float *inv_valid_count, size_t rows)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    const float ll = strided_sum(rows, [&](size_t i) { return row_loss[i]; });
    const float lv = strided_sum(rows, [&](size_t i) { return row_valid[i]; });
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
    const float ll = strided_sum(rows, [&](size_t i) { return row_loss[i]; });
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
    // out-of-range ids count (their loss is NaN), as in finalize
    const float n = strided_sum(rows, [&](size_t i) {
        const int t = targets[i];
        return (t >= 0 && t != ignore_index) ? 1.0f : 0.0f;
    });
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
    const bool vec = sizeof(T) == 2 && (classes % 8U) == 0U && (((uintptr_t)lr | (uintptr_t)dr | (uintptr_t)bias) % 16U) == 0U;
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
        const uint4 *rv = reinterpret_cast<const uint4 *>(lr), *bv = reinterpret_cast<const uint4 *>(bias);
        uint4 *dv = reinterpret_cast<uint4 *>(dr);
        for (size_t v = threadIdx.x; v < classes / 8U; v += blockDim.x) {
            float x[8];
            raw8<T>(rv[v], bv, v, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x[e] = grad_of(v * 8U + (size_t)e, apply_softcap(x[e], cap, inv_cap));
            }
            dv[v] = make_uint4(pack2<T>::down(x[0], x[1]), pack2<T>::down(x[2], x[3]), pack2<T>::down(x[4], x[5]), pack2<T>::down(x[6], x[7]));
        }
    } else {
        for (size_t c = threadIdx.x; c < classes; c += blockDim.x) {
            gdb_io<T>::st(dr, c, grad_of(c, eff_logit<T>(gdb_io<T>::ld(lr, c), bias, c, cap, inv_cap)));
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Loss statistics and logits gradient of rows whose chunk holds ALL classes, in one pass: the row is read once into
// registers (NV 16-byte vectors per thread, 32 * wpr threads per row), the soft-capped logits, their maximum, the
// exponentials and their sum are formed there, the per-row loss is written and the row is overwritten in place with
//   dlogit = (exp(soft - max) / sum - 1[target]) * max(0, 1 - (soft / cap)^2) * grad_loss * scale / valid_rows
// (metal_lm_cross_entropy.metal:184-203 and :294-310 evaluated together). Against online update + backward chunk this
// halves the special-function work (soft-capping once instead of twice per element, one exponential instead of two)
// and reads the logits once. The number of valid rows comes in as counts[0] (known from the targets before the
// forward pass), so the gradient seed does not wait for the loss reduction.
// Rows of a block are independent: each row's warps meet at their own named barrier, and a row without a usable
// target only has its gradient cleared. A block walks over the rows with the grid's stride; the vectors of its next
// row are already in flight while the current one is worked on, so the loads never wait for the arithmetic.
constexpr int LMF_BLOCK = 256;
constexpr int LMF_MAX_WPR = LMF_BLOCK / 32;
// Vectors per thread. Measured on 18432 rows of 2048 classes: 4 (126 registers, 16 warps per SM) 60 us inside the train step,
// 2 (80 registers, 24 warps) 63 us, 8 (one warp per row, 8 warps per SM) 28 us more than 4.
constexpr int LMF_VECTORS = 4;

// 2^x and 1/x in one special-function instruction each; results below the normal range are flushed to zero (__expf keeps
// them, which costs a range test and two scalings per call; no term this kernel forms can tell the difference).
__device__ __forceinline__ float exp2_ftz(float x)
{
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rcp_ftz(float x)
{
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
constexpr float LOG2E = 1.4426950408889634f;

// Two FP32 values in one 64-bit register pair: sm_100 multiplies, adds and fuses both halves in one instruction, which
// halves the issue slots of the arithmetic between the special-function calls (each half rounds as the scalar instruction does).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_make(float lo, float hi)
{
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_split(f32x2 p, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// tanh(raw / cap) = 1 - 2 / (1 + E), E = exp(2 raw / cap) = 2^(raw * arg_scale): one form for both signs (E = inf gives 1,
// E = 0 gives -1), absolute error about 2e-7, i.e. 6e-6 on a logit capped at 30 - far below the spacing of the 16-bit logits
// it is computed from. (The reference's form, metal_lm_cross_entropy.metal:13-31, takes |y|, divides and restores the sign,
// with a pass-through below 2^-12 that only matters for the relative error of logits the softmax cannot tell from 0.)
__device__ __forceinline__ f32x2 softcap_tanh2(f32x2 raw, f32x2 arg_scale, f32x2 one, f32x2 minus_two)
{
    float a0, a1, d0, d1;
    f2_split(f2_mul(raw, arg_scale), a0, a1);
    f2_split(f2_add(f2_make(exp2_ftz(a0), exp2_ftz(a1)), one), d0, d1);
    return f2_fma(f2_make(rcp_ftz(d0), rcp_ftz(d1)), minus_two, one);
}
__device__ __forceinline__ float softcap_tanh1(float raw, float arg_scale)
{
    return __fmaf_rn(rcp_ftz(__fadd_rn(exp2_ftz(__fmul_rn(raw, arg_scale)), 1.0f)), -2.0f, 1.0f);
}
template <typename T> struct max2_16;
template <> struct max2_16<__half> {
    static constexpr uint32_t LOWEST = 0xFBFFFBFFU;
    static __device__ __forceinline__ uint32_t of(uint32_t a, uint32_t b)
    {
        const __half2 r = __hmax2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
};
template <> struct max2_16<__nv_bfloat16> {
    static constexpr uint32_t LOWEST = 0xFF7FFF7FU;
    static __device__ __forceinline__ uint32_t of(uint32_t a, uint32_t b)
    {
        const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&a), *reinterpret_cast<const __nv_bfloat162 *>(&b));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
};
__device__ __forceinline__ void row_barrier(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

constexpr int LMF_NO_ROW = INT_MIN;   // target value standing for "no such row" in the row loop

template <typename T, int NV, bool CAP>
__global__ void __launch_bounds__(LMF_BLOCK, 2) lmce_fused_rows_kernel(T *logits, const T *bias, const int *targets,
                                                                                     const float *grad_loss, const float *counts, float *row_loss,
                                                                                     size_t rows, int nvec, int wpr, float scale, float cap,
                                                                                     float inv_cap, int ignore_index)
{
    gdb_pdl_sync();
    __shared__ float red[2][LMF_MAX_WPR][LMF_MAX_WPR];
    __shared__ float target_soft[LMF_MAX_WPR];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rib = warp / wpr, wr = warp - rib * wpr;     // row within the block, warp within the row
    const int rpb = (LMF_BLOCK / 32) / wpr;                // rows a block works on at a time
    const int tpr = wpr * 32, tr = wr * 32 + lane;
    const size_t groups = (rows + (size_t)rpb - 1U) / (size_t)rpb;
    const uint4 *bv = reinterpret_cast<const uint4 *>(bias);
    const float valid = counts[0];
    const float seed = grad_loss[0] * scale * (valid > 0.0f ? 1.0f / valid : 0.0f);

    // the row's vectors of this thread and its target; a row without a usable target is not read
    auto fetch = [&](size_t group, uint4 (&dst)[NV], int &t) {
        const size_t row = group * (size_t)rpb + (size_t)rib;
        t = (group < groups && row < rows) ? targets[row] : LMF_NO_ROW;
        const bool usable = t >= 0 && t != ignore_index && t < nvec * 8;
        const uint4 *rv = reinterpret_cast<const uint4 *>(logits) + row * (size_t)nvec;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = tr + i * tpr;
            dst[i] = (usable && v < nvec) ? rv[v] : make_uint4(0U, 0U, 0U, 0U);
        }
    };

    uint4 cur[NV], nxt[NV];
    int t, t_next;
    fetch(blockIdx.x, cur, t);
    for (size_t group = blockIdx.x; group < groups; group += gridDim.x) {
        fetch(group + gridDim.x, nxt, t_next);             // in flight while this row is worked on
        const size_t row = group * (size_t)rpb + (size_t)rib;
        uint4 *rv = reinterpret_cast<uint4 *>(logits) + row * (size_t)nvec;
        if (t == LMF_NO_ROW) {
            // past the last row: nothing to do (the other rows of the block carry on)
        } else if (t < 0 || t == ignore_index || t >= nvec * 8) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = tr + i * tpr;
                if (v < nvec) rv[v] = make_uint4(0U, 0U, 0U, 0U);
            }
            if (tr == 0) {
                row_loss[row] = (t < 0 || t == ignore_index) ? 0.0f : __int_as_float(0x7fc00000);
            }
        } else {
            // u[] = tanh(raw / cap) (raw itself without capping), two per register pair: soft = unit * u with unit = cap (1
            // without capping). The soft-capping keeps the order of the logits, so the row maximum is taken over the raw
            // 16-bit pairs (one packed instruction for two classes) and capped once.
            const f32x2 one = f2_make(1.0f, 1.0f), minus_one = f2_make(-1.0f, -1.0f), minus_two = f2_make(-2.0f, -2.0f);
            const float arg_scale = 2.0f * LOG2E * inv_cap;
            const f32x2 arg_scale2 = f2_make(arg_scale, arg_scale);
            f32x2 u[NV * 4];
            uint32_t hm = max2_16<T>::LOWEST;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = tr + i * tpr;
                if (v < nvec) {
                    uint4 a = cur[i];
                    if (bv != nullptr) {
                        const uint4 b = bv[v];
                        a.x = pack2<T>::add(a.x, b.x);
                        a.y = pack2<T>::add(a.y, b.y);
                        a.z = pack2<T>::add(a.z, b.z);
                        a.w = pack2<T>::add(a.w, b.w);
                    }
                    hm = max2_16<T>::of(max2_16<T>::of(hm, a.x), max2_16<T>::of(a.y, max2_16<T>::of(a.z, a.w)));
                    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 r = pack2<T>::up(w[q]);
                        const f32x2 raw = f2_make(r.x, r.y);
                        u[i * 4 + q] = CAP ? softcap_tanh2(raw, arg_scale2, one, minus_two) : raw;
                    }
                }
            }
            const float2 hmf = pack2<T>::up(hm);
            float um = fmaxf(hmf.x, hmf.y);
            if (CAP) um = softcap_tanh1(um, arg_scale);
            um = gdb_warp_max(um);
            if (wpr > 1) {
                if (lane == 0) red[0][rib][wr] = um;
                row_barrier(rib + 1, tpr);
                um = red[0][rib][0];
                for (int k = 1; k < wpr; ++k) um = fmaxf(um, red[0][rib][k]);
            }
            // u[] <- exp(soft - max) * d(soft)/d(raw); the thread that holds the target class keeps its two numbers
            const float unit = CAP ? cap : 1.0f;
            const float c1 = unit * LOG2E, c0 = -um * c1;
            const f32x2 c1_2 = f2_make(c1, c1), c0_2 = f2_make(c0, c0);
            f32x2 s2 = f2_make(0.0f, 0.0f);
            float tgt_u = 0.0f, tgt_exp = 0.0f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = tr + i * tpr;
                if (v < nvec) {
                    const unsigned rel = (unsigned)(t - v * 8);
                    f32x2 ex[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float a0, a1;
                        f2_split(f2_fma(u[i * 4 + q], c1_2, c0_2), a0, a1);
                        ex[q] = f2_make(exp2_ftz(a0), exp2_ftz(a1));
                        s2 = f2_add(s2, ex[q]);
                    }
                    if (rel < 8U) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float u0, u1, e0, e1;
                            f2_split(u[i * 4 + q], u0, u1);
                            f2_split(ex[q], e0, e1);
                            if (rel == (unsigned)(2 * q)) {
                                tgt_u = u0;
                                tgt_exp = e0;
                            }
                            if (rel == (unsigned)(2 * q + 1)) {
                                tgt_u = u1;
                                tgt_exp = e1;
                            }
                        }
                        target_soft[rib] = unit * tgt_u;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        u[i * 4 + q] = CAP ? f2_mul(ex[q], f2_fma(f2_mul(u[i * 4 + q], u[i * 4 + q]), minus_one, one)) : ex[q];
                    }
                }
            }
            float s_lo, s_hi;
            f2_split(s2, s_lo, s_hi);
            float s = gdb_warp_sum(s_lo + s_hi);
            if (wpr > 1) {
                if (lane == 0) red[1][rib][wr] = s;
                row_barrier(rib + 1, tpr);
                s = red[1][rib][0];
                for (int k = 1; k < wpr; ++k) s += red[1][rib][k];
            } else {
                __syncwarp();
            }
            if (tr == 0) {
                row_loss[row] = logf(s) + unit * um - target_soft[rib];
            }
            const float inv_sum = 1.0f / s;
            const float k = inv_sum * seed;
            const f32x2 k2 = f2_make(k, k);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = tr + i * tpr;
                if (v >= nvec) continue;
                const unsigned rel = (unsigned)(t - v * 8);
                float g[8];
#pragma unroll
                for (int q = 0; q < 4; ++q) f2_split(f2_mul(u[i * 4 + q], k2), g[2 * q], g[2 * q + 1]);
                if (rel < 8U) {                             // the target class: (p - 1) * slope * seed, as the reference orders it
                    const float slope = CAP ? fmaf(-tgt_u, tgt_u, 1.0f) : 1.0f;
                    const float gt = (tgt_exp * inv_sum - 1.0f) * slope * seed;
#pragma unroll
                    for (int e = 0; e < 8; ++e) g[e] = rel == (unsigned)e ? gt : g[e];
                }
                rv[v] = make_uint4(pack2<T>::down(g[0], g[1]), pack2<T>::down(g[2], g[3]), pack2<T>::down(g[4], g[5]), pack2<T>::down(g[6], g[7]));
            }
            if (wpr > 1) {
                row_barrier(rib + 1, tpr);                  // target_soft and red[] are rewritten by the next row
            } else {
                __syncwarp();
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
        t = t_next;
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

namespace {
template <typename T, int NV>
void launch_fused_rows(gd_backend *be, unsigned groups, bool capped, void *lp, const void *bp, const int *tp, const float *gl, const float *cp,
                       float *rl, size_t rows, int nvec, int wpr, float scale, float cap, float inv_cap, int ignore_index)
{
    // one wave of resident blocks, each walking over the row groups
    static int per_sm[2] = {0, 0};
    int &resident = per_sm[capped ? 1 : 0];
    if (resident == 0) {
        int n = 0;
        const cudaError_t e = capped ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, lmce_fused_rows_kernel<T, NV, true>, LMF_BLOCK, 0)
                                     : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, lmce_fused_rows_kernel<T, NV, false>, LMF_BLOCK, 0);
        resident = (e == cudaSuccess && n > 0) ? n : 1;
    }
    const unsigned wave = (unsigned)(be->sm_count > 0 ? be->sm_count : 1) * (unsigned)resident;
    const unsigned grid = groups < wave ? groups : wave;
    if (capped) {
        gdb_launch(lmce_fused_rows_kernel<T, NV, true>, grid, LMF_BLOCK, 0, be->stream, (T *)lp, (const T *)bp, tp, gl, cp, rl, rows, nvec, wpr, scale, cap, inv_cap, ignore_index);
    } else {
        gdb_launch(lmce_fused_rows_kernel<T, NV, false>, grid, LMF_BLOCK, 0, be->stream, (T *)lp, (const T *)bp, tp, gl, cp, rl, rows, nvec, wpr, scale, cap, inv_cap, ignore_index);
    }
}
}  // namespace

extern "C" gd_status gdb200_lm_cross_entropy_fused_rows(gd_backend *be, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *bias,
                                                        const gd_backend_tensor_view *targets, const gd_backend_tensor_view *grad_loss,
                                                        const gd_backend_tensor_view *counts, const gd_backend_tensor_view *row_loss, float scale,
                                                        float logits_softcap, int32_t ignore_index)
{
    chunk_shape cs;
    if (be == NULL || logits == NULL || targets == NULL || grad_loss == NULL || counts == NULL || row_loss == NULL ||
        !(logits_softcap >= 0.0f) || !chunk_dims(logits, targets, &cs) || row_loss->count != cs.rows || grad_loss->count != 1U ||
        counts->count == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t dt = logits->dtype;
    if (!half_dt(dt)) {
        return GD_ERR_UNSUPPORTED;
    }
    void *lp = gdb_tv_ptr(logits, dt);
    const void *bp = NULL;
    if (bias != NULL) {
        if (bias->count != cs.classes || (bp = gdb_tv_ptr(bias, dt)) == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const int *tp = (const int *)gdb_tv_ptr(targets, GDB_DTYPE_I32);
    const float *gl = (const float *)gdb_tv_ptr(grad_loss, GDB_DTYPE_F32), *cp = (const float *)gdb_tv_ptr(counts, GDB_DTYPE_F32);
    float *rl = (float *)gdb_tv_ptr(row_loss, GDB_DTYPE_F32);
    if (lp == NULL || tp == NULL || gl == NULL || cp == NULL || rl == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    // the whole row sits in the registers of at most 256 threads, LMF_VECTORS 16-byte vectors each; longer or unaligned rows
    // take the three-entry path
    if ((cs.classes % 8U) != 0U || (((uintptr_t)lp | (uintptr_t)bp) % 16U) != 0U || cs.classes / 8U > (size_t)(LMF_BLOCK * LMF_VECTORS)) {
        return GD_ERR_UNSUPPORTED;
    }
    const int nvec = (int)(cs.classes / 8U);
    int wpr = 1;
    while (wpr * 32 * LMF_VECTORS < nvec) {
        wpr <<= 1;
    }
    const unsigned rpb = (unsigned)((LMF_BLOCK / 32) / wpr);
    const unsigned groups = (unsigned)((cs.rows + rpb - 1U) / rpb);
    const float inv_cap = logits_softcap > 0.0f ? 1.0f / logits_softcap : 0.0f;
    const bool capped = logits_softcap > 0.0f;
    if (dt == GDB_DTYPE_F16) {
        launch_fused_rows<__half, LMF_VECTORS>(be, groups, capped, lp, bp, tp, gl, cp, rl, cs.rows, nvec, wpr, scale, logits_softcap, inv_cap, (int)ignore_index);
    } else {
        launch_fused_rows<__nv_bfloat16, LMF_VECTORS>(be, groups, capped, lp, bp, tp, gl, cp, rl, cs.rows, nvec, wpr, scale, logits_softcap, inv_cap, (int)ignore_index);
    }
    return gdb_launched(be, "lm_cross_entropy_fused_rows");
}

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
