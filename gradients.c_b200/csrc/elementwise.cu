// HBM-bound elementwise kernels: add (with numpy-style broadcast), relu, dropout family,
// SwiGLU family. 16-byte vector loads/stores on the aligned fast paths, grid-stride loops
// sized to a few waves of the SM count.
//
// Reference arithmetic: src/ops/add/metal_add.metal, src/ops/_shared/binary/metal_binary_common.h:68-128
// (broadcast rule), src/ops/dropout/metal_dropout.metal:6-140 + metal_dropout.m:145-155
// (keep rule and threshold), src/ops/swiglu/metal_swiglu.metal:6-151.
#include "common.cuh"
#include "decode_parts.cuh"

#include <math.h>

namespace {

// ------------------------------------------------------------------ add / relu
struct bcast_desc {
    uint32_t rank;
    uint32_t shape[8];
    uint64_t xs[8];
    uint64_t ys[8];
};

// OP: 0 add, 1 mul, 2 sub; computed in FP32 and rounded once to the storage type (for 16-bit storage that equals
// the reference's half-precision arithmetic, src/ops/{add,mul,sub}/metal_*.metal).
enum { BIN_ADD = 0, BIN_MUL = 1, BIN_SUB = 2 };
template <int OP>
__device__ __forceinline__ float binop(float a, float b)
{
    return OP == BIN_ADD ? a + b : (OP == BIN_MUL ? a * b : a - b);
}

template <typename T, int OP>
__global__ void add_direct_kernel(const T *x, const T *y, T *out, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        gdb_io<T>::st(out, i, binop<OP>(gdb_io<T>::ld(x, i), gdb_io<T>::ld(y, i)));
    }
}
template <typename T, int OP>
__global__ void add_direct_vec8_kernel(const uint4 *x, const uint4 *y, uint4 *out, size_t vecs)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        gdb_vec8<T> a, b;
        a.raw = x[i];
        b.raw = y[i];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a.set(e, binop<OP>(a.get(e), b.get(e)));
        }
        out[i] = a.raw;
    }
}
// out[r, c] = x[r, c] + y[c]; cols % 8 == 0, all pointers 16-byte aligned.
template <typename T, int OP>
__global__ void add_row_vec8_kernel(const uint4 *x, const uint4 *y, uint4 *out, size_t vecs, unsigned row_vecs)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        gdb_vec8<T> a, b;
        a.raw = x[i];
        b.raw = __ldg(&y[i % row_vecs]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a.set(e, binop<OP>(a.get(e), b.get(e)));
        }
        out[i] = a.raw;
    }
}
template <typename T, int OP>
__global__ void add_bcast_kernel(const T *x, const T *y, T *out, size_t n, bcast_desc d)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        size_t rem = i, xo = 0, yo = 0;
        for (int dim = (int)d.rank - 1; dim >= 0; --dim) {
            const size_t idx = rem % d.shape[dim];
            rem /= d.shape[dim];
            xo += idx * d.xs[dim];
            yo += idx * d.ys[dim];
        }
        gdb_io<T>::st(out, i, binop<OP>(gdb_io<T>::ld(x, xo), gdb_io<T>::ld(y, yo)));
    }
}

template <typename T>
__global__ void relu_kernel(const T *x, T *y, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = gdb_io<T>::ld(x, i);
        gdb_io<T>::st(y, i, v > 0.0f ? v : 0.0f);
    }
}
template <typename T>
__global__ void relu_backward_kernel(const T *x, const T *g, T *dx, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        gdb_io<T>::st(dx, i, gdb_io<T>::ld(x, i) > 0.0f ? gdb_io<T>::ld(g, i) : 0.0f);
    }
}

bool bcast_stride(const gd_backend_tensor_view *arg, const gd_backend_tensor_view *out, uint32_t dim, uint64_t *stride)
{
    if (arg->rank > out->rank || out->rank > 8U) {
        return false;
    }
    const uint32_t prefix = out->rank - arg->rank;
    if (out->shape[dim] <= 0) {
        return false;
    }
    if (dim < prefix) {
        *stride = 0;
        return true;
    }
    const int64_t ad = arg->shape[dim - prefix], st = arg->strides[dim - prefix];
    if (ad == out->shape[dim] && st >= 0) {
        *stride = (uint64_t)st;
        return true;
    }
    if (ad == 1) {
        *stride = 0;
        return true;
    }
    return false;
}

template <typename T, int OP>
gd_status add_typed(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y,
                    const gd_backend_tensor_view *out, const bcast_desc &d, bool direct, bool row)
{
    const T *xp = (const T *)(x->buffer->dptr + x->offset);
    const T *yp = (const T *)(y->buffer->dptr + y->offset);
    T *op = (T *)(out->buffer->dptr + out->offset);
    const size_t n = out->count;
    const bool al16 = (((uintptr_t)xp | (uintptr_t)yp | (uintptr_t)op) % 16U) == 0U;
    if constexpr (sizeof(T) == 2) {
        if (direct && al16 && (n % 8U) == 0U) {
            gdb_launch(add_direct_vec8_kernel<T, OP>, gdb_grid_for(n / 8U, 256, be, 8), 256, 0, be->stream, (const uint4 *)xp, (const uint4 *)yp, (uint4 *)op, n / 8U);
            return gdb_launched(be, OP == BIN_ADD ? "add" : (OP == BIN_MUL ? "mul" : "sub"));
        }
        if (!direct && row && al16 && (d.shape[d.rank - 1] % 8U) == 0U) {
            gdb_launch(add_row_vec8_kernel<T, OP>, gdb_grid_for(n / 8U, 256, be, 8), 256, 0, be->stream, (const uint4 *)xp, (const uint4 *)yp, (uint4 *)op, n / 8U, d.shape[d.rank - 1] / 8U);
            return gdb_launched(be, OP == BIN_ADD ? "add" : (OP == BIN_MUL ? "mul" : "sub"));
        }
    }
    if (direct) {
        gdb_launch(add_direct_kernel<T, OP>, gdb_grid_for(n, 256, be, 8), 256, 0, be->stream, xp, yp, op, n);
    } else {
        gdb_launch(add_bcast_kernel<T, OP>, gdb_grid_for(n, 256, be, 8), 256, 0, be->stream, xp, yp, op, n, d);
    }
    return gdb_launched(be, OP == BIN_ADD ? "add" : (OP == BIN_MUL ? "mul" : "sub"));
}

// ------------------------------------------------------------------ dropout
__device__ __forceinline__ bool dropout_keep(uint64_t seed, uint64_t index, unsigned threshold) { return gdb_dropout_keep(seed, index, threshold); }
unsigned dropout_threshold(float p) { return gdb_dropout_threshold(p); }

// MODE 0: y = dropout(x), write mask. MODE 1: y = residual + dropout(x), write mask.
// MODE 2: dx = g * keep(seed) * scale (recompute). MODE 3: dx = g * mask * scale.
template <typename T, int MODE>
__global__ void dropout_kernel(const T *x, const T *residual, const unsigned char *mask_in, T *y,
                               unsigned char *mask_out, size_t n, float scale, uint64_t seed, unsigned threshold)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        bool keep;
        if (MODE == 3) {
            keep = mask_in[i] != 0;
        } else {
            keep = dropout_keep(seed, (uint64_t)i, threshold);
        }
        // the dropped value is rounded to storage precision before the residual add,
        // as in the reference (metal_dropout.metal:129-140)
        const float dropped = keep ? gdb_io<T>::rnd(gdb_io<T>::ld(x, i) * scale) : 0.0f;
        if (MODE == 0 || MODE == 1) {
            mask_out[i] = keep ? 1 : 0;
        }
        gdb_io<T>::st(y, i, MODE == 1 ? gdb_io<T>::ld(residual, i) + dropped : dropped);
    }
}

template <typename T, int MODE>
__global__ void dropout_vec8_kernel(const uint4 *x, const uint4 *residual, const uint2 *mask_in, uint4 *y,
                                    uint2 *mask_out, size_t vecs, float scale, uint64_t seed, unsigned threshold)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        gdb_vec8<T> xv, rv;
        xv.raw = x[v];
        if (MODE == 1) {
            rv.raw = residual[v];
        }
        uint2 m = make_uint2(0U, 0U);
        if (MODE == 3) {
            m = mask_in[v];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            bool keep;
            unsigned *mw = e < 4 ? &m.x : &m.y;
            const unsigned sh = 8U * (unsigned)(e & 3);
            if (MODE == 3) {
                keep = ((*mw >> sh) & 255U) != 0U;
            } else {
                keep = dropout_keep(seed, (uint64_t)v * 8U + (uint64_t)e, threshold);
                *mw |= (keep ? 1U : 0U) << sh;
            }
            const float dropped = keep ? gdb_io<T>::rnd(xv.get(e) * scale) : 0.0f;
            xv.set(e, MODE == 1 ? rv.get(e) + dropped : dropped);
        }
        y[v] = xv.raw;
        if (MODE == 0 || MODE == 1) {
            mask_out[v] = m;
        }
    }
}

template <typename T, int MODE>
gd_status dropout_launch(gd_backend *be, const void *x, const void *residual, const void *mask_in, void *y,
                         void *mask_out, size_t n, float scale, uint64_t seed, unsigned threshold)
{
    const uintptr_t al = (uintptr_t)x | (uintptr_t)y | (MODE == 1 ? (uintptr_t)residual : 0U);
    const uintptr_t mal = (MODE == 3 ? (uintptr_t)mask_in : 0U) | ((MODE == 0 || MODE == 1) ? (uintptr_t)mask_out : 0U);
    if constexpr (sizeof(T) == 2) {
        if ((n % 8U) == 0U && (al % 16U) == 0U && (mal % 8U) == 0U) {
            gdb_launch(dropout_vec8_kernel<T, MODE>, gdb_grid_for(n / 8U, 256, be, 8), 256, 0, be->stream, (const uint4 *)x, (const uint4 *)residual, (const uint2 *)mask_in, (uint4 *)y, (uint2 *)mask_out,
                n / 8U, scale, seed, threshold);
            return gdb_launched(be, "dropout");
        }
    }
    {
        gdb_launch(dropout_kernel<T, MODE>, gdb_grid_for(n, 256, be, 8), 256, 0, be->stream, (const T *)x, (const T *)residual, (const unsigned char *)mask_in, (T *)y, (unsigned char *)mask_out,
            n, scale, seed, threshold);
    }
    return gdb_launched(be, "dropout");
}

template <int MODE>
gd_status dropout_dispatch(gd_backend *be, uint32_t dtype, const void *x, const void *residual, const void *mask_in,
                           void *y, void *mask_out, size_t n, float scale, uint64_t seed, unsigned threshold)
{
    if (dtype == GDB_DTYPE_F16) {
        return dropout_launch<__half, MODE>(be, x, residual, mask_in, y, mask_out, n, scale, seed, threshold);
    }
    if (dtype == GDB_DTYPE_BF16) {
        return dropout_launch<__nv_bfloat16, MODE>(be, x, residual, mask_in, y, mask_out, n, scale, seed, threshold);
    }
    if (dtype == GDB_DTYPE_F32) {
        return dropout_launch<float, MODE>(be, x, residual, mask_in, y, mask_out, n, scale, seed, threshold);
    }
    return GD_ERR_UNSUPPORTED;
}

bool dropout_p_ok(float p) { return p >= 0.0f && p < 1.0f; }

// ------------------------------------------------------------------ SwiGLU
__device__ __forceinline__ float swiglu_sigmoid(float x) { return gdb_swiglu_sigmoid(x); }

// out[r, c] = x1[r, c] * silu(x2[r, c]); x1/x2 rows may live in one [rows, 2H] tensor.
template <typename T>
__global__ void swiglu_fwd_kernel(const T *x1, const T *x2, T *out, size_t rows, size_t h, size_t in_ld)
{
    gdb_pdl_sync();
    const size_t n = rows * h, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t r = i / h, c = i - r * h;
        const float z = gdb_io<T>::ld(x2, r * in_ld + c);
        gdb_io<T>::st(out, i, gdb_io<T>::ld(x1, r * in_ld + c) * (z * swiglu_sigmoid(z)));
    }
}
template <typename T>
__global__ void swiglu_fwd_vec8_kernel(const uint4 *x1, const uint4 *x2, uint4 *out, unsigned rows, unsigned hv, unsigned in_ldv)
{
    gdb_pdl_sync();
    // 32-bit index arithmetic (the host checks rows * hv < 2^32): a 64-bit division per 16-byte vector costs more than the gate
    const unsigned n = rows * hv, stride = gridDim.x * blockDim.x;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned r = i / hv, c = i - r * hv;
        gdb_vec8<T> a, b;
        a.raw = x1[(size_t)r * in_ldv + c];
        b.raw = x2[(size_t)r * in_ldv + c];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float z = b.get(e);
            a.set(e, a.get(e) * (z * swiglu_sigmoid(z)));
        }
        out[i] = a.raw;
    }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T *x1, const T *x2, const T *go, T *dx1, T *dx2,
                                  size_t rows, size_t h, size_t in_ld, size_t out_ld)
{
    gdb_pdl_sync();
    const size_t n = rows * h, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t r = i / h, c = i - r * h;
        const float z = gdb_io<T>::ld(x2, r * in_ld + c);
        const float g = gdb_io<T>::ld(go, i);
        const float s = swiglu_sigmoid(z);
        if (dx1 != nullptr) {
            gdb_io<T>::st(dx1, r * out_ld + c, g * (z * s));
        }
        if (dx2 != nullptr) {
            gdb_io<T>::st(dx2, r * out_ld + c, g * gdb_io<T>::ld(x1, r * in_ld + c) * (s * (1.0f + z * (1.0f - s))));
        }
    }
}
template <typename T>
__global__ void swiglu_bwd_vec8_kernel(const uint4 *x1, const uint4 *x2, const uint4 *go, uint4 *dx1, uint4 *dx2,
                                       unsigned rows, unsigned hv, unsigned in_ldv, unsigned out_ldv)
{
    gdb_pdl_sync();
    const unsigned n = rows * hv, stride = gridDim.x * blockDim.x;   // 32-bit index arithmetic, see the forward kernel
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned r = i / hv, c = i - r * hv;
        // packed conversions (two elements per instruction both ways); the arithmetic per element is unchanged
        float a[8], b[8], g[8], d1[8], d2[8];
        gdb_dec::unpack8<T>(x1[(size_t)r * in_ldv + c], a);
        gdb_dec::unpack8<T>(x2[(size_t)r * in_ldv + c], b);
        gdb_dec::unpack8<T>(go[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float z = b[e], s = swiglu_sigmoid(z), gv = g[e];
            d1[e] = gv * (z * s);
            d2[e] = gv * a[e] * (s * (1.0f + z * (1.0f - s)));
        }
        using pk = gdb_dec::pack2<T>;
        dx1[(size_t)r * out_ldv + c] = make_uint4(pk::down(d1[0], d1[1]), pk::down(d1[2], d1[3]), pk::down(d1[4], d1[5]), pk::down(d1[6], d1[7]));
        dx2[(size_t)r * out_ldv + c] = make_uint4(pk::down(d2[0], d2[1]), pk::down(d2[2], d2[3]), pk::down(d2[4], d2[5]), pk::down(d2[6], d2[7]));
    }
}

template <typename T>
gd_status swiglu_fwd_typed(gd_backend *be, const void *x1, const void *x2, void *out, size_t rows, size_t h, size_t in_ld)
{
    const uintptr_t al = (uintptr_t)x1 | (uintptr_t)x2 | (uintptr_t)out;
    if ((al % 16U) == 0U && (h % 8U) == 0U && (in_ld % 8U) == 0U && rows * (h / 8U) < 0xffffffffULL && in_ld / 8U < 0xffffffffULL) {
        gdb_launch(swiglu_fwd_vec8_kernel<T>, gdb_grid_for(rows * h / 8U, 256, be, 8), 256, 0, be->stream, (const uint4 *)x1, (const uint4 *)x2, (uint4 *)out, (unsigned)rows, (unsigned)(h / 8U), (unsigned)(in_ld / 8U));
    } else {
        gdb_launch(swiglu_fwd_kernel<T>, gdb_grid_for(rows * h, 256, be, 8), 256, 0, be->stream, (const T *)x1, (const T *)x2, (T *)out, rows, h, in_ld);
    }
    return gdb_launched(be, "swiglu_forward");
}
template <typename T>
gd_status swiglu_bwd_typed(gd_backend *be, const void *x1, const void *x2, const void *go, void *dx1, void *dx2,
                           size_t rows, size_t h, size_t in_ld, size_t out_ld)
{
    const uintptr_t al = (uintptr_t)x1 | (uintptr_t)x2 | (uintptr_t)go | (uintptr_t)dx1 | (uintptr_t)dx2;
    if (dx1 != NULL && dx2 != NULL && (al % 16U) == 0U && (h % 8U) == 0U && (in_ld % 8U) == 0U && (out_ld % 8U) == 0U && rows * (h / 8U) < 0xffffffffULL && in_ld / 8U < 0xffffffffULL && out_ld / 8U < 0xffffffffULL) {
        gdb_launch(swiglu_bwd_vec8_kernel<T>, gdb_grid_for(rows * h / 8U, 256, be, 8), 256, 0, be->stream, (const uint4 *)x1, (const uint4 *)x2, (const uint4 *)go, (uint4 *)dx1, (uint4 *)dx2, (unsigned)rows, (unsigned)(h / 8U), (unsigned)(in_ld / 8U), (unsigned)(out_ld / 8U));
    } else {
        gdb_launch(swiglu_bwd_kernel<T>, gdb_grid_for(rows * h, 256, be, 8), 256, 0, be->stream, (const T *)x1, (const T *)x2, (const T *)go, (T *)dx1, (T *)dx2, rows, h, in_ld, out_ld);
    }
    return gdb_launched(be, "swiglu_backward");
}

bool half_dtype(uint32_t dt) { return dt == GDB_DTYPE_F16 || dt == GDB_DTYPE_BF16; }

}  // namespace

// Broadcasting binary op (src/core/backend_generated.h:14-28): out = x OP y with numpy-style broadcasting of x and y.
template <int OP>
static gd_status binary_entry(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *out)
{
    bcast_desc d;
    bool direct = true;
    if (be == NULL || x == NULL || y == NULL || out == NULL || x->dtype != out->dtype || y->dtype != out->dtype ||
        out->rank > 8U || x->rank > out->rank || y->rank > out->rank) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(out->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    if (gdb_tv_ptr(x, x->dtype) == NULL || gdb_tv_ptr(y, y->dtype) == NULL || gdb_tv_ptr(out, out->dtype) == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (out->count == 0U) {
        return GD_OK;
    }
    memset(&d, 0, sizeof(d));
    d.rank = out->rank == 0U ? 1U : out->rank;
    if (out->rank == 0U) {
        d.shape[0] = 1U;
    }
    uint64_t contiguous = 1;
    for (int dim = (int)out->rank - 1; dim >= 0; --dim) {
        const uint32_t xp = out->rank - x->rank, yp = out->rank - y->rank;
        const int64_t xd = (uint32_t)dim < xp ? 1 : x->shape[dim - xp];
        const int64_t yd = (uint32_t)dim < yp ? 1 : y->shape[dim - yp];
        if (out->shape[dim] != (xd > yd ? xd : yd) || !bcast_stride(x, out, (uint32_t)dim, &d.xs[dim]) ||
            !bcast_stride(y, out, (uint32_t)dim, &d.ys[dim])) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        d.shape[dim] = (uint32_t)out->shape[dim];
        if (out->shape[dim] != 1 && (d.xs[dim] != contiguous || d.ys[dim] != contiguous)) {
            direct = false;
        }
        contiguous *= (uint64_t)out->shape[dim];
    }
    // row broadcast: x is the full contiguous tensor and y repeats along every leading dim
    bool row = !direct && out->rank >= 1U && x->count == out->count && d.ys[out->rank - 1U] == 1U;
    if (row) {
        uint64_t c = 1;
        for (int dim = (int)out->rank - 1; dim >= 0; --dim) {
            if (out->shape[dim] != 1 && d.xs[dim] != c) {
                row = false;
            }
            if (dim < (int)out->rank - 1 && out->shape[dim] != 1 && d.ys[dim] != 0U) {
                row = false;
            }
            c *= (uint64_t)out->shape[dim];
        }
    }
    if (out->dtype == GDB_DTYPE_F16) {
        return add_typed<__half, OP>(be, x, y, out, d, direct, row);
    }
    if (out->dtype == GDB_DTYPE_BF16) {
        return add_typed<__nv_bfloat16, OP>(be, x, y, out, d, direct, row);
    }
    return add_typed<float, OP>(be, x, y, out, d, direct, row);
}

extern "C" {

gd_status gd_backend_add(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *out)
{
    return binary_entry<BIN_ADD>(be, x, y, out);
}
gd_status gd_backend_mul(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *out)
{
    return binary_entry<BIN_MUL>(be, x, y, out);
}
gd_status gd_backend_sub(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *out)
{
    return binary_entry<BIN_SUB>(be, x, y, out);
}

gd_status gd_backend_relu(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y)
{
    if (be == NULL || x == NULL || y == NULL || x->dtype != y->dtype || x->count != y->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype);
    void *yp = gdb_tv_ptr(y, y->dtype);
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    if (xp == NULL || yp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x->count == 0U) {
        return GD_OK;
    }
    const unsigned grid = gdb_grid_for(x->count, 256, be, 8);
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(relu_kernel<__half>, grid, 256, 0, be->stream, (const __half *)xp, (__half *)yp, x->count);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(relu_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, (__nv_bfloat16 *)yp, x->count);
    } else {
        gdb_launch(relu_kernel<float>, grid, 256, 0, be->stream, (const float *)xp, (float *)yp, x->count);
    }
    return gdb_launched(be, "relu");
}

gd_status gd_backend_relu_backward(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x)
{
    if (be == NULL || x == NULL || grad_out == NULL || grad_x == NULL || x->dtype != grad_out->dtype ||
        x->dtype != grad_x->dtype || x->count != grad_out->count || x->count != grad_x->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *gp = gdb_tv_ptr(grad_out, x->dtype);
    void *dp = gdb_tv_ptr(grad_x, x->dtype);
    if (xp == NULL || gp == NULL || dp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x->count == 0U) {
        return GD_OK;
    }
    const unsigned grid = gdb_grid_for(x->count, 256, be, 8);
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(relu_backward_kernel<__half>, grid, 256, 0, be->stream, (const __half *)xp, (const __half *)gp, (__half *)dp, x->count);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(relu_backward_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, (const __nv_bfloat16 *)gp, (__nv_bfloat16 *)dp, x->count);
    } else {
        gdb_launch(relu_backward_kernel<float>, grid, 256, 0, be->stream, (const float *)xp, (const float *)gp, (float *)dp, x->count);
    }
    return gdb_launched(be, "relu_backward");
}

gd_status gd_backend_dropout_forward(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *mask, float p, uint64_t seed)
{
    if (be == NULL || x == NULL || y == NULL || mask == NULL || !dropout_p_ok(p) || x->dtype != y->dtype ||
        !gdb_same_shape(x, y) || mask->count != x->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype);
    void *yp = gdb_tv_ptr(y, y->dtype), *mp = gdb_tv_ptr(mask, GDB_DTYPE_U8);
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    if (xp == NULL || yp == NULL || mp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x->count == 0U) {
        return GD_OK;
    }
    return dropout_dispatch<0>(be, x->dtype, xp, NULL, NULL, yp, mp, x->count, 1.0f / (1.0f - p), seed, dropout_threshold(p));
}

gd_status gd_backend_dropout_add_forward(gd_backend *be, const gd_backend_tensor_view *residual, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *mask, float p, uint64_t seed)
{
    if (be == NULL || residual == NULL || x == NULL || y == NULL || mask == NULL || !dropout_p_ok(p) ||
        x->dtype != y->dtype || residual->dtype != x->dtype || !gdb_same_shape(x, y) ||
        !gdb_same_shape(x, residual) || mask->count != x->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!half_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;  // the reference entry is F16-only
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *rp = gdb_tv_ptr(residual, x->dtype);
    void *yp = gdb_tv_ptr(y, y->dtype), *mp = gdb_tv_ptr(mask, GDB_DTYPE_U8);
    if (xp == NULL || rp == NULL || yp == NULL || mp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x->count == 0U) {
        return GD_OK;
    }
    return dropout_dispatch<1>(be, x->dtype, xp, rp, NULL, yp, mp, x->count, 1.0f / (1.0f - p), seed, dropout_threshold(p));
}

gd_status gd_backend_dropout_backward(gd_backend *be, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x, float p, uint64_t seed)
{
    if (be == NULL || grad_out == NULL || grad_x == NULL || !dropout_p_ok(p) || grad_out->dtype != grad_x->dtype ||
        !gdb_same_shape(grad_out, grad_x)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(grad_out->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *gp = gdb_tv_ptr(grad_out, grad_out->dtype);
    void *dp = gdb_tv_ptr(grad_x, grad_x->dtype);
    if (gp == NULL || dp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (grad_out->count == 0U) {
        return GD_OK;
    }
    return dropout_dispatch<2>(be, grad_out->dtype, gp, NULL, NULL, dp, NULL, grad_out->count, 1.0f / (1.0f - p), seed, dropout_threshold(p));
}

gd_status gd_backend_dropout_backward_mask(gd_backend *be, const gd_backend_tensor_view *mask, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x, float scale)
{
    if (be == NULL || mask == NULL || grad_out == NULL || grad_x == NULL || !(scale > 0.0f) || scale != scale ||
        grad_out->dtype != grad_x->dtype || !gdb_same_shape(grad_out, grad_x) || mask->count != grad_out->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(grad_out->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *gp = gdb_tv_ptr(grad_out, grad_out->dtype), *mp = gdb_tv_ptr(mask, GDB_DTYPE_U8);
    void *dp = gdb_tv_ptr(grad_x, grad_x->dtype);
    if (gp == NULL || dp == NULL || mp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (grad_out->count == 0U) {
        return GD_OK;
    }
    return dropout_dispatch<3>(be, grad_out->dtype, gp, NULL, mp, dp, NULL, grad_out->count, scale, 0U, 0U);
}

gd_status gd_backend_swiglu_forward(gd_backend *be, const gd_backend_tensor_view *x1, const gd_backend_tensor_view *x2, const gd_backend_tensor_view *out)
{
    if (be == NULL || x1 == NULL || x2 == NULL || out == NULL || x1->dtype != x2->dtype || x1->dtype != out->dtype ||
        x1->count != x2->count || x1->count != out->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!half_dtype(x1->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *a = gdb_tv_ptr(x1, x1->dtype), *b = gdb_tv_ptr(x2, x1->dtype);
    void *o = gdb_tv_ptr(out, x1->dtype);
    if (a == NULL || b == NULL || o == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x1->count == 0U) {
        return GD_OK;
    }
    // one logical row: the kernels index x1/x2 by row * in_ld + c
    return x1->dtype == GDB_DTYPE_F16 ? swiglu_fwd_typed<__half>(be, a, b, o, 1U, x1->count, x1->count)
                                      : swiglu_fwd_typed<__nv_bfloat16>(be, a, b, o, 1U, x1->count, x1->count);
}

gd_status gd_backend_swiglu_backward(gd_backend *be, const gd_backend_tensor_view *x1, const gd_backend_tensor_view *x2, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x1, const gd_backend_tensor_view *grad_x2)
{
    if (be == NULL || x1 == NULL || x2 == NULL || grad_out == NULL || (grad_x1 == NULL && grad_x2 == NULL) ||
        x1->dtype != x2->dtype || x1->dtype != grad_out->dtype || x1->count != x2->count || x1->count != grad_out->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!half_dtype(x1->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *a = gdb_tv_ptr(x1, x1->dtype), *b = gdb_tv_ptr(x2, x1->dtype), *g = gdb_tv_ptr(grad_out, x1->dtype);
    void *d1 = grad_x1 != NULL ? gdb_tv_ptr(grad_x1, x1->dtype) : NULL;
    void *d2 = grad_x2 != NULL ? gdb_tv_ptr(grad_x2, x1->dtype) : NULL;
    if (a == NULL || b == NULL || g == NULL || (grad_x1 != NULL && (d1 == NULL || grad_x1->count != x1->count)) ||
        (grad_x2 != NULL && (d2 == NULL || grad_x2->count != x1->count))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (x1->count == 0U) {
        return GD_OK;
    }
    return x1->dtype == GDB_DTYPE_F16
               ? swiglu_bwd_typed<__half>(be, a, b, g, d1, d2, 1U, x1->count, x1->count, x1->count)
               : swiglu_bwd_typed<__nv_bfloat16>(be, a, b, g, d1, d2, 1U, x1->count, x1->count, x1->count);
}

// x12 [..., 2H] -> out [..., H], x1 = first half of each row (metal_swiglu.metal:113-116).
gd_status gd_backend_swiglu_split_forward(gd_backend *be, const gd_backend_tensor_view *x12, const gd_backend_tensor_view *out)
{
    if (be == NULL || x12 == NULL || out == NULL || x12->dtype != out->dtype || x12->rank == 0U || x12->rank > 8U ||
        x12->rank != out->rank) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!half_dtype(x12->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const int64_t two_h = x12->shape[x12->rank - 1U], h = out->shape[out->rank - 1U];
    if (h <= 0 || two_h != 2 * h || x12->count != 2U * out->count || (out->count % (size_t)h) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned char *xp = (const unsigned char *)gdb_tv_ptr(x12, x12->dtype);
    void *op = gdb_tv_ptr(out, out->dtype);
    if (xp == NULL || op == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t rows = out->count / (size_t)h;
    return x12->dtype == GDB_DTYPE_F16
               ? swiglu_fwd_typed<__half>(be, xp, xp + (size_t)h * 2U, op, rows, (size_t)h, (size_t)two_h)
               : swiglu_fwd_typed<__nv_bfloat16>(be, xp, xp + (size_t)h * 2U, op, rows, (size_t)h, (size_t)two_h);
}

gd_status gd_backend_swiglu_split_backward(gd_backend *be, const gd_backend_tensor_view *x12, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *grad_x12)
{
    if (be == NULL || x12 == NULL || grad_out == NULL || grad_x12 == NULL || x12->dtype != grad_out->dtype ||
        x12->dtype != grad_x12->dtype || x12->rank == 0U || x12->rank > 8U || grad_out->rank != x12->rank ||
        !gdb_same_shape(x12, grad_x12)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!half_dtype(x12->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const int64_t two_h = x12->shape[x12->rank - 1U], h = grad_out->shape[grad_out->rank - 1U];
    if (h <= 0 || two_h != 2 * h || x12->count != 2U * grad_out->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned char *xp = (const unsigned char *)gdb_tv_ptr(x12, x12->dtype);
    const void *gp = gdb_tv_ptr(grad_out, x12->dtype);
    unsigned char *dp = (unsigned char *)gdb_tv_ptr(grad_x12, x12->dtype);
    if (xp == NULL || gp == NULL || dp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t rows = grad_out->count / (size_t)h;
    return x12->dtype == GDB_DTYPE_F16
               ? swiglu_bwd_typed<__half>(be, xp, xp + (size_t)h * 2U, gp, dp, dp + (size_t)h * 2U, rows, (size_t)h, (size_t)two_h, (size_t)two_h)
               : swiglu_bwd_typed<__nv_bfloat16>(be, xp, xp + (size_t)h * 2U, gp, dp, dp + (size_t)h * 2U, rows, (size_t)h, (size_t)two_h, (size_t)two_h);
}

}  // extern "C"
