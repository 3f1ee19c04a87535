// Backend entries off the gpt_lm path that the reference's other examples and C tests use: sigmoid / tanh (with both
// backward forms), the mul backward fast paths, MSE and Huber losses, PoWLU gates and permute. All are one pass over
// their operands (HBM-bound, launch-bound at test sizes); arithmetic is FP32 with one rounding to the storage type,
// following the reference's Metal kernels cited at each entry.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------ unary activations
// OP 0: sigmoid (src/ops/sigmoid/metal_sigmoid.metal:6-20), 1: tanh (src/ops/tanh/metal_tanh.metal:6-27).
template <int OP>
__device__ __forceinline__ float act_forward(float x)
{
    if (OP == 0) {
        return 1.0f / (1.0f + expf(-x));
    }
    const float e = expf(-2.0f * fabsf(x));
    const float y = (1.0f - e) / (1.0f + e);
    return x < 0.0f ? -y : y;
}
template <int OP>
__device__ __forceinline__ float act_grad_from_y(float y, float g)
{
    return OP == 0 ? g * y * (1.0f - y) : g * (1.0f - y * y);
}

// MODE 0: y = f(x); 1: dx = g * f'(x) from the input; 2: dx = g * f'(y) from the saved output (a = y).
template <typename T, int OP, int MODE>
__global__ void act_kernel(const T *__restrict__ a, const T *__restrict__ g, T *__restrict__ out, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = gdb_io<T>::ld(a, i);
        float r;
        if (MODE == 0) {
            r = act_forward<OP>(v);
        } else {
            r = act_grad_from_y<OP>(MODE == 1 ? act_forward<OP>(v) : v, gdb_io<T>::ld(g, i));
        }
        gdb_io<T>::st(out, i, r);
    }
}

template <int OP, int MODE>
gd_status act_entry(gd_backend *be, const gd_backend_tensor_view *a, const gd_backend_tensor_view *g, const gd_backend_tensor_view *out,
                    const char *what)
{
    if (be == NULL || a == NULL || out == NULL || (MODE != 0 && g == NULL) || a->count == 0U || a->dtype != out->dtype ||
        !gdb_same_shape(a, out) || (MODE != 0 && (g->dtype != a->dtype || !gdb_same_shape(a, g)))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(a->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *ap = gdb_tv_ptr(a, a->dtype), *gp = MODE != 0 ? gdb_tv_ptr(g, a->dtype) : NULL;
    void *op = gdb_tv_ptr(out, a->dtype);
    if (ap == NULL || op == NULL || (MODE != 0 && gp == NULL)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const unsigned grid = gdb_grid_for(a->count, 256, be, 8);
    if (a->dtype == GDB_DTYPE_F16) {
        gdb_launch(act_kernel<__half, OP, MODE>, grid, 256, 0, be->stream, (const __half *)ap, (const __half *)gp, (__half *)op, a->count);
    } else if (a->dtype == GDB_DTYPE_BF16) {
        gdb_launch(act_kernel<__nv_bfloat16, OP, MODE>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)ap, (const __nv_bfloat16 *)gp,
                   (__nv_bfloat16 *)op, a->count);
    } else {
        gdb_launch(act_kernel<float, OP, MODE>, grid, 256, 0, be->stream, (const float *)ap, (const float *)gp, (float *)op, a->count);
    }
    return gdb_launched(be, what);
}

// ------------------------------------------------------------------ mul backward fast paths
template <typename T>
__global__ void mul_backward_direct_kernel(const T *__restrict__ x, const T *__restrict__ y, const T *__restrict__ g, T *__restrict__ dx,
                                           T *__restrict__ dy, size_t n)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float gv = gdb_io<T>::ld(g, i);
        gdb_io<T>::st(dx, i, gv * gdb_io<T>::ld(y, i));
        gdb_io<T>::st(dy, i, gv * gdb_io<T>::ld(x, i));
    }
}

// dst[j] = sum_r g[r, j] * o[r, j]: a block owns 32 columns, its 8 warps take rows round-robin (coalesced 32-wide row
// reads), partial sums meet in shared memory and are added in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
mul_reduce_suffix_kernel(const T *__restrict__ g, const T *__restrict__ o, T *__restrict__ dst, size_t repeats, size_t cols)
{
    gdb_pdl_sync();
    __shared__ float sh[8][33];
    const int cx = threadIdx.x & 31, gy = threadIdx.x >> 5;
    const size_t c = (size_t)blockIdx.x * 32 + cx;
    float s = 0.0f;
    if (c < cols) {
        for (size_t r = gy; r < repeats; r += 8) {
            s += gdb_io<T>::ld(g, r * cols + c) * gdb_io<T>::ld(o, r * cols + c);
        }
    }
    sh[gy][cx] = s;
    __syncthreads();
    if (gy == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += sh[w][cx];
        gdb_io<T>::st(dst, c, t);
    }
}

// ------------------------------------------------------------------ pairwise losses
// LOSS 0: squared error (src/ops/mse/metal_mse.metal), 1: Huber (src/ops/huber/metal_huber.metal:8-18).
template <int LOSS>
__device__ __forceinline__ float loss_value(float d, float delta)
{
    if (LOSS == 0) {
        return d * d;
    }
    const float ad = fabsf(d);
    return ad <= delta ? 0.5f * d * d : delta * (ad - 0.5f * delta);
}
template <int LOSS>
__device__ __forceinline__ float loss_grad(float d, float delta)
{
    if (LOSS == 0) {
        return d;
    }
    return fabsf(d) <= delta ? d : (d < 0.0f ? -delta : delta);
}

// out[chunk] = scale * sum over the chunk; one block per chunk, fixed summation order.
template <typename T, int LOSS>
__global__ void __launch_bounds__(256)
loss_forward_kernel(const T *__restrict__ x, const T *__restrict__ y, float *__restrict__ out, size_t count, size_t chunk, float scale, float delta)
{
    gdb_pdl_sync();
    __shared__ float sh[8];
    const size_t begin = (size_t)blockIdx.x * chunk;
    const size_t end = begin + chunk < count ? begin + chunk : count;
    float acc = 0.0f;
    for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
        acc += loss_value<LOSS>(gdb_io<T>::ld(x, i) - gdb_io<T>::ld(y, i), delta);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffU, acc, d);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += sh[w];
        out[blockIdx.x] = t * scale;
    }
}

template <typename T, int LOSS>
__global__ void loss_backward_kernel(const T *__restrict__ x, const T *__restrict__ y, const float *__restrict__ grad_out, T *__restrict__ dx,
                                     T *__restrict__ dy, size_t n, float scale, float delta)
{
    gdb_pdl_sync();
    const float g = grad_out[0] * scale;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float d = loss_grad<LOSS>(gdb_io<T>::ld(x, i) - gdb_io<T>::ld(y, i), delta) * g;
        if (dx != nullptr) gdb_io<T>::st(dx, i, d);
        if (dy != nullptr) gdb_io<T>::st(dy, i, -d);
    }
}

template <int LOSS>
gd_status loss_forward_entry(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *out,
                             uint64_t chunk_size, float scale, float delta)
{
    // argument rules of src/ops/_shared/loss/metal_pairwise_loss_common.h:160-190
    if (be == NULL || x == NULL || y == NULL || out == NULL || !(scale == scale) || chunk_size == 0U || chunk_size > 0xffffffffULL ||
        x->count == 0U || x->dtype != y->dtype || !gdb_same_shape(x, y) || out->dtype != GDB_DTYPE_F32 || x->count > 0xffffffffULL ||
        (LOSS == 1 && !(delta > 0.0f))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!gdb_is_float_dtype(x->dtype)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint64_t chunks = ((uint64_t)x->count + chunk_size - 1U) / chunk_size;
    if (out->count != (size_t)chunks) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *yp = gdb_tv_ptr(y, x->dtype);
    float *op = (float *)gdb_tv_ptr(out, GDB_DTYPE_F32);
    if (xp == NULL || yp == NULL || op == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const unsigned grid = (unsigned)chunks;
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(loss_forward_kernel<__half, LOSS>, grid, 256, 0, be->stream, (const __half *)xp, (const __half *)yp, op, x->count,
                   (size_t)chunk_size, scale, delta);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(loss_forward_kernel<__nv_bfloat16, LOSS>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, (const __nv_bfloat16 *)yp, op,
                   x->count, (size_t)chunk_size, scale, delta);
    } else {
        gdb_launch(loss_forward_kernel<float, LOSS>, grid, 256, 0, be->stream, (const float *)xp, (const float *)yp, op, x->count,
                   (size_t)chunk_size, scale, delta);
    }
    return gdb_launched(be, LOSS == 0 ? "mse_forward" : "huber_forward");
}

template <int LOSS>
gd_status loss_backward_entry(gd_backend *be, const gd_backend_tensor_view *x, const gd_backend_tensor_view *y, const gd_backend_tensor_view *grad_out,
                              const gd_backend_tensor_view *grad_x, const gd_backend_tensor_view *grad_y, float scale, float delta)
{
    // argument rules of src/ops/_shared/loss/metal_pairwise_loss_common.h:193-230
    if (be == NULL || x == NULL || y == NULL || grad_out == NULL || (grad_x == NULL && grad_y == NULL) || !(scale == scale) ||
        x->count == 0U || x->dtype != y->dtype || !gdb_same_shape(x, y) || grad_out->dtype != GDB_DTYPE_F32 || grad_out->rank != 0U ||
        grad_out->count != 1U || x->count > 0xffffffffULL || !gdb_is_float_dtype(x->dtype) || (LOSS == 1 && !(delta > 0.0f))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    for (const gd_backend_tensor_view *gv : {grad_x, grad_y}) {
        if (gv != NULL && (gv->dtype != x->dtype || !gdb_same_shape(x, gv) || gdb_tv_ptr(gv, x->dtype) == NULL)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *yp = gdb_tv_ptr(y, x->dtype);
    const float *gp = (const float *)gdb_tv_ptr(grad_out, GDB_DTYPE_F32);
    void *dxp = grad_x != NULL ? gdb_tv_ptr(grad_x, x->dtype) : NULL, *dyp = grad_y != NULL ? gdb_tv_ptr(grad_y, x->dtype) : NULL;
    if (xp == NULL || yp == NULL || gp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const unsigned grid = gdb_grid_for(x->count, 256, be, 8);
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(loss_backward_kernel<__half, LOSS>, grid, 256, 0, be->stream, (const __half *)xp, (const __half *)yp, gp, (__half *)dxp,
                   (__half *)dyp, x->count, scale, delta);
    } else if (x->dtype == GDB_DTYPE_BF16) {
        gdb_launch(loss_backward_kernel<__nv_bfloat16, LOSS>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, (const __nv_bfloat16 *)yp, gp,
                   (__nv_bfloat16 *)dxp, (__nv_bfloat16 *)dyp, x->count, scale, delta);
    } else {
        gdb_launch(loss_backward_kernel<float, LOSS>, grid, 256, 0, be->stream, (const float *)xp, (const float *)yp, gp, (float *)dxp,
                   (float *)dyp, x->count, scale, delta);
    }
    return gdb_launched(be, LOSS == 0 ? "mse_backward" : "huber_backward");
}

// ------------------------------------------------------------------ PoWLU (src/ops/powlu/metal_powlu.metal:25-76)
__device__ __forceinline__ float powlu_sigmoid(float x)
{
    const float e = expf(-fabsf(x));
    const float inv = 1.0f / (1.0f + e);
    return x >= 0.0f ? inv : e * inv;
}
// gate(z, m) = z * sigmoid(z) for z <= 0, z^(m / (sqrt(z) + 1)) * sigmoid(z) for z > 0; *grad = d gate / dz.
__device__ __forceinline__ float powlu_gate_and_grad(float z, float m, float *grad)
{
    const float s = powlu_sigmoid(z);
    if (!(z > 0.0f)) {
        *grad = s * (1.0f + z * (1.0f - s));
        return z * s;
    }
    const float zp = fmaxf(z, 0x1p-24f);
    const float r = sqrtf(zp), rp1 = r + 1.0f;
    const float a = m / rp1, lz = logf(zp);
    const float gate = expf(a * lz) * s;
    const float da = -m / (2.0f * r * rp1 * rp1);
    *grad = gate * (a / zp + da * lz + (1.0f - s));
    return gate;
}

// x1 / x2 rows may live in one [rows, 2H] tensor (in_ld = 2H) or in two [rows, H] tensors (in_ld = H).
template <typename T>
__global__ void powlu_fwd_kernel(const T *__restrict__ x1, const T *__restrict__ x2, T *__restrict__ out, size_t rows, size_t h, size_t in_ld, float m)
{
    gdb_pdl_sync();
    const size_t n = rows * h, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t r = i / h, c = i - r * h;
        float unused;
        gdb_io<T>::st(out, i, gdb_io<T>::ld(x1, r * in_ld + c) * powlu_gate_and_grad(gdb_io<T>::ld(x2, r * in_ld + c), m, &unused));
    }
}
template <typename T>
__global__ void powlu_bwd_kernel(const T *__restrict__ x1, const T *__restrict__ x2, const T *__restrict__ go, T *__restrict__ dx1,
                                 T *__restrict__ dx2, size_t rows, size_t h, size_t ld, float m)
{
    gdb_pdl_sync();
    const size_t n = rows * h, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t r = i / h, c = i - r * h;
        float dgate;
        const float gate = powlu_gate_and_grad(gdb_io<T>::ld(x2, r * ld + c), m, &dgate);
        const float g = gdb_io<T>::ld(go, i);
        if (dx1 != nullptr) gdb_io<T>::st(dx1, r * ld + c, g * gate);
        if (dx2 != nullptr) gdb_io<T>::st(dx2, r * ld + c, g * gdb_io<T>::ld(x1, r * ld + c) * dgate);
    }
}

bool powlu_dtype(uint32_t dt) { return dt == GDB_DTYPE_F16 || dt == GDB_DTYPE_BF16; }

bool powlu_split_shape(const gd_backend_tensor_view *x12, const gd_backend_tensor_view *out)
{
    if (x12->rank == 0U || x12->rank != out->rank || x12->rank > 8U || x12->shape[x12->rank - 1U] <= 0 ||
        (x12->shape[x12->rank - 1U] & 1) != 0 || out->shape[out->rank - 1U] != x12->shape[x12->rank - 1U] / 2) {
        return false;
    }
    for (uint32_t a = 0; a + 1U < x12->rank; ++a) {
        if (x12->shape[a] != out->shape[a]) {
            return false;
        }
    }
    return x12->count == out->count * 2U;
}

gd_status powlu_launch_fwd(gd_backend *be, uint32_t dt, const void *x1, const void *x2, void *out, size_t rows, size_t h, size_t ld, float m)
{
    cudaSetDevice(be->device);
    const unsigned grid = gdb_grid_for(rows * h, 256, be, 8);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(powlu_fwd_kernel<__half>, grid, 256, 0, be->stream, (const __half *)x1, (const __half *)x2, (__half *)out, rows, h, ld, m);
    } else {
        gdb_launch(powlu_fwd_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)x1, (const __nv_bfloat16 *)x2,
                   (__nv_bfloat16 *)out, rows, h, ld, m);
    }
    return gdb_launched(be, "powlu_forward");
}
gd_status powlu_launch_bwd(gd_backend *be, uint32_t dt, const void *x1, const void *x2, const void *go, void *dx1, void *dx2, size_t rows, size_t h,
                           size_t ld, float m)
{
    cudaSetDevice(be->device);
    const unsigned grid = gdb_grid_for(rows * h, 256, be, 8);
    if (dt == GDB_DTYPE_F16) {
        gdb_launch(powlu_bwd_kernel<__half>, grid, 256, 0, be->stream, (const __half *)x1, (const __half *)x2, (const __half *)go, (__half *)dx1,
                   (__half *)dx2, rows, h, ld, m);
    } else {
        gdb_launch(powlu_bwd_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)x1, (const __nv_bfloat16 *)x2,
                   (const __nv_bfloat16 *)go, (__nv_bfloat16 *)dx1, (__nv_bfloat16 *)dx2, rows, h, ld, m);
    }
    return gdb_launched(be, "powlu_backward");
}

// ------------------------------------------------------------------ permute (src/ops/permute/metal_permute.metal:4-28)
struct permute_desc {
    uint32_t rank;
    uint64_t dst_shape[8];
    uint64_t src_stride[8];   // stride in the source of the axis that output axis d reads
};
template <typename U>
__global__ void permute_kernel(const U *__restrict__ src, U *__restrict__ dst, size_t n, permute_desc d)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        size_t rem = i, so = 0;
        for (int a = (int)d.rank - 1; a >= 0; --a) {
            const size_t coord = rem % d.dst_shape[a];
            rem /= d.dst_shape[a];
            so += coord * d.src_stride[a];
        }
        dst[i] = src[so];
    }
}

bool contiguous_view(const gd_backend_tensor_view *v)
{
    int64_t expected = 1;
    if (v->rank > 8U) {
        return false;
    }
    for (int a = (int)v->rank - 1; a >= 0; --a) {
        if (v->shape[a] <= 0 || v->strides[a] != expected) {
            return false;
        }
        expected *= v->shape[a];
    }
    return true;
}

}  // namespace

extern "C" {

typedef const gd_backend_tensor_view *TV;

gd_status gd_backend_sigmoid(gd_backend *be, TV x, TV y) { return act_entry<0, 0>(be, x, NULL, y, "sigmoid"); }
gd_status gd_backend_sigmoid_backward(gd_backend *be, TV x, TV grad_out, TV grad_x) { return act_entry<0, 1>(be, x, grad_out, grad_x, "sigmoid_backward"); }
gd_status gd_backend_sigmoid_backward_from_output(gd_backend *be, TV y, TV grad_out, TV grad_x)
{
    return act_entry<0, 2>(be, y, grad_out, grad_x, "sigmoid_backward_from_output");
}
gd_status gd_backend_tanh(gd_backend *be, TV x, TV y) { return act_entry<1, 0>(be, x, NULL, y, "tanh"); }
gd_status gd_backend_tanh_backward(gd_backend *be, TV x, TV grad_out, TV grad_x) { return act_entry<1, 1>(be, x, grad_out, grad_x, "tanh_backward"); }
gd_status gd_backend_tanh_backward_from_output(gd_backend *be, TV y, TV grad_out, TV grad_x)
{
    return act_entry<1, 2>(be, y, grad_out, grad_x, "tanh_backward_from_output");
}

// grad_x = grad_out * y, grad_y = grad_out * x for equal shapes (src/ops/mul/metal_mul.metal gd_mul_backward_direct_kernel).
gd_status gd_backend_mul_backward_direct(gd_backend *be, TV x, TV y, TV grad_out, TV grad_x, TV grad_y)
{
    if (be == NULL || x == NULL || y == NULL || grad_out == NULL || grad_x == NULL || grad_y == NULL || x->count == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    for (TV v : {y, grad_out, grad_x, grad_y}) {
        if (v->dtype != x->dtype || !gdb_same_shape(x, v)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    if (!powlu_dtype(x->dtype)) {
        return GD_ERR_UNSUPPORTED;   // the reference entry is F16-only
    }
    const void *xp = gdb_tv_ptr(x, x->dtype), *yp = gdb_tv_ptr(y, x->dtype), *gp = gdb_tv_ptr(grad_out, x->dtype);
    void *dxp = gdb_tv_ptr(grad_x, x->dtype), *dyp = gdb_tv_ptr(grad_y, x->dtype);
    if (xp == NULL || yp == NULL || gp == NULL || dxp == NULL || dyp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const unsigned grid = gdb_grid_for(x->count, 256, be, 8);
    if (x->dtype == GDB_DTYPE_F16) {
        gdb_launch(mul_backward_direct_kernel<__half>, grid, 256, 0, be->stream, (const __half *)xp, (const __half *)yp, (const __half *)gp,
                   (__half *)dxp, (__half *)dyp, x->count);
    } else {
        gdb_launch(mul_backward_direct_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)xp, (const __nv_bfloat16 *)yp,
                   (const __nv_bfloat16 *)gp, (__nv_bfloat16 *)dxp, (__nv_bfloat16 *)dyp, x->count);
    }
    return gdb_launched(be, "mul_backward_direct");
}

// dst[j] = sum_r grad_out[r, j] * other[r, j], r over count / dst.count repeats (gd_mul_reduce_suffix_kernel).
gd_status gd_backend_mul_reduce_suffix(gd_backend *be, TV grad_out, TV other, TV dst)
{
    if (be == NULL || grad_out == NULL || other == NULL || dst == NULL || grad_out->count == 0U || dst->count == 0U ||
        grad_out->dtype != other->dtype || grad_out->dtype != dst->dtype || !gdb_same_shape(grad_out, other) ||
        grad_out->count > 0xffffffffULL || (grad_out->count % dst->count) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!powlu_dtype(dst->dtype)) {
        return GD_ERR_UNSUPPORTED;
    }
    const void *gp = gdb_tv_ptr(grad_out, dst->dtype), *op = gdb_tv_ptr(other, dst->dtype);
    void *dp = gdb_tv_ptr(dst, dst->dtype);
    if (gp == NULL || op == NULL || dp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const size_t cols = dst->count, repeats = grad_out->count / dst->count;
    const unsigned grid = (unsigned)((cols + 31U) / 32U);
    if (dst->dtype == GDB_DTYPE_F16) {
        gdb_launch(mul_reduce_suffix_kernel<__half>, grid, 256, 0, be->stream, (const __half *)gp, (const __half *)op, (__half *)dp, repeats, cols);
    } else {
        gdb_launch(mul_reduce_suffix_kernel<__nv_bfloat16>, grid, 256, 0, be->stream, (const __nv_bfloat16 *)gp, (const __nv_bfloat16 *)op,
                   (__nv_bfloat16 *)dp, repeats, cols);
    }
    return gdb_launched(be, "mul_reduce_suffix");
}

gd_status gd_backend_mse_forward(gd_backend *be, TV x, TV y, TV out, uint64_t chunk_size, float scale)
{
    return loss_forward_entry<0>(be, x, y, out, chunk_size, scale, 0.0f);
}
gd_status gd_backend_mse_backward(gd_backend *be, TV x, TV y, TV grad_out, TV grad_x, TV grad_y, float scale)
{
    return loss_backward_entry<0>(be, x, y, grad_out, grad_x, grad_y, scale, 0.0f);
}
gd_status gd_backend_huber_forward(gd_backend *be, TV x, TV y, TV out, uint64_t chunk_size, float scale, float delta)
{
    return loss_forward_entry<1>(be, x, y, out, chunk_size, scale, delta);
}
gd_status gd_backend_huber_backward(gd_backend *be, TV x, TV y, TV grad_out, TV grad_x, TV grad_y, float scale, float delta)
{
    return loss_backward_entry<1>(be, x, y, grad_out, grad_x, grad_y, scale, delta);
}

// out = x1 * gate(x2, m) (src/ops/powlu/metal_powlu.m:108-150).
gd_status gd_backend_powlu_forward(gd_backend *be, TV x1, TV x2, TV out, float m)
{
    if (be == NULL || x1 == NULL || x2 == NULL || out == NULL || x1->count == 0U || !(m == m) || x1->dtype != x2->dtype ||
        x1->dtype != out->dtype || !gdb_same_shape(x1, x2) || !gdb_same_shape(x1, out)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (!powlu_dtype(x1->dtype)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *p1 = gdb_tv_ptr(x1, x1->dtype), *p2 = gdb_tv_ptr(x2, x1->dtype);
    void *po = gdb_tv_ptr(out, x1->dtype);
    if (p1 == NULL || p2 == NULL || po == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return powlu_launch_fwd(be, x1->dtype, p1, p2, po, 1, x1->count, x1->count, m);
}

gd_status gd_backend_powlu_backward(gd_backend *be, TV x1, TV x2, TV grad_out, TV grad_x1, TV grad_x2, float m)
{
    if (be == NULL || x1 == NULL || x2 == NULL || grad_out == NULL || (grad_x1 == NULL && grad_x2 == NULL) || x1->count == 0U || !(m == m) ||
        !powlu_dtype(x1->dtype)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    for (TV v : {x2, grad_out, grad_x1, grad_x2}) {
        if (v != NULL && (v->dtype != x1->dtype || !gdb_same_shape(x1, v) || gdb_tv_ptr(v, x1->dtype) == NULL)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    const void *p1 = gdb_tv_ptr(x1, x1->dtype);
    if (p1 == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return powlu_launch_bwd(be, x1->dtype, p1, gdb_tv_ptr(x2, x1->dtype), gdb_tv_ptr(grad_out, x1->dtype),
                            grad_x1 != NULL ? gdb_tv_ptr(grad_x1, x1->dtype) : NULL, grad_x2 != NULL ? gdb_tv_ptr(grad_x2, x1->dtype) : NULL, 1,
                            x1->count, x1->count, m);
}

// x12 [..., 2H] = [x1 | x2] -> out [..., H] (src/ops/powlu/metal_powlu.metal:128-152).
gd_status gd_backend_powlu_split_forward(gd_backend *be, TV x12, TV out, float m)
{
    if (be == NULL || x12 == NULL || out == NULL || out->count == 0U || !(m == m) || x12->dtype != out->dtype || !powlu_dtype(x12->dtype) ||
        !contiguous_view(x12) || !contiguous_view(out) || !powlu_split_shape(x12, out)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned char *p = (const unsigned char *)gdb_tv_ptr(x12, x12->dtype);
    void *po = gdb_tv_ptr(out, out->dtype);
    if (p == NULL || po == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t h = (size_t)out->shape[out->rank - 1U], rows = out->count / h;
    return powlu_launch_fwd(be, x12->dtype, p, p + h * 2U, po, rows, h, 2U * h, m);
}

gd_status gd_backend_powlu_split_backward(gd_backend *be, TV x12, TV grad_out, TV grad_x12, float m)
{
    if (be == NULL || x12 == NULL || grad_out == NULL || grad_x12 == NULL || grad_out->count == 0U || !(m == m) || x12->dtype != grad_out->dtype ||
        x12->dtype != grad_x12->dtype || !powlu_dtype(x12->dtype) || !contiguous_view(x12) || !contiguous_view(grad_out) ||
        !contiguous_view(grad_x12) || !gdb_same_shape(x12, grad_x12) || !powlu_split_shape(x12, grad_out)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned char *p = (const unsigned char *)gdb_tv_ptr(x12, x12->dtype);
    const void *pg = gdb_tv_ptr(grad_out, x12->dtype);
    unsigned char *pd = (unsigned char *)gdb_tv_ptr(grad_x12, x12->dtype);
    if (p == NULL || pg == NULL || pd == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t h = (size_t)grad_out->shape[grad_out->rank - 1U], rows = grad_out->count / h;
    return powlu_launch_bwd(be, x12->dtype, p, p + h * 2U, pg, pd, pd + h * 2U, rows, h, 2U * h, m);
}

// dst = src.permute(axes) for contiguous tensors (argument rules of src/ops/permute/metal_permute.m:180-219).
gd_status gd_backend_permute(gd_backend *be, TV src, TV dst, const gd_backend_permute_args *args)
{
    if (be == NULL || src == NULL || dst == NULL || args == NULL || src->buffer == NULL || dst->buffer == NULL || src->dtype != dst->dtype ||
        src->rank != dst->rank || src->rank != args->rank || args->rank > 8U || args->active_rank > args->rank || args->count == 0U ||
        args->count > 0xffffffffULL || src->count != (size_t)args->count || dst->count != (size_t)args->count || args->inner == 0U ||
        !contiguous_view(src) || !contiguous_view(dst)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    unsigned seen = 0;
    for (uint32_t d = 0; d < args->rank; ++d) {
        if (args->axes[d] >= args->rank || (seen & (1U << args->axes[d])) != 0U) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        seen |= 1U << args->axes[d];
    }
    const size_t es = (src->dtype == GDB_DTYPE_U8) ? 1U : ((src->dtype == GDB_DTYPE_F16 || src->dtype == GDB_DTYPE_BF16) ? 2U
                      : ((src->dtype == GDB_DTYPE_F32 || src->dtype == GDB_DTYPE_I32) ? 4U : 0U));
    if (es == 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    uint64_t inner = 1;
    permute_desc pd;
    memset(&pd, 0, sizeof(pd));
    pd.rank = args->rank;
    for (uint32_t d = 0; d < args->rank; ++d) {
        if (dst->shape[d] != src->shape[args->axes[d]]) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        pd.dst_shape[d] = (uint64_t)dst->shape[d];
        pd.src_stride[d] = (uint64_t)src->strides[args->axes[d]];
    }
    for (uint32_t d = args->active_rank; d < args->rank; ++d) {
        if (args->axes[d] != d) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        inner *= (uint64_t)dst->shape[d];
    }
    if (inner != args->inner) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const void *sp = gdb_tv_ptr(src, src->dtype);
    void *dp = gdb_tv_ptr(dst, dst->dtype);
    if (sp == NULL || dp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    cudaSetDevice(be->device);
    const size_t n = (size_t)args->count;
    const unsigned grid = gdb_grid_for(n, 256, be, 8);
    if (es == 1U) {
        gdb_launch(permute_kernel<uint8_t>, grid, 256, 0, be->stream, (const uint8_t *)sp, (uint8_t *)dp, n, pd);
    } else if (es == 2U) {
        gdb_launch(permute_kernel<uint16_t>, grid, 256, 0, be->stream, (const uint16_t *)sp, (uint16_t *)dp, n, pd);
    } else {
        gdb_launch(permute_kernel<uint32_t>, grid, 256, 0, be->stream, (const uint32_t *)sp, (uint32_t *)dp, n, pd);
    }
    return gdb_launched(be, "permute");
}

}  // extern "C"
