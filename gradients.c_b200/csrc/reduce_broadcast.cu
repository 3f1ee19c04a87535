// Contiguous reductions and broadcasts used by the reference's reduce_sum / reduce_mean /
// sum_to_shape capsules (the materialised cross-entropy mean and the batch-gradient reduction
// of broadcast matmul go through them). Semantics: src/core/backend.h:241-262,359-368 and
// src/ops/_shared/reduce/metal_reduce.metal:48-480. FP32 accumulation, one rounding at the store.
#include "common.cuh"

namespace {

__device__ __forceinline__ float ld_any(const void *p, size_t i, uint32_t dt)
{
    if (dt == GDB_DTYPE_F16) return __half2float(((const __half *)p)[i]);
    if (dt == GDB_DTYPE_BF16) return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
    return ((const float *)p)[i];
}
__device__ __forceinline__ void st_any(void *p, size_t i, uint32_t dt, float v)
{
    if (dt == GDB_DTYPE_F16) ((__half *)p)[i] = __float2half_rn(v);
    else if (dt == GDB_DTYPE_BF16) ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
    else ((float *)p)[i] = v;
}

// dst[j] = scale * sum(src[j*chunk, min((j+1)*chunk, n))), chunk = ceil(n / dst_count); one block per j.
__global__ void reduce_contiguous_kernel(const void *src, void *dst, size_t n, size_t dst_count, uint32_t sdt, uint32_t ddt, float scale)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    const size_t chunk = (n + dst_count - 1) / dst_count;
    for (size_t j = blockIdx.x; j < dst_count; j += gridDim.x) {
        const size_t begin = j * chunk, end = begin + chunk < n ? begin + chunk : n;
        float acc = 0.0f;
        for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) acc += ld_any(src, i, sdt);
        acc = gdb_block_sum(acc, sh);
        if (threadIdx.x == 0) st_any(dst, j, ddt, acc * scale);
    }
}

// dst[o, i] = scale * sum_a src[o, a, i]
__global__ void reduce_axis_kernel(const void *src, void *dst, size_t outer, size_t axis, size_t inner, uint32_t dt, float scale)
{
    gdb_pdl_sync();
    const size_t n = outer * inner, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        const size_t o = e / inner, i = e - o * inner;
        float acc = 0.0f;
        for (size_t a = 0; a < axis; ++a) acc += ld_any(src, (o * axis + a) * inner + i, dt);
        st_any(dst, e, dt, acc * scale);
    }
}
// dst[o, a, i] = scale * src[o, i]
__global__ void broadcast_axis_kernel(const void *src, void *dst, size_t outer, size_t axis, size_t inner, uint32_t dt, float scale)
{
    gdb_pdl_sync();
    const size_t n = outer * axis * inner, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        const size_t i = e % inner, o = e / (axis * inner);
        st_any(dst, e, dt, ld_any(src, o * inner + i, dt) * scale);
    }
}

struct nd_desc {
    uint32_t rank;
    uint32_t big[8];     // shape of the larger tensor
    uint64_t small_stride[8];  // element stride of the smaller tensor per big dim (0 = broadcast)
};

// dst (big) [e] = scale * src (small)[mapped e]
__global__ void broadcast_to_kernel(const void *src, void *dst, size_t n, nd_desc d, uint32_t sdt, uint32_t ddt, float scale)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        size_t rem = e, so = 0;
        for (int k = (int)d.rank - 1; k >= 0; --k) {
            so += (rem % d.big[k]) * d.small_stride[k];
            rem /= d.big[k];
        }
        st_any(dst, e, ddt, ld_any(src, so, sdt) * scale);
    }
}

// dst (small) [j] = scale * sum over the src (big) elements that broadcast to j. One warp per j.
__global__ void reduce_broadcast_kernel(const void *src, void *dst, size_t small_n, size_t big_n, nd_desc d,
                                        uint32_t small_shape_packed_rank, const uint32_t *unused, uint32_t dt, float scale)
{
    gdb_pdl_sync();
    (void)small_shape_packed_rank;
    (void)unused;
    const int lane = threadIdx.x & 31;
    const size_t w = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= small_n) {
        return;
    }
    // offset in the big tensor of the kept coordinates of w, then walk the reduced dims only
    size_t rem = w, base = 0, big_stride = 1, reduced_n = 1;
    size_t bstride[8];
    for (int k = (int)d.rank - 1; k >= 0; --k) {
        bstride[k] = big_stride;
        big_stride *= d.big[k];
        if (d.small_stride[k] != 0) {
            base += (rem % d.big[k]) * bstride[k];
            rem /= d.big[k];
        } else {
            reduced_n *= d.big[k];
        }
    }
    (void)big_n;
    float acc = 0.0f;
    for (size_t r = lane; r < reduced_n; r += 32) {
        size_t rr = r, off = base;
        for (int k = (int)d.rank - 1; k >= 0; --k) {
            if (d.small_stride[k] == 0) {
                off += (rr % d.big[k]) * bstride[k];
                rr /= d.big[k];
            }
        }
        acc += ld_any(src, off, dt);
    }
    acc = gdb_warp_sum(acc);
    if (lane == 0) st_any(dst, w, dt, acc * scale);
}

bool view_ok(const gd_backend_tensor_view *v)
{
    return v != NULL && v->rank <= 8U && gdb_is_float_dtype(v->dtype) && gdb_tv_ptr(v, v->dtype) != NULL;
}

// Right-aligned broadcast map from `small` onto `big`; false when shapes are incompatible.
bool make_desc(const gd_backend_tensor_view *small, const gd_backend_tensor_view *big, nd_desc *d)
{
    if (small->rank > big->rank) {
        return false;
    }
    memset(d, 0, sizeof(*d));
    d->rank = big->rank;
    const uint32_t prefix = big->rank - small->rank;
    uint64_t stride = 1;
    for (int k = (int)big->rank - 1; k >= 0; --k) {
        d->big[k] = (uint32_t)big->shape[k];
        if ((uint32_t)k < prefix) {
            d->small_stride[k] = 0;
            continue;
        }
        const int64_t sd = small->shape[k - prefix];
        if (sd == big->shape[k]) {
            d->small_stride[k] = sd == 1 ? 0 : stride;
        } else if (sd == 1) {
            d->small_stride[k] = 0;
        } else {
            return false;
        }
        stride *= (uint64_t)sd;
    }
    return true;
}

}  // namespace

extern "C" {

gd_status gd_backend_reduce_contiguous(gd_backend *be, const gd_backend_tensor_view *src, const gd_backend_tensor_view *dst, float scale)
{
    if (be == NULL || !view_ok(src) || !view_ok(dst) || dst->count == 0U || src->count < dst->count) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const unsigned grid = (unsigned)(dst->count < 65535U * 4U ? dst->count : 65535U * 4U);
    gdb_launch(reduce_contiguous_kernel, grid, 256, 0, be->stream, gdb_tv_ptr(src, src->dtype), gdb_tv_ptr(dst, dst->dtype), src->count, dst->count, src->dtype, dst->dtype, scale);
    return gdb_launched(be, "reduce_contiguous");
}

static gd_status axis_common(gd_backend *be, const gd_backend_tensor_view *full, const gd_backend_tensor_view *reduced, uint32_t axis, float scale, bool reduce)
{
    if (be == NULL || !view_ok(full) || !view_ok(reduced) || full->dtype != reduced->dtype || axis >= full->rank) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    size_t outer = 1, inner = 1;
    for (uint32_t k = 0; k < axis; ++k) outer *= (size_t)full->shape[k];
    for (uint32_t k = axis + 1; k < full->rank; ++k) inner *= (size_t)full->shape[k];
    const size_t a = (size_t)full->shape[axis];
    if (a == 0U || full->count != outer * a * inner || reduced->count != outer * inner) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (full->count == 0U) {
        return GD_OK;
    }
    void *fp = gdb_tv_ptr(full, full->dtype), *rp = gdb_tv_ptr(reduced, reduced->dtype);
    if (reduce) {
        gdb_launch(reduce_axis_kernel, gdb_grid_for(outer * inner, 256, be, 8), 256, 0, be->stream, fp, rp, outer, a, inner, full->dtype, scale);
    } else {
        gdb_launch(broadcast_axis_kernel, gdb_grid_for(full->count, 256, be, 8), 256, 0, be->stream, rp, fp, outer, a, inner, full->dtype, scale);
    }
    return gdb_launched(be, reduce ? "reduce_axis" : "broadcast_axis");
}

gd_status gd_backend_reduce_axis(gd_backend *be, const gd_backend_tensor_view *src, const gd_backend_tensor_view *dst, uint32_t axis, float scale)
{
    return axis_common(be, src, dst, axis, scale, true);
}
gd_status gd_backend_broadcast_axis(gd_backend *be, const gd_backend_tensor_view *src, const gd_backend_tensor_view *dst, uint32_t axis, float scale)
{
    return axis_common(be, dst, src, axis, scale, false);
}

gd_status gd_backend_broadcast_to(gd_backend *be, const gd_backend_tensor_view *src, const gd_backend_tensor_view *dst, float scale)
{
    nd_desc d;
    if (be == NULL || !view_ok(src) || !view_ok(dst) || src->dtype != dst->dtype || !make_desc(src, dst, &d)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (dst->count == 0U) {
        return GD_OK;
    }
    gdb_launch(broadcast_to_kernel, gdb_grid_for(dst->count, 256, be, 8), 256, 0, be->stream, gdb_tv_ptr(src, src->dtype), gdb_tv_ptr(dst, dst->dtype), dst->count, d, src->dtype, dst->dtype, scale);
    return gdb_launched(be, "broadcast_to");
}

// dst[i] = src[0] * scale; same dtype, or an F32 scalar into a 16-bit destination.
gd_status gd_backend_broadcast_scalar(gd_backend *be, const gd_backend_tensor_view *src, const gd_backend_tensor_view *dst, float scale)
{
    nd_desc d;
    if (be == NULL || !view_ok(src) || !view_ok(dst) || src->count < 1U ||
        !(src->dtype == dst->dtype || src->dtype == GDB_DTYPE_F32)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (dst->count == 0U) {
        return GD_OK;
    }
    memset(&d, 0, sizeof(d));
    d.rank = 1;
    d.big[0] = (uint32_t)dst->count;
    d.small_stride[0] = 0;
    gdb_launch(broadcast_to_kernel, gdb_grid_for(dst->count, 256, be, 8), 256, 0, be->stream, gdb_tv_ptr(src, src->dtype), gdb_tv_ptr(dst, dst->dtype), dst->count, d, src->dtype, dst->dtype, scale);
    return gdb_launched(be, "broadcast_scalar");
}

gd_status gd_backend_reduce_broadcast(gd_backend *be, const gd_backend_tensor_view *src, const gd_backend_tensor_view *dst, float scale)
{
    nd_desc d;
    if (be == NULL || !view_ok(src) || !view_ok(dst) || src->dtype != dst->dtype || !make_desc(dst, src, &d)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (dst->count == 0U) {
        return GD_OK;
    }
    const size_t warps = dst->count;
    gdb_launch(reduce_broadcast_kernel, (unsigned)((warps + 3) / 4), 128, 0, be->stream, gdb_tv_ptr(src, src->dtype), gdb_tv_ptr(dst, dst->dtype), dst->count, src->count, d, 0U, (const uint32_t *)nullptr, src->dtype, scale);
    return gdb_launched(be, "reduce_broadcast");
}

}  // extern "C"
