// Slice copies used by concat / split (multi-prompt prefill gathers last rows through
// gd_backend_concat_to_full). Slice semantics: src/core/backend.h:579-615.
#include "common.cuh"

namespace {

// TO_FULL: full[o, off + a, r] = slice[o, a, r]; else slice[...] = full[...].
template <typename U, bool TO_FULL>
__global__ void slice_copy_kernel(const U *src, U *dst, size_t count, size_t slice_span, size_t full_span, size_t lead)
{
    gdb_pdl_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const size_t o = i / slice_span, r = i - o * slice_span;
        const size_t f = o * full_span + lead + r;
        if (TO_FULL) {
            dst[f] = src[i];
        } else {
            dst[i] = src[f];
        }
    }
}

template <bool TO_FULL>
gd_status slice_copy(gd_backend *be, const gd_backend_tensor_view *slice, const gd_backend_tensor_view *full,
                     uint64_t count, uint64_t inner, uint64_t slice_axis, uint64_t full_axis, uint64_t axis_offset)
{
    if (be == NULL || slice == NULL || full == NULL || slice->dtype != full->dtype || inner == 0U || slice_axis == 0U ||
        full_axis == 0U || axis_offset > full_axis || slice_axis > full_axis - axis_offset || slice->count != count ||
        (count % (slice_axis * inner)) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t es = gdb_dtype_size(slice->dtype);
    if (es == 0U) {
        return GD_ERR_UNSUPPORTED;
    }
    const size_t outer = count / (slice_axis * inner);
    if (full->count != outer * full_axis * inner) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    void *sp = gdb_tv_ptr(slice, slice->dtype), *fp = gdb_tv_ptr(full, full->dtype);
    if (sp == NULL || fp == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    const size_t ss = slice_axis * inner, fs = full_axis * inner, lead = axis_offset * inner;
    const unsigned grid = gdb_grid_for(count, 256, be, 8);
    const void *src = TO_FULL ? sp : fp;
    void *dst = TO_FULL ? fp : sp;
    if (es == 1U) {
        gdb_launch(slice_copy_kernel<unsigned char, TO_FULL>, grid, 256, 0, be->stream, (const unsigned char *)src, (unsigned char *)dst, count, ss, fs, lead);
    } else if (es == 2U) {
        gdb_launch(slice_copy_kernel<unsigned short, TO_FULL>, grid, 256, 0, be->stream, (const unsigned short *)src, (unsigned short *)dst, count, ss, fs, lead);
    } else {
        gdb_launch(slice_copy_kernel<unsigned, TO_FULL>, grid, 256, 0, be->stream, (const unsigned *)src, (unsigned *)dst, count, ss, fs, lead);
    }
    return gdb_launched(be, "slice_copy");
}

}  // namespace

#define TV const gd_backend_tensor_view *

extern "C" {

gd_status gd_backend_concat_to_full(gd_backend *be, TV src, TV dst, const gd_backend_concat_args *a)
{
    return a == NULL ? GD_ERR_INVALID_ARGUMENT : slice_copy<true>(be, src, dst, a->count, a->inner, a->slice_axis, a->full_axis, a->axis_offset);
}
gd_status gd_backend_concat_from_full(gd_backend *be, TV src, TV dst, const gd_backend_concat_args *a)
{
    return a == NULL ? GD_ERR_INVALID_ARGUMENT : slice_copy<false>(be, dst, src, a->count, a->inner, a->slice_axis, a->full_axis, a->axis_offset);
}
gd_status gd_backend_split_from_full(gd_backend *be, TV full, TV slice, const gd_backend_split_args *a)
{
    return a == NULL ? GD_ERR_INVALID_ARGUMENT : slice_copy<false>(be, slice, full, a->count, a->inner, a->slice_axis, a->full_axis, a->axis_offset);
}
gd_status gd_backend_split_to_full(gd_backend *be, TV slice, TV full, const gd_backend_split_args *a)
{
    return a == NULL ? GD_ERR_INVALID_ARGUMENT : slice_copy<true>(be, slice, full, a->count, a->inner, a->slice_axis, a->full_axis, a->axis_offset);
}


}  // extern "C"
