// AMP loss-scale state machine, global-norm gradient clipping and the AdamW update.
//
// Reference arithmetic: src/backends/metal/primitives/amp/metal_amp.metal:59-166,
// src/optim/adamw/metal_adamw.metal:35-270 and metal_adamw.m:146-190 (host-side constants).
// The reference issues three launches per parameter tensor; here the descriptor array is
// copied into kernel parameters and ONE launch covers up to 64 tensors (prepare / update /
// commit stay separate launches because update reads state that commit rewrites).
#include "common.cuh"

#include <math.h>

namespace {

constexpr int MT_MAX = 64;          // tensors per multi-tensor launch
constexpr unsigned NORM_BLOCK = 1024;  // elements per gradient-norm partial (reference: 1024)
constexpr unsigned NORM_GROUP = 8;     // partial slots handled by one block of the norm kernel

__device__ __forceinline__ float load_as_float(const void *p, size_t i, uint32_t dtype)
{
    if (dtype == GDB_DTYPE_F16) {
        return __half2float(((const __half *)p)[i]);
    }
    if (dtype == GDB_DTYPE_BF16) {
        return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
    }
    return ((const float *)p)[i];
}
__device__ __forceinline__ void store_from_float(void *p, size_t i, uint32_t dtype, float v)
{
    if (dtype == GDB_DTYPE_F16) {
        ((__half *)p)[i] = __float2half_rn(v);
    } else if (dtype == GDB_DTYPE_BF16) {
        ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
    } else {
        ((float *)p)[i] = v;
    }
}

// ------------------------------------------------------------------ AMP
__global__ void amp_begin_kernel(float *scale, int *flags, float min_scale, float max_scale)
{
    gdb_pdl_sync();
    const float s = fminf(fmaxf(scale[0], min_scale), max_scale);
    scale[0] = s;
    scale[1] = 1.0f / s;
    flags[1] = 0;
}
__global__ void amp_finish_kernel(float *scale, unsigned *flags, float growth, float backoff, float min_scale,
                                  float max_scale, unsigned interval)
{
    gdb_pdl_sync();
    const bool found = flags[1] != 0U;
    float s = scale[0];
    unsigned tracker = flags[0];
    flags[2] = found ? 1U : 0U;
    if (found) {
        s = fmaxf(s * backoff, min_scale);
        tracker = 0U;
    } else {
        tracker += 1U;
        if (tracker >= interval) {
            s = fminf(s * growth, max_scale);
            tracker = 0U;
        }
    }
    scale[0] = s;
    scale[1] = 1.0f / s;
    flags[0] = tracker;
}
// dst[i] = (src ? src[i] : 1) * scale[0]
__global__ void amp_scale_kernel(void *dst, const void *src, size_t n, uint32_t dtype, const float *scale)
{
    gdb_pdl_sync();
    const float s = scale[0];
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        store_from_float(dst, i, dtype, src != nullptr ? load_as_float(src, i, dtype) * s : s);
    }
}

struct unscale_batch {
    void *grad[MT_MAX];
    size_t count[MT_MAX];
    uint32_t dtype[MT_MAX];
    const float *inv_scale[MT_MAX];
    int *found_inf[MT_MAX];
    unsigned block_start[MT_MAX + 1];
    int n;
};
__global__ void amp_unscale_kernel(unscale_batch b)
{
    gdb_pdl_sync();
    int t = 0;
    while (t + 1 < b.n && blockIdx.x >= b.block_start[t + 1]) {
        ++t;
    }
    const size_t base = (size_t)(blockIdx.x - b.block_start[t]) * NORM_BLOCK;
    const float inv = b.inv_scale[t][0];
    bool bad = false;
    for (unsigned j = threadIdx.x; j < NORM_BLOCK; j += blockDim.x) {
        const size_t i = base + j;
        if (i < b.count[t]) {
            const float g = load_as_float(b.grad[t], i, b.dtype[t]) * inv;
            bad = bad || !isfinite(g);
            store_from_float(b.grad[t], i, b.dtype[t], g);
        }
    }
    if (bad) {
        *b.found_inf[t] = 1;
    }
}

// ------------------------------------------------------------------ gradient norm / clip
struct norm_batch {
    const void *grad[MT_MAX];
    size_t count[MT_MAX];
    uint32_t dtype[MT_MAX];
    float *partial[MT_MAX];
    unsigned block_start[MT_MAX + 1];
    const float *grad_scale;
    int *found_inf;  // nullable
    int n;
};
__global__ void grad_norm_stage_kernel(norm_batch b)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    int t = 0;
    while (t + 1 < b.n && blockIdx.x >= b.block_start[t + 1]) {
        ++t;
    }
    // one block covers NORM_GROUP partial slots (8192 elements) and writes the first of them; the
    // other slots of the group stay zero (the host clears the partial range before this launch)
    const unsigned local = blockIdx.x - b.block_start[t];
    const size_t base = (size_t)local * NORM_BLOCK * NORM_GROUP;
    const float gs = b.grad_scale[0];
    float sum = 0.0f;
    bool bad = false;
    const uint32_t dt = b.dtype[t];
    const unsigned char *gp = (const unsigned char *)b.grad[t];
    if ((dt == GDB_DTYPE_F16 || dt == GDB_DTYPE_BF16) && ((uintptr_t)(gp + base * 2U) % 16U) == 0U &&
        base + (size_t)NORM_BLOCK * NORM_GROUP <= b.count[t]) {
        // full group of 16-bit gradients: 16-byte loads, 8 elements each
        const uint4 *v = reinterpret_cast<const uint4 *>(gp + base * 2U);
        for (unsigned j = threadIdx.x; j < NORM_BLOCK * NORM_GROUP / 8U; j += blockDim.x) {
            const uint4 raw = __ldg(&v[j]);
            const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float g0, g1;
                if (dt == GDB_DTYPE_F16) {
                    g0 = gdb_io<__half>::up((unsigned short)(w[e] & 0xffffU));
                    g1 = gdb_io<__half>::up((unsigned short)(w[e] >> 16));
                } else {
                    g0 = gdb_io<__nv_bfloat16>::up((unsigned short)(w[e] & 0xffffU));
                    g1 = gdb_io<__nv_bfloat16>::up((unsigned short)(w[e] >> 16));
                }
                g0 *= gs;
                g1 *= gs;
                bad = bad || !isfinite(g0) || !isfinite(g1);
                sum = fmaf(g0, g0, sum);
                sum = fmaf(g1, g1, sum);
            }
        }
    } else {
        for (unsigned j = threadIdx.x; j < NORM_BLOCK * NORM_GROUP; j += blockDim.x) {
            const size_t i = base + j;
            if (i < b.count[t]) {
                const float g = load_as_float(b.grad[t], i, dt) * gs;
                bad = bad || !isfinite(g);
                sum = fmaf(g, g, sum);
            }
        }
    }
    if (bad && b.found_inf != nullptr) {
        *b.found_inf = 1;
    }
    sum = gdb_block_sum(sum, sh);
    if (threadIdx.x == 0) {
        b.partial[t][(size_t)local * NORM_GROUP] = sum;
    }
}
__global__ void grad_clip_finalize_kernel(const float *partials, size_t n, float *out, const float *grad_scale,
                                          float max_norm, float eps)
{
    gdb_pdl_sync();
    __shared__ float sh[33];
    float sum = 0.0f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        sum += partials[i];
    }
    sum = gdb_block_sum(sum, sh);
    if (threadIdx.x == 0) {
        const float total = sqrtf(sum);
        float scale = max_norm / (total + eps);
        if (!isfinite(total)) {
            scale = 0.0f;
        } else if (!(scale < 1.0f)) {
            scale = 1.0f;
        }
        out[0] = scale * grad_scale[0];
        out[1] = total;
    }
}

// ------------------------------------------------------------------ AdamW
struct adamw_item {
    void *param;
    float *master;          // nullable
    const void *grad;
    const float *grad_scale;  // nullable
    const int *found_inf;     // nullable
    float *m, *v;
    float *beta1_power, *beta2_power, *step_scale, *decay_scale, *eps_scaled;  // device state, nullable
    unsigned *param_step, *optimizer_step;
    size_t count;
    uint32_t param_dtype, grad_dtype;
    uint32_t bias_correction, update_optimizer_step;
    float lr, beta1, beta2, eps, weight_decay;
    float host_step_scale, host_decay_scale, host_eps_scaled;
};
// One launch takes up to ADAMW_BATCH tensors (the struct travels as a kernel parameter: 8.3 KB of the 32 KB sm_100 allows), which
// covers every parameter of a gpt_lm of up to four blocks in one update launch.
constexpr int ADAMW_BATCH = 48;
struct adamw_batch {
    adamw_item it[ADAMW_BATCH];
    unsigned block_start[ADAMW_BATCH + 1];
    int n;
};
// The per-tensor step scalars (metal_adamw.metal:59-88, src/optim/adamw.c:1570-1640): bias corrections from the running beta
// powers, which adamw_commit_kernel advances after the update.
struct adamw_scalars {
    float step_scale, decay_scale, eps_scaled;
};
__device__ __forceinline__ adamw_scalars adamw_step_scalars(const adamw_item &a)
{
    const float b1p = __fmul_rn(a.beta1_power[0], a.beta1);
    const float b2p = __fmul_rn(a.beta2_power[0], a.beta2);
    const float bc1 = a.bias_correction ? __fsub_rn(1.0f, b1p) : 1.0f;
    const float bc2 = a.bias_correction ? __fsub_rn(1.0f, b2p) : 1.0f;
    const float bc2s = sqrtf(bc2);
    adamw_scalars r;
    r.step_scale = __fdiv_rn(__fmul_rn(a.lr, bc2s), bc1);
    r.decay_scale = __fmul_rn(a.lr, a.weight_decay);
    r.eps_scaled = __fmul_rn(a.eps, bc2s);
    return r;
}

// What adamw_commit_kernel needs of a tensor: 2.7 KB for a full batch, where the whole adamw_batch is 8.3 KB (kernel parameters
// above 4 KB take a slower path into the launch).
struct adamw_commit_item {
    float *beta1_power, *beta2_power;
    unsigned *param_step, *optimizer_step;
    const int *found_inf;
    float beta1, beta2;
    uint32_t update_optimizer_step;
};
struct adamw_commit_batch {
    adamw_commit_item it[ADAMW_BATCH];
    int n;
};
__global__ void adamw_commit_kernel(adamw_commit_batch b)
{
    gdb_pdl_sync();
    const int t = threadIdx.x;
    if (t >= b.n) {
        return;
    }
    const adamw_commit_item &a = b.it[t];
    if (a.beta1_power == nullptr || (a.found_inf != nullptr && *a.found_inf != 0)) {
        return;
    }
    a.beta1_power[0] = __fmul_rn(a.beta1_power[0], a.beta1);
    a.beta2_power[0] = __fmul_rn(a.beta2_power[0], a.beta2);
    a.param_step[0] += 1U;
    if (a.update_optimizer_step) {
        a.optimizer_step[0] += 1U;
    }
}

constexpr unsigned ADAMW_BLOCK_ELEMS = 2048;  // elements per block (256 threads x 8)

__global__ void adamw_update_kernel(adamw_batch b)
{
    gdb_pdl_sync();
    int t = 0;
    while (t + 1 < b.n && blockIdx.x >= b.block_start[t + 1]) {
        ++t;
    }
    const adamw_item &a = b.it[t];
    if (a.found_inf != nullptr && *a.found_inf != 0) {
        return;  // overflow: the whole update is skipped (metal_adamw.metal:117)
    }
    const float gs = a.grad_scale != nullptr ? a.grad_scale[0] : 1.0f;
    float step_scale = a.host_step_scale, decay_scale = a.host_decay_scale, eps_scaled = a.host_eps_scaled;
    if (a.beta1_power != nullptr) {
        // device-side state: every block forms the tensor's step scalars itself (a dozen operations; the beta powers do not
        // change before adamw_commit_kernel), and the tensor's first block leaves them in the state where the reference keeps them
        const adamw_scalars sc = adamw_step_scalars(a);
        step_scale = sc.step_scale;
        decay_scale = sc.decay_scale;
        eps_scaled = sc.eps_scaled;
        if (blockIdx.x == b.block_start[t] && threadIdx.x == 0) {
            a.step_scale[0] = sc.step_scale;
            a.decay_scale[0] = sc.decay_scale;
            a.eps_scaled[0] = sc.eps_scaled;
        }
    } else if (a.step_scale != nullptr) {
        step_scale = a.step_scale[0];
        decay_scale = a.decay_scale[0];
        eps_scaled = a.eps_scaled[0];
    }
    const float omb1 = __fsub_rn(1.0f, a.beta1), omb2 = __fsub_rn(1.0f, a.beta2);
    const size_t base = (size_t)(blockIdx.x - b.block_start[t]) * ADAMW_BLOCK_ELEMS;
    // Full block of 16-bit parameters / gradients with FP32 masters: every thread owns 8 consecutive elements and moves
    // them with 16-byte accesses; the arithmetic per element is the one of the scalar loop below, operation for operation.
    if (a.master != nullptr && a.param_dtype == a.grad_dtype && (a.param_dtype == GDB_DTYPE_F16 || a.param_dtype == GDB_DTYPE_BF16) &&
        base + ADAMW_BLOCK_ELEMS <= a.count &&
        (((uintptr_t)((const unsigned char *)a.grad + base * 2U) | (uintptr_t)((unsigned char *)a.param + base * 2U) |
          (uintptr_t)(a.master + base) | (uintptr_t)(a.m + base) | (uintptr_t)(a.v + base)) % 16U) == 0U) {
        const size_t i0 = base + (size_t)threadIdx.x * 8U;
        const bool f16 = a.param_dtype == GDB_DTYPE_F16;
        const uint4 graw = __ldg(reinterpret_cast<const uint4 *>((const unsigned char *)a.grad + i0 * 2U));
        const unsigned gw[4] = {graw.x, graw.y, graw.z, graw.w};
        float pm[8], mm[8], vv8[8];
        *reinterpret_cast<float4 *>(pm) = *reinterpret_cast<const float4 *>(a.master + i0);
        *reinterpret_cast<float4 *>(pm + 4) = *reinterpret_cast<const float4 *>(a.master + i0 + 4);
        *reinterpret_cast<float4 *>(mm) = *reinterpret_cast<const float4 *>(a.m + i0);
        *reinterpret_cast<float4 *>(mm + 4) = *reinterpret_cast<const float4 *>(a.m + i0 + 4);
        *reinterpret_cast<float4 *>(vv8) = *reinterpret_cast<const float4 *>(a.v + i0);
        *reinterpret_cast<float4 *>(vv8 + 4) = *reinterpret_cast<const float4 *>(a.v + i0 + 4);
        unsigned pw[4];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const unsigned short bits = (unsigned short)((e & 1) ? (gw[e >> 1] >> 16) : (gw[e >> 1] & 0xffffU));
            float g = f16 ? gdb_io<__half>::up(bits) : gdb_io<__nv_bfloat16>::up(bits);
            g = gs == 0.0f ? 0.0f : __fmul_rn(g, gs);
            const float p = pm[e];
            const float m_new = fmaf(a.beta1, mm[e], __fmul_rn(omb1, g));
            const float v_new = fmaf(a.beta2, vv8[e], __fmul_rn(__fmul_rn(omb2, g), g));
            const float denom = __fadd_rn(sqrtf(v_new), eps_scaled);
            const float p_new = __fsub_rn(__fsub_rn(p, __fdiv_rn(__fmul_rn(step_scale, m_new), denom)), __fmul_rn(decay_scale, p));
            mm[e] = m_new;
            vv8[e] = v_new;
            pm[e] = p_new;
            const unsigned pb = f16 ? gdb_io<__half>::down(p_new) : gdb_io<__nv_bfloat16>::down(p_new);
            if (e & 1) pw[e >> 1] |= pb << 16; else pw[e >> 1] = pb;
        }
        *reinterpret_cast<float4 *>(a.master + i0) = *reinterpret_cast<const float4 *>(pm);
        *reinterpret_cast<float4 *>(a.master + i0 + 4) = *reinterpret_cast<const float4 *>(pm + 4);
        *reinterpret_cast<float4 *>(a.m + i0) = *reinterpret_cast<const float4 *>(mm);
        *reinterpret_cast<float4 *>(a.m + i0 + 4) = *reinterpret_cast<const float4 *>(mm + 4);
        *reinterpret_cast<float4 *>(a.v + i0) = *reinterpret_cast<const float4 *>(vv8);
        *reinterpret_cast<float4 *>(a.v + i0 + 4) = *reinterpret_cast<const float4 *>(vv8 + 4);
        *reinterpret_cast<uint4 *>((unsigned char *)a.param + i0 * 2U) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        return;
    }
#pragma unroll 4
    for (unsigned j = threadIdx.x; j < ADAMW_BLOCK_ELEMS; j += 256) {
        const size_t i = base + j;
        if (i >= a.count) {
            break;
        }
        float g = load_as_float(a.grad, i, a.grad_dtype);
        g = gs == 0.0f ? 0.0f : __fmul_rn(g, gs);
        const float p = a.master != nullptr ? a.master[i] : load_as_float(a.param, i, a.param_dtype);
        const float m_new = fmaf(a.beta1, a.m[i], __fmul_rn(omb1, g));
        const float v_new = fmaf(a.beta2, a.v[i], __fmul_rn(__fmul_rn(omb2, g), g));
        const float denom = __fadd_rn(sqrtf(v_new), eps_scaled);
        const float p_new = __fsub_rn(__fsub_rn(p, __fdiv_rn(__fmul_rn(step_scale, m_new), denom)), __fmul_rn(decay_scale, p));
        a.m[i] = m_new;
        a.v[i] = v_new;
        if (a.master != nullptr) {
            a.master[i] = p_new;
        }
        store_from_float(a.param, i, a.param_dtype, p_new);
    }
}

bool rng(gd_backend_buffer *b, size_t off, size_t n) { return gdb_range_ok(b, off, n); }

gd_status fill_adamw_item(const gd_backend_adamw_desc *d, adamw_item *it)
{
    const size_t pes = gdb_dtype_size(d->param_dtype), ges = gdb_dtype_size(d->grad_dtype);
    if (d->count == 0U || !gdb_is_float_dtype(d->param_dtype) || !gdb_is_float_dtype(d->grad_dtype) ||
        !rng(d->param_buffer, d->param_offset, d->count * pes) || !rng(d->grad_buffer, d->grad_offset, d->count * ges) ||
        !rng(d->m_buffer, d->m_offset, d->count * 4U) || !rng(d->v_buffer, d->v_offset, d->count * 4U) ||
        (d->has_master && !rng(d->master_buffer, d->master_offset, d->count * 4U)) ||
        (d->has_grad_scale && !rng(d->grad_scale_buffer, d->grad_scale_offset, 4U)) ||
        (d->has_found_inf && !rng(d->found_inf_buffer, d->found_inf_offset, 4U))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (d->has_device_state &&
        (!rng(d->state_f32_buffer, d->beta1_power_offset, 4U) || !rng(d->state_f32_buffer, d->beta2_power_offset, 4U) ||
         !rng(d->state_f32_buffer, d->step_scale_offset, 4U) || !rng(d->state_f32_buffer, d->decay_scale_offset, 4U) ||
         !rng(d->state_f32_buffer, d->eps_scaled_offset, 4U) || !rng(d->state_i32_buffer, d->param_step_offset, 4U) ||
         !rng(d->state_i32_buffer, d->optimizer_step_offset, 4U))) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (d->has_master == 0U && d->param_dtype != GDB_DTYPE_F32 && d->param_dtype != GDB_DTYPE_F16 && d->param_dtype != GDB_DTYPE_BF16) {
        return GD_ERR_UNSUPPORTED;
    }
    memset(it, 0, sizeof(*it));
    it->param = d->param_buffer->dptr + d->param_offset;
    it->master = d->has_master ? (float *)(d->master_buffer->dptr + d->master_offset) : NULL;
    it->grad = d->grad_buffer->dptr + d->grad_offset;
    it->grad_scale = d->has_grad_scale ? (const float *)(d->grad_scale_buffer->dptr + d->grad_scale_offset) : NULL;
    it->found_inf = d->has_found_inf ? (const int *)(d->found_inf_buffer->dptr + d->found_inf_offset) : NULL;
    it->m = (float *)(d->m_buffer->dptr + d->m_offset);
    it->v = (float *)(d->v_buffer->dptr + d->v_offset);
    if (d->has_device_state) {
        unsigned char *f = d->state_f32_buffer->dptr, *i32 = d->state_i32_buffer->dptr;
        it->beta1_power = (float *)(f + d->beta1_power_offset);
        it->beta2_power = (float *)(f + d->beta2_power_offset);
        it->step_scale = (float *)(f + d->step_scale_offset);
        it->decay_scale = (float *)(f + d->decay_scale_offset);
        it->eps_scaled = (float *)(f + d->eps_scaled_offset);
        it->param_step = (unsigned *)(i32 + d->param_step_offset);
        it->optimizer_step = (unsigned *)(i32 + d->optimizer_step_offset);
    }
    it->count = d->count;
    it->param_dtype = d->param_dtype;
    it->grad_dtype = d->grad_dtype;
    it->bias_correction = d->bias_correction != 0U;
    it->update_optimizer_step = d->update_optimizer_step != 0U;
    it->lr = d->lr;
    it->beta1 = d->beta1;
    it->beta2 = d->beta2;
    it->eps = d->eps;
    it->weight_decay = d->weight_decay;
    const float bc2s = d->has_device_state ? 1.0f : sqrtf(d->bias_correction2);
    const float bc1 = d->has_device_state ? 1.0f : d->bias_correction1;
    it->host_step_scale = d->lr * bc2s / bc1;
    it->host_decay_scale = d->lr * d->weight_decay;
    it->host_eps_scaled = d->eps * bc2s;
    return GD_OK;
}

bool amp_desc_ok(const gd_backend_amp_state_desc *d)
{
    return d != NULL && rng(d->scale_buffer, d->scale_offset, 8U) && rng(d->flags_buffer, d->flags_offset, 12U) &&
           (d->scale_offset % 4U) == 0U && (d->flags_offset % 4U) == 0U;
}

}  // namespace

extern "C" {

gd_status gd_backend_amp_begin_step(gd_backend *be, const gd_backend_amp_state_desc *d)
{
    if (be == NULL || !amp_desc_ok(d)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gdb_launch(amp_begin_kernel, 1, 1, 0, be->stream, (float *)(d->scale_buffer->dptr + d->scale_offset),
                                              (int *)(d->flags_buffer->dptr + d->flags_offset), d->min_scale, d->max_scale);
    return gdb_launched(be, "amp_begin_step");
}

gd_status gd_backend_amp_finish_step(gd_backend *be, const gd_backend_amp_state_desc *d)
{
    if (be == NULL || !amp_desc_ok(d)) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    gdb_launch(amp_finish_kernel, 1, 1, 0, be->stream, (float *)(d->scale_buffer->dptr + d->scale_offset),
                                               (unsigned *)(d->flags_buffer->dptr + d->flags_offset), d->growth_factor,
                                               d->backoff_factor, d->min_scale, d->max_scale, d->growth_interval);
    return gdb_launched(be, "amp_finish_step");
}

gd_status gd_backend_amp_fill_scale(gd_backend *be, gd_backend_buffer *dst_buffer, size_t dst_offset, size_t count, uint32_t dtype, gd_backend_buffer *scale_buffer, size_t scale_offset)
{
    const size_t es = gdb_dtype_size(dtype);
    if (be == NULL || !gdb_is_float_dtype(dtype) || !rng(dst_buffer, dst_offset, count * es) || (dst_offset % es) != 0U ||
        !rng(scale_buffer, scale_offset, 4U) || (scale_offset % 4U) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    gdb_launch(amp_scale_kernel, gdb_grid_for(count, 256, be, 8), 256, 0, be->stream, dst_buffer->dptr + dst_offset, (const void *)nullptr, count, dtype, (const float *)(scale_buffer->dptr + scale_offset));
    return gdb_launched(be, "amp_fill_scale");
}

gd_status gd_backend_amp_scale(gd_backend *be, gd_backend_buffer *dst_buffer, size_t dst_offset, gd_backend_buffer *src_buffer, size_t src_offset, size_t count, uint32_t dtype, gd_backend_buffer *scale_buffer, size_t scale_offset)
{
    const size_t es = gdb_dtype_size(dtype);
    if (be == NULL || !gdb_is_float_dtype(dtype) || !rng(dst_buffer, dst_offset, count * es) || (dst_offset % es) != 0U ||
        !rng(src_buffer, src_offset, count * es) || (src_offset % es) != 0U || !rng(scale_buffer, scale_offset, 4U) ||
        (scale_offset % 4U) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (count == 0U) {
        return GD_OK;
    }
    gdb_launch(amp_scale_kernel, gdb_grid_for(count, 256, be, 8), 256, 0, be->stream, dst_buffer->dptr + dst_offset, src_buffer->dptr + src_offset, count, dtype, (const float *)(scale_buffer->dptr + scale_offset));
    return gdb_launched(be, "amp_scale");
}

gd_status gd_backend_amp_unscale_batch(gd_backend *be, const gd_backend_amp_unscale_desc *descs, uint32_t desc_count)
{
    if (desc_count == 0U) {
        return GD_OK;
    }
    if (be == NULL || descs == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    for (uint32_t i = 0; i < desc_count; ++i) {
        const gd_backend_amp_unscale_desc *d = &descs[i];
        const size_t es = gdb_dtype_size(d->grad_dtype);
        if (!gdb_is_float_dtype(d->grad_dtype) || !rng(d->grad_buffer, d->grad_offset, d->count * es) ||
            !rng(d->inv_scale_buffer, d->inv_scale_offset, 4U) || !rng(d->found_inf_buffer, d->found_inf_offset, 4U)) {
            return GD_ERR_INVALID_ARGUMENT;
        }
    }
    for (uint32_t start = 0; start < desc_count; start += MT_MAX) {
        unscale_batch b;
        memset(&b, 0, sizeof(b));
        unsigned blocks = 0;
        for (uint32_t i = start; i < desc_count && b.n < MT_MAX; ++i) {
            const gd_backend_amp_unscale_desc *d = &descs[i];
            if (d->count == 0U) {
                continue;
            }
            b.grad[b.n] = d->grad_buffer->dptr + d->grad_offset;
            b.count[b.n] = d->count;
            b.dtype[b.n] = d->grad_dtype;
            b.inv_scale[b.n] = (const float *)(d->inv_scale_buffer->dptr + d->inv_scale_offset);
            b.found_inf[b.n] = (int *)(d->found_inf_buffer->dptr + d->found_inf_offset);
            b.block_start[b.n] = blocks;
            blocks += (unsigned)((d->count + NORM_BLOCK - 1U) / NORM_BLOCK);
            b.n += 1;
        }
        b.block_start[b.n] = blocks;
        if (blocks == 0U) {
            continue;
        }
        gdb_launch(amp_unscale_kernel, blocks, 256, 0, be->stream, b);
        gd_status st = gdb_launched(be, "amp_unscale");
        if (st != GD_OK) {
            return st;
        }
    }
    return GD_OK;
}

gd_status gd_backend_amp_unscale(gd_backend *be, const gd_backend_amp_unscale_desc *desc)
{
    return desc == NULL ? GD_ERR_INVALID_ARGUMENT : gd_backend_amp_unscale_batch(be, desc, 1U);
}

// Partials are laid out as in the reference: one float per 1024 gradient elements, tensor after
// tensor, contiguous from descs[0].partial_offset (metal_adamw.m:414-437).
gd_status gd_backend_grad_clip_scale(gd_backend *be, const gd_backend_grad_norm_desc *descs, uint32_t desc_count, gd_backend_buffer *scale_buffer, size_t scale_offset, float max_norm, float eps)
{
    if (desc_count == 0U) {
        return GD_OK;
    }
    if (be == NULL || descs == NULL || !(max_norm > 0.0f) || !isfinite(max_norm) || !(eps > 0.0f) || !isfinite(eps) ||
        !rng(scale_buffer, scale_offset, 8U) || (scale_offset % 4U) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    size_t running = descs[0].partial_offset, total_partials = 0;
    for (uint32_t i = 0; i < desc_count; ++i) {
        const gd_backend_grad_norm_desc *d = &descs[i];
        const size_t es = gdb_dtype_size(d->grad_dtype);
        const size_t need = (d->count + NORM_BLOCK - 1U) / NORM_BLOCK;
        if (!gdb_is_float_dtype(d->grad_dtype) || !rng(d->grad_buffer, d->grad_offset, d->count * es) ||
            d->partial_buffer != descs[0].partial_buffer || d->partial_offset != running ||
            d->grad_scale_buffer != descs[0].grad_scale_buffer || d->grad_scale_offset != descs[0].grad_scale_offset ||
            d->partial_count < need || !rng(d->partial_buffer, d->partial_offset, d->partial_count * 4U) ||
            !rng(d->grad_scale_buffer, d->grad_scale_offset, 4U) ||
            (d->has_found_inf && !rng(d->found_inf_buffer, d->found_inf_offset, 4U))) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        running += d->partial_count * 4U;
        total_partials += d->partial_count;
    }
    if (total_partials == 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const float *gscale = (const float *)(descs[0].grad_scale_buffer->dptr + descs[0].grad_scale_offset);
    float *partials = (float *)(descs[0].partial_buffer->dptr + descs[0].partial_offset);
    // Unused tail slots of each tensor's partial range must read as zero in the finalize sum.
    cudaError_t e = cudaMemsetAsync(partials, 0, total_partials * 4U, be->stream);
    be->launches += 1U;
    if (e != cudaSuccess) {
        return gdb_fail(be, e, "grad_clip partial clear");
    }
    for (uint32_t start = 0; start < desc_count; start += MT_MAX) {
        norm_batch b;
        memset(&b, 0, sizeof(b));
        unsigned blocks = 0;
        b.grad_scale = gscale;
        for (uint32_t i = start; i < desc_count && i < start + MT_MAX; ++i) {
            const gd_backend_grad_norm_desc *d = &descs[i];
            if (d->count == 0U) {
                continue;
            }
            b.grad[b.n] = d->grad_buffer->dptr + d->grad_offset;
            b.count[b.n] = d->count;
            b.dtype[b.n] = d->grad_dtype;
            b.partial[b.n] = (float *)(d->partial_buffer->dptr + d->partial_offset);
            if (d->has_found_inf) {
                b.found_inf = (int *)(d->found_inf_buffer->dptr + d->found_inf_offset);
            }
            b.block_start[b.n] = blocks;
            blocks += (unsigned)((d->count + NORM_BLOCK * NORM_GROUP - 1U) / (NORM_BLOCK * NORM_GROUP));
            b.n += 1;
        }
        b.block_start[b.n] = blocks;
        if (blocks == 0U) {
            continue;
        }
        gdb_launch(grad_norm_stage_kernel, blocks, 256, 0, be->stream, b);
        gd_status st = gdb_launched(be, "grad_norm_stage");
        if (st != GD_OK) {
            return st;
        }
    }
    gdb_launch(grad_clip_finalize_kernel, 1, 1024, 0, be->stream, partials, total_partials, (float *)(scale_buffer->dptr + scale_offset), gscale, max_norm, eps);
    return gdb_launched(be, "grad_clip_finalize");
}

gd_status gd_backend_adamw_batch(gd_backend *be, const gd_backend_adamw_desc *descs, uint32_t desc_count)
{
    if (desc_count == 0U) {
        return GD_OK;
    }
    if (be == NULL || descs == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    // validate everything before the first launch so a bad descriptor leaves no partial update
    {
        adamw_item tmp;
        for (uint32_t i = 0; i < desc_count; ++i) {
            gd_status st = fill_adamw_item(&descs[i], &tmp);
            if (st != GD_OK) {
                return st;
            }
        }
    }
    for (uint32_t start = 0; start < desc_count; start += (uint32_t)ADAMW_BATCH) {
        adamw_batch b;
        memset(&b, 0, sizeof(b));
        unsigned blocks = 0;
        bool any_state = false;
        for (uint32_t i = start; i < desc_count && i < start + (uint32_t)ADAMW_BATCH; ++i) {
            (void)fill_adamw_item(&descs[i], &b.it[b.n]);
            any_state = any_state || b.it[b.n].beta1_power != NULL;
            b.block_start[b.n] = blocks;
            blocks += (unsigned)((descs[i].count + ADAMW_BLOCK_ELEMS - 1U) / ADAMW_BLOCK_ELEMS);
            b.n += 1;
        }
        b.block_start[b.n] = blocks;
        gd_status st;
        // (the step scalars of tensors with device-side state are formed inside the update kernel)
        gdb_launch(adamw_update_kernel, blocks, 256, 0, be->stream, b);
        st = gdb_launched(be, "adamw_update");
        if (st != GD_OK) {
            return st;
        }
        if (any_state) {
            adamw_commit_batch cb;
            memset(&cb, 0, sizeof(cb));
            cb.n = b.n;
            for (int i = 0; i < b.n; ++i) {
                const adamw_item &a = b.it[i];
                adamw_commit_item &c = cb.it[i];
                c.beta1_power = a.beta1_power;
                c.beta2_power = a.beta2_power;
                c.param_step = a.param_step;
                c.optimizer_step = a.optimizer_step;
                c.found_inf = a.found_inf;
                c.beta1 = a.beta1;
                c.beta2 = a.beta2;
                c.update_optimizer_step = a.update_optimizer_step;
            }
            gdb_launch(adamw_commit_kernel, 1, 64, 0, be->stream, cb);
            st = gdb_launched(be, "adamw_commit");
            if (st != GD_OK) {
                return st;
            }
        }
    }
    return GD_OK;
}

gd_status gd_backend_adamw(gd_backend *be, const gd_backend_adamw_desc *desc)
{
    return desc == NULL ? GD_ERR_INVALID_ARGUMENT : gd_backend_adamw_batch(be, desc, 1U);
}

}  // extern "C"
