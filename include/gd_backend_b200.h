/*
 * gd_backend_b200.h - C ABI of the B200 (sm_100a) CUDA backend for gradients.c.
 *
 * The shared library libgd_backend_b200.so defines every global symbol that the
 * gradients.c host runtime binds at its backend boundary (reference:
 * src/core/backend.h:144-791 and src/core/backend_generated.h:6-43, 109 functions).
 * The reference selects a backend at link time (one set of gd_backend_* symbols per
 * build, Makefile:57-73), so linking libgradients.a against this library instead of
 * src/backends/null/ is the whole integration.
 *
 * Struct layouts below are binary-compatible with the reference's view/descriptor
 * structs (src/core/backend.h:21-140,301-305,321-325,528-537,579-639,671-689); the
 * field order is part of the ABI. If the reference's own header is already included
 * (GD_CORE_BACKEND_H defined) the type section is skipped and only the additive
 * gdb200_* entry points are declared.
 *
 * Conventions shared by all entries (reference: src/core/backend.h and the behaviour of
 * src/backends/metal/backend_metal.m:340-394,534-897):
 *   - first argument is the backend handle; return value is a gd_status code
 *     (include/gradients/status.h:8-19); arguments are validated and byte ranges are
 *     checked against the buffer size; nothing aborts.
 *   - `offset` fields are byte offsets into `buffer`; matrix views carry `row_bytes`.
 *   - dtype codes are gd_dtype values (include/gradients/tensor.h:49-57).
 *   - all work is enqueued on one in-order CUDA stream; gd_backend_flush waits for it.
 *   - all 109 entries of the vtable are implemented; a dtype or shape that an entry does
 *     not take is answered with GD_ERR_UNSUPPORTED (the code the reference's null backend
 *     gives, src/backends/null/backend_null.c), never with a silent fallback.
 */
#ifndef GD_BACKEND_B200_H
#define GD_BACKEND_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GD_CORE_BACKEND_H /* reference header not present: declare the ABI ourselves */

#ifndef GRADIENTS_STATUS_H
/* include/gradients/status.h:8-19 */
typedef enum gd_status {
    GD_OK = 0,
    GD_ERR_INVALID_ARGUMENT = -1,
    GD_ERR_OUT_OF_MEMORY = -2,
    GD_ERR_FROZEN = -3,
    GD_ERR_BUSY = -4,
    GD_ERR_BAD_STATE = -5,
    GD_ERR_UNSUPPORTED = -6,
    GD_ERR_INTERNAL = -7,
    GD_ERR_NOT_IMPLEMENTED = -8,
    GD_ERR_IO = -9
} gd_status;
#endif

/* gd_dtype codes travel as uint32_t (include/gradients/tensor.h:49-57). */
enum {
    GDB_DTYPE_F16 = 1,
    GDB_DTYPE_BF16 = 2,
    GDB_DTYPE_F32 = 3,
    GDB_DTYPE_I32 = 4,
    GDB_DTYPE_U8 = 5,
    GDB_DTYPE_U16 = 6
};

typedef struct gd_backend gd_backend;               /* opaque, src/core/backend.h:10 */
typedef struct gd_backend_buffer gd_backend_buffer; /* opaque, src/core/backend.h:11 */
typedef struct gd_backend_fence { void *handle; } gd_backend_fence; /* :13-15 */

/* src/core/backend.h:17-19 has only the Metal kind; this backend reports 2. */
typedef enum gd_backend_kind { GD_BACKEND_METAL = 1, GD_BACKEND_CUDA_B200 = 2 } gd_backend_kind;

/* ---- views (src/core/backend.h:21-50,132-140) ---- */
typedef struct gd_backend_matrix_view {
    gd_backend_buffer *buffer;
    size_t offset;
    uint32_t rows, cols;
    size_t row_bytes;
    uint32_t dtype;
} gd_backend_matrix_view;

#define GD_BACKEND_MAX_BATCH_DIMS 6U
typedef struct gd_backend_batched_matrix_view {
    gd_backend_buffer *buffer;
    size_t offset;
    uint32_t rows, cols;
    size_t row_bytes;
    uint32_t dtype;
    uint32_t batch_rank, batch_count;
    uint32_t batch_shape[GD_BACKEND_MAX_BATCH_DIMS];
    size_t batch_strides[GD_BACKEND_MAX_BATCH_DIMS];
} gd_backend_batched_matrix_view;

typedef struct gd_backend_vector_view {
    gd_backend_buffer *buffer;
    size_t offset;
    uint32_t length;
    uint32_t dtype;
} gd_backend_vector_view;

typedef struct gd_backend_tensor_view {
    gd_backend_buffer *buffer;
    size_t offset;
    size_t count;
    uint32_t dtype;
    uint32_t rank;
    int64_t shape[8];
    int64_t strides[8];
} gd_backend_tensor_view;

/* ---- optimizer / AMP descriptors (src/core/backend.h:52-130) ---- */
typedef struct gd_backend_adamw_desc {
    gd_backend_buffer *param_buffer;      size_t param_offset;
    gd_backend_buffer *master_buffer;     size_t master_offset;     /* optional FP32 masters */
    gd_backend_buffer *grad_buffer;       size_t grad_offset;
    gd_backend_buffer *grad_scale_buffer; size_t grad_scale_offset; /* optional F32 multiplier */
    gd_backend_buffer *found_inf_buffer;  size_t found_inf_offset;  /* optional I32 skip flag */
    gd_backend_buffer *m_buffer;          size_t m_offset;
    gd_backend_buffer *v_buffer;          size_t v_offset;
    gd_backend_buffer *state_f32_buffer;  /* optional device scalar state */
    size_t beta1_power_offset, beta2_power_offset, step_scale_offset, decay_scale_offset, eps_scaled_offset;
    gd_backend_buffer *state_i32_buffer;  /* optional device step counters */
    size_t param_step_offset, optimizer_step_offset;
    size_t count;
    uint32_t param_dtype, grad_dtype;
    uint32_t has_master, has_grad_scale, has_found_inf, has_device_state;
    uint32_t bias_correction, update_optimizer_step;
    float lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2;
} gd_backend_adamw_desc;

typedef struct gd_backend_amp_state_desc {
    gd_backend_buffer *scale_buffer; size_t scale_offset; /* F32[2]: scale, 1/scale */
    gd_backend_buffer *flags_buffer; size_t flags_offset; /* I32[3]: growth_tracker, found_inf, last_found_inf */
    float growth_factor, backoff_factor, min_scale, max_scale;
    uint32_t growth_interval;
} gd_backend_amp_state_desc;

typedef struct gd_backend_amp_unscale_desc {
    gd_backend_buffer *grad_buffer; size_t grad_offset;
    size_t count;
    uint32_t grad_dtype;
    gd_backend_buffer *inv_scale_buffer; size_t inv_scale_offset;
    gd_backend_buffer *found_inf_buffer; size_t found_inf_offset;
} gd_backend_amp_unscale_desc;

typedef struct gd_backend_grad_norm_desc {
    gd_backend_buffer *grad_buffer; size_t grad_offset;
    size_t count;
    uint32_t grad_dtype;
    gd_backend_buffer *partial_buffer; size_t partial_offset; size_t partial_count;
    gd_backend_buffer *grad_scale_buffer; size_t grad_scale_offset;
    gd_backend_buffer *found_inf_buffer; size_t found_inf_offset;
    uint32_t has_found_inf;
} gd_backend_grad_norm_desc;

/* ---- per-op argument blocks ---- */
typedef struct gd_backend_embedding_args { uint64_t ids_count, vocab, dim; } gd_backend_embedding_args; /* :301-305 */
typedef struct gd_backend_rope_args { float theta; uint32_t n_dims; uint32_t interleaved; } gd_backend_rope_args; /* :321-325 */
typedef struct gd_backend_rms_norm_args { /* :528-537 */
    uint64_t rows, cols, row_blocks;
    float eps;
    uint32_t simdgroups, wgrad_simdgroups, wgrad_row_block, reserved0;
} gd_backend_rms_norm_args;
typedef struct gd_backend_concat_args { uint64_t count, inner, slice_axis, full_axis, axis_offset; } gd_backend_concat_args; /* :579-585 */
typedef struct gd_backend_split_args { uint64_t count, inner, slice_axis, full_axis, axis_offset; } gd_backend_split_args;   /* :598-604 */
typedef struct gd_backend_permute_args { /* :617-624 */
    uint64_t count, inner;
    uint32_t rank, active_rank;
    uint32_t axes[8];
    uint32_t reserved0;
} gd_backend_permute_args;
typedef struct gd_backend_minimax_m3_sparse_args { /* :632-639 */
    float scale;
    uint32_t block_size, topk, init_blocks, local_blocks, max_seqlen;
} gd_backend_minimax_m3_sparse_args;
typedef struct gd_backend_sdpa_varlen_args { /* :671-678 */
    float scale;
    uint32_t causal, sliding_window, prefix_len, max_seqlen, use_forward_stats;
} gd_backend_sdpa_varlen_args;
typedef struct gd_backend_sdpa_decode_args { /* :680-685 */
    float scale;
    uint32_t sliding_window, prefix_len;
    int32_t cache_pos;
} gd_backend_sdpa_decode_args;
typedef struct gd_backend_kv_cache_append_args { int32_t cache_pos; } gd_backend_kv_cache_append_args; /* :687-689 */

#define GDB_TV const gd_backend_tensor_view *
#define GDB_MV const gd_backend_matrix_view *
#define GDB_BV const gd_backend_batched_matrix_view *
#define GDB_VV const gd_backend_vector_view *

/* ---- lifecycle, buffers, stream scope, fences (src/core/backend.h:144-158,788-791) ---- */
gd_status gd_backend_create_default(gd_backend **out_backend);
void gd_backend_destroy(gd_backend *backend);
gd_backend_kind gd_backend_kind_query(const gd_backend *backend);
const char *gd_backend_name(const gd_backend *backend);
gd_status gd_backend_buffer_create(gd_backend *backend, size_t nbytes, gd_backend_buffer **out_buffer);
void gd_backend_buffer_destroy(gd_backend_buffer *buffer);
size_t gd_backend_buffer_nbytes(const gd_backend_buffer *buffer);
void *gd_backend_buffer_host_ptr(gd_backend_buffer *buffer);
bool gd_backend_buffer_is_host_visible(const gd_backend_buffer *buffer);
gd_status gd_backend_scope_begin(gd_backend *backend);
gd_status gd_backend_flush(gd_backend *backend);
gd_status gd_backend_record_fence(gd_backend *backend, gd_backend_fence *out_fence);
void gd_backend_fence_destroy(gd_backend_fence *fence);
bool gd_backend_fence_is_complete(gd_backend_fence *fence);
gd_status gd_backend_fence_wait(gd_backend_fence *fence);

/* ---- transfers and initialisers (:160-185) ---- */
gd_status gd_backend_upload(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, const void *src, size_t nbytes);
gd_status gd_backend_download(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, void *dst, size_t nbytes);
gd_status gd_backend_fill(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, size_t count, size_t elem_size, uint32_t pattern);
gd_status gd_backend_rand_uniform(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, size_t count, uint32_t dtype, uint64_t seed, float low, float high);

/* ---- dense contractions (:187-223). matmul: y = x w; _nt: y = x w^T (w stored [y.cols, x.cols]);
 * _tn: y = x^T w (x stored [inner, y.rows]); linear: y = x w + bias (bias added in FP32 before the
 * single rounding); reduce_rows: y[c] = sum_r x[r,c]. F16/BF16 storage, FP32 accumulation. ---- */
gd_status gd_backend_matmul(gd_backend *backend, GDB_MV x, GDB_MV w, GDB_MV y);
gd_status gd_backend_matmul_nt(gd_backend *backend, GDB_MV x, GDB_MV w, GDB_MV y);
gd_status gd_backend_matmul_tn(gd_backend *backend, GDB_MV x, GDB_MV w, GDB_MV y);
gd_status gd_backend_batched_matmul(gd_backend *backend, GDB_BV x, GDB_BV w, GDB_BV y);
gd_status gd_backend_batched_matmul_nt(gd_backend *backend, GDB_BV x, GDB_BV w, GDB_BV y);
gd_status gd_backend_batched_matmul_tn(gd_backend *backend, GDB_BV x, GDB_BV w, GDB_BV y);
gd_status gd_backend_linear(gd_backend *backend, GDB_MV x, GDB_MV w, GDB_VV bias, GDB_MV y);
gd_status gd_backend_reduce_rows(gd_backend *backend, GDB_MV x, GDB_VV y);

/* ---- gradient plumbing (:224-240): dst += src (F16 rounds every add); dst = src * scale ---- */
gd_status gd_backend_accumulate(gd_backend *backend, gd_backend_buffer *dst_buffer, size_t dst_offset, gd_backend_buffer *src_buffer, size_t src_offset, size_t count, uint32_t dtype);
gd_status gd_backend_scale(gd_backend *backend, gd_backend_buffer *dst_buffer, size_t dst_offset, gd_backend_buffer *src_buffer, size_t src_offset, size_t count, uint32_t dtype, float scale);

/* ---- elementwise, generated group (src/core/backend_generated.h:6-43) ---- */
gd_status gd_backend_relu(gd_backend *backend, GDB_TV x, GDB_TV y);
gd_status gd_backend_relu_backward(gd_backend *backend, GDB_TV x, GDB_TV grad_out, GDB_TV grad_x);
gd_status gd_backend_add(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV out);
gd_status gd_backend_mul(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV out);
gd_status gd_backend_sub(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV out);
gd_status gd_backend_sigmoid(gd_backend *backend, GDB_TV x, GDB_TV y);
gd_status gd_backend_sigmoid_backward(gd_backend *backend, GDB_TV x, GDB_TV grad_out, GDB_TV grad_x);
gd_status gd_backend_tanh(gd_backend *backend, GDB_TV x, GDB_TV y);
gd_status gd_backend_tanh_backward(gd_backend *backend, GDB_TV x, GDB_TV grad_out, GDB_TV grad_x);

/* ---- dropout (:273-299): keep iff top 24 bits of splitmix64(seed+i) >= ceil(p*2^24) ---- */
gd_status gd_backend_dropout_forward(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV mask, float p, uint64_t seed);
gd_status gd_backend_dropout_add_forward(gd_backend *backend, GDB_TV residual, GDB_TV x, GDB_TV y, GDB_TV mask, float p, uint64_t seed);
gd_status gd_backend_dropout_backward(gd_backend *backend, GDB_TV grad_out, GDB_TV grad_x, float p, uint64_t seed);
gd_status gd_backend_dropout_backward_mask(gd_backend *backend, GDB_TV mask, GDB_TV grad_out, GDB_TV grad_x, float scale);

/* ---- embedding (:307-319): invalid ids give NaN rows forward and are skipped backward ---- */
gd_status gd_backend_embedding_forward(gd_backend *backend, GDB_TV table, GDB_TV ids, GDB_TV out, const gd_backend_embedding_args *args);
gd_status gd_backend_embedding_backward(gd_backend *backend, GDB_TV grad_out, GDB_TV ids, GDB_TV grad_table, GDB_TV scratch, const gd_backend_embedding_args *args);

/* ---- rotary embedding (:327-358) ---- */
gd_status gd_backend_rope(gd_backend *backend, GDB_TV x, GDB_TV pos_ids, GDB_TV out, const gd_backend_rope_args *args);
gd_status gd_backend_rope_backward(gd_backend *backend, GDB_TV grad_out, GDB_TV pos_ids, GDB_TV grad_x, const gd_backend_rope_args *args);
gd_status gd_backend_qkv_split_rope_forward(gd_backend *backend, GDB_TV qkv, GDB_TV pos_ids, GDB_TV q, GDB_TV k, GDB_TV v, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args);
gd_status gd_backend_qkv_split_rope_backward(gd_backend *backend, GDB_TV grad_q, GDB_TV grad_k, GDB_TV grad_v, GDB_TV pos_ids, GDB_TV grad_qkv, uint32_t n_heads, uint32_t head_dim, const gd_backend_rope_args *args);

/* ---- gated MLP (:509-526): out = x1 * silu(x2); split form takes x12 = [x1 | x2] ---- */
gd_status gd_backend_swiglu_forward(gd_backend *backend, GDB_TV x1, GDB_TV x2, GDB_TV out);
gd_status gd_backend_swiglu_backward(gd_backend *backend, GDB_TV x1, GDB_TV x2, GDB_TV grad_out, GDB_TV grad_x1, GDB_TV grad_x2);
gd_status gd_backend_swiglu_split_forward(gd_backend *backend, GDB_TV x12, GDB_TV out);
gd_status gd_backend_swiglu_split_backward(gd_backend *backend, GDB_TV x12, GDB_TV grad_out, GDB_TV grad_x12);

/* ---- RMSNorm (:539-577) ---- */
gd_status gd_backend_rms_norm_forward(gd_backend *backend, GDB_TV x, GDB_TV weight, GDB_TV out, const gd_backend_rms_norm_args *args);
gd_status gd_backend_rms_norm_forward_stats(gd_backend *backend, GDB_TV x, GDB_TV weight, GDB_TV out, GDB_TV inv_rms, const gd_backend_rms_norm_args *args);
gd_status gd_backend_rms_norm_inv(gd_backend *backend, GDB_TV x, GDB_TV inv_rms, const gd_backend_rms_norm_args *args);
gd_status gd_backend_rms_norm_backward(gd_backend *backend, GDB_TV x, GDB_TV weight, GDB_TV grad_out, GDB_TV grad_x, const gd_backend_rms_norm_args *args);
gd_status gd_backend_rms_norm_backward_stats(gd_backend *backend, GDB_TV x, GDB_TV weight, GDB_TV inv_rms, GDB_TV grad_out, GDB_TV grad_x, const gd_backend_rms_norm_args *args);
gd_status gd_backend_rms_norm_weight_backward_stats(gd_backend *backend, GDB_TV x, GDB_TV inv_rms, GDB_TV grad_out, GDB_TV grad_weight, GDB_TV partial, const gd_backend_rms_norm_args *args);

/* ---- attention and KV cache (:691-750) ---- */
gd_status gd_backend_sdpa_varlen(gd_backend *backend, GDB_TV q, GDB_TV k, GDB_TV v, GDB_TV cu_seqlens, GDB_TV out, GDB_TV stats, const gd_backend_sdpa_varlen_args *args);
gd_status gd_backend_sdpa_varlen_backward(gd_backend *backend, GDB_TV grad_out, GDB_TV q, GDB_TV k, GDB_TV v, GDB_TV cu_seqlens, GDB_TV grad_q, GDB_TV grad_k, GDB_TV grad_v, GDB_TV stats, const gd_backend_sdpa_varlen_args *args);
gd_status gd_backend_sdpa_decode(gd_backend *backend, GDB_TV q, GDB_TV k_cache, GDB_TV v_cache, GDB_TV cache_pos, GDB_TV out, const gd_backend_sdpa_decode_args *args);
gd_status gd_backend_sdpa_decode_at(gd_backend *backend, GDB_TV q, GDB_TV k_cache, GDB_TV v_cache, GDB_TV out, const gd_backend_sdpa_decode_args *args);
gd_status gd_backend_sdpa_decode_positions(gd_backend *backend, GDB_TV q, GDB_TV k_cache, GDB_TV v_cache, GDB_TV cache_pos, GDB_TV out, const gd_backend_sdpa_decode_args *args);
gd_status gd_backend_kv_cache_append_at(gd_backend *backend, GDB_TV k_cache, GDB_TV v_cache, GDB_TV k_new, GDB_TV v_new, const gd_backend_kv_cache_append_args *args);
gd_status gd_backend_kv_cache_append_positions(gd_backend *backend, GDB_TV k_cache, GDB_TV v_cache, GDB_TV cache_pos, GDB_TV k_new, GDB_TV v_new, const gd_backend_kv_cache_append_args *args);
gd_status gd_backend_kv_cache_append_packed(gd_backend *backend, GDB_TV k_cache, GDB_TV v_cache, GDB_TV cache_pos, GDB_TV cu_seqlens, GDB_TV k_new, GDB_TV v_new, const gd_backend_kv_cache_append_args *args);

/* ---- losses (:381-450) ---- */
gd_status gd_backend_cross_entropy_loss(gd_backend *backend, GDB_TV logits, GDB_TV targets, GDB_TV row_loss);
gd_status gd_backend_cross_entropy_loss_stats(gd_backend *backend, GDB_TV logits, GDB_TV targets, GDB_TV row_loss, GDB_TV row_max, GDB_TV row_inv_sum);
gd_status gd_backend_cross_entropy_backward(gd_backend *backend, GDB_TV logits, GDB_TV targets, GDB_TV grad_loss, GDB_TV grad_logits, float scale);
gd_status gd_backend_cross_entropy_backward_stats(gd_backend *backend, GDB_TV logits, GDB_TV targets, GDB_TV row_max, GDB_TV row_inv_sum, GDB_TV grad_loss, GDB_TV grad_logits, float scale);
gd_status gd_backend_lm_cross_entropy_online_update(gd_backend *backend, GDB_TV logits_chunk, GDB_TV bias_chunk, GDB_TV targets, GDB_TV row_loss, GDB_TV row_max, GDB_TV row_inv_sum, uint64_t class_start, uint64_t total_classes, float logits_softcap);
gd_status gd_backend_lm_cross_entropy_finalize(gd_backend *backend, GDB_TV targets, GDB_TV row_loss, GDB_TV row_max, GDB_TV row_inv_sum, GDB_TV row_valid, uint64_t total_classes, int32_t ignore_index);
gd_status gd_backend_lm_cross_entropy_reduce_normalize(gd_backend *backend, GDB_TV row_loss, GDB_TV row_valid, GDB_TV loss, GDB_TV inv_valid_count);
gd_status gd_backend_lm_cross_entropy_backward_chunk(gd_backend *backend, GDB_TV logits_chunk, GDB_TV bias_chunk, GDB_TV targets, GDB_TV row_max, GDB_TV row_inv_sum, GDB_TV grad_loss, GDB_TV inv_valid_count, GDB_TV grad_logits_chunk, uint64_t class_start, uint64_t total_classes, float scale, float logits_softcap, int32_t ignore_index);

/* ---- AMP loss scaling, gradient clipping, AdamW (:752-786) ---- */
gd_status gd_backend_amp_begin_step(gd_backend *backend, const gd_backend_amp_state_desc *desc);
gd_status gd_backend_amp_finish_step(gd_backend *backend, const gd_backend_amp_state_desc *desc);
gd_status gd_backend_amp_fill_scale(gd_backend *backend, gd_backend_buffer *dst_buffer, size_t dst_offset, size_t count, uint32_t dtype, gd_backend_buffer *scale_buffer, size_t scale_offset);
gd_status gd_backend_amp_scale(gd_backend *backend, gd_backend_buffer *dst_buffer, size_t dst_offset, gd_backend_buffer *src_buffer, size_t src_offset, size_t count, uint32_t dtype, gd_backend_buffer *scale_buffer, size_t scale_offset);
gd_status gd_backend_amp_unscale(gd_backend *backend, const gd_backend_amp_unscale_desc *desc);
gd_status gd_backend_amp_unscale_batch(gd_backend *backend, const gd_backend_amp_unscale_desc *descs, uint32_t desc_count);
gd_status gd_backend_grad_clip_scale(gd_backend *backend, const gd_backend_grad_norm_desc *descs, uint32_t desc_count, gd_backend_buffer *scale_buffer, size_t scale_offset, float max_norm, float eps);
gd_status gd_backend_adamw(gd_backend *backend, const gd_backend_adamw_desc *desc);
gd_status gd_backend_adamw_batch(gd_backend *backend, const gd_backend_adamw_desc *descs, uint32_t desc_count);

/* ---- layout copies (:587-630); concat_to_full is used by multi-prompt prefill ---- */
gd_status gd_backend_concat_to_full(gd_backend *backend, GDB_TV src, GDB_TV dst, const gd_backend_concat_args *args);
gd_status gd_backend_concat_from_full(gd_backend *backend, GDB_TV src, GDB_TV dst, const gd_backend_concat_args *args);
gd_status gd_backend_split_from_full(gd_backend *backend, GDB_TV full, GDB_TV slice, const gd_backend_split_args *args);
gd_status gd_backend_split_to_full(gd_backend *backend, GDB_TV slice, GDB_TV full, const gd_backend_split_args *args);
gd_status gd_backend_permute(gd_backend *backend, GDB_TV src, GDB_TV dst, const gd_backend_permute_args *args);

/* ---- entries off the gpt_lm path, used by the reference's other examples and tests (src/core/backend.h:243-268,
 * 355-382, 452-506). F16 / BF16 / F32 unless noted. reduce_* / broadcast_*: sums and broadcasts of contiguous tensors
 * times `scale`. *_backward_from_output: gradients from the saved forward output. mul_backward_direct and
 * mul_reduce_suffix: 16-bit fast paths of the mul backward. mse / huber: per-chunk partial sums (F32) forward,
 * +/- grad_out[0] * scale * d backward into either optional gradient. powlu: out = x1 * gate(x2, m), 16-bit. ---- */
gd_status gd_backend_reduce_contiguous(gd_backend *backend, GDB_TV src, GDB_TV dst, float scale);
gd_status gd_backend_reduce_axis(gd_backend *backend, GDB_TV src, GDB_TV dst, uint32_t axis, float scale);
gd_status gd_backend_broadcast_axis(gd_backend *backend, GDB_TV src, GDB_TV dst, uint32_t axis, float scale);
gd_status gd_backend_broadcast_to(gd_backend *backend, GDB_TV src, GDB_TV dst, float scale);
gd_status gd_backend_broadcast_scalar(gd_backend *backend, GDB_TV src, GDB_TV dst, float scale);
gd_status gd_backend_reduce_broadcast(gd_backend *backend, GDB_TV src, GDB_TV dst, float scale);
gd_status gd_backend_sigmoid_backward_from_output(gd_backend *backend, GDB_TV sigmoid_out, GDB_TV grad_out, GDB_TV grad_x);
gd_status gd_backend_tanh_backward_from_output(gd_backend *backend, GDB_TV tanh_out, GDB_TV grad_out, GDB_TV grad_x);
gd_status gd_backend_mul_backward_direct(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV grad_out, GDB_TV grad_x, GDB_TV grad_y);
gd_status gd_backend_mul_reduce_suffix(gd_backend *backend, GDB_TV grad_out, GDB_TV other, GDB_TV dst);
gd_status gd_backend_mse_forward(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV out, uint64_t chunk_size, float scale);
gd_status gd_backend_mse_backward(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV grad_out, GDB_TV grad_x, GDB_TV grad_y, float scale);
gd_status gd_backend_huber_forward(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV out, uint64_t chunk_size, float scale, float delta);
gd_status gd_backend_huber_backward(gd_backend *backend, GDB_TV x, GDB_TV y, GDB_TV grad_out, GDB_TV grad_x, GDB_TV grad_y, float scale, float delta);
gd_status gd_backend_powlu_forward(gd_backend *backend, GDB_TV x1, GDB_TV x2, GDB_TV out, float m);
gd_status gd_backend_powlu_backward(gd_backend *backend, GDB_TV x1, GDB_TV x2, GDB_TV grad_out, GDB_TV grad_x1, GDB_TV grad_x2, float m);
gd_status gd_backend_powlu_split_forward(gd_backend *backend, GDB_TV x12, GDB_TV out, float m);
gd_status gd_backend_powlu_split_backward(gd_backend *backend, GDB_TV x12, GDB_TV grad_out, GDB_TV grad_x12, float m);
/* MiniMax-M3 block-sparse attention (src/core/backend.h:632-668): index_q / index_k [N, Hkv, Dh] -> topk_idx I32 [Hkv, N, topk]
 * (sequence-local block ids, -1 padded); q [N, Hq, Dh], k / v [N, Hkv, Dh], Dh <= 64, topk <= 16, block_size <= 128; stats F32 [N, Hq, 3]
 * is scratch of the backward. Rows of a sequence beyond max_seqlen are not visited. */
gd_status gd_backend_minimax_m3_index_topk(gd_backend *backend, GDB_TV index_q, GDB_TV index_k, GDB_TV cu_seqlens, GDB_TV topk_idx, const gd_backend_minimax_m3_sparse_args *args);
gd_status gd_backend_minimax_m3_sparse_attention(gd_backend *backend, GDB_TV q, GDB_TV k, GDB_TV v, GDB_TV cu_seqlens, GDB_TV topk_idx, GDB_TV out, const gd_backend_minimax_m3_sparse_args *args);
gd_status gd_backend_minimax_m3_sparse_attention_backward(gd_backend *backend, GDB_TV grad_out, GDB_TV q, GDB_TV k, GDB_TV v, GDB_TV cu_seqlens, GDB_TV topk_idx, GDB_TV grad_q, GDB_TV grad_k, GDB_TV grad_v, GDB_TV stats, const gd_backend_minimax_m3_sparse_args *args);

#undef GDB_TV
#undef GDB_MV
#undef GDB_BV
#undef GDB_VV

#endif /* !GD_CORE_BACKEND_H */

/* ==================================================================================
 * Additive entry points (no counterpart in the reference). The reference ABI links and
 * runs without them; they exist for measurement, data parallelism and foreign-function
 * callers that cannot hold the opaque structs.
 * ================================================================================== */

/* Raw device address of byte `offset` of a buffer (for ctypes/FFI tests and NCCL staging). */
void *gdb200_buffer_device_ptr(gd_backend_buffer *buffer, size_t offset);
/* The CUDA stream (cudaStream_t) every entry of this backend enqueues on. */
void *gdb200_stream(gd_backend *backend);
/* CUDA device ordinal the backend was created on (GD_CUDA_DEVICE, else LOCAL_RANK, else 0). */
int gdb200_device(const gd_backend *backend);
/* Number of kernel launches issued by this backend since creation (all entries). */
uint64_t gdb200_launch_count(const gd_backend *backend);
/* Last CUDA error string seen by the backend ("" if none); storage owned by the backend. */
const char *gdb200_last_error(const gd_backend *backend);
/* Select the GEMM implementation: 0 = automatic (tcgen05 when the shape/alignment allows,
 * else the portable tiled kernel), 1 = force the portable kernel, 2 = require tcgen05 and
 * fail with GD_ERR_UNSUPPORTED when it cannot run, 3 = automatic without the CTA-pair
 * (cta_group::2) kernel, for A/B measurements. Returns the previous value. */
int gdb200_set_gemm_mode(gd_backend *backend, int mode);
/* Select the sdpa_varlen forward implementation: 0 = automatic (tcgen05 / tensor-memory kernel when
 * head_dim is 64 and the storage is 16-bit, else the mma.sync flash kernels), 1 = mma.sync flash
 * kernels only, for A/B measurements. Returns the previous value. */
int gdb200_set_attention_mode(gd_backend *backend, int mode);
/* Event pair timing helper: records an event on the backend stream and returns an opaque
 * handle; gdb200_event_elapsed_ms synchronises on `stop` and returns milliseconds. */
void *gdb200_event_record(gd_backend *backend);
float gdb200_event_elapsed_ms(void *start, void *stop);
void gdb200_event_destroy(void *event);
/* Page-locked host memory for upload sources / download targets (cudaMallocHost / cudaFreeHost). */
void *gdb200_pinned_alloc(size_t nbytes);
void gdb200_pinned_free(void *p);
/* Stream-ordered copies between page-locked host memory and a buffer, enqueued behind the submitted work and not
 * waited for (gd_backend_upload / gd_backend_download are synchronous, src/core/backend.h upload/download). They
 * are the device half of the reference's data-slot ring: the next batch is staged while the device still works on
 * the previous one and a fence guards reuse (src/core/memory.c:1149-1208, src/dataset/dataloader.c:487-492). The
 * host range must not be written (upload) or read (download) until a fence recorded after the call has completed. */
gd_status gdb200_upload_async(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, const void *pinned_src, size_t nbytes);
gd_status gdb200_download_async(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, void *pinned_dst, size_t nbytes);
/* Benchmark instrumentation: bracket every dense-contraction dispatch with a CUDA event pair on
 * the backend stream; read returns the number of launches, their summed device time and the
 * algorithmic FLOPs / bytes (2MNK and one pass over each operand) accumulated since enable. */
void gdb200_gemm_profile_enable(gd_backend *backend, int enable);
gd_status gdb200_gemm_profile_read(gd_backend *backend, uint64_t *launches, double *total_ms, double *flops, double *bytes);
/* Overwrite a private buffer larger than L2 so that the next kernel starts with a cold L2. */
gd_status gdb200_flush_l2(gd_backend *backend);

/* y = round(round(x w^T) + bias), w stored [y.cols, x.cols]: gd_backend_matmul_nt followed by the
 * row-broadcast gd_backend_add of the reference's linear_transposed_weight capsule
 * (src/ops/linear_transposed_weight/core_linear_transposed_weight.c:51-79) in one kernel, with the
 * same two roundings, so results are bit-identical to the two-call sequence. */
gd_status gdb200_matmul_nt_bias(gd_backend *backend, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                                const gd_backend_vector_view *bias, const gd_backend_matrix_view *y);

/* out [M, F] = x1 * silu(x2) with [x1 | x2] = round(round(x w^T) + bias), w stored [2F, K]: gdb200_matmul_nt_bias followed by
 * gd_backend_swiglu_split_forward (the up / gate projection of examples/gpt_lm/gpt_lm_shared.c:1032-1046) in one
 * launch, bit-identical to the two calls; the [M, 2F] intermediate is not written. Built for decode (M <= 64, K a
 * multiple of 128, 16-byte aligned rows); GD_ERR_UNSUPPORTED otherwise, and the caller issues the two calls. */
gd_status gdb200_matmul_nt_bias_swiglu(gd_backend *backend, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                                       const gd_backend_vector_view *bias, const gd_backend_matrix_view *out);
/* Training form of the same fusion: up_gate [M, 2F] = round(round(x w^T) + bias) (kept for the backward pass) AND
 * act [M, F] = swiglu_split(up_gate) from one contraction whose epilogue reads the x1 and the x2 accumulator tile together
 * (the reference composes matmul_nt, add and swiglu_split: src/ops/linear_transposed_weight/core_linear_transposed_weight.c:51-79,
 * src/ops/swiglu_split_linear/core_swiglu_split_linear.c:226-301). Bit-identical to those three calls, which also run when the
 * fused kernel does not take the shape. */
gd_status gdb200_matmul_nt_bias_swiglu_both(gd_backend *backend, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                                            const gd_backend_vector_view *bias, const gd_backend_matrix_view *up_gate,
                                            const gd_backend_matrix_view *act);
/* Backward counterpart: d_up_gate [M, 2F] = swiglu_split_backward(up_gate, round(g w^T)) with w stored [F, K] (the down
 * projection's weight): gd_backend_matmul_nt into a scratch [M, F] followed by gd_backend_swiglu_split_backward
 * (src/ops/swiglu_split_linear/core_swiglu_split_linear.c:303-420), in one launch and without the scratch. Bit-identical to the two
 * calls; GD_ERR_UNSUPPORTED when the fused kernel does not take the shape (the caller then makes the two calls). */
gd_status gdb200_matmul_nt_swiglu_backward(gd_backend *backend, const gd_backend_matrix_view *g, const gd_backend_matrix_view *w,
                                           const gd_backend_matrix_view *up_gate, const gd_backend_matrix_view *d_up_gate);

/* gd_backend_rms_norm_backward_stats and gd_backend_rms_norm_weight_backward_stats (src/core/backend.h, the two calls of
 * src/ops/rms_norm/core_rms_norm_bwd.c) from ONE pass over x and grad_out: grad_x exactly as the first entry computes it
 * (with accumulate != 0 it is added into grad_x: round, add, round, as gd_backend_accumulate after the entry would), and
 * grad_weight = sum over rows of grad_out * x * inv_rms through FP32 partials [row_blocks, cols] summed in a fixed order.
 * 16-bit storage, cols <= 512 and a multiple of 8; GD_ERR_UNSUPPORTED otherwise (the caller then makes the two calls). */
gd_status gdb200_rms_norm_backward_with_weight(gd_backend *backend, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                               const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                               const gd_backend_tensor_view *grad_x, int32_t accumulate,
                                               const gd_backend_tensor_view *grad_weight, const gd_backend_tensor_view *partial,
                                               const gd_backend_rms_norm_args *args);

/* The same launch with a second output: grad_dropped = gd_backend_dropout_backward_mask(mask, grad_x, scale) (src/core/backend.h;
 * src/ops/dropout_add/core_dropout_add.c backward), formed from the stored grad_x after the optional accumulation, bit for bit
 * what the separate entry writes. For a residual stream whose next consumer of the gradient is the dropout in front of a
 * residual add (gpt_lm: examples/gpt_lm/gpt_lm_shared.c:602-749, every norm's input gradient meets one). mask U8 and
 * grad_dropped, both [rows, cols], are required here. grad_dropped_colsum (optional, [cols]) = sum over the rows of grad_dropped
 * in FP32, rounded once: gd_backend_reduce_rows of it up to the order of the FP32 sum (the bias gradient of the projection whose
 * output went through the dropout); `partial` then has to hold 2 * row_blocks * cols elements. */
gd_status gdb200_rms_norm_backward_with_weight_dropout(gd_backend *backend, const gd_backend_tensor_view *x, const gd_backend_tensor_view *weight,
                                                       const gd_backend_tensor_view *inv_rms, const gd_backend_tensor_view *grad_out,
                                                       const gd_backend_tensor_view *grad_x, int32_t accumulate,
                                                       const gd_backend_tensor_view *grad_weight, const gd_backend_tensor_view *partial,
                                                       const gd_backend_rms_norm_args *args, const gd_backend_tensor_view *mask,
                                                       const gd_backend_tensor_view *grad_dropped, float scale,
                                                       const gd_backend_tensor_view *grad_dropped_colsum);

/* The head of the gpt_lm forward pass (examples/gpt_lm/gpt_lm_shared.c:751-790) in one launch: x = dropout(embedding(table, ids))
 * with the keep mask written, normed = rms_norm(x, weight) and inv_rms saved, i.e. gd_backend_embedding_forward,
 * gd_backend_dropout_forward and gd_backend_rms_norm_forward_stats (src/core/backend.h) with the same rounding points, the same
 * keep decision per element index (seed as gd_backend_dropout_forward takes it) and NaN rows for ids outside the table: bit for bit
 * the three entries' x, mask and normed. table [vocab, cols] and x / normed [ids, cols] in F16 or BF16, cols a multiple of 8,
 * 16-byte aligned; GD_ERR_UNSUPPORTED otherwise (the caller then makes the three calls). */
gd_status gdb200_embedding_dropout_rms_norm(gd_backend *backend, const gd_backend_tensor_view *table, const gd_backend_tensor_view *ids,
                                            const gd_backend_tensor_view *weight, const gd_backend_tensor_view *x, const gd_backend_tensor_view *mask,
                                            const gd_backend_tensor_view *normed, const gd_backend_tensor_view *inv_rms, float eps, float p,
                                            uint64_t seed);

/* Fused LM cross entropy of a logits matrix that holds ALL classes (one chunk), loss statistics and logits gradient from ONE
 * pass: gd_backend_lm_cross_entropy_online_update + _finalize + _backward_chunk (src/core/backend.h, called by
 * src/ops/lm_cross_entropy/core_lm_cross_entropy.c:452-675 and :876-890) for a caller that knows the gradient seed and the
 * number of valid target rows before the loss is reduced. logits [rows, classes] holds the matmul logits on entry and
 * dlogits = (softmax(soft) - 1[target]) * max(0, 1 - (soft / cap)^2) * grad_loss[0] * scale / counts[0] on return, with
 * soft = softcap(round(logit + bias)); row_loss[row] = logsumexp(soft) - soft[target], 0 for an ignored target (negative or
 * equal to ignore_index) and NaN for one past the classes; such rows get a zero gradient. counts (F32, element 0) = valid
 * target rows of the batch the loss is a mean over. The arithmetic differs from the three entries in three places: the row
 * maximum is found before the exponentials instead of by an online merge; tanh(y) of the soft-capping is 1 - 2 / (1 + exp(2 y))
 * with a reciprocal estimate (absolute error about 2e-7, against the reference's sign(y) (1 - e) / (1 + e), e = exp(-2 |y|));
 * and the capping's slope is 1 - tanh^2 instead of max(0, 1 - (soft / cap)^2). Measured on 18432 x 2048 logits capped at 30:
 * row losses within 6e-6 of the FP32 oracle (the three entries: 4e-6), 2e-5 of the 16-bit gradient elements differ from the
 * three entries' in their last bit. 16-bit storage, classes a multiple of 8 and at most 8192, 16-byte aligned rows;
 * GD_ERR_UNSUPPORTED otherwise, with logits untouched (the caller then makes the three calls). */
gd_status gdb200_lm_cross_entropy_fused_rows(gd_backend *backend, const gd_backend_tensor_view *logits, const gd_backend_tensor_view *bias,
                                             const gd_backend_tensor_view *targets, const gd_backend_tensor_view *grad_loss,
                                             const gd_backend_tensor_view *counts, const gd_backend_tensor_view *row_loss, float scale,
                                             float logits_softcap, int32_t ignore_index);

/* gd_backend_sdpa_varlen_backward (src/core/backend.h:699-709) for a caller that still holds the forward output `out`
 * [N, Hq, Dh] and can lend FP32 scratch `dq_accum` of q's element count: D = rowsum(grad_out o out) replaces the
 * query-stationary recomputation, and dK, dV and dQ come from one key-stationary pass (dQ accumulated in dq_accum, then
 * rounded). Needs the forward's statistics (args->use_forward_stats) and head_dim 64; every other case runs exactly
 * as gd_backend_sdpa_varlen_backward. Results agree with it to FP32 rounding of D (out is a rounded tensor). */
gd_status gdb200_sdpa_varlen_backward_with_output(gd_backend *backend, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *q,
                                                  const gd_backend_tensor_view *k, const gd_backend_tensor_view *v,
                                                  const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *out,
                                                  const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k,
                                                  const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *stats,
                                                  const gd_backend_tensor_view *dq_accum, const gd_backend_sdpa_varlen_args *args);
/* The same call for a caller whose next step reads the query gradient in FP32: where the one-pass kernel ran, the rounding
 * pass is skipped, the unrounded gradient stays in dq_accum, grad_q is left untouched and *query_grad_in_accum is 1; in every
 * other case grad_q is written as above and *query_grad_in_accum is 0.
 * gdb200_qkv_split_rope_backward_q32 is gd_backend_qkv_split_rope_backward (src/core/backend.h; src/ops/qkv_split_rope) with the
 * query gradient taken from such an FP32 tensor [N, heads, head_dim] and rounded to the storage type on load: the same bits as
 * the rounding pass followed by the reference entry. Vector path only (half-split rotation of the whole head, head_dim a multiple
 * of 16, 16-byte aligned tensors), GD_ERR_UNSUPPORTED otherwise. */
gd_status gdb200_sdpa_varlen_backward_with_output_q32(gd_backend *backend, const gd_backend_tensor_view *grad_out, const gd_backend_tensor_view *q,
                                                      const gd_backend_tensor_view *k, const gd_backend_tensor_view *v,
                                                      const gd_backend_tensor_view *cu_seqlens, const gd_backend_tensor_view *out,
                                                      const gd_backend_tensor_view *grad_q, const gd_backend_tensor_view *grad_k,
                                                      const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *stats,
                                                      const gd_backend_tensor_view *dq_accum, const gd_backend_sdpa_varlen_args *args,
                                                      int32_t *query_grad_in_accum);
gd_status gdb200_qkv_split_rope_backward_q32(gd_backend *backend, const gd_backend_tensor_view *grad_q_f32, const gd_backend_tensor_view *grad_k,
                                             const gd_backend_tensor_view *grad_v, const gd_backend_tensor_view *pos_ids,
                                             const gd_backend_tensor_view *grad_qkv, uint32_t n_heads, uint32_t head_dim,
                                             const gd_backend_rope_args *args);

/* Weight and bias gradient of a linear layer in one pass over the upstream gradient (no counterpart in the reference,
 * which calls matmul_tn and reduce_rows, src/ops/linear_transposed_weight/core_linear_transposed_weight_bwd.c:31-167):
 * y[M, N] = x^T w with x stored [K, M] and w stored [K, N] (as gd_backend_matmul_tn), and colsum[m] = sum_k x[k, m]
 * (as gd_backend_reduce_rows(x)). Shapes the fused kernel does not take run as those two entries. */
gd_status gdb200_matmul_tn_colsum(gd_backend *backend, const gd_backend_matrix_view *x, const gd_backend_matrix_view *w,
                                  const gd_backend_matrix_view *y, const gd_backend_vector_view *colsum);

/* Embedding table gradient with no allocation (no counterpart in the reference). Same result as
 * gd_backend_embedding_backward, but the FP32 accumulation table is a fixed device array inside the
 * library instead of a caller-provided scratch tensor, for callers that cannot allocate: a runtime
 * whose arenas already own all device memory, or an FFI caller holding only raw device pointers.
 * Pointers are device pointers on the current device; stream is a cudaStream_t or NULL.
 * Limits: vocab * dim <= gdb200_embedding_backward_static_max_elems() (1 Mi floats, 4 MiB resident on
 * every GPU that loads the library), else GD_ERR_INVALID_ARGUMENT with a message from
 * gdb200_embedding_backward_static_error(). Calls share the array: each clears what it uses, and
 * calls that overlap on the GPU race. The first call on a device resolves the array's device
 * address and should be made outside of stream capture. */
gd_status gdb200_embedding_backward_static(void *stream, const void *grad_out, const int32_t *ids, void *grad_table,
                                           uint64_t ids_count, uint64_t vocab, uint64_t dim, uint32_t dtype);
const char *gdb200_embedding_backward_static_error(void);
uint64_t gdb200_embedding_backward_static_max_elems(void);

/* Native sequencing of one gpt_lm training step (no counterpart in the reference's backend ABI; it
 * replays the call sequence of the reference's host: src/train/trainer.c:75-223,
 * examples/gpt_lm/gpt_lm_shared.c:602-823, src/optim/adamw.c:2163-2270). The caller lays out
 * parameters (storage dtype) in params_buffer and, in state_buffer, FP32 masters / m / v per
 * parameter, the AdamW device scalars F32 [5][n_params] and I32 [n_params + 1], the gradient-norm
 * partials (sum of ceil(count / 1024) floats), the clip scale F32[2] and the AMP state F32[2] + I32[3].
 * Parameter order: token_embedding; per block attn_norm_w, qkv w/b, attn_proj w/b, mlp_norm_w,
 * up_gate w/b, down_proj w/b; final_norm_w; lm_head weight (when untied); lm_head_bias.
 * Activations and gradients are bump-allocated from scratch_buffer from offset 0. */
#define GDB200_GPT_MAX_LAYERS 64
#define GDB200_GPT_MAX_PARAMS (1 + 10 * GDB200_GPT_MAX_LAYERS + 3)
typedef struct gdb200_gpt_spec {
    gd_backend_buffer *params_buffer, *state_buffer, *scratch_buffer;
    size_t scratch_bytes;
    int32_t vocab_size, context_length, d_model, n_layers, n_heads, head_dim, mlp_hidden, tied_lm_head;
    int32_t sdpa_window, pad_token_id, lm_ce_chunk, n_params, dp_world;
    uint32_t dtype;
    float dropout_p, logits_softcap, rms_eps, rope_theta;
    uint64_t dropout_seed;
    float adam_beta1, adam_beta2, adam_eps, grad_clip_norm;
    float amp_growth_factor, amp_backoff_factor, amp_min_scale, amp_max_scale;
    uint32_t amp_growth_interval;
    size_t state_f32_offset, state_i32_offset, partials_offset, clip_scale_offset, amp_scale_offset, amp_flags_offset;
    size_t param_offset[GDB200_GPT_MAX_PARAMS], param_count[GDB200_GPT_MAX_PARAMS];
    size_t master_offset[GDB200_GPT_MAX_PARAMS], m_offset[GDB200_GPT_MAX_PARAMS], v_offset[GDB200_GPT_MAX_PARAMS];
    float weight_decay[GDB200_GPT_MAX_PARAMS];
    /* Valid target rows of the GLOBAL batch when this batch is one shard of it and the caller knows the figure;
     * 0 = count the shard and, with a data-parallel communicator attached, sum the counts over the ranks. */
    float global_valid_rows;
} gdb200_gpt_spec;
typedef struct gdb200_gpt_batch {
    gd_backend_buffer *buffer;  /* I32 fields: input ids, targets, positions [n_tokens]; cu_seqlens [n_cu] */
    size_t input_ids_offset, targets_offset, positions_offset, cu_seqlens_offset;
    int64_t n_tokens, n_cu;
} gdb200_gpt_batch;
/* Enqueues forward, backward (loss scaled by the AMP state), gradient exchange when a data-parallel
 * communicator is attached and spec->dp_world > 1, clipping, AdamW and the scaler update. The mean
 * loss (F32 scalar) is left at *loss_offset of scratch_buffer. Under data parallelism the loss and the
 * gradients are those of the GLOBAL batch: every rank divides by the number of valid target rows of all
 * ranks (one scalar all-reduce that overlaps the forward pass), the gradient sum over the ranks needs no
 * further division, and the reported loss is the global mean on every rank. */
gd_status gdb200_gpt_train_step(gd_backend *backend, const gdb200_gpt_spec *spec, const gdb200_gpt_batch *batch,
                                uint64_t step, float lr, size_t *loss_offset, size_t *scratch_used);
/* Scratch-buffer offsets of the parameter gradients the last gdb200_gpt_train_step produced, in parameter order
 * (storage dtype, still multiplied by the loss scale; summed over the ranks under data parallelism). They stay valid
 * until the scratch arena is written again. Returns the number of parameters; at most `capacity` offsets are stored. */
int32_t gdb200_gpt_train_step_grad_offsets(const gd_backend *backend, size_t *offsets, int32_t capacity);

/* Expansion of a batch of compact GPT-LM records on the device. The reference expands each record on a loader
 * thread (examples/gpt_lm/main.c:873-970: u16 tokens[context_length + 1] and the record's I32 segment lengths ->
 * I32 input ids, next-token targets with cross-document targets replaced by pad_id, positions restarting per
 * segment) and its packed-sequence collate generates cu_seqlens from all lengths of the batch
 * (src/dataset/gdds_dataset.c:2191-2224); with this entry a step uploads 2 bytes per token instead of 12.
 * segment_lengths holds the records' length lists one after another and record_offsets[r] the index of record r's
 * first length in it (record_offsets[n_records] = n_segments: the per-sample offsets the reference's collate
 * keeps for a packed-sequence field, gdds_dataset.c:2181-2186). The outputs are the fields of
 * gdb200_gpt_batch (n_tokens = n_records * context_length, n_cu = n_segments + 1). Input the reference's transform
 * rejects with GD_ERR_INVALID_ARGUMENT is reported asynchronously: *status (I32 in the buffer) receives 0 or
 * GDB200_COMPACT_* flags, the outputs are then unspecified but stay inside their ranges. */
enum {
    GDB200_COMPACT_BAD_TOKEN = 1,   /* a token id >= vocab_size (main.c:934-939) */
    GDB200_COMPACT_BAD_LENGTH = 2,  /* a segment length <= 0 (main.c:946) */
    GDB200_COMPACT_BAD_COVER = 4    /* the lengths of a record do not add up to context_length (main.c:946,957) */
};
typedef struct gdb200_gpt_compact_batch {
    gd_backend_buffer *buffer;
    size_t tokens_offset;           /* in:  U16 [n_records, context_length + 1] */
    size_t segment_lengths_offset;  /* in:  I32 [n_segments] */
    size_t record_offsets_offset;   /* in:  I32 [n_records + 1] */
    size_t input_ids_offset, targets_offset, positions_offset;  /* out: I32 [n_records * context_length] */
    size_t cu_seqlens_offset;       /* out: I32 [n_segments + 1] */
    size_t status_offset;           /* out: I32 */
    int64_t n_records, n_segments;
    int32_t context_length, vocab_size, pad_id, im_start_id, im_end_id;
} gdb200_gpt_compact_batch;
gd_status gdb200_gpt_compact_expand(gd_backend *backend, const gdb200_gpt_compact_batch *batch);

/* Device-side greedy sampling (no counterpart in the reference's backend ABI: the reference downloads
 * the logits and samples on the host, examples/gpt_lm/gpt_lm_shared.c:1322,1371-1442). logits [rows,
 * classes] F16/BF16/F32; softcap > 0 applies cap * tanh(x / cap) first; non-finite values count as
 * -inf; the FIRST maximum wins (:1393). out_ids: I32 [rows]. */
gd_status gdb200_argmax_rows(gd_backend *backend, const gd_backend_tensor_view *logits, float softcap,
                             const gd_backend_tensor_view *out_ids);

/* Greedy KV-cache decode with the token feedback kept on the device (replays gpt_block_decode_cached,
 * examples/gpt_lm/gpt_lm_shared.c:961-1115,1204-1246, and the argmax rule of :1388-1398).
 * cache_buffer holds per layer K and V caches [batch, capacity, n_heads, head_dim] in the storage
 * dtype. io_buffer holds I32 words: tokens [batch] (ids fed to the next step, replaced by each step's
 * argmax), positions [batch] (cache slot / rotary position of that id, incremented by each step),
 * out_tokens [max_steps, batch] and one step counter (the row of out_tokens the next step writes;
 * steps beyond max_steps are not recorded). Only spec's model fields, params_buffer / param_offset,
 * scratch_buffer and scratch_bytes are used. */
typedef struct gdb200_gpt_decode_state {
    gd_backend_buffer *cache_buffer, *io_buffer;
    size_t k_cache_offset[GDB200_GPT_MAX_LAYERS], v_cache_offset[GDB200_GPT_MAX_LAYERS];
    size_t tokens_offset, positions_offset, out_tokens_offset, step_counter_offset;
    int32_t batch, capacity, max_steps;
} gdb200_gpt_decode_state;
/* Enqueues n_steps decode steps without any host synchronisation. use_graph == 0: one launch per operation, step after
 * step. use_graph != 0: where the shapes allow (16-bit storage, at most 64 sequences, head_dim 64, d_model 128 / 256 / 512,
 * mlp_hidden a multiple of 128, the cos / sin table of the rotation in use) ALL steps run in one persistent cooperative
 * kernel (one CTA per SM in clusters of two, grid barriers between the phases of a step; a barrier that is not reached within
 * its bounded wait stores code 398 in the error word and ends the kernel); otherwise the first step runs eagerly, the second is
 * recorded as a CUDA graph and the rest replay it. The three forms generate the same ids. */
gd_status gdb200_gpt_decode_steps(gd_backend *backend, const gdb200_gpt_spec *spec, const gdb200_gpt_decode_state *state,
                                  int32_t n_steps, int32_t use_graph, size_t *scratch_used);

/* Failure detection without a fault (the reference reports a failed command buffer as GD_ERR_INTERNAL at flush,
 * src/backends/metal/backend_metal.m:569-573; here every device-side wait is bounded and reports through an error word
 * that flush / fence_wait read). gdb200_inject_device_error stores `code` in that word in stream order;
 * gdb200_selftest_bounded_wait runs a one-warp kernel that polls an mbarrier nobody arrives at for at most max_iters
 * (<= 2^20) iterations, stores code 399 and returns. After either, gd_backend_flush returns GD_ERR_INTERNAL once,
 * gdb200_last_error names the code, and the backend stays usable. */
gd_status gdb200_inject_device_error(gd_backend *backend, int32_t code);
gd_status gdb200_selftest_bounded_wait(gd_backend *backend, uint32_t max_iters);

/* Data-parallel gradient exchange (the reference has no collective; one process per GPU).
 * id_bytes is the 128-byte ncclUniqueId produced by gdb200_dp_unique_id on rank 0. */
gd_status gdb200_dp_unique_id(void *id_bytes_128);
gd_status gdb200_dp_init(gd_backend *backend, const void *id_bytes_128, int rank, int world);
/* In-place sum all-reduce of `count` elements of dtype (F16/BF16/F32) on the comm stream,
 * ordered after everything already enqueued on the compute stream. */
gd_status gdb200_dp_all_reduce(gd_backend *backend, gd_backend_buffer *buffer, size_t offset, size_t count, uint32_t dtype);
/* Make the compute stream wait for all outstanding all-reduces. Polls the communicator's asynchronous error state
 * (GD_ERR_INTERNAL when it reports one); with GDB200_DP_TIMEOUT_MS > 0 in the environment the host also waits, at most
 * that long, for the collectives to complete and returns GD_ERR_INTERNAL when they do not (a peer that never joined). */
gd_status gdb200_dp_join(gd_backend *backend);
/* The polling loop behind that wait, with the two queries as callbacks (completed: 1 = done; failed: non-zero = the
 * communicator reports an error) so that it can be exercised without a GPU. *reason: 0 ok, 1 error reported, 2 timeout. */
gd_status gdb200_dp_wait_with(int (*completed)(void *), int (*failed)(void *), void *user, uint32_t timeout_ms, int32_t *reason);
void gdb200_dp_shutdown(gd_backend *backend);

#ifdef __cplusplus
}
#endif

#endif /* GD_BACKEND_B200_H */
