// Native sequencing of one gpt_lm training step over the backend entries (host code only).
//
// The reference drives a training step from C (src/train/trainer.c:75-223 ->
// examples/gpt_lm/gpt_lm_shared.c:602-823 -> op capsules -> tape backward -> src/optim/adamw.c:2163);
// a Python host issuing the same ~170 backend calls per step costs more host time than the B200
// needs to execute them. This file issues exactly the same gd_backend_* call sequence as
// host/gpt_lm.py + host/ops.py + host/optim.py (same scratch tensors, same rounding points, same
// gradient-accumulation order), with a bump allocator over the caller's scratch buffer, so the two
// hosts are interchangeable and are checked against each other in the tests. Parameters, optimizer
// state and the AMP scaler state are laid out by the caller and described by gdb200_gpt_spec.
//
// With a data-parallel communicator attached (gdb200_dp_init) all parameter gradients are allocated as
// one contiguous range and summed across ranks with ONE all-reduce after the backward pass (or, with
// GDB200_DP_OVERLAP=1, one per block as soon as the block's backward has been enqueued). The loss is
// normalised by the number of valid target rows of ALL ranks (counted and all-reduced at the start of
// the step), so the summed gradients are those of the global batch without a division by the world size.
#include "common.cuh"
#include "decode_parts.cuh"

#include <math.h>
#include <stdlib.h>
#include <algorithm>
#include <utility>
#include <vector>

namespace {

struct Ten {
    gd_backend_buffer *buf;
    size_t off;
    uint32_t dt;
    uint32_t rank;
    int64_t shape[4];
    size_t count() const
    {
        size_t n = 1;
        for (uint32_t i = 0; i < rank; ++i) n *= (size_t)shape[i];
        return n;
    }
};

gd_backend_tensor_view tv(const Ten &t)
{
    gd_backend_tensor_view v;
    memset(&v, 0, sizeof(v));
    v.buffer = t.buf;
    v.offset = t.off;
    v.count = t.count();
    v.dtype = t.dt;
    v.rank = t.rank;
    int64_t stride = 1;
    for (int d = (int)t.rank - 1; d >= 0; --d) {
        v.shape[d] = t.shape[d];
        v.strides[d] = stride;
        stride *= t.shape[d];
    }
    return v;
}

gd_backend_matrix_view mv(const Ten &t, uint32_t rows, uint32_t cols, size_t row_offset = 0)
{
    gd_backend_matrix_view v;
    const size_t es = gdb_dtype_size(t.dt);
    v.buffer = t.buf;
    v.row_bytes = (size_t)cols * es;
    v.offset = t.off + row_offset * v.row_bytes;
    v.rows = rows;
    v.cols = cols;
    v.dtype = t.dt;
    return v;
}

gd_backend_vector_view vv(const Ten &t, size_t start, uint32_t length)
{
    gd_backend_vector_view v;
    v.buffer = t.buf;
    v.offset = t.off + start * gdb_dtype_size(t.dt);
    v.length = length;
    v.dtype = t.dt;
    return v;
}

uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}

constexpr uint64_t SITE_EMBED = 0x9E3779B97F4A7C15ULL, SITE_ATTN = 0xBF58476D1CE4E5B9ULL, SITE_MLP = 0x94D049BB133111EBULL;

struct Step {
    gd_backend *be;
    const gdb200_gpt_spec *s;
    size_t top;
    gd_status st;
    const char *where;

    Ten alloc(uint32_t dt, std::initializer_list<int64_t> shape, size_t align = 256)
    {
        Ten t;
        memset(&t, 0, sizeof(t));
        t.buf = s->scratch_buffer;
        t.dt = dt;
        t.rank = (uint32_t)shape.size();
        int i = 0;
        for (int64_t d : shape) t.shape[i++] = d;
        const size_t bytes = (t.count() == 0 ? 1 : t.count()) * gdb_dtype_size(dt);
        const size_t off = (top + align - 1) & ~(align - 1);
        if (off + bytes > s->scratch_bytes) {
            if (st == GD_OK) {
                st = GD_ERR_OUT_OF_MEMORY;
                where = "scratch arena";
            }
            t.off = 0;
            return t;
        }
        t.off = off;
        top = off + bytes;
        return t;
    }
    bool ok(gd_status r, const char *what)
    {
        if (r != GD_OK && st == GD_OK) {
            st = r;
            where = what;
        }
        return st == GD_OK;
    }
    Ten param(int idx, std::initializer_list<int64_t> shape) const
    {
        Ten t;
        memset(&t, 0, sizeof(t));
        t.buf = s->params_buffer;
        t.off = s->param_offset[idx];
        t.dt = s->dtype;
        t.rank = (uint32_t)shape.size();
        int i = 0;
        for (int64_t d : shape) t.shape[i++] = d;
        return t;
    }
    Ten fill(Ten t, uint32_t pattern)
    {
        ok(gd_backend_fill(be, t.buf, t.off, t.count(), gdb_dtype_size(t.dt), pattern), "fill");
        return t;
    }
    // dst += src with the storage rounding after the add (gradient accumulation)
    void accumulate(const Ten &dst, const Ten &src) { ok(gd_backend_accumulate(be, dst.buf, dst.off, src.buf, src.off, src.count(), src.dt), "accumulate"); }
};

gd_backend_rms_norm_args rms_args(int64_t rows, int64_t cols, float eps)
{
    gd_backend_rms_norm_args a;
    memset(&a, 0, sizeof(a));
    const uint64_t rb = rows >= 4096 ? 128U : 64U;  // src/ops/rms_norm/core_rms_norm.c:9-11
    a.rows = (uint64_t)rows;
    a.cols = (uint64_t)cols;
    a.row_blocks = ((uint64_t)rows + rb - 1U) / rb;
    a.eps = eps;
    a.simdgroups = 8;
    a.wgrad_simdgroups = 8;
    a.wgrad_row_block = (uint32_t)rb;
    return a;
}

struct LayerSave {
    Ten x, normed, inv1, qkv, q, k, v, stats, attn, mask1, resid, normed2, inv2, up_gate, act, mask2;
};

// y = x w^T + b (fused, reference rounding), w stored [n, k]
Ten linear_t(Step &c, const Ten &x, const Ten &w, const Ten &b, int64_t m, int64_t k, int64_t n)
{
    Ten y = c.alloc(x.dt, {m, n});
    gd_backend_matrix_view xm = mv(x, (uint32_t)m, (uint32_t)k), wm = mv(w, (uint32_t)n, (uint32_t)k), ym = mv(y, (uint32_t)m, (uint32_t)n);
    gd_backend_vector_view bv = vv(b, 0, (uint32_t)n);
    c.ok(gdb200_matmul_nt_bias(c.be, &xm, &wm, &bv, &ym), "matmul_nt_bias");
    return y;
}

// backward of y = x w^T + b: dx = g w, dw = g^T x, db = colsum(g)
void linear_t_backward(Step &c, const Ten &x, const Ten &w, const Ten &g, int64_t m, int64_t k, int64_t n, Ten *dx, const Ten &dw, const Ten &db)
{
    gd_backend_matrix_view gm = mv(g, (uint32_t)m, (uint32_t)n), wm = mv(w, (uint32_t)n, (uint32_t)k), xm = mv(x, (uint32_t)m, (uint32_t)k);
    if (dx != NULL) {
        *dx = c.alloc(x.dt, {m, k});
        gd_backend_matrix_view dxm = mv(*dx, (uint32_t)m, (uint32_t)k);
        c.ok(gd_backend_matmul(c.be, &gm, &wm, &dxm), "matmul(dX)");
    }
    // dW = g^T x and db = colsum(g) from one pass over g
    gd_backend_matrix_view dwm = mv(dw, (uint32_t)n, (uint32_t)k);
    gd_backend_vector_view dbv = vv(db, 0, (uint32_t)n);
    c.ok(gdb200_matmul_tn_colsum(c.be, &gm, &xm, &dwm, &dbv), "matmul_tn_colsum(dW, db)");
}

Ten rms_forward(Step &c, const Ten &x, const Ten &w, int64_t rows, int64_t cols, Ten *inv)
{
    gd_backend_rms_norm_args a = rms_args(rows, cols, c.s->rms_eps);
    Ten out = c.alloc(x.dt, {rows, cols});
    *inv = c.alloc(GDB_DTYPE_F32, {rows});
    gd_backend_tensor_view xv = tv(x), wv = tv(w), ov = tv(out), iv = tv(*inv);
    c.ok(gd_backend_rms_norm_forward_stats(c.be, &xv, &wv, &ov, &iv, &a), "rms_norm_forward_stats");
    return out;
}

// `accum` != NULL: the input gradient is added into *accum (rounded, then added, then rounded: the two calls
// rms_norm_backward_stats + accumulate in one launch) and *accum is returned.
Ten dropout_mask_backward(Step &c, const Ten &mask, const Ten &g, float scale);

// dx (accumulated into *accum when given) and the weight gradient of an RMSNorm; with `mask`, *dropped = the gradient of the
// dropped branch that feeds the same residual stream, dropout_backward_mask(mask, dx, scale), and with `dropped_colsum` its
// sum over the rows (the bias gradient of the branch's last projection), from the same launch where the one-pass kernel takes
// the shape (separate launches otherwise).
Ten rms_backward(Step &c, const Ten &x, const Ten &w, const Ten &inv, const Ten &g, int64_t rows, int64_t cols, const Ten &dw,
                 const Ten *accum = nullptr, const Ten *mask = nullptr, float mask_scale = 1.0f, Ten *dropped = nullptr,
                 const Ten *dropped_colsum = nullptr)
{
    gd_backend_rms_norm_args a = rms_args(rows, cols, c.s->rms_eps);
    Ten dx = accum != nullptr ? *accum : c.alloc(x.dt, {rows, cols});
    gd_backend_tensor_view xv = tv(x), wv = tv(w), iv = tv(inv), gv = tv(g), dxv = tv(dx), dwv = tv(dw);
    if (mask != nullptr) {
        // GDB200_RMS_BWD_DROPOUT=0: the dropout backward stays a launch of its own
        static const bool fuse_mask = !(getenv("GDB200_RMS_BWD_DROPOUT") != NULL && getenv("GDB200_RMS_BWD_DROPOUT")[0] == '0');
        static const bool split = getenv("GDB200_RMS_BWD_SPLIT") != NULL;
        if (fuse_mask && !split && c.st == GD_OK) {
            const size_t mark = c.top;
            Ten out = dropped->buf != NULL ? *dropped : c.alloc(x.dt, {rows, cols});   // the caller's buffer when it has one
            const int64_t prow = std::max<int64_t>((int64_t)a.row_blocks, 2 * (int64_t)c.be->sm_count);
            Ten partial = c.alloc(GDB_DTYPE_F32, {prow, cols});
            gd_backend_tensor_view pv = tv(partial), mv8 = tv(*mask), ov = tv(out), csv;
            if (dropped_colsum != nullptr) csv = tv(*dropped_colsum);
            gd_status r = gdb_rms_norm_backward_with_weight(c.be, &xv, &wv, &iv, &gv, &dxv, accum != nullptr, &dwv, &pv, &a, &mv8, &ov, mask_scale,
                                                            dropped_colsum != nullptr ? &csv : NULL);
            if (r != GD_ERR_UNSUPPORTED) {
                c.ok(r, "rms_norm_backward + weight gradient + dropout backward");
                *dropped = out;
                return dx;
            }
            c.top = mark;
        }
        Ten plain = rms_backward(c, x, w, inv, g, rows, cols, dw, accum);
        if (dropped->buf != NULL) {
            gd_backend_tensor_view mvw = tv(*mask), pv = tv(plain), dv = tv(*dropped);
            c.ok(gd_backend_dropout_backward_mask(c.be, &mvw, &pv, &dv, mask_scale), "dropout_backward_mask");
        } else {
            *dropped = dropout_mask_backward(c, *mask, plain, mask_scale);
        }
        if (dropped_colsum != nullptr) {
            gd_backend_matrix_view gm = mv(*dropped, (uint32_t)rows, (uint32_t)cols);
            gd_backend_vector_view dbv = vv(*dropped_colsum, 0, (uint32_t)cols);
            c.ok(gd_backend_reduce_rows(c.be, &gm, &dbv), "reduce_rows(dropped gradient)");
        }
        return plain;
    }
    {
        // input and weight gradient from one pass over x and g where the fused kernel takes the shape (GDB200_RMS_BWD_SPLIT=1: two passes)
        static const bool split = getenv("GDB200_RMS_BWD_SPLIT") != NULL;
        if (!split && c.st == GD_OK) {
            const int64_t prow = std::max<int64_t>((int64_t)a.row_blocks, 2 * (int64_t)c.be->sm_count);
            Ten partial = c.alloc(GDB_DTYPE_F32, {prow, cols});
            gd_backend_tensor_view pv = tv(partial);
            gd_status r = gdb_rms_norm_backward_with_weight(c.be, &xv, &wv, &iv, &gv, &dxv, accum != nullptr, &dwv, &pv, &a, NULL, NULL, 1.0f, NULL);
            if (r != GD_ERR_UNSUPPORTED) {
                c.ok(r, "rms_norm_backward + weight gradient");
                return dx;
            }
        }
    }
    if (accum != nullptr) {
        c.ok(gdb_rms_norm_backward_accumulate(c.be, &xv, &wv, &iv, &gv, &dxv, &a), "rms_norm_backward_stats + accumulate");
    } else {
        c.ok(gd_backend_rms_norm_backward_stats(c.be, &xv, &wv, &iv, &gv, &dxv, &a), "rms_norm_backward_stats");
    }
    Ten partial = c.alloc(GDB_DTYPE_F32, {(int64_t)a.row_blocks, cols});
    gd_backend_tensor_view pv = tv(partial);
    c.ok(gd_backend_rms_norm_weight_backward_stats(c.be, &xv, &iv, &gv, &dwv, &pv, &a), "rms_norm_weight_backward_stats");
    return dx;
}

Ten dropout_mask_backward(Step &c, const Ten &mask, const Ten &g, float scale)
{
    Ten dx = c.alloc(g.dt, {g.shape[0], g.shape[1]});
    gd_backend_tensor_view mvw = tv(mask), gv = tv(g), dv = tv(dx);
    c.ok(gd_backend_dropout_backward_mask(c.be, &mvw, &gv, &dv, scale), "dropout_backward_mask");
    return dx;
}

}  // namespace

extern "C" gd_status gdb200_gpt_train_step(gd_backend *be, const gdb200_gpt_spec *s, const gdb200_gpt_batch *batch,
                                           uint64_t step, float lr, size_t *loss_offset, size_t *scratch_used)
{
    if (be == NULL || s == NULL || batch == NULL || loss_offset == NULL || s->n_layers <= 0 || s->n_layers > GDB200_GPT_MAX_LAYERS ||
        batch->n_tokens <= 0 || s->n_heads * s->head_dim != s->d_model) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    Step c;
    c.be = be;
    c.s = s;
    c.top = 0;
    c.st = GD_OK;
    c.where = "";
    const int64_t T = batch->n_tokens, D = s->d_model, F = s->mlp_hidden, V = s->vocab_size, H = s->n_heads, Dh = s->head_dim;
    const int L = s->n_layers;
    const uint32_t dt = s->dtype;
    const bool drop = s->dropout_p > 0.0f;
    const float drop_scale = 1.0f / (1.0f - s->dropout_p);
    const int P_FINAL = 1 + 10 * L, P_LMW = s->tied_lm_head ? 0 : P_FINAL + 1, P_LMB = P_FINAL + (s->tied_lm_head ? 1 : 2);
    const int n_params = P_LMB + 1;
    if (n_params != s->n_params) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    auto data_tensor = [&](size_t off, int64_t n) {
        Ten t;
        memset(&t, 0, sizeof(t));
        t.buf = batch->buffer;
        t.off = off;
        t.dt = GDB_DTYPE_I32;
        t.rank = 1;
        t.shape[0] = n;
        return t;
    };
    const Ten ids = data_tensor(batch->input_ids_offset, T), tgt = data_tensor(batch->targets_offset, T);
    const Ten pos = data_tensor(batch->positions_offset, T), cu = data_tensor(batch->cu_seqlens_offset, batch->n_cu);
    auto seed_of = [&](uint64_t site, uint64_t layer) { return splitmix64(s->dropout_seed ^ site ^ (layer << 32) ^ step); };

    // ---- AMP scaler: clamp the scale, clear found_inf (first use of the step) ----
    gd_backend_amp_state_desc amp;
    memset(&amp, 0, sizeof(amp));
    amp.scale_buffer = s->state_buffer;
    amp.scale_offset = s->amp_scale_offset;
    amp.flags_buffer = s->state_buffer;
    amp.flags_offset = s->amp_flags_offset;
    amp.growth_factor = s->amp_growth_factor;
    amp.backoff_factor = s->amp_backoff_factor;
    amp.min_scale = s->amp_min_scale;
    amp.max_scale = s->amp_max_scale;
    amp.growth_interval = s->amp_growth_interval;

    // ---- loss normaliser of a sharded batch: the number of valid target rows of the GLOBAL batch ----
    // Known from the targets alone, so it is counted and summed over the ranks first and the collective
    // hides behind the forward pass. A caller that knows the figure passes it in spec->global_valid_rows.
    const bool dp = be->dp != NULL && s->dp_world > 1;
    const bool global_norm = dp || s->global_valid_rows > 0.0f;
    Ten counts;
    memset(&counts, 0, sizeof(counts));
    if (global_norm) {
        counts = c.alloc(GDB_DTYPE_F32, {2});
        gd_backend_tensor_view tgv0 = tv(tgt), cv0 = tv(counts);
        c.ok(gdb_lm_ce_count_valid(be, &tgv0, s->pad_token_id, &cv0), "lm_ce_count_valid");
        if (s->global_valid_rows > 0.0f) {
            uint32_t bits;
            memcpy(&bits, &s->global_valid_rows, sizeof(bits));
            c.ok(gd_backend_fill(be, counts.buf, counts.off, 1, sizeof(float), bits), "fill(global rows)");
        } else {
            c.ok(gdb200_dp_all_reduce(be, counts.buf, counts.off, 1, GDB_DTYPE_F32), "dp_all_reduce(valid rows)");
        }
    }

    // ---------------------------------------------------------------- forward
    const Ten emb_w = c.param(0, {V, D});
    gd_backend_embedding_args ea = {(uint64_t)T, (uint64_t)V, (uint64_t)D};
    Ten x, emb_mask, next_normed, next_inv;
    bool have_next_norm = false;   // the norm in front of the next block came out of the launch that formed its input
    memset(&emb_mask, 0, sizeof(emb_mask));
    bool embedded = false;
    if (drop && L > 0 && c.st == GD_OK) {
        // embedding gather, its dropout and the first block's norm in one launch where the fused kernel takes the shape
        // (GDB200_FUSE_EMBED=0: the three entries)
        static const bool fuse_embed = !(getenv("GDB200_FUSE_EMBED") != NULL && getenv("GDB200_FUSE_EMBED")[0] == '0');
        const size_t mark = c.top;
        x = c.alloc(dt, {T, D});
        emb_mask = c.alloc(GDB_DTYPE_U8, {T, D});
        Ten nrm = c.alloc(dt, {T, D}), iv = c.alloc(GDB_DTYPE_F32, {T});
        const Ten w0 = c.param(1, {D});
        gd_backend_tensor_view a = tv(emb_w), b = tv(ids), wv = tv(w0), y = tv(x), m = tv(emb_mask), nv = tv(nrm), ivv = tv(iv);
        const gd_status st = fuse_embed ? gdb_embedding_dropout_rms_norm(be, &a, &b, &wv, &y, &m, &nv, &ivv, (size_t)T, (size_t)D, (size_t)V, s->rms_eps,
                                                                         s->dropout_p, splitmix64(s->dropout_seed ^ SITE_EMBED ^ step))
                                        : GD_ERR_UNSUPPORTED;
        if (st == GD_OK) {
            next_normed = nrm;
            next_inv = iv;
            have_next_norm = true;
            embedded = true;
        } else {
            if (st != GD_ERR_UNSUPPORTED) c.ok(st, "embedding + dropout + rms_norm");
            c.top = mark;
        }
    }
    if (!embedded) {
        Ten x0 = c.alloc(dt, {T, D});
        {
            gd_backend_tensor_view a = tv(emb_w), b = tv(ids), o = tv(x0);
            c.ok(gd_backend_embedding_forward(be, &a, &b, &o, &ea), "embedding_forward");
        }
        x = x0;
        if (drop) {
            x = c.alloc(dt, {T, D});
            emb_mask = c.alloc(GDB_DTYPE_U8, {T, D});
            gd_backend_tensor_view a = tv(x0), y = tv(x), m = tv(emb_mask);
            c.ok(gd_backend_dropout_forward(be, &a, &y, &m, s->dropout_p, splitmix64(s->dropout_seed ^ SITE_EMBED ^ step)), "dropout_forward");
        }
    }
    std::vector<LayerSave> saves((size_t)L);
    gd_backend_rope_args rope = {s->rope_theta, (uint32_t)Dh, 0U};
    gd_backend_sdpa_varlen_args sa;
    memset(&sa, 0, sizeof(sa));
    sa.scale = (float)(1.0 / sqrt((double)Dh));
    sa.causal = 1;
    sa.sliding_window = (uint32_t)s->sdpa_window;
    sa.max_seqlen = (uint32_t)s->context_length;
    // sum = residual + dropout(y) and normed = rms_norm(sum, w) (inv_rms saved): one launch when the fused kernel takes the
    // shape, else dropout_add_forward (or add) followed by rms_norm_forward_stats
    auto residual_then_norm = [&](const Ten &residual, const Ten &y, const Ten &w, uint64_t seed, Ten *sum, Ten *mask, Ten *normed, Ten *inv) {
        *sum = c.alloc(dt, {T, D});
        memset(mask, 0, sizeof(*mask));
        if (drop) {
            *mask = c.alloc(GDB_DTYPE_U8, {T, D});
            Ten nrm = c.alloc(dt, {T, D}), iv = c.alloc(GDB_DTYPE_F32, {T});
            gd_backend_tensor_view r = tv(residual), a = tv(y), wv = tv(w), sv_ = tv(*sum), m = tv(*mask), nv = tv(nrm), ivv = tv(iv);
            gd_status st = c.st == GD_OK ? gdb_dropout_add_rms_norm(be, &r, &a, &wv, &sv_, &m, &nv, &ivv, (size_t)T, (size_t)D, s->rms_eps, s->dropout_p, seed)
                                         : GD_ERR_UNSUPPORTED;
            if (st == GD_OK) {
                *normed = nrm;
                *inv = iv;
                return;
            }
            if (st != GD_ERR_UNSUPPORTED) {
                c.ok(st, "dropout_add + rms_norm");
            }
            c.ok(gd_backend_dropout_add_forward(be, &r, &a, &sv_, &m, s->dropout_p, seed), "dropout_add_forward");
        } else {
            gd_backend_tensor_view r = tv(residual), a = tv(y), sv_ = tv(*sum);
            c.ok(gd_backend_add(be, &r, &a, &sv_), "add");
        }
        *normed = rms_forward(c, *sum, w, T, D, inv);
    };
    for (int i = 0; i < L && c.st == GD_OK; ++i) {
        LayerSave &sv = saves[(size_t)i];
        const int pb = 1 + 10 * i;
        sv.x = x;
        if (have_next_norm) {
            sv.normed = next_normed;   // produced together with the previous block's residual add
            sv.inv1 = next_inv;
        } else {
            sv.normed = rms_forward(c, x, c.param(pb + 0, {D}), T, D, &sv.inv1);
        }
        sv.qkv = linear_t(c, sv.normed, c.param(pb + 1, {3 * D, D}), c.param(pb + 2, {3 * D}), T, D, 3 * D);
        sv.q = c.alloc(dt, {T, H, Dh});
        sv.k = c.alloc(dt, {T, H, Dh});
        sv.v = c.alloc(dt, {T, H, Dh});
        {
            gd_backend_tensor_view a = tv(sv.qkv), p = tv(pos), q = tv(sv.q), k = tv(sv.k), v = tv(sv.v);
            c.ok(gd_backend_qkv_split_rope_forward(be, &a, &p, &q, &k, &v, (uint32_t)H, (uint32_t)Dh, &rope), "qkv_split_rope_forward");
        }
        sv.attn = c.alloc(dt, {T, D});
        sv.stats = c.alloc(GDB_DTYPE_F32, {T, H, 3});
        {
            Ten attn3 = sv.attn;
            attn3.rank = 3;
            attn3.shape[0] = T;
            attn3.shape[1] = H;
            attn3.shape[2] = Dh;
            gd_backend_tensor_view q = tv(sv.q), k = tv(sv.k), v = tv(sv.v), cv = tv(cu), o = tv(attn3), stv = tv(sv.stats);
            sa.use_forward_stats = 0;
            c.ok(gd_backend_sdpa_varlen(be, &q, &k, &v, &cv, &o, &stv, &sa), "sdpa_varlen");
        }
        Ten proj = linear_t(c, sv.attn, c.param(pb + 3, {D, D}), c.param(pb + 4, {D}), T, D, D);
        memset(&sv.mask2, 0, sizeof(sv.mask2));
        residual_then_norm(x, proj, c.param(pb + 5, {D}), seed_of(SITE_ATTN, (uint64_t)i), &sv.resid, &sv.mask1, &sv.normed2, &sv.inv2);
        // up / gate projection and the SwiGLU gate: one contraction whose epilogue writes both (same bits as the three calls)
        sv.up_gate = c.alloc(dt, {T, 2 * F});
        sv.act = c.alloc(dt, {T, F});
        {
            const Ten w = c.param(pb + 6, {2 * F, D}), b = c.param(pb + 7, {2 * F});
            gd_backend_matrix_view xm = mv(sv.normed2, (uint32_t)T, (uint32_t)D), wm = mv(w, (uint32_t)(2 * F), (uint32_t)D);
            gd_backend_matrix_view um = mv(sv.up_gate, (uint32_t)T, (uint32_t)(2 * F)), am = mv(sv.act, (uint32_t)T, (uint32_t)F);
            gd_backend_vector_view bv = vv(b, 0, (uint32_t)(2 * F));
            c.ok(gdb200_matmul_nt_bias_swiglu_both(be, &xm, &wm, &bv, &um, &am), "matmul_nt_bias + swiglu_split");
        }
        Ten mlp = c.alloc(dt, {T, D});
        {
            const Ten w = c.param(pb + 8, {F, D}), b = c.param(pb + 9, {D});
            gd_backend_matrix_view am = mv(sv.act, (uint32_t)T, (uint32_t)F), wm = mv(w, (uint32_t)F, (uint32_t)D), ym = mv(mlp, (uint32_t)T, (uint32_t)D);
            gd_backend_vector_view bv = vv(b, 0, (uint32_t)D);
            c.ok(gd_backend_linear(be, &am, &wm, &bv, &ym), "linear(down_proj)");
        }
        // the norm that consumes this block's output: the next block's attention norm, or the final norm
        Ten out;
        residual_then_norm(sv.resid, mlp, i + 1 < L ? c.param(1 + 10 * (i + 1), {D}) : c.param(P_FINAL, {D}), seed_of(SITE_MLP, (uint64_t)i), &out,
                           &sv.mask2, &next_normed, &next_inv);
        have_next_norm = true;
        x = out;
    }
    const Ten final_w = c.param(P_FINAL, {D});
    Ten inv_f, final_norm;
    if (have_next_norm) {
        final_norm = next_normed;
        inv_f = next_inv;
    } else {
        final_norm = rms_forward(c, x, final_w, T, D, &inv_f);
    }

    // ---- fused LM cross entropy (chunked over the vocabulary, src/ops/lm_cross_entropy/core_lm_cross_entropy.c:452-675) ----
    const Ten lm_w = c.param(P_LMW, {V, D}), lm_b = c.param(P_LMB, {V});
    Ten row_loss = c.alloc(GDB_DTYPE_F32, {T}), row_max = c.alloc(GDB_DTYPE_F32, {T});
    Ten row_inv_sum = c.alloc(GDB_DTYPE_F32, {T}), row_valid = c.alloc(GDB_DTYPE_F32, {T});
    Ten inv_valid = c.alloc(GDB_DTYPE_F32, {});
    Ten loss = c.alloc(GDB_DTYPE_F32, {});
    const int64_t chunk = s->lm_ce_chunk > 0 && s->lm_ce_chunk < V ? s->lm_ce_chunk : V;
    const bool single = chunk >= V;
    Ten saved_logits;
    memset(&saved_logits, 0, sizeof(saved_logits));
    gd_backend_tensor_view tgv = tv(tgt), rlv = tv(row_loss), rmv = tv(row_max), rsv = tv(row_inv_sum), rvv = tv(row_valid), ivv = tv(inv_valid), lov = tv(loss);
    // One chunk holding all classes: loss statistics and logits gradient come from ONE pass over the logits
    // (gdb200_lm_cross_entropy_fused_rows), which needs the gradient seed (the loss scale) and the number of valid rows
    // before the loss exists; both are known here. GDB200_LMCE_FUSED=0 keeps online update + finalize + backward chunk.
    static int lmce_fused = -1;
    if (lmce_fused < 0) {
        const char *env = getenv("GDB200_LMCE_FUSED");
        lmce_fused = (env != NULL && env[0] == '0') ? 0 : 1;
    }
    bool fused_ce = false;
    Ten seed;
    memset(&seed, 0, sizeof(seed));
    if (single && lmce_fused != 0) {
        if (!global_norm) {
            counts = c.alloc(GDB_DTYPE_F32, {2});
            gd_backend_tensor_view cv0 = tv(counts);
            c.ok(gdb_lm_ce_count_valid(be, &tgv, s->pad_token_id, &cv0), "lm_ce_count_valid");
        }
        c.ok(gd_backend_amp_begin_step(be, &amp), "amp_begin_step");
        seed = c.alloc(GDB_DTYPE_F32, {});
        c.ok(gd_backend_amp_fill_scale(be, seed.buf, seed.off, 1, GDB_DTYPE_F32, s->state_buffer, s->amp_scale_offset), "amp_fill_scale");
        Ten logits = c.alloc(dt, {T, V});
        gd_backend_matrix_view hm = mv(final_norm, (uint32_t)T, (uint32_t)D), wm = mv(lm_w, (uint32_t)V, (uint32_t)D), lm = mv(logits, (uint32_t)T, (uint32_t)V);
        c.ok(gd_backend_matmul_nt(be, &hm, &wm, &lm), "matmul_nt(logits)");
        saved_logits = logits;
        if (c.st == GD_OK) {
            if (dp && !(s->global_valid_rows > 0.0f)) c.ok(gdb200_dp_join(be), "dp_join(valid rows)");
            gd_backend_tensor_view lv = tv(logits), bv = tv(lm_b), sdv = tv(seed), cv1 = tv(counts);
            const gd_status fst = gdb200_lm_cross_entropy_fused_rows(be, &lv, &bv, &tgv, &sdv, &cv1, &rlv, 1.0f, s->logits_softcap, s->pad_token_id);
            if (fst == GD_OK) {
                fused_ce = true;
                c.ok(gdb_lm_ce_reduce_normalize_global(be, &rlv, &cv1, &lov, &ivv), "lm_ce_reduce_normalize(rows)");
                if (dp) c.ok(gdb200_dp_all_reduce(be, loss.buf, loss.off, 1, GDB_DTYPE_F32), "dp_all_reduce(loss)");
            } else if (fst != GD_ERR_UNSUPPORTED) {
                c.ok(fst, "lm_ce_fused_rows");
            }
        }
    }
    const size_t ce_mark = c.top;
    if (!fused_ce) {
        c.fill(row_loss, 0U);
        c.fill(row_max, 0xFF800000U);
        c.fill(row_inv_sum, 0U);
        c.fill(row_valid, 0U);
    }
    for (int64_t start = 0; start < V && c.st == GD_OK && !fused_ce; start += chunk) {
        const int64_t cc = chunk < V - start ? chunk : V - start;
        if (!single) c.top = ce_mark;
        // (when the one-pass kernel declined, its logits are intact and are used as they are)
        const bool have_logits = single && saved_logits.buf != NULL;
        Ten logits = have_logits ? saved_logits : c.alloc(dt, {T, cc});
        gd_backend_matrix_view hm = mv(final_norm, (uint32_t)T, (uint32_t)D), wm = mv(lm_w, (uint32_t)cc, (uint32_t)D, (size_t)start), lm = mv(logits, (uint32_t)T, (uint32_t)cc);
        if (!have_logits) c.ok(gd_backend_matmul_nt(be, &hm, &wm, &lm), "matmul_nt(logits)");
        Ten bchunk = lm_b;
        bchunk.off += (size_t)start * gdb_dtype_size(dt);
        bchunk.shape[0] = cc;
        gd_backend_tensor_view lv = tv(logits), bv = tv(bchunk);
        c.ok(gd_backend_lm_cross_entropy_online_update(be, &lv, &bv, &tgv, &rlv, &rmv, &rsv, (uint64_t)start, (uint64_t)V, s->logits_softcap), "lm_ce_online_update");
        if (single) saved_logits = logits;
    }
    if (fused_ce) {
        // loss and 1 / valid rows are already written
    } else {
    c.ok(gd_backend_lm_cross_entropy_finalize(be, &tgv, &rlv, &rmv, &rsv, &rvv, (uint64_t)V, s->pad_token_id), "lm_ce_finalize");
    if (global_norm) {
        // loss = this rank's share of the global mean; the shares are summed below so that every rank reports the mean
        gd_backend_tensor_view cv1 = tv(counts);
        if (dp && !(s->global_valid_rows > 0.0f)) c.ok(gdb200_dp_join(be), "dp_join(valid rows)");
        c.ok(gdb_lm_ce_reduce_normalize_global(be, &rlv, &cv1, &lov, &ivv), "lm_ce_reduce_normalize(global)");
        if (dp) c.ok(gdb200_dp_all_reduce(be, loss.buf, loss.off, 1, GDB_DTYPE_F32), "dp_all_reduce(loss)");
    } else {
        c.ok(gd_backend_lm_cross_entropy_reduce_normalize(be, &rlv, &rvv, &lov, &ivv), "lm_ce_reduce_normalize");
    }
    }
    *loss_offset = loss.off;
    if (c.st != GD_OK) {
        snprintf(be->last_error, sizeof(be->last_error), "gpt step forward: %s", c.where);
        return c.st;
    }

    // ---------------------------------------------------------------- backward
    if (seed.buf == NULL) {
        c.ok(gd_backend_amp_begin_step(be, &amp), "amp_begin_step");
        seed = c.alloc(GDB_DTYPE_F32, {});
        c.ok(gd_backend_amp_fill_scale(be, seed.buf, seed.off, 1, GDB_DTYPE_F32, s->state_buffer, s->amp_scale_offset), "amp_fill_scale");
    }

    std::vector<Ten> grads((size_t)n_params);
    const size_t es = gdb_dtype_size(dt);
    // contiguous gradient storage for a run of parameters (16-byte aligned pieces): one all-reduce range
    auto alloc_grads = [&](int first, int count, size_t *range_off, size_t *range_elems) {
        size_t total = 0;
        for (int p = first; p < first + count; ++p) total += (s->param_count[p] + 7U) & ~(size_t)7U;
        Ten block = c.alloc(dt, {(int64_t)total});
        size_t cursor = 0;
        for (int p = first; p < first + count; ++p) {
            Ten g = block;
            g.off = block.off + cursor * es;
            g.shape[0] = (int64_t)s->param_count[p];
            grads[(size_t)p] = g;
            cursor += (s->param_count[p] + 7U) & ~(size_t)7U;
        }
        *range_off = block.off;
        *range_elems = total;
    };
    // Default: ONE all-reduce over the whole (contiguous) gradient range after the backward pass. GDB200_DP_OVERLAP=1
    // issues one collective per transformer block as soon as that block's backward is enqueued instead; on 2 and 8
    // B200s that was slower (4.07 vs 4.01 ms per step at 8 GPUs): the collective's CTAs compete with the persistent
    // GEMM / attention grids for SMs, and five 2-8 MB messages cost more than one 25 MB message.
    static int dp_overlap = -1;
    if (dp_overlap < 0) {
        const char *env = getenv("GDB200_DP_OVERLAP");
        dp_overlap = (env != NULL && env[0] == '1') ? 1 : 0;
    }
    std::vector<std::pair<size_t, size_t>> deferred;
    auto reduce_range = [&](size_t off, size_t elems) {
        if (!dp) return;
        if (dp_overlap) {
            c.ok(gdb200_dp_all_reduce(be, s->scratch_buffer, off, elems, dt), "dp_all_reduce");
        } else {
            deferred.push_back(std::make_pair(off, elems));
        }
    };

    // head: final norm weight, LM head weight (when untied) and bias
    size_t head_off = 0, head_elems = 0;
    alloc_grads(P_FINAL, n_params - P_FINAL, &head_off, &head_elems);
    Ten emb_grad;  // token embedding gradient: last to become final
    {
        size_t eo = 0, ee = 0;
        alloc_grads(0, 1, &eo, &ee);
        emb_grad = grads[0];
    }
    // the blocks' gradients follow directly, so that all parameter gradients form one address range
    std::vector<size_t> blk_off((size_t)L), blk_elems((size_t)L);
    for (int i = L - 1; i >= 0; --i) alloc_grads(1 + 10 * i, 10, &blk_off[(size_t)i], &blk_elems[(size_t)i]);
    const size_t all_grads_end = c.top;
    // padding elements between the pieces take part in the all-reduce: keep them finite (one clear over the whole range)
    c.ok(gd_backend_fill(be, s->scratch_buffer, head_off, (all_grads_end - head_off) / es, es, 0U), "gradient range clear");
    Ten dh = c.alloc(dt, {T, D});
    if (!single) c.fill(dh, 0U);
    Ten dh_part;
    if (!single) dh_part = c.alloc(dt, {T, D});
    Ten lmw_grad = s->tied_lm_head ? emb_grad : grads[(size_t)P_LMW];
    const size_t bwd_mark = c.top;
    gd_backend_tensor_view sdv = tv(seed);
    for (int64_t start = 0; start < V && c.st == GD_OK; start += chunk) {
        const int64_t cc = chunk < V - start ? chunk : V - start;
        Ten logits = saved_logits;
        gd_backend_matrix_view hm = mv(final_norm, (uint32_t)T, (uint32_t)D), wm = mv(lm_w, (uint32_t)cc, (uint32_t)D, (size_t)start);
        if (!single) {
            c.top = bwd_mark;
            logits = c.alloc(dt, {T, cc});
            gd_backend_matrix_view lm = mv(logits, (uint32_t)T, (uint32_t)cc);
            c.ok(gd_backend_matmul_nt(be, &hm, &wm, &lm), "matmul_nt(logits bwd)");
        }
        Ten bchunk = lm_b;
        bchunk.off += (size_t)start * es;
        bchunk.shape[0] = cc;
        gd_backend_tensor_view lv = tv(logits), bv = tv(bchunk);
        if (!fused_ce) {
            c.ok(gd_backend_lm_cross_entropy_backward_chunk(be, &lv, &bv, &tgv, &rmv, &rsv, &sdv, &ivv, &lv, (uint64_t)start, (uint64_t)V, 1.0f,
                                                            s->logits_softcap, s->pad_token_id), "lm_ce_backward_chunk");
        }
        gd_backend_matrix_view lm = mv(logits, (uint32_t)T, (uint32_t)cc);
        gd_backend_matrix_view dhm = mv(single ? dh : dh_part, (uint32_t)T, (uint32_t)D);
        c.ok(gd_backend_matmul(be, &lm, &wm, &dhm), "matmul(d_hidden)");
        if (!single) c.accumulate(dh, dh_part);
        gd_backend_matrix_view dwm = mv(lmw_grad, (uint32_t)cc, (uint32_t)D, (size_t)start);
        gd_backend_vector_view dbv = vv(grads[(size_t)P_LMB], (size_t)start, (uint32_t)cc);
        c.ok(gdb200_matmul_tn_colsum(be, &lm, &hm, &dwm, &dbv), "matmul_tn_colsum(d_lm_w, d_lm_b)");
    }
    // Every RMSNorm backward below feeds the residual gradient, whose next consumer is the backward of the dropout in front of
    // the residual add (the MLP branch, the attention branch, the embedding): that gradient comes out of the same launch.
    // Two buffers in front of the blocks' scratch: `to_mlp` is written by the norm in front of a block boundary (final norm, norm 1)
    // and read by the MLP branch of the block below it (or by the embedding), `to_attn` is written by norm 2 and read in its block.
    Ten to_mlp, to_attn;
    memset(&to_mlp, 0, sizeof(to_mlp));
    memset(&to_attn, 0, sizeof(to_attn));
    if (drop) {
        to_mlp = c.alloc(dt, {T, D});
        to_attn = c.alloc(dt, {T, D});
    }
    // (the block below reads `to_mlp` as the gradient of its down projection's output: that projection's bias gradient, the sum of
    // `to_mlp` over the rows, comes out of the same launch too)
    const Ten *first_mask = !drop ? nullptr : (L > 0 ? &saves[(size_t)L - 1].mask2 : &emb_mask);
    Ten gx = rms_backward(c, x, final_w, inv_f, dh, T, D, grads[(size_t)P_FINAL], nullptr, first_mask, drop_scale, &to_mlp,
                          drop && L > 0 ? &grads[(size_t)(1 + 10 * (L - 1)) + 9] : nullptr);
    reduce_range(head_off, head_elems);

    for (int i = L - 1; i >= 0 && c.st == GD_OK; --i) {
        LayerSave &sv = saves[(size_t)i];
        const int pb = 1 + 10 * i;
        const size_t goff = blk_off[(size_t)i], gelems = blk_elems[(size_t)i];
        // Everything else this block's backward allocates is dead once the block is done (the gradient that flows on
        // lives in the buffer that came in), so the space is reused by the next block: backward scratch is O(1) in depth.
        const size_t layer_mark = c.top;
        // out = resid + dropout(mlp)
        Ten g_mlp = drop ? to_mlp : gx;
        Ten g_resid = gx;  // adopted: later contributions accumulate into this buffer
        // down projection y = act w + b (w stored [F, D]): dW = act^T g, db = colsum(g), dact = g w^T
        {
            const Ten w = c.param(pb + 8, {F, D});
            gd_backend_matrix_view am = mv(sv.act, (uint32_t)T, (uint32_t)F), gm = mv(g_mlp, (uint32_t)T, (uint32_t)D), wm = mv(w, (uint32_t)F, (uint32_t)D);
            gd_backend_matrix_view dwm = mv(grads[(size_t)pb + 8], (uint32_t)F, (uint32_t)D);
            c.ok(gd_backend_matmul_tn(be, &am, &gm, &dwm), "matmul_tn(d_down_w)");
            if (!drop) {   // with dropout the norm in front of this block has written it together with g_mlp
                gd_backend_vector_view dbv = vv(grads[(size_t)pb + 9], 0, (uint32_t)D);
                c.ok(gd_backend_reduce_rows(be, &gm, &dbv), "reduce_rows(d_down_b)");
            }
            // d_act = g w^T and the SwiGLU backward in its epilogue; the two separate calls when the fused kernel declines
            Ten d_up = c.alloc(dt, {T, 2 * F});
            gd_backend_matrix_view ugm = mv(sv.up_gate, (uint32_t)T, (uint32_t)(2 * F)), dum = mv(d_up, (uint32_t)T, (uint32_t)(2 * F));
            // (measured on the benchmark step: the fused launch takes as long as the two it replaces, 3.114 against 3.109 ms per
            // step, because the epilogue then carries two special-function evaluations and two 16-byte loads per element; it
            // saves the [T, F] scratch, so it is what GDB200_FUSE_SWIGLU_BWD=1 selects)
            static int fuse_bwd = -1;
            if (fuse_bwd < 0) {
                const char *env = getenv("GDB200_FUSE_SWIGLU_BWD");
                fuse_bwd = (env != NULL && env[0] == '1') ? 1 : 0;
            }
            gd_status fst = (c.st == GD_OK && fuse_bwd) ? gdb200_matmul_nt_swiglu_backward(be, &gm, &wm, &ugm, &dum) : GD_ERR_UNSUPPORTED;
            if (fst == GD_ERR_UNSUPPORTED) {
                Ten dact = c.alloc(dt, {T, F});
                gd_backend_matrix_view dam = mv(dact, (uint32_t)T, (uint32_t)F);
                c.ok(gd_backend_matmul_nt(be, &gm, &wm, &dam), "matmul_nt(d_act)");
                gd_backend_tensor_view xv = tv(sv.up_gate), dav = tv(dact), duv = tv(d_up);
                c.ok(gd_backend_swiglu_split_backward(be, &xv, &dav, &duv), "swiglu_split_backward");
            } else {
                c.ok(fst, "matmul_nt(d_act) + swiglu_split_backward");
            }
            Ten dn2;
            linear_t_backward(c, sv.normed2, c.param(pb + 6, {2 * F, D}), d_up, T, D, 2 * F, &dn2, grads[(size_t)pb + 6], grads[(size_t)pb + 7]);
            rms_backward(c, sv.resid, c.param(pb + 5, {D}), sv.inv2, dn2, T, D, grads[(size_t)pb + 5], &g_resid, drop ? &sv.mask1 : nullptr, drop_scale,
                         &to_attn);
        }
        // resid = x + dropout(proj)
        Ten g_proj = drop ? to_attn : g_resid;
        Ten d_attn;
        linear_t_backward(c, sv.attn, c.param(pb + 3, {D, D}), g_proj, T, D, D, &d_attn, grads[(size_t)pb + 3], grads[(size_t)pb + 4]);
        Ten dq = c.alloc(dt, {T, H, Dh}), dk = c.alloc(dt, {T, H, Dh}), dv = c.alloc(dt, {T, H, Dh}), acc;
        int32_t q_in_acc = 0;
        memset(&acc, 0, sizeof(acc));
        {
            Ten g3 = d_attn;
            g3.rank = 3;
            g3.shape[0] = T;
            g3.shape[1] = H;
            g3.shape[2] = Dh;
            gd_backend_tensor_view gv = tv(g3), q = tv(sv.q), k = tv(sv.k), v = tv(sv.v), cv = tv(cu), dqv = tv(dq), dkv = tv(dk), dvv = tv(dv), stv = tv(sv.stats);
            sa.use_forward_stats = 1;
            // the forward output is still held for the projection's weight gradient: one attention pass instead of two
            Ten attn3 = sv.attn;
            attn3.rank = 3;
            attn3.shape[0] = T;
            attn3.shape[1] = H;
            attn3.shape[2] = Dh;
            acc = c.alloc(GDB_DTYPE_F32, {T, H, Dh});
            gd_backend_tensor_view ov = tv(attn3), av = tv(acc);
            // the query gradient may stay in the FP32 accumulator: the RoPE backward below rounds it on load (GDB200_DQ_F32=0:
            // a conversion pass in between, as the reference's two entries imply)
            static const bool dq_f32 = !(getenv("GDB200_DQ_F32") != NULL && getenv("GDB200_DQ_F32")[0] == '0');
            // (only where that RoPE backward takes its vector path: half-split rotation of the whole head, head_dim a multiple of 16)
            if (dq_f32 && rope.interleaved == 0U && rope.n_dims == (uint32_t)Dh && (Dh % 16) == 0) {
                c.ok(gdb200_sdpa_varlen_backward_with_output_q32(be, &gv, &q, &k, &v, &cv, &ov, &dqv, &dkv, &dvv, &stv, &av, &sa, &q_in_acc), "sdpa_varlen_backward");
            } else {
                c.ok(gdb200_sdpa_varlen_backward_with_output(be, &gv, &q, &k, &v, &cv, &ov, &dqv, &dkv, &dvv, &stv, &av, &sa), "sdpa_varlen_backward");
            }
        }
        Ten dqkv = c.alloc(dt, {T, 3 * D});
        {
            gd_backend_tensor_view a = tv(dq), a32 = tv(acc), b = tv(dk), v = tv(dv), p = tv(pos), o = tv(dqkv);
            if (q_in_acc != 0) {
                c.ok(gdb200_qkv_split_rope_backward_q32(be, &a32, &b, &v, &p, &o, (uint32_t)H, (uint32_t)Dh, &rope), "qkv_split_rope_backward(FP32 dq)");
            } else {
                c.ok(gd_backend_qkv_split_rope_backward(be, &a, &b, &v, &p, &o, (uint32_t)H, (uint32_t)Dh, &rope), "qkv_split_rope_backward");
            }
        }
        Ten dn1;
        linear_t_backward(c, sv.normed, c.param(pb + 1, {3 * D, D}), dqkv, T, D, 3 * D, &dn1, grads[(size_t)pb + 1], grads[(size_t)pb + 2]);
        // (this block's g_mlp in `to_mlp` is dead by now: the next reader is the block below, or the embedding after the first block)
        const Ten *next_mask = !drop ? nullptr : (i > 0 ? &saves[(size_t)i - 1].mask2 : &emb_mask);
        rms_backward(c, sv.x, c.param(pb + 0, {D}), sv.inv1, dn1, T, D, grads[(size_t)pb + 0], &g_resid, next_mask, drop_scale, &to_mlp,
                     drop && i > 0 ? &grads[(size_t)(pb - 10) + 9] : nullptr);
        gx = g_resid;
        reduce_range(goff, gelems);
        c.top = layer_mark;
    }
    if (drop) gx = to_mlp;
    {
        // embedding table gradient; with a tied LM head the head contribution is already in emb_grad
        Ten target = emb_grad;
        if (s->tied_lm_head) target = c.alloc(dt, {V, D});
        Ten scratch = c.alloc(GDB_DTYPE_F32, {V, D});
        Ten t2 = target;
        t2.rank = 2;
        t2.shape[0] = V;
        t2.shape[1] = D;
        gd_backend_tensor_view gv = tv(gx), iv = tv(ids), tvw = tv(t2), sv2 = tv(scratch);
        c.ok(gd_backend_embedding_backward(be, &gv, &iv, &tvw, &sv2, &ea), "embedding_backward");
        if (s->tied_lm_head) c.accumulate(emb_grad, target);
        reduce_range(emb_grad.off, (size_t)V * (size_t)D);
    }
    if (c.st != GD_OK) {
        snprintf(be->last_error, sizeof(be->last_error), "gpt step backward: %s", c.where);
        return c.st;
    }

    // ---------------------------------------------------------------- optimizer (src/optim/adamw.c:2163-2270)
    gd_backend_buffer *scale_buf = s->state_buffer;
    size_t inv_scale_off = s->amp_scale_offset + sizeof(float);
    if (dp) {
        if (!deferred.empty()) {
            // one collective over the whole gradient range (alignment gaps between the pieces ride along)
            c.ok(gdb200_dp_all_reduce(be, s->scratch_buffer, head_off, (all_grads_end - head_off) / es, dt), "dp_all_reduce");
        }
        // every rank divided by the global row count already: the sum over ranks IS the gradient of the global mean loss
        c.ok(gdb200_dp_join(be), "dp_join");
    }
    std::vector<gd_backend_grad_norm_desc> nd((size_t)n_params);
    std::vector<gd_backend_adamw_desc> ad((size_t)n_params);
    size_t partial_index = 0;
    for (int p = 0; p < n_params; ++p) {
        const size_t groups = (s->param_count[p] + 1023U) / 1024U;
        gd_backend_grad_norm_desc &d = nd[(size_t)p];
        memset(&d, 0, sizeof(d));
        d.grad_buffer = grads[(size_t)p].buf;
        d.grad_offset = grads[(size_t)p].off;
        d.count = s->param_count[p];
        d.grad_dtype = dt;
        d.partial_buffer = s->state_buffer;
        d.partial_offset = s->partials_offset + partial_index * sizeof(float);
        d.partial_count = groups;
        d.grad_scale_buffer = scale_buf;
        d.grad_scale_offset = inv_scale_off;
        d.found_inf_buffer = s->state_buffer;
        d.found_inf_offset = s->amp_flags_offset + sizeof(int32_t);
        d.has_found_inf = 1;
        partial_index += groups;
        gd_backend_adamw_desc &a = ad[(size_t)p];
        memset(&a, 0, sizeof(a));
        a.param_buffer = s->params_buffer;
        a.param_offset = s->param_offset[p];
        a.master_buffer = s->state_buffer;
        a.master_offset = s->master_offset[p];
        a.has_master = 1;
        a.grad_buffer = d.grad_buffer;
        a.grad_offset = d.grad_offset;
        a.grad_scale_buffer = s->state_buffer;
        a.grad_scale_offset = s->clip_scale_offset;
        a.has_grad_scale = 1;
        a.found_inf_buffer = s->state_buffer;
        a.found_inf_offset = d.found_inf_offset;
        a.has_found_inf = 1;
        a.m_buffer = s->state_buffer;
        a.m_offset = s->m_offset[p];
        a.v_buffer = s->state_buffer;
        a.v_offset = s->v_offset[p];
        a.state_f32_buffer = s->state_buffer;
        a.beta1_power_offset = s->state_f32_offset + ((size_t)0 * (size_t)n_params + (size_t)p) * 4U;
        a.beta2_power_offset = s->state_f32_offset + ((size_t)1 * (size_t)n_params + (size_t)p) * 4U;
        a.step_scale_offset = s->state_f32_offset + ((size_t)2 * (size_t)n_params + (size_t)p) * 4U;
        a.decay_scale_offset = s->state_f32_offset + ((size_t)3 * (size_t)n_params + (size_t)p) * 4U;
        a.eps_scaled_offset = s->state_f32_offset + ((size_t)4 * (size_t)n_params + (size_t)p) * 4U;
        a.state_i32_buffer = s->state_buffer;
        a.param_step_offset = s->state_i32_offset + (size_t)p * 4U;
        a.optimizer_step_offset = s->state_i32_offset + (size_t)n_params * 4U;
        a.count = s->param_count[p];
        a.param_dtype = dt;
        a.grad_dtype = dt;
        a.has_device_state = 1;
        a.bias_correction = 1;
        a.update_optimizer_step = p == 0 ? 1U : 0U;
        a.lr = lr;
        a.beta1 = s->adam_beta1;
        a.beta2 = s->adam_beta2;
        a.eps = s->adam_eps;
        a.weight_decay = s->weight_decay[p];
        a.bias_correction1 = a.bias_correction2 = 1.0f;
    }
    be->last_grad_count = n_params;
    for (int p = 0; p < n_params; ++p) be->last_grad_offset[p] = grads[(size_t)p].off;
    c.ok(gd_backend_grad_clip_scale(be, nd.data(), (uint32_t)n_params, s->state_buffer, s->clip_scale_offset, s->grad_clip_norm, 1.0e-6f), "grad_clip_scale");
    c.ok(gd_backend_adamw_batch(be, ad.data(), (uint32_t)n_params), "adamw_batch");
    c.ok(gd_backend_amp_finish_step(be, &amp), "amp_finish_step");
    if (scratch_used != NULL) {
        *scratch_used = c.top;
    }
    if (c.st != GD_OK) {
        snprintf(be->last_error, sizeof(be->last_error), "gpt step optimizer: %s", c.where);
    }
    return c.st;
}

extern "C" int32_t gdb200_gpt_train_step_grad_offsets(const gd_backend *be, size_t *offsets, int32_t capacity)
{
    if (be == NULL) return 0;
    for (int32_t p = 0; p < be->last_grad_count && p < capacity && offsets != NULL; ++p) offsets[p] = be->last_grad_offset[p];
    return be->last_grad_count;
}

// ---------------------------------------------------------------------------------------------
// Greedy KV-cache decode with the token feedback on the device.
//
// The reference samples on the host: every decode step downloads logits [B, V], applies the soft
// cap and picks the first maximum (examples/gpt_lm/gpt_lm_shared.c:1322,1388-1398), then uploads the
// next ids, positions and cache positions (:1652-1661). Here the same rule runs in a kernel and the
// ids / positions stay in device memory, so a run of decode steps needs no host round trip; one
// step is recorded once as a CUDA graph and replayed.
namespace {

// One block per row: softcap, non-finite -> -inf, first maximum wins. Writes the winner to
// tokens[row] (the next step's input) and to out_tokens[*step_counter, row]; positions[row] += 1.
template <typename T>
__global__ void argmax_rows_kernel(const T *__restrict__ logits, uint32_t classes, float softcap, int32_t *__restrict__ ids_out,
                                   int32_t *__restrict__ out_tokens, const int32_t *step_counter, int32_t max_steps,
                                   int32_t *__restrict__ positions, uint32_t rows, unsigned *tickets, int32_t *step_counter_rw)
{
    gdb_pdl_sync();
    const uint32_t row = blockIdx.x;
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    const int32_t id = gdb_dec::argmax_row<T>(logits + (size_t)row * classes, classes, softcap, sv, si);
    {
        if (threadIdx.x == 0) {
            ids_out[row] = id;
            if (out_tokens != nullptr) {
                const int32_t t = *step_counter;
                if (t >= 0 && t < max_steps) out_tokens[(size_t)t * rows + row] = id;
            }
            if (positions != nullptr) positions[row] += 1;
            if (tickets != nullptr) {
                // every block reads *step_counter before it takes a ticket, so the last one may advance it
                __threadfence();
                if (atomicAdd(tickets, 1U) == gridDim.x - 1U) {
                    *tickets = 0U;
                    *step_counter_rw += 1;
                }
            }
        }
    }
}

gd_status argmax_launch(gd_backend *be, const gd_backend_tensor_view *logits, float softcap, int32_t *ids_out, int32_t *out_tokens,
                        int32_t *counter, int32_t max_steps, int32_t *positions)
{
    // with a step counter, the last block of the launch advances it (ticket word reserved for this kernel)
    unsigned *tickets = counter != nullptr ? gdb_tickets(be) + (GDB_TICKET_WORDS - 1) : nullptr;
    if (logits == NULL || logits->rank != 2 || logits->shape[0] <= 0 || logits->shape[1] <= 0) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const uint32_t rows = (uint32_t)logits->shape[0], classes = (uint32_t)logits->shape[1];
    const void *x = gdb_tv_ptr(logits, logits->dtype);
    if (x == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    switch (logits->dtype) {
    case GDB_DTYPE_F16:
        gdb_launch(argmax_rows_kernel<__half>, rows, 256, 0, be->stream, (const __half *)x, classes, softcap, ids_out, out_tokens, counter, max_steps, positions, rows, tickets, counter);
        break;
    case GDB_DTYPE_BF16:
        gdb_launch(argmax_rows_kernel<__nv_bfloat16>, rows, 256, 0, be->stream, (const __nv_bfloat16 *)x, classes, softcap, ids_out, out_tokens, counter, max_steps, positions, rows, tickets, counter);
        break;
    case GDB_DTYPE_F32:
        gdb_launch(argmax_rows_kernel<float>, rows, 256, 0, be->stream, (const float *)x, classes, softcap, ids_out, out_tokens, counter, max_steps, positions, rows, tickets, counter);
        break;
    default:
        return GD_ERR_UNSUPPORTED;
    }
    return gdb_launched(be, "argmax_rows");
}

Ten i32_tensor(gd_backend_buffer *buf, size_t off, int64_t n)
{
    Ten t;
    memset(&t, 0, sizeof(t));
    t.buf = buf;
    t.off = off;
    t.dt = GDB_DTYPE_I32;
    t.rank = 1;
    t.shape[0] = n;
    return t;
}

// Enqueues one decode step (gpt_block_decode_cached, examples/gpt_lm/gpt_lm_shared.c:961-1115, and the
// logits head :1204-1246) followed by the device-side argmax and counter advance.
gd_status decode_step_body(gd_backend *be, const gdb200_gpt_spec *s, const gdb200_gpt_decode_state *d, size_t *scratch_used)
{
    Step c;
    c.be = be;
    c.s = s;
    c.top = 0;
    c.st = GD_OK;
    c.where = "";
    const int64_t B = d->batch, D = s->d_model, F = s->mlp_hidden, V = s->vocab_size, H = s->n_heads, Dh = s->head_dim, CAP = d->capacity;
    const int L = s->n_layers;
    const uint32_t dt = s->dtype;
    const int P_FINAL = 1 + 10 * L, P_LMW = s->tied_lm_head ? 0 : P_FINAL + 1, P_LMB = P_FINAL + (s->tied_lm_head ? 1 : 2);
    const Ten ids = i32_tensor(d->io_buffer, d->tokens_offset, B), pos = i32_tensor(d->io_buffer, d->positions_offset, B);
    Ten x = c.alloc(dt, {B, D});
    gd_backend_embedding_args ea = {(uint64_t)B, (uint64_t)V, (uint64_t)D};
    {
        const Ten emb_w = c.param(0, {V, D});
        gd_backend_tensor_view a = tv(emb_w), b = tv(ids), o = tv(x);
        c.ok(gd_backend_embedding_forward(be, &a, &b, &o, &ea), "embedding_forward");
    }
    gd_backend_rope_args rope = {s->rope_theta, (uint32_t)Dh, 0U};
    gd_backend_sdpa_decode_args da;
    memset(&da, 0, sizeof(da));
    da.scale = (float)(1.0 / sqrt((double)Dh));
    da.sliding_window = (uint32_t)s->sdpa_window;
    gd_backend_kv_cache_append_args ka = {0};
    // out = x + y and normed = rms_norm(out, w) in one launch when the vector path applies, else the two calls
    auto add_then_rms = [&](const Ten &xa, const Ten &ya, const Ten &w, Ten *sum, Ten *normed) {
        *sum = c.alloc(dt, {B, D});
        *normed = c.alloc(dt, {B, D});
        gd_backend_tensor_view xv = tv(xa), yv = tv(ya), wv = tv(w), sv = tv(*sum), nv = tv(*normed);
        gd_status r = gdb_add_rms_norm(be, &xv, &yv, &wv, &sv, &nv, (size_t)B, (size_t)D, s->rms_eps);
        if (r == GD_ERR_UNSUPPORTED) {
            c.ok(gd_backend_add(be, &xv, &yv, &sv), "add");
            gd_backend_rms_norm_args a = rms_args(B, D, s->rms_eps);
            r = gd_backend_rms_norm_forward(be, &sv, &wv, &nv, &a);
        }
        c.ok(r, "add + rms_norm");
    };
    Ten inv0;
    Ten normed = rms_forward(c, x, c.param(1, {D}), B, D, &inv0);
    for (int i = 0; i < L && c.st == GD_OK; ++i) {
        const int pb = 1 + 10 * i;
        Ten qkv = linear_t(c, normed, c.param(pb + 1, {3 * D, D}), c.param(pb + 2, {3 * D}), B, D, 3 * D);
        Ten q = c.alloc(dt, {B, 1, H, Dh});
        Ten kc, vc;
        memset(&kc, 0, sizeof(kc));
        kc.buf = d->cache_buffer;
        kc.dt = dt;
        kc.rank = 4;
        kc.shape[0] = B;
        kc.shape[1] = CAP;
        kc.shape[2] = H;
        kc.shape[3] = Dh;
        vc = kc;
        kc.off = d->k_cache_offset[i];
        vc.off = d->v_cache_offset[i];
        Ten attn = c.alloc(dt, {B, 1, H, Dh});
        {
            Ten q3 = q;
            q3.rank = 3;
            q3.shape[0] = B;
            q3.shape[1] = H;
            q3.shape[2] = Dh;
            gd_backend_tensor_view a = tv(qkv), pv = tv(pos), q3v = tv(q3), kcv = tv(kc), vcv = tv(vc), qv = tv(q), ov = tv(attn);
            // rotated key / value go straight into their cache slots; fall back to split + append when that path does not apply
            gd_status r = gdb_qkv_rope_append(be, &a, &pv, &q3v, &kcv, &vcv, (uint32_t)H, (uint32_t)Dh, (uint32_t)CAP, &rope);
            if (r == GD_ERR_UNSUPPORTED) {
                Ten k = c.alloc(dt, {B, 1, H, Dh}), v = c.alloc(dt, {B, 1, H, Dh});
                Ten k3 = k, v3 = v;
                for (Ten *t : {&k3, &v3}) {
                    t->rank = 3;
                    t->shape[0] = B;
                    t->shape[1] = H;
                    t->shape[2] = Dh;
                }
                gd_backend_tensor_view k3v = tv(k3), v3v = tv(v3), kn = tv(k), vn = tv(v);
                c.ok(gd_backend_qkv_split_rope_forward(be, &a, &pv, &q3v, &k3v, &v3v, (uint32_t)H, (uint32_t)Dh, &rope), "qkv_split_rope_forward");
                r = gd_backend_kv_cache_append_positions(be, &kcv, &vcv, &pv, &kn, &vn, &ka);
            }
            c.ok(r, "rope + kv append");
            c.ok(gd_backend_sdpa_decode_positions(be, &qv, &kcv, &vcv, &pv, &ov, &da), "sdpa_decode_positions");
        }
        Ten proj = linear_t(c, attn, c.param(pb + 3, {D, D}), c.param(pb + 4, {D}), B, D, D);
        Ten resid, normed2;
        add_then_rms(x, proj, c.param(pb + 5, {D}), &resid, &normed2);
        Ten act = c.alloc(dt, {B, F});
        {
            // up / gate projection and the gate in one launch when the 64-row kernel takes the shape, else the two calls
            const Ten w = c.param(pb + 6, {2 * F, D}), bv = c.param(pb + 7, {2 * F});
            const size_t es = gdb_dtype_size(dt);
            gd_status r = GD_ERR_UNSUPPORTED;
            if (c.st == GD_OK && be->gemm_mode != 1 && be->gemm_mode != 2) {
                r = gdb_gemm_skinny_swiglu(be, dt, normed2.buf->dptr + normed2.off, (size_t)D * es, w.buf->dptr + w.off, (size_t)D * es,
                                           bv.buf->dptr + bv.off, act.buf->dptr + act.off, (size_t)F * es, (uint32_t)B, (uint32_t)F, (uint32_t)D);
            }
            if (r == GD_ERR_UNSUPPORTED) {
                Ten up_gate = linear_t(c, normed2, w, bv, B, D, 2 * F);
                gd_backend_tensor_view a = tv(up_gate), o = tv(act);
                r = gd_backend_swiglu_split_forward(be, &a, &o);
            }
            c.ok(r, "up_gate linear + swiglu");
        }
        Ten mlp = c.alloc(dt, {B, D});
        {
            const Ten w = c.param(pb + 8, {F, D}), b = c.param(pb + 9, {D});
            gd_backend_matrix_view am = mv(act, (uint32_t)B, (uint32_t)F), wm = mv(w, (uint32_t)F, (uint32_t)D), ym = mv(mlp, (uint32_t)B, (uint32_t)D);
            gd_backend_vector_view bv = vv(b, 0, (uint32_t)D);
            c.ok(gd_backend_linear(be, &am, &wm, &bv, &ym), "linear(down_proj)");
        }
        // residual add fused with the norm that consumes it: the next block's attention norm, or the final norm
        Ten out;
        add_then_rms(resid, mlp, i + 1 < L ? c.param(1 + 10 * (i + 1), {D}) : c.param(P_FINAL, {D}), &out, &normed);
        x = out;
    }
    Ten final_norm = normed;
    Ten logits = linear_t(c, final_norm, c.param(P_LMW, {V, D}), c.param(P_LMB, {V}), B, D, V);
    if (c.st == GD_OK) {
        gd_backend_tensor_view lv = tv(logits);
        int32_t *io = (int32_t *)gdb_raw_ptr(d->io_buffer, 0, gd_backend_buffer_nbytes(d->io_buffer));
        if (io == NULL) {
            return GD_ERR_INVALID_ARGUMENT;
        }
        int32_t *tok = io + d->tokens_offset / 4U, *posp = io + d->positions_offset / 4U;
        int32_t *outp = io + d->out_tokens_offset / 4U, *cnt = io + d->step_counter_offset / 4U;
        c.ok(argmax_launch(be, &lv, s->logits_softcap, tok, outp, cnt, d->max_steps, posp), "argmax_rows");
    }
    if (scratch_used != NULL) {
        *scratch_used = c.top;
    }
    if (c.st != GD_OK) {
        snprintf(be->last_error, sizeof(be->last_error), "gpt decode step: %s", c.where);
    }
    return c.st;
}

// The whole run of decode steps in one persistent kernel (decode_mega.cu) where its shapes allow; GD_ERR_UNSUPPORTED
// otherwise (the caller then enqueues one launch per operation).
gd_status decode_steps_persistent(gd_backend *be, const gdb200_gpt_spec *s, const gdb200_gpt_decode_state *d, int32_t n_steps, size_t *scratch_used)
{
    const int64_t B = d->batch, D = s->d_model, F = s->mlp_hidden, V = s->vocab_size, H = s->n_heads, Dh = s->head_dim, CAP = d->capacity;
    const int L = s->n_layers;
    const uint32_t dt = s->dtype;
    if (!gdb_decode_mega_supported(be, dt, (int)B, (int)D, (int)F, (int)V, (int)H, (int)Dh, L)) {
        return GD_ERR_UNSUPPORTED;
    }
    if ((long long)n_steps * (5 * L + 2) * be->sm_count >= (1LL << 30)) {
        return GD_ERR_UNSUPPORTED;   // the barrier counter of one launch has 31 bits
    }
    const size_t es = gdb_dtype_size(dt);
    Step c;
    c.be = be;
    c.s = s;
    c.top = 0;
    c.st = GD_OK;
    c.where = "";
    gdb_mega_args a;
    memset(&a, 0, sizeof(a));
    bool aligned = true;
    auto pptr = [&](int idx, size_t count) -> const void * {
        const void *p = gdb_raw_ptr(s->params_buffer, s->param_offset[idx], count * es);
        if (p == NULL || ((uintptr_t)p % 16U) != 0U) aligned = false;
        return p;
    };
    const int P_FINAL = 1 + 10 * L, P_LMW = s->tied_lm_head ? 0 : P_FINAL + 1, P_LMB = P_FINAL + (s->tied_lm_head ? 1 : 2);
    a.emb = pptr(0, (size_t)(V * D));
    a.w_final = pptr(P_FINAL, (size_t)D);
    a.w_lm = pptr(P_LMW, (size_t)(V * D));
    a.b_lm = pptr(P_LMB, (size_t)V);
    const size_t counts[10] = {(size_t)D, (size_t)(3 * D * D), (size_t)(3 * D), (size_t)(D * D), (size_t)D,
                               (size_t)D, (size_t)(2 * F * D), (size_t)(2 * F), (size_t)(F * D), (size_t)D};
    const size_t cache_bytes = (size_t)(B * CAP * H * Dh) * es;
    for (int i = 0; i < L; ++i) {
        for (int j = 0; j < 10; ++j) a.lw[i][j] = pptr(1 + 10 * i + j, counts[j]);
        a.kc[i] = gdb_raw_ptr(d->cache_buffer, d->k_cache_offset[i], cache_bytes);
        a.vc[i] = gdb_raw_ptr(d->cache_buffer, d->v_cache_offset[i], cache_bytes);
        if (a.kc[i] == NULL || a.vc[i] == NULL || (((uintptr_t)a.kc[i] | (uintptr_t)a.vc[i]) % 16U) != 0U) aligned = false;
    }
    if (!aligned) {
        return GD_ERR_UNSUPPORTED;
    }
    gd_backend_rope_args rope = {s->rope_theta, (uint32_t)Dh, 0U};
    gd_status st = gdb_rope_params_for_decode(be, (uint32_t)H, (uint32_t)Dh, &rope, (size_t)B, &a.rope);
    if (st != GD_OK) {
        return st;
    }
    a.rope_table = be->rope_table;
    a.B = (int)B;
    a.D = (int)D;
    a.F = (int)F;
    a.V = (int)V;
    a.H = (int)H;
    a.L = L;
    a.CAP = (int)CAP;
    a.window = s->sdpa_window;
    // the key splits the stand-alone attention entry uses for this shape (the same partition gives the same bits)
    a.splits = gdb_dec::decode_choose_splits(be->sm_count, (int)B, 1, (int)H, (int)Dh, (int)CAP, 32);
    a.max_steps = d->max_steps;
    a.n_steps = n_steps;
    a.eps = s->rms_eps;
    a.scale = (float)(1.0 / sqrt((double)Dh));
    a.softcap = s->logits_softcap;
    auto act = [&](int64_t cols) -> void * {
        Ten t = c.alloc(dt, {B, cols});
        return t.buf != NULL ? (void *)(t.buf->dptr + t.off) : NULL;
    };
    a.xbuf = act(D);
    a.resid = act(D);
    a.q = act(D);
    a.attn = act(D);
    a.act = act(F);
    a.logits = act(V);
    Ten sync = c.alloc(GDB_DTYPE_I32, {4});
    if (c.st != GD_OK) {
        snprintf(be->last_error, sizeof(be->last_error), "gpt decode steps: %s", c.where);
        return c.st;
    }
    a.sync = (unsigned *)(sync.buf->dptr + sync.off);
    int32_t *io = (int32_t *)gdb_raw_ptr(d->io_buffer, 0, gd_backend_buffer_nbytes(d->io_buffer));
    if (io == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    a.tokens = io + d->tokens_offset / 4U;
    a.positions = io + d->positions_offset / 4U;
    a.out_tokens = io + d->out_tokens_offset / 4U;
    a.step_counter = io + d->step_counter_offset / 4U;
    a.err_flag = (int *)be->err_flag;
    st = gd_backend_fill(be, sync.buf, sync.off, sync.count(), 4U, 0U);
    if (st != GD_OK) {
        return st;
    }
    // GDB200_DECODE_TIMELINE=1 (diagnostic): time stamps after every grid barrier, printed per phase as a mean over the steps
    const int per_step = 5 * L + 2;
    Ten tl;
    const bool want_tl = getenv("GDB200_DECODE_TIMELINE") != NULL;
    if (want_tl) {
        tl = c.alloc(GDB_DTYPE_F32, {(int64_t)n_steps * per_step * 2});
        if (c.st == GD_OK) a.timeline = (unsigned long long *)(tl.buf->dptr + tl.off);
    }
    if (scratch_used != NULL) {
        *scratch_used = c.top;
    }
    st = gdb_decode_mega_launch(be, dt, &a);
    if (st == GD_OK && a.timeline != NULL && n_steps > 2) {
        std::vector<unsigned long long> h((size_t)n_steps * per_step);
        if (cudaStreamSynchronize(be->stream) == cudaSuccess &&
            cudaMemcpy(h.data(), a.timeline, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess) {
            static const char *names[5] = {"A qkv+rope", "B attention", "C proj", "D upgate", "E down"};
            fprintf(stderr, "decode timeline, mean ns per phase over steps 1..%d (%.1f us per step)\n", n_steps - 1,
                    (double)(h.back() - h[(size_t)per_step - 1]) / 1000.0 / (double)(n_steps - 1));
            for (int k = 0; k < per_step; ++k) {
                double sum = 0.0;
                for (int stp = 1; stp < n_steps; ++stp) {
                    const size_t i = (size_t)stp * per_step + k;
                    sum += (double)(h[i] - h[i - 1]);
                }
                if (k < 5 * L) {
                    fprintf(stderr, "  layer %d %-12s %8.0f\n", k / 5, names[k % 5], sum / (n_steps - 1));
                } else {
                    fprintf(stderr, "  %-20s %8.0f\n", k == 5 * L ? "F logits" : "G argmax", sum / (n_steps - 1));
                }
            }
        }
    }
    return st;
}

}  // namespace

extern "C" gd_status gdb200_argmax_rows(gd_backend *be, const gd_backend_tensor_view *logits, float softcap, const gd_backend_tensor_view *out_ids)
{
    if (be == NULL || logits == NULL || out_ids == NULL || logits->rank != 2 || out_ids->count != (size_t)logits->shape[0]) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    int32_t *out = (int32_t *)gdb_tv_ptr(out_ids, GDB_DTYPE_I32);
    if (out == NULL) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    return argmax_launch(be, logits, softcap, out, nullptr, nullptr, 0, nullptr);
}

extern "C" gd_status gdb200_gpt_decode_steps(gd_backend *be, const gdb200_gpt_spec *s, const gdb200_gpt_decode_state *d, int32_t n_steps,
                                             int32_t use_graph, size_t *scratch_used)
{
    if (be == NULL || s == NULL || d == NULL || n_steps < 0 || d->batch <= 0 || d->capacity <= 0 || s->n_layers <= 0 ||
        s->n_layers > GDB200_GPT_MAX_LAYERS || s->n_heads * s->head_dim != s->d_model || d->cache_buffer == NULL || d->io_buffer == NULL ||
        ((d->tokens_offset | d->positions_offset | d->out_tokens_offset | d->step_counter_offset) % 4U) != 0U) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    const size_t io_bytes = gd_backend_buffer_nbytes(d->io_buffer);
    if (d->tokens_offset + (size_t)d->batch * 4U > io_bytes || d->positions_offset + (size_t)d->batch * 4U > io_bytes ||
        d->step_counter_offset + 4U > io_bytes || d->out_tokens_offset + (size_t)d->max_steps * (size_t)d->batch * 4U > io_bytes) {
        return GD_ERR_INVALID_ARGUMENT;
    }
    if (n_steps == 0) {
        return GD_OK;
    }
    if (use_graph) {
        gd_status pst = decode_steps_persistent(be, s, d, n_steps, scratch_used);
        if (pst != GD_ERR_UNSUPPORTED) {
            return pst;
        }
    }
    int done = 0;
    // The first step runs eagerly: it performs the one-time kernel attribute set-up that must not
    // happen while a stream is being captured.
    gd_status st = decode_step_body(be, s, d, scratch_used);
    if (st != GD_OK) {
        return st;
    }
    done = 1;
    if (use_graph && n_steps - done >= 2) {
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        const uint64_t launches0 = be->launches;
        cudaError_t e = cudaStreamBeginCapture(be->stream, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) {
            return gdb_fail(be, e, "decode graph: begin capture");
        }
        st = decode_step_body(be, s, d, nullptr);
        e = cudaStreamEndCapture(be->stream, &graph);
        const uint64_t per_step = be->launches - launches0;
        be->launches = launches0;
        if (st != GD_OK || e != cudaSuccess || graph == nullptr) {
            if (graph != nullptr) cudaGraphDestroy(graph);
            return st != GD_OK ? st : gdb_fail(be, e, "decode graph: end capture");
        }
        e = cudaGraphInstantiate(&exec, graph, 0);
        if (e != cudaSuccess) {
            cudaGraphDestroy(graph);
            return gdb_fail(be, e, "decode graph: instantiate");
        }
        for (; done < n_steps; ++done) {
            e = cudaGraphLaunch(exec, be->stream);
            if (e != cudaSuccess) {
                break;
            }
            be->launches += per_step;
        }
        // the graph objects may be released while launches are in flight; execution keeps its own references
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) {
            return gdb_fail(be, e, "decode graph: launch");
        }
        return GD_OK;
    }
    for (; done < n_steps; ++done) {
        st = decode_step_body(be, s, d, nullptr);
        if (st != GD_OK) {
            return st;
        }
    }
    return GD_OK;
}
