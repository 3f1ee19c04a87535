"""Op capsules of the gpt_lm path: validate -> allocate scratch -> backend call -> record.

Each function mirrors the reference capsule of the same name (src/ops/<op>/core_*.c and
autograd_*.c): same argument meaning, same scratch tensors, same backend entry sequence and
the same backward rules. Outputs live in the scratch arena of the current step.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

from . import abi
from .abi import F16, BF16, F32, I32, U8
from .runtime import Context, Tensor

byref = C.byref

RMS_WGRAD_ROW_BLOCK_SMALL = 64        # src/ops/rms_norm/core_rms_norm.c:9-11
RMS_WGRAD_ROW_BLOCK_LARGE = 128
RMS_WGRAD_LARGE_ROWS = 4096
LM_CE_DEFAULT_CHUNK = 2048            # src/ops/lm_cross_entropy/core_lm_cross_entropy.c:14
F32_NEG_INF_PATTERN = 0xFF800000      # :15
# gd_linear_transposed_weight: use the additive fused entry instead of the reference's two-call
# sequence (matmul_nt, then add). Both give bit-identical results; tests exercise both.
FUSE_BIAS_ADD = True
# gd_sdpa_varlen's backward through gdb200_sdpa_varlen_backward_with_output (False: the reference entry, two passes)
SDPA_BACKWARD_WITH_OUTPUT = True


def _tvp(t: Optional[Tensor]):
    return byref(t.tv()) if t is not None else None


def _flat2(t: Tensor) -> tuple[int, int]:
    cols = t.shape[-1]
    return t.count // cols, cols


# --------------------------------------------------------------------------- embedding
def gd_embedding(ctx: Context, table: Tensor, ids: Tensor) -> Tensor:
    """out = table[ids]; reference src/ops/embedding/core_embedding.c:158 (bwd :191)."""
    vocab, dim = table.shape
    out = ctx.scratch_empty(table.dtype, (ids.count, dim), "embedding")
    args = abi.EmbeddingArgs(ids.count, vocab, dim)
    ctx.check(ctx.lib.gd_backend_embedding_forward(ctx.backend, _tvp(table), _tvp(ids), _tvp(out), byref(args)), "embedding_forward")
    out.requires_grad = table.requires_grad
    if table.requires_grad:
        def backward():
            if out.grad is None:
                return
            dtable = ctx.scratch_empty(table.dtype, table.shape, "d_table")
            scratch = ctx.scratch_empty(F32, table.shape, "d_table_f32") if table.dtype != F32 else None
            ctx.check(ctx.lib.gd_backend_embedding_backward(ctx.backend, _tvp(out.grad), _tvp(ids), _tvp(dtable),
                                                            _tvp(scratch), byref(args)), "embedding_backward")
            ctx.accumulate_grad(table, dtable)
        ctx.record(backward)
    return out


# --------------------------------------------------------------------------- dropout
def _dropout_backward_mask(ctx: Context, mask: Tensor, grad_out: Tensor, scale: float) -> Tensor:
    dx = ctx.scratch_empty(grad_out.dtype, grad_out.shape, "d_dropout")
    ctx.check(ctx.lib.gd_backend_dropout_backward_mask(ctx.backend, _tvp(mask), _tvp(grad_out), _tvp(dx), scale), "dropout_backward_mask")
    return dx


def gd_dropout(ctx: Context, x: Tensor, p: float, training: bool, seed: int) -> Tensor:
    """Inverted dropout with a saved u8 mask (src/ops/dropout/core_dropout.c:183-345).
    Eval mode or p == 0 returns x itself."""
    if not training or p == 0.0:
        return x
    y = ctx.scratch_empty(x.dtype, x.shape, "dropout")
    mask = ctx.scratch_empty(U8, x.shape, "dropout_mask")
    ctx.check(ctx.lib.gd_backend_dropout_forward(ctx.backend, _tvp(x), _tvp(y), _tvp(mask), p, seed & (2**64 - 1)), "dropout_forward")
    y.requires_grad = x.requires_grad
    if x.requires_grad:
        scale = 1.0 / (1.0 - p)

        def backward():
            if y.grad is not None:
                ctx.accumulate_grad(x, _dropout_backward_mask(ctx, mask, y.grad, scale))
        ctx.record(backward)
    return y


def gd_add(ctx: Context, x: Tensor, y: Tensor) -> Tensor:
    """out = x + y with trailing-dimension broadcast of y (src/ops/add/core_add.c)."""
    out = ctx.scratch_empty(x.dtype, x.shape, "add")
    ctx.check(ctx.lib.gd_backend_add(ctx.backend, _tvp(x), _tvp(y), _tvp(out)), "add")
    out.requires_grad = x.requires_grad or y.requires_grad
    if out.requires_grad:
        def backward():
            if out.grad is None:
                return
            ctx.accumulate_grad(x, out.grad)
            if y.requires_grad:
                if y.count == out.count:
                    ctx.accumulate_grad(y, out.grad)
                else:
                    rows, cols = out.count // y.count, y.count
                    dy = ctx.scratch_empty(y.dtype, y.shape, "d_add_bias")
                    mv, vv = out.grad.mv(rows, cols), dy.vv()
                    ctx.check(ctx.lib.gd_backend_reduce_rows(ctx.backend, byref(mv), byref(vv)), "reduce_rows")
                    ctx.accumulate_grad(y, dy)
        ctx.record(backward)
    return out


def gd_dropout_add(ctx: Context, residual: Tensor, x: Tensor, p: float, training: bool, seed: int) -> Tensor:
    """y = residual + dropout(x) fused (src/ops/dropout/core_dropout.c:348-432); eval or
    p == 0 degrades to gd_add (:391-393)."""
    if not training or p == 0.0:
        return gd_add(ctx, residual, x)
    y = ctx.scratch_empty(x.dtype, x.shape, "dropout_add")
    mask = ctx.scratch_empty(U8, x.shape, "dropout_add_mask")
    ctx.check(ctx.lib.gd_backend_dropout_add_forward(ctx.backend, _tvp(residual), _tvp(x), _tvp(y), _tvp(mask), p,
                                                     seed & (2**64 - 1)), "dropout_add_forward")
    y.requires_grad = residual.requires_grad or x.requires_grad
    if y.requires_grad:
        scale = 1.0 / (1.0 - p)

        def backward():
            if y.grad is None:
                return
            if x.requires_grad:
                ctx.accumulate_grad(x, _dropout_backward_mask(ctx, mask, y.grad, scale))
            ctx.accumulate_grad(residual, y.grad)
        ctx.record(backward)
    return y


# --------------------------------------------------------------------------- rms_norm
def _rms_args(rows: int, cols: int, eps: float) -> abi.RmsNormArgs:
    rb = RMS_WGRAD_ROW_BLOCK_LARGE if rows >= RMS_WGRAD_LARGE_ROWS else RMS_WGRAD_ROW_BLOCK_SMALL
    a = abi.RmsNormArgs()
    a.rows, a.cols, a.row_blocks, a.eps = rows, cols, (rows + rb - 1) // rb, eps
    a.simdgroups, a.wgrad_simdgroups, a.wgrad_row_block = 8, 8, rb
    return a


def gd_rms_norm(ctx: Context, x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """y = x * w * rsqrt(mean(x^2) + eps), saving inv_rms (src/ops/rms_norm/core_rms_norm.c:210,271,319)."""
    rows, cols = _flat2(x)
    args = _rms_args(rows, cols, eps)
    out = ctx.scratch_empty(x.dtype, x.shape, "rms_norm")
    needs_grad = ctx.grad_enabled and (x.requires_grad or weight.requires_grad)
    if needs_grad:
        inv = ctx.scratch_empty(F32, (rows,), "inv_rms")
        ctx.check(ctx.lib.gd_backend_rms_norm_forward_stats(ctx.backend, _tvp(x), _tvp(weight), _tvp(out), _tvp(inv), byref(args)), "rms_norm_forward_stats")
    else:
        ctx.check(ctx.lib.gd_backend_rms_norm_forward(ctx.backend, _tvp(x), _tvp(weight), _tvp(out), byref(args)), "rms_norm_forward")
    out.requires_grad = needs_grad
    if needs_grad:
        def backward():
            if out.grad is None:
                return
            if x.requires_grad:
                dx = ctx.scratch_empty(x.dtype, x.shape, "d_rms_x")
                ctx.check(ctx.lib.gd_backend_rms_norm_backward_stats(ctx.backend, _tvp(x), _tvp(weight), _tvp(inv), _tvp(out.grad), _tvp(dx), byref(args)), "rms_norm_backward_stats")
                ctx.accumulate_grad(x, dx)
            if weight.requires_grad:
                dw = ctx.scratch_empty(weight.dtype, weight.shape, "d_rms_w")
                partial = ctx.scratch_empty(F32, (args.row_blocks, cols), "rms_partial")
                ctx.check(ctx.lib.gd_backend_rms_norm_weight_backward_stats(ctx.backend, _tvp(x), _tvp(inv), _tvp(out.grad), _tvp(dw), _tvp(partial), byref(args)), "rms_norm_weight_backward_stats")
                ctx.accumulate_grad(weight, dw)
        ctx.record(backward)
    return out


# --------------------------------------------------------------------------- linear family
def _matmul(ctx: Context, fn, x_mv, w_mv, y_mv, what: str) -> None:
    ctx.check(fn(ctx.backend, byref(x_mv), byref(w_mv), byref(y_mv)), what)


def _reduce_rows(ctx: Context, g: Tensor, rows: int, cols: int, like: Tensor) -> Tensor:
    db = ctx.scratch_empty(like.dtype, like.shape, "d_bias")
    mv, vv = g.mv(rows, cols), db.vv()
    ctx.check(ctx.lib.gd_backend_reduce_rows(ctx.backend, byref(mv), byref(vv)), "reduce_rows")
    return db


def gd_linear_transposed_weight(ctx: Context, x: Tensor, w: Tensor, bias: Optional[Tensor]) -> Tensor:
    """y = x w^T (+ bias through a separate add), w stored [N, K]
    (src/ops/linear_transposed_weight/core_linear_transposed_weight.c:7-103, bwd _bwd.c:31-167):
    dX = dY w (matmul), dW = dY^T x (matmul_tn), db = reduce_rows(dY)."""
    m, k = _flat2(x)
    n = w.shape[0]
    assert w.shape[1] == k
    lib = ctx.lib
    y = ctx.scratch_empty(x.dtype, x.shape[:-1] + (n,), "linear_t")
    out = y
    if bias is None:
        _matmul(ctx, lib.gd_backend_matmul_nt, x.mv(m, k), w.mv(n, k), y.mv(m, n), "matmul_nt")
    elif FUSE_BIAS_ADD:
        # one kernel with the same two roundings as matmul_nt + add (bit-identical results)
        xm, wm, bv, ym = x.mv(m, k), w.mv(n, k), bias.vv(), y.mv(m, n)
        ctx.check(lib.gdb200_matmul_nt_bias(ctx.backend, byref(xm), byref(wm), byref(bv), byref(ym)), "matmul_nt_bias")
    else:
        _matmul(ctx, lib.gd_backend_matmul_nt, x.mv(m, k), w.mv(n, k), y.mv(m, n), "matmul_nt")
        out = ctx.scratch_empty(x.dtype, y.shape, "linear_t_bias")
        ctx.check(lib.gd_backend_add(ctx.backend, _tvp(y), _tvp(bias), _tvp(out)), "add(bias)")
    needs = x.requires_grad or w.requires_grad or (bias is not None and bias.requires_grad)
    out.requires_grad = needs
    if needs:
        def backward():
            g = out.grad
            if g is None:
                return
            if x.requires_grad:
                dx = ctx.scratch_empty(x.dtype, x.shape, "d_linear_t_x")
                _matmul(ctx, lib.gd_backend_matmul, g.mv(m, n), w.mv(n, k), dx.mv(m, k), "matmul(dX)")
                ctx.accumulate_grad(x, dx)
            if w.requires_grad:
                dw = ctx.scratch_empty(w.dtype, w.shape, "d_linear_t_w")
                _matmul(ctx, lib.gd_backend_matmul_tn, g.mv(m, n), x.mv(m, k), dw.mv(n, k), "matmul_tn(dW)")
                ctx.accumulate_grad(w, dw)
            if bias is not None and bias.requires_grad:
                ctx.accumulate_grad(bias, _reduce_rows(ctx, g, m, n, bias))
        ctx.record(backward)
    return out


def gd_linear_backward(ctx: Context, x: Tensor, w: Tensor, bias: Optional[Tensor], g: Tensor,
                       need_x: bool, need_w: bool, need_b: bool):
    """Backward of y = x w + b with w stored [K, N] (src/ops/linear/core_linear_bwd.c:30-155):
    dX = dY w^T (matmul_nt), dW = x^T dY (matmul_tn), db = reduce_rows(dY)."""
    m, k = _flat2(x)
    n = w.shape[1]
    lib = ctx.lib
    dx = dw = db = None
    if need_x:
        dx = ctx.scratch_empty(x.dtype, x.shape, "d_linear_x")
        _matmul(ctx, lib.gd_backend_matmul_nt, g.mv(m, n), w.mv(k, n), dx.mv(m, k), "matmul_nt(dX)")
    if need_w:
        dw = ctx.scratch_empty(w.dtype, w.shape, "d_linear_w")
        _matmul(ctx, lib.gd_backend_matmul_tn, x.mv(m, k), g.mv(m, n), dw.mv(k, n), "matmul_tn(dW)")
    if need_b:
        db = _reduce_rows(ctx, g, m, n, bias)
    return dx, dw, db


def gd_linear(ctx: Context, x: Tensor, w: Tensor, bias: Optional[Tensor]) -> Tensor:
    """y = x w + b fused, w stored [K, N] (src/ops/linear/core_linear.c:7-74)."""
    m, k = _flat2(x)
    n = w.shape[1]
    assert w.shape[0] == k
    y = ctx.scratch_empty(x.dtype, x.shape[:-1] + (n,), "linear")
    xm, wm, ym = x.mv(m, k), w.mv(k, n), y.mv(m, n)
    if bias is not None:
        bv = bias.vv()
        ctx.check(ctx.lib.gd_backend_linear(ctx.backend, byref(xm), byref(wm), byref(bv), byref(ym)), "linear")
    else:
        ctx.check(ctx.lib.gd_backend_matmul(ctx.backend, byref(xm), byref(wm), byref(ym)), "matmul")
    needs = x.requires_grad or w.requires_grad or (bias is not None and bias.requires_grad)
    y.requires_grad = needs
    if needs:
        def backward():
            if y.grad is None:
                return
            dx, dw, db = gd_linear_backward(ctx, x, w, bias, y.grad, x.requires_grad, w.requires_grad,
                                            bias is not None and bias.requires_grad)
            if dx is not None:
                ctx.accumulate_grad(x, dx)
            if dw is not None:
                ctx.accumulate_grad(w, dw)
            if db is not None:
                ctx.accumulate_grad(bias, db)
        ctx.record(backward)
    return y


# --------------------------------------------------------------------------- swiglu
def gd_swiglu_split(ctx: Context, x12: Tensor) -> Tensor:
    """out = x1 * silu(x2) with x12 = [x1 | x2] on the last axis (src/ops/swiglu/core_swiglu.c:340)."""
    h = x12.shape[-1] // 2
    out = ctx.scratch_empty(x12.dtype, x12.shape[:-1] + (h,), "swiglu")
    ctx.check(ctx.lib.gd_backend_swiglu_split_forward(ctx.backend, _tvp(x12), _tvp(out)), "swiglu_split_forward")
    out.requires_grad = x12.requires_grad
    if x12.requires_grad:
        def backward():
            if out.grad is not None:
                ctx.accumulate_grad(x12, _swiglu_split_backward(ctx, x12, out.grad))
        ctx.record(backward)
    return out


def _swiglu_split_backward(ctx: Context, x12: Tensor, g: Tensor) -> Tensor:
    dx12 = ctx.scratch_empty(x12.dtype, x12.shape, "d_swiglu")
    ctx.check(ctx.lib.gd_backend_swiglu_split_backward(ctx.backend, _tvp(x12), _tvp(g), _tvp(dx12)), "swiglu_split_backward")
    return dx12


def gd_swiglu_split_linear(ctx: Context, x12: Tensor, w: Tensor, bias: Optional[Tensor]) -> Tensor:
    """y = linear(swiglu_split(x12), w, b), activation saved for backward
    (src/ops/swiglu_split_linear/core_swiglu_split_linear.c:226-301; bwd :303-407:
    dW, db from the activation, dact = dY w^T, dx12 through the SwiGLU backward)."""
    h = x12.shape[-1] // 2
    m = x12.count // x12.shape[-1]
    n = w.shape[1]
    act = ctx.scratch_empty(x12.dtype, x12.shape[:-1] + (h,), "swiglu_act")
    ctx.check(ctx.lib.gd_backend_swiglu_split_forward(ctx.backend, _tvp(x12), _tvp(act)), "swiglu_split_forward")
    y = ctx.scratch_empty(x12.dtype, x12.shape[:-1] + (n,), "swiglu_linear")
    am, wm, ym = act.mv(m, h), w.mv(h, n), y.mv(m, n)
    if bias is not None:
        bv = bias.vv()
        ctx.check(ctx.lib.gd_backend_linear(ctx.backend, byref(am), byref(wm), byref(bv), byref(ym)), "linear")
    else:
        ctx.check(ctx.lib.gd_backend_matmul(ctx.backend, byref(am), byref(wm), byref(ym)), "matmul")
    needs = x12.requires_grad or w.requires_grad or (bias is not None and bias.requires_grad)
    y.requires_grad = needs
    if needs:
        def backward():
            g = y.grad
            if g is None:
                return
            need_b = bias is not None and bias.requires_grad
            if w.requires_grad or need_b:
                _, dw, db = gd_linear_backward(ctx, act, w, bias, g, False, w.requires_grad, need_b)
                if dw is not None:
                    ctx.accumulate_grad(w, dw)
                if db is not None:
                    ctx.accumulate_grad(bias, db)
            if x12.requires_grad:
                dact, _, _ = gd_linear_backward(ctx, act, w, bias, g, True, False, False)
                ctx.accumulate_grad(x12, _swiglu_split_backward(ctx, x12, dact))
        ctx.record(backward)
    return y


# --------------------------------------------------------------------------- rope / attention
def gd_qkv_split_rope(ctx: Context, qkv: Tensor, positions: Tensor, n_heads: int, head_dim: int,
                      theta: float = 10000.0, interleaved: bool = False):
    """qkv [N, 3*H*Dh] -> q, k (rotated), v [N, H, Dh] (src/ops/qkv_split_rope/core_qkv_split_rope.c:148,184)."""
    n = qkv.shape[0]
    args = abi.RopeArgs(theta, head_dim, 1 if interleaved else 0)
    q = ctx.scratch_empty(qkv.dtype, (n, n_heads, head_dim), "q")
    k = ctx.scratch_empty(qkv.dtype, (n, n_heads, head_dim), "k")
    v = ctx.scratch_empty(qkv.dtype, (n, n_heads, head_dim), "v")
    ctx.check(ctx.lib.gd_backend_qkv_split_rope_forward(ctx.backend, _tvp(qkv), _tvp(positions), _tvp(q), _tvp(k), _tvp(v),
                                                        n_heads, head_dim, byref(args)), "qkv_split_rope_forward")
    for t in (q, k, v):
        t.requires_grad = qkv.requires_grad
    if qkv.requires_grad:
        def backward():
            if q.grad is None and k.grad is None and v.grad is None:
                return
            gs = []
            for t in (q, k, v):
                gs.append(t.grad if t.grad is not None else ctx.zeros(ctx.scratch, t.dtype, t.shape, "zero_grad"))
            dqkv = ctx.scratch_empty(qkv.dtype, qkv.shape, "d_qkv")
            ctx.check(ctx.lib.gd_backend_qkv_split_rope_backward(ctx.backend, _tvp(gs[0]), _tvp(gs[1]), _tvp(gs[2]), _tvp(positions),
                                                                 _tvp(dqkv), n_heads, head_dim, byref(args)), "qkv_split_rope_backward")
            ctx.accumulate_grad(qkv, dqkv)
        ctx.record(backward)
    return q, k, v


def gd_sdpa_varlen(ctx: Context, q: Tensor, k: Tensor, v: Tensor, cu_seqlens: Tensor, *, scale: float = 0.0,
                   causal: bool = True, sliding_window: int = 0, prefix_len: int = 0, max_seqlen: int = 0) -> Tensor:
    """Packed causal/windowed attention (src/ops/sdpa_varlen/core_sdpa_varlen.c:167,272). Forward
    statistics [N, H, 3] are saved when a gradient is needed; scale <= 0 means 1/sqrt(Dh)
    computed in double (:48-51); max_seqlen == 0 means N (:37-42)."""
    n, hq, dh = q.shape
    if scale <= 0.0:
        scale = float(1.0 / math.sqrt(float(dh)))
    args = abi.SdpaVarlenArgs(scale, 1 if causal else 0, sliding_window, prefix_len, max_seqlen or n, 0)
    needs = ctx.grad_enabled and (q.requires_grad or k.requires_grad or v.requires_grad)
    out = ctx.scratch_empty(q.dtype, q.shape, "attn")
    stats = ctx.scratch_empty(F32, (n, hq, 3), "attn_stats") if needs else None
    ctx.check(ctx.lib.gd_backend_sdpa_varlen(ctx.backend, _tvp(q), _tvp(k), _tvp(v), _tvp(cu_seqlens), _tvp(out), _tvp(stats),
                                             byref(args)), "sdpa_varlen")
    out.requires_grad = needs
    if needs:
        def backward():
            if out.grad is None:
                return
            dq = ctx.scratch_empty(q.dtype, q.shape, "dq")
            dk = ctx.scratch_empty(k.dtype, k.shape, "dk")
            dv = ctx.scratch_empty(v.dtype, v.shape, "dv")
            bargs = abi.SdpaVarlenArgs(scale, args.causal, sliding_window, prefix_len, args.max_seqlen, 1)
            if SDPA_BACKWARD_WITH_OUTPUT:
                # the capsule still holds the forward output: the additive entry runs one attention pass where it can
                acc = ctx.scratch_empty(F32, q.shape, "dq_accum")
                ctx.check(ctx.lib.gdb200_sdpa_varlen_backward_with_output(ctx.backend, _tvp(out.grad), _tvp(q), _tvp(k), _tvp(v), _tvp(cu_seqlens),
                                                                          _tvp(out), _tvp(dq), _tvp(dk), _tvp(dv), _tvp(stats), _tvp(acc),
                                                                          byref(bargs)), "sdpa_varlen_backward")
            else:
                ctx.check(ctx.lib.gd_backend_sdpa_varlen_backward(ctx.backend, _tvp(out.grad), _tvp(q), _tvp(k), _tvp(v), _tvp(cu_seqlens),
                                                                  _tvp(dq), _tvp(dk), _tvp(dv), _tvp(stats), byref(bargs)), "sdpa_varlen_backward")
            ctx.accumulate_grad(q, dq)
            ctx.accumulate_grad(k, dk)
            ctx.accumulate_grad(v, dv)
        ctx.record(backward)
    return out


def gd_kv_cache_append_packed(ctx: Context, k_cache: Tensor, v_cache: Tensor, cache_pos: Tensor, cu_seqlens: Tensor,
                              k_new: Tensor, v_new: Tensor) -> None:
    """Append packed rows [N, H, Dh] at cache_pos[b] + t (src/ops/kv_cache_append/core_kv_cache_append.c:302)."""
    a = abi.KvCacheAppendArgs(0)
    ctx.check(ctx.lib.gd_backend_kv_cache_append_packed(ctx.backend, _tvp(k_cache), _tvp(v_cache), _tvp(cache_pos), _tvp(cu_seqlens),
                                                        _tvp(k_new), _tvp(v_new), byref(a)), "kv_cache_append_packed")


def gd_kv_cache_append_positions(ctx: Context, k_cache: Tensor, v_cache: Tensor, cache_pos: Tensor, k_new: Tensor, v_new: Tensor) -> None:
    """Append [B, Tnew, H, Dh] rows at per-batch positions (core_kv_cache_append.c:345)."""
    a = abi.KvCacheAppendArgs(0)
    ctx.check(ctx.lib.gd_backend_kv_cache_append_positions(ctx.backend, _tvp(k_cache), _tvp(v_cache), _tvp(cache_pos), _tvp(k_new),
                                                           _tvp(v_new), byref(a)), "kv_cache_append_positions")


def gd_sdpa_decode_positions(ctx: Context, q: Tensor, k_cache: Tensor, v_cache: Tensor, cache_pos: Tensor, *,
                             scale: float = 0.0, sliding_window: int = 0, prefix_len: int = 0) -> Tensor:
    """q [B, Tq, H, Dh] against the caches with live keys [0, pos[b] + Tq) (src/ops/sdpa_decode/core_sdpa_decode.c:315)."""
    if scale <= 0.0:
        scale = float(1.0 / math.sqrt(float(q.shape[-1])))
    a = abi.SdpaDecodeArgs(scale, sliding_window, prefix_len, 0)
    out = ctx.scratch_empty(q.dtype, q.shape, "decode_attn")
    ctx.check(ctx.lib.gd_backend_sdpa_decode_positions(ctx.backend, _tvp(q), _tvp(k_cache), _tvp(v_cache), _tvp(cache_pos), _tvp(out),
                                                       byref(a)), "sdpa_decode_positions")
    return out


# --------------------------------------------------------------------------- fused LM cross entropy
def lm_ce_chunk_classes(classes: int) -> int:
    env = os.environ.get("GD_LM_CE_CHUNK_SIZE", "")
    chunk = int(env) if env.isdigit() and int(env) != 0 else LM_CE_DEFAULT_CHUNK
    return max(1, min(chunk, classes))


def gd_lm_cross_entropy_softcapped_bias_ignore(ctx: Context, hidden: Tensor, weight: Tensor, bias: Optional[Tensor],
                                               targets: Tensor, logits_softcap: float, ignore_index: int,
                                               shard_share: float = 1.0) -> Tensor:
    """Mean cross entropy of softcap(hidden w^T + b) against targets, computed chunk by chunk
    over the vocabulary with an online (max, sum) merge; returns a scalar F32 tensor
    (src/ops/lm_cross_entropy/core_lm_cross_entropy.c:452-675, backward :676-974).
    `shard_share` = valid target rows of this batch / valid target rows of the global batch it is a shard of:
    loss and 1/valid_count are multiplied by it, so the loss is the shard's share of the global mean and the
    backward pass divides by the global count (data parallelism; 1.0 = the reference's local normaliser)."""
    lib = ctx.lib
    rows, k = _flat2(hidden)
    n = weight.shape[0]
    row_loss = ctx.zeros(ctx.scratch, F32, (rows,), "row_loss")
    row_max = ctx.scratch_empty(F32, (rows,), "row_max")
    ctx.fill(row_max, F32_NEG_INF_PATTERN)
    row_inv_sum = ctx.zeros(ctx.scratch, F32, (rows,), "row_inv_sum")
    row_valid = ctx.zeros(ctx.scratch, F32, (rows,), "row_valid")
    inv_valid = ctx.scratch_empty(F32, (), "inv_valid_count")
    loss = ctx.scratch_empty(F32, (), "loss")
    needs = ctx.grad_enabled and (hidden.requires_grad or weight.requires_grad or (bias is not None and bias.requires_grad))
    chunk = lm_ce_chunk_classes(n)
    single = chunk >= n
    saved_logits = None
    scratch_mark = ctx.scratch.top
    for start in range(0, n, chunk):
        cc = min(chunk, n - start)
        if not (needs and single):
            ctx.scratch.top = scratch_mark  # chunk logits are freed after the update
        logits = ctx.scratch_empty(hidden.dtype, (rows, cc), "logits_chunk")
        _matmul(ctx, lib.gd_backend_matmul_nt, hidden.mv(rows, k), weight.mv(cc, k, row_offset=start), logits.mv(rows, cc), "matmul_nt(logits)")
        bvp = None
        if bias is not None:
            bchunk = Tensor(ctx, bias.arena, bias.offset + start * abi.DTYPE_SIZE[bias.dtype], bias.dtype, (cc,))
            bvp = _tvp(bchunk)
        ctx.check(lib.gd_backend_lm_cross_entropy_online_update(ctx.backend, _tvp(logits), bvp, _tvp(targets), _tvp(row_loss), _tvp(row_max),
                                                                _tvp(row_inv_sum), start, n, logits_softcap), "lm_ce_online_update")
        if needs and single:
            saved_logits = logits
    ctx.check(lib.gd_backend_lm_cross_entropy_finalize(ctx.backend, _tvp(targets), _tvp(row_loss), _tvp(row_max), _tvp(row_inv_sum),
                                                       _tvp(row_valid), n, ignore_index), "lm_ce_finalize")
    ctx.check(lib.gd_backend_lm_cross_entropy_reduce_normalize(ctx.backend, _tvp(row_loss), _tvp(row_valid), _tvp(loss), _tvp(inv_valid)), "lm_ce_reduce_normalize")
    if shard_share != 1.0:
        for t in (loss, inv_valid):
            ctx.check(lib.gd_backend_scale(ctx.backend, t.buffer, t.offset, t.buffer, t.offset, 1, F32, float(shard_share)), "scale(shard share)")
    loss.requires_grad = needs
    if needs:
        def backward():
            g = loss.grad
            if g is None:
                return
            need_h, need_w = hidden.requires_grad, weight.requires_grad
            need_b = bias is not None and bias.requires_grad
            dh = dw = db = None
            if need_h:
                dh = ctx.scratch_empty(hidden.dtype, hidden.shape, "d_hidden") if single else ctx.zeros(ctx.scratch, hidden.dtype, hidden.shape, "d_hidden")
                partial = None if single else ctx.scratch_empty(hidden.dtype, hidden.shape, "d_hidden_part")
            if need_w:
                dw = ctx.scratch_empty(weight.dtype, weight.shape, "d_lm_w")
            if need_b:
                db = ctx.scratch_empty(bias.dtype, bias.shape, "d_lm_b")
            for start in range(0, n, chunk):
                cc = min(chunk, n - start)
                if saved_logits is not None and single:
                    logits = saved_logits
                else:
                    logits = ctx.scratch_empty(hidden.dtype, (rows, cc), "logits_chunk_bwd")
                    _matmul(ctx, lib.gd_backend_matmul_nt, hidden.mv(rows, k), weight.mv(cc, k, row_offset=start), logits.mv(rows, cc), "matmul_nt(logits bwd)")
                bvp = None
                if bias is not None:
                    bchunk = Tensor(ctx, bias.arena, bias.offset + start * abi.DTYPE_SIZE[bias.dtype], bias.dtype, (cc,))
                    bvp = _tvp(bchunk)
                # dlogits overwrite the logits chunk in place (core_lm_cross_entropy.c:876-890)
                ctx.check(lib.gd_backend_lm_cross_entropy_backward_chunk(ctx.backend, _tvp(logits), bvp, _tvp(targets), _tvp(row_max), _tvp(row_inv_sum),
                                                                         _tvp(g), _tvp(inv_valid), _tvp(logits), start, n, 1.0, logits_softcap,
                                                                         ignore_index), "lm_ce_backward_chunk")
                if need_h:
                    dst = dh if single else partial
                    _matmul(ctx, lib.gd_backend_matmul, logits.mv(rows, cc), weight.mv(cc, k, row_offset=start), dst.mv(rows, k), "matmul(d_hidden)")
                    if not single:
                        ctx.check(lib.gd_backend_accumulate(ctx.backend, dh.buffer, dh.offset, partial.buffer, partial.offset, dh.count, dh.dtype), "accumulate")
                if need_w:
                    _matmul(ctx, lib.gd_backend_matmul_tn, logits.mv(rows, cc), hidden.mv(rows, k), dw.mv(cc, k, row_offset=start), "matmul_tn(d_lm_w)")
                if need_b:
                    mv, vv = logits.mv(rows, cc), db.vv(start, cc)
                    ctx.check(lib.gd_backend_reduce_rows(ctx.backend, byref(mv), byref(vv)), "reduce_rows(d_lm_b)")
            if dh is not None:
                ctx.accumulate_grad(hidden, dh)
            if dw is not None:
                ctx.accumulate_grad(weight, dw)
            if db is not None:
                ctx.accumulate_grad(bias, db)
        ctx.record(backward)
    return loss
