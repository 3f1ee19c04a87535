"""CPU oracle for the gpt_lm hot path: PyTorch-CPU / numpy restatements of every op.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module; it is used by
tests/, by the smoke check and by bench.py's CPU-baseline and reference arms as the checker.

Style follows the reference's own oracle scripts (FP32 math on CPU, results rounded to the
storage dtype at the points where the reference stores a tensor): src/ops/linear/fwd.py:120-183,
src/ops/rms_norm/fwd.py, src/ops/dropout/fwd.py:140-150 (numpy splitmix64 mask),
src/ops/embedding/fwd.py. Ops that have no oracle script in the reference restate the CPU
references embedded in its C tests and the arithmetic of its Metal kernels; each function
names the lines it follows.

Parity pin: the functions here are checked against (a) the reference-side functions of the
reference's own oracle scripts imported from the reference tree and (b) the CPU reference
functions of the reference's C tests compiled from the reference tree (oracle/ref_harness.c);
the resulting vectors are committed under tests/golden/ (see tests/golden/make_golden.py).

Tensors are torch.float32 CPU tensors holding values that are exactly representable in the
storage dtype ("f16" or "bf16"); integer tensors are int32/int64.
"""
from __future__ import annotations

import math

import numpy as np
import torch

MASK64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def rnd(x: torch.Tensor, dtype: str = "f16") -> torch.Tensor:
    """Round FP32 values to the storage grid and return them as FP32."""
    if dtype == "f16":
        return x.to(torch.float16).to(torch.float32)
    if dtype == "bf16":
        return x.to(torch.bfloat16).to(torch.float32)
    return x.to(torch.float32)


# --------------------------------------------------------------------------- integer helpers
def splitmix64(x: np.ndarray) -> np.ndarray:
    """src/backends/metal/primitives/random/metal_random.metal:8-14 (uint64 wrap-around)."""
    with np.errstate(over="ignore"):
        x = (x.astype(np.uint64) + np.uint64(0x9E3779B97F4A7C15))
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def dropout_threshold(p: float) -> int:
    """src/ops/dropout/metal_dropout.m:145-155; p is the float32 probability."""
    t = math.ceil(float(np.float32(p)) * 16777216.0)
    return 0 if t <= 0 else (16777216 if t >= 16777216 else int(t))


def dropout_keep_mask(count: int, p: float, seed: int) -> np.ndarray:
    """keep[i] = top-24 bits of splitmix64(seed + i) >= ceil(p * 2^24) (metal_dropout.metal:14-19)."""
    with np.errstate(over="ignore"):
        idx = np.arange(count, dtype=np.uint64) + np.uint64(seed & 0xFFFFFFFFFFFFFFFF)
    r = splitmix64(idx)
    mant = ((r >> np.uint64(40)) & np.uint64(0xFFFFFF)).astype(np.int64)
    return (mant >= dropout_threshold(p)).astype(np.uint8)


def rand_uniform(count: int, seed: int, low: float, high: float) -> np.ndarray:
    """metal_random.metal:16-30: u = mant24 / 2^24, v = low + (high - low) * u in FP32."""
    with np.errstate(over="ignore"):
        idx = np.arange(count, dtype=np.uint64) + np.uint64(seed & 0xFFFFFFFFFFFFFFFF)
    mant = ((splitmix64(idx) >> np.uint64(40)) & np.uint64(0xFFFFFF)).astype(np.float32)
    u = mant * np.float32(1.0 / 16777216.0)
    return (np.float32(low) + (np.float32(high) - np.float32(low)) * u).astype(np.float32)


def mask_allowed(i: np.ndarray, j: np.ndarray, causal: bool, window: int, prefix: int) -> np.ndarray:
    """Attention mask rule, src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55 (vectorised)."""
    ok = np.ones(np.broadcast(i, j).shape, dtype=bool)
    if causal:
        if prefix > 0:
            ok &= np.where(i < prefix, j < prefix, j <= i)
        else:
            ok &= j <= i
    if window > 0:
        if prefix > 0:
            ok &= ~((i >= prefix) & (j >= prefix) & ((i - j) >= window))
        else:
            ok &= (i - j) < window
    return ok


# --------------------------------------------------------------------------- embedding / dropout
def embedding_forward(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """src/ops/embedding/metal_embedding.metal:60-83: invalid ids give NaN rows."""
    vocab = table.shape[0]
    ids = ids.to(torch.int64)
    bad = (ids < 0) | (ids >= vocab)
    out = table[ids.clamp(0, vocab - 1)].clone()
    out[bad] = float("nan")
    return out


def embedding_backward(grad_out: torch.Tensor, ids: torch.Tensor, vocab: int, dtype: str = "f16") -> torch.Tensor:
    """FP32 scatter-add then one rounding (metal_embedding.metal:109-179); invalid ids skipped."""
    ids = ids.to(torch.int64)
    ok = (ids >= 0) & (ids < vocab)
    acc = torch.zeros((vocab, grad_out.shape[1]), dtype=torch.float32)
    acc.index_add_(0, ids[ok], grad_out[ok])
    return rnd(acc, dtype)


def dropout_forward(x: torch.Tensor, p: float, seed: int, dtype: str = "f16"):
    """y = round(x / (1 - p)) where kept else 0, plus the u8 mask (metal_dropout.metal:21-30)."""
    keep = torch.from_numpy(dropout_keep_mask(x.numel(), p, seed)).reshape(x.shape)
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(p))
    y = torch.where(keep.bool(), rnd(x * float(scale), dtype), torch.zeros_like(x))
    return y, keep


def dropout_add_forward(residual: torch.Tensor, x: torch.Tensor, p: float, seed: int, dtype: str = "f16"):
    """y = residual + dropout(x): the dropped value is rounded first, then the sum is rounded
    (metal_dropout.metal:129-140)."""
    dropped, keep = dropout_forward(x, p, seed, dtype)
    return rnd(residual + dropped, dtype), keep


def dropout_backward_mask(mask: torch.Tensor, grad_out: torch.Tensor, scale: float, dtype: str = "f16") -> torch.Tensor:
    return torch.where(mask.bool(), rnd(grad_out * float(np.float32(scale)), dtype), torch.zeros_like(grad_out))


# --------------------------------------------------------------------------- RMSNorm
def rms_norm_forward(x: torch.Tensor, w: torch.Tensor, eps: float, dtype: str = "f16"):
    """src/ops/rms_norm/metal_rms_norm.metal:29-66: inv = rsqrt(mean(x^2) + eps), y = x * w * inv."""
    inv = torch.rsqrt((x * x).sum(dim=-1) / x.shape[-1] + eps)
    return rnd(x * w * inv[..., None], dtype), inv


def rms_norm_backward(x, w, inv, g, dtype: str = "f16"):
    """dx = inv * g * w - x * inv^3 / cols * sum(g * w * x) (:225-262); dw = sum_rows g * x * inv (:414-447)."""
    cols = x.shape[-1]
    a = (g * w * x).sum(dim=-1, keepdim=True)
    inv_ = inv[..., None]
    dx = inv_ * g * w - x * (inv_ ** 3 / cols) * a
    dw = (g * x * inv_).reshape(-1, cols).sum(dim=0)
    return rnd(dx, dtype), rnd(dw, dtype)


# --------------------------------------------------------------------------- linear family
def linear_transposed_weight_forward(x, w, bias, dtype: str = "f16"):
    """y = round(round(x w^T) + b): GEMM result rounded, bias added by a separate rounded add
    (src/ops/linear_transposed_weight/core_linear_transposed_weight.c:51-79)."""
    y = rnd(x @ w.t(), dtype)
    return rnd(y + bias, dtype) if bias is not None else y


def linear_transposed_weight_backward(x, w, g, dtype: str = "f16"):
    """dX = dY w, dW = dY^T x, db = sum_rows dY (core_linear_transposed_weight_bwd.c:104-160)."""
    return rnd(g @ w, dtype), rnd(g.t() @ x, dtype), rnd(g.sum(dim=0), dtype)


def linear_forward(x, w, bias, dtype: str = "f16"):
    """y = round(x w + b), bias added in FP32 before the single rounding, w stored [K, N]
    (src/ops/_shared/gemm/metal_gemm_common.h:124-133; src/ops/linear/fwd.py:120-126)."""
    y = x @ w
    return rnd(y + bias if bias is not None else y, dtype)


def linear_backward(x, w, g, dtype: str = "f16"):
    """dX = dY w^T, dW = x^T dY, db = sum_rows dY (src/ops/linear/core_linear_bwd.c:100-140)."""
    return rnd(g @ w.t(), dtype), rnd(x.t() @ g, dtype), rnd(g.sum(dim=0), dtype)


# --------------------------------------------------------------------------- SwiGLU
def _sigmoid(z: torch.Tensor) -> torch.Tensor:
    e = torch.exp(-z.abs())
    inv = 1.0 / (1.0 + e)
    return torch.where(z >= 0, inv, e * inv)  # metal_swiglu.metal:11-16


def swiglu_split_forward(x12: torch.Tensor, dtype: str = "f16") -> torch.Tensor:
    """out = x1 * (x2 * sigmoid(x2)), x12 = [x1 | x2] (src/ops/swiglu/metal_swiglu.metal:18-34,94-116)."""
    h = x12.shape[-1] // 2
    x1, x2 = x12[..., :h], x12[..., h:]
    return rnd(x1 * (x2 * _sigmoid(x2)), dtype)


def swiglu_split_backward(x12: torch.Tensor, go: torch.Tensor, dtype: str = "f16") -> torch.Tensor:
    """dx1 = go * gate, dx2 = go * x1 * s * (1 + z * (1 - s)) (metal_swiglu.metal:18-52)."""
    h = x12.shape[-1] // 2
    x1, z = x12[..., :h], x12[..., h:]
    s = _sigmoid(z)
    return torch.cat([rnd(go * (z * s), dtype), rnd(go * x1 * (s * (1.0 + z * (1.0 - s))), dtype)], dim=-1)


# --------------------------------------------------------------------------- RoPE
def rope_cos_sin(positions: torch.Tensor, n_dims: int, theta: float):
    """angle = pos * 2^(pair * (-2 log2(theta) / n_dims)), all in FP32
    (src/ops/qkv_split_rope/metal_qkv_split_rope.metal:6-11, metal_qkv_split_rope.m:228)."""
    freq_scale = np.float32(-2.0) * np.float32(np.log2(np.float32(theta))) / np.float32(n_dims)
    pair = torch.arange(n_dims // 2, dtype=torch.float32)
    inv = torch.exp2(pair * float(freq_scale))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang), torch.sin(ang)


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    # x [N, H, Dh]; NeoX pairs (c, c + Dh/2) or interleaved pairs (2c, 2c + 1) (metal :13-25)
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
    else:
        half = x.shape[-1] // 2
        a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    ra, rb = a * c - b * s, a * s + b * c
    if interleaved:
        return torch.stack([ra, rb], dim=-1).reshape(x.shape)
    return torch.cat([ra, rb], dim=-1)


def qkv_split_rope_forward(qkv, positions, n_heads: int, head_dim: int, theta: float = 10000.0,
                           interleaved: bool = False, dtype: str = "f16"):
    """qkv [N, 3*H*Dh] = [Q | K | V] per token -> q, k rotated, v copied (metal :57-104)."""
    n = qkv.shape[0]
    q, k, v = (t.reshape(n, n_heads, head_dim) for t in qkv.split(n_heads * head_dim, dim=1))
    cos, sin = rope_cos_sin(positions, head_dim, theta)
    return rnd(_rotate(q, cos, sin, interleaved), dtype), rnd(_rotate(k, cos, sin, interleaved), dtype), v.clone()


def qkv_split_rope_backward(gq, gk, gv, positions, theta: float = 10000.0, interleaved: bool = False, dtype: str = "f16"):
    """Same rotation with sin_sign = -1, re-packed to [N, 3*H*Dh] (metal :106-160)."""
    n, h, dh = gq.shape
    cos, sin = rope_cos_sin(positions, dh, theta)
    dq, dk = rnd(_rotate(gq, cos, -sin, interleaved), dtype), rnd(_rotate(gk, cos, -sin, interleaved), dtype)
    return torch.cat([dq.reshape(n, -1), dk.reshape(n, -1), gv.reshape(n, -1)], dim=1)


# --------------------------------------------------------------------------- attention
def _segment_mask(t: int, causal: bool, window: int, prefix: int) -> torch.Tensor:
    i = np.arange(t)[:, None]
    j = np.arange(t)[None, :]
    return torch.from_numpy(mask_allowed(i, j, causal, window, prefix))


def sdpa_varlen_forward(q, k, v, cu_seqlens, scale: float = 0.0, causal: bool = True, window: int = 0,
                        prefix: int = 0, dtype: str = "f16"):
    """Packed attention per (segment, head) with FP32 softmax; rows with no allowed key give zeros
    (tests/test_sdpa_varlen.c:158-230, metal_sdpa_varlen.metal:137-228). Returns (out, stats) with
    stats [N, Hq, 2] = (row max of scaled scores, sum of exp)."""
    n, hq, dh = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    if scale <= 0.0:
        scale = float(np.float32(1.0 / math.sqrt(float(dh))))
    out = torch.zeros_like(q)
    stats = torch.zeros((n, hq, 2), dtype=torch.float32)
    cu = [int(c) for c in cu_seqlens]
    for b in range(len(cu) - 1):
        s0, s1 = cu[b], cu[b + 1]
        t = s1 - s0
        if t <= 0:
            continue
        allowed = _segment_mask(t, causal, window, prefix)
        qs = q[s0:s1].transpose(0, 1)                                  # [Hq, T, Dh]
        ks = k[s0:s1].transpose(0, 1).repeat_interleave(group, dim=0)  # [Hq, T, Dh]
        vs = v[s0:s1].transpose(0, 1).repeat_interleave(group, dim=0)
        s = (qs @ ks.transpose(1, 2)) * scale
        s = s.masked_fill(~allowed[None], float("-inf"))
        m = s.max(dim=-1).values
        any_key = allowed.any(dim=-1)[None].expand_as(m)
        m_safe = torch.where(any_key, m, torch.zeros_like(m))
        e = torch.exp(s - m_safe[..., None])
        e = torch.where(allowed[None], e, torch.zeros_like(e))
        l = e.sum(dim=-1)
        o = (e @ vs) / torch.where(l > 0, l, torch.ones_like(l))[..., None]
        o = torch.where((l > 0)[..., None], o, torch.zeros_like(o))
        out[s0:s1] = o.transpose(0, 1)
        stats[s0:s1, :, 0] = torch.where(any_key, m, torch.full_like(m, float("-inf"))).transpose(0, 1)
        stats[s0:s1, :, 1] = l.transpose(0, 1)
    return rnd(out, dtype), stats


def sdpa_varlen_backward(go, q, k, v, cu_seqlens, scale: float = 0.0, causal: bool = True, window: int = 0,
                         prefix: int = 0, dtype: str = "f16"):
    """D = sum_j P dP, dS = P (dP - D), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO, group heads
    summed into their KV head (tests/test_sdpa_varlen.c:232-371, metal_sdpa_varlen.metal:230-533)."""
    n, hq, dh = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    if scale <= 0.0:
        scale = float(np.float32(1.0 / math.sqrt(float(dh))))
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    cu = [int(c) for c in cu_seqlens]
    for b in range(len(cu) - 1):
        s0, s1 = cu[b], cu[b + 1]
        t = s1 - s0
        if t <= 0:
            continue
        allowed = _segment_mask(t, causal, window, prefix)
        qs = q[s0:s1].transpose(0, 1)
        ks = k[s0:s1].transpose(0, 1).repeat_interleave(group, dim=0)
        vs = v[s0:s1].transpose(0, 1).repeat_interleave(group, dim=0)
        gs = go[s0:s1].transpose(0, 1)
        s = (qs @ ks.transpose(1, 2)) * scale
        s = s.masked_fill(~allowed[None], float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        e = torch.where(allowed[None], torch.exp(s - m), torch.zeros_like(s))
        l = e.sum(dim=-1, keepdim=True)
        p = e / torch.where(l > 0, l, torch.ones_like(l))
        dp = gs @ vs.transpose(1, 2)
        d = (p * dp).sum(dim=-1, keepdim=True)
        ds = p * (dp - d) * scale
        dq[s0:s1] = (ds @ ks).transpose(0, 1)
        dkh = ds.transpose(1, 2) @ qs        # [Hq, T, Dh]
        dvh = p.transpose(1, 2) @ gs
        dk[s0:s1] = dkh.reshape(hkv, group, t, dh).sum(dim=1).transpose(0, 1)
        dv[s0:s1] = dvh.reshape(hkv, group, t, dh).sum(dim=1).transpose(0, 1)
    return rnd(dq, dtype), rnd(dk, dtype), rnd(dv, dtype)


def kv_cache_append(k_cache, v_cache, k_new, v_new, cache_pos, cu_seqlens=None):
    """In-place append; packed form when cu_seqlens is given. Rows whose destination would exceed
    the capacity are dropped for the whole sequence (src/ops/kv_cache_append/metal_kv_cache_append.metal:30-122)."""
    b, tmax = k_cache.shape[0], k_cache.shape[1]
    for i in range(b):
        pos = int(cache_pos[i]) if hasattr(cache_pos, "__len__") else int(cache_pos)
        if cu_seqlens is not None:
            s0, s1 = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
            rows_k, rows_v = k_new[s0:s1], v_new[s0:s1]
        else:
            rows_k, rows_v = k_new[i], v_new[i]
        t = rows_k.shape[0]
        if pos < 0 or pos + t > tmax:
            continue
        k_cache[i, pos:pos + t] = rows_k
        v_cache[i, pos:pos + t] = rows_v


def sdpa_decode(q, k_cache, v_cache, cache_pos, scale: float = 0.0, window: int = 0, prefix: int = 0, dtype: str = "f16"):
    """q [B, Tq, Hq, Dh] against cache rows [0, pos + Tq); query t sits at position pos + t
    (tests/test_sdpa_varlen.c:604-677, src/ops/sdpa_decode/metal_sdpa_decode.metal:31-281)."""
    bsz, tq, hq, dh = q.shape
    tmax, hkv = k_cache.shape[1], k_cache.shape[2]
    group = hq // hkv
    if scale <= 0.0:
        scale = float(np.float32(1.0 / math.sqrt(float(dh))))
    out = torch.zeros_like(q)
    for b in range(bsz):
        pos = int(cache_pos[b]) if hasattr(cache_pos, "__len__") else int(cache_pos)
        if pos < 0:
            continue
        live = min(pos + tq, tmax)
        i = (pos + np.arange(tq))[:, None]
        j = np.arange(live)[None, :]
        allowed = torch.from_numpy(mask_allowed(i, j, True, window, prefix))
        qs = q[b].transpose(0, 1)
        ks = k_cache[b, :live].transpose(0, 1).repeat_interleave(group, dim=0)
        vs = v_cache[b, :live].transpose(0, 1).repeat_interleave(group, dim=0)
        s = ((qs @ ks.transpose(1, 2)) * scale).masked_fill(~allowed[None], float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        e = torch.where(allowed[None], torch.exp(s - m), torch.zeros_like(s))
        l = e.sum(dim=-1, keepdim=True)
        o = (e @ vs) / torch.where(l > 0, l, torch.ones_like(l))
        out[b] = torch.where(l > 0, o, torch.zeros_like(o)).transpose(0, 1)
    return rnd(out, dtype)


# --------------------------------------------------------------------------- fused LM cross entropy
def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """cap * tanh(x / cap) with the linear branch below 2^-12 (metal_lm_cross_entropy.metal:13-31)."""
    if cap <= 0.0:
        return x
    y = x * float(np.float32(1.0) / np.float32(cap))
    ay = y.abs()
    e = torch.exp(-2.0 * ay)
    t = (1.0 - e) / (1.0 + e)
    t = torch.where(y < 0, -t, t)
    t = torch.where(ay < 0.000244140625, y, t)
    return cap * t


def lm_cross_entropy_forward(hidden, weight, bias, targets, cap: float, ignore_index: int, dtype: str = "f16"):
    """Mean over valid rows of logsumexp(soft) - soft[target], soft = softcap(round(round(h w^T) + b))
    (metal_lm_cross_entropy.metal:89-252; tests/test_lm_cross_entropy.c:168-296). Returns a dict
    with the loss and the saved statistics."""
    return lm_cross_entropy_from_logits(rnd(hidden @ weight.t(), dtype), bias, targets, cap, ignore_index, dtype)


def lm_cross_entropy_from_logits(logits, bias, targets, cap: float, ignore_index: int, dtype: str = "f16"):
    """The statistics of lm_cross_entropy_forward from storage-precision matmul logits [rows, classes] that hold all classes."""
    raw = rnd(logits + bias, dtype) if bias is not None else logits
    soft = softcap(raw, cap)
    tg = targets.to(torch.int64)
    v = logits.shape[-1]
    ignored = (tg < 0) | (tg == ignore_index)
    oob = (~ignored) & (tg >= v)
    m = soft.max(dim=-1).values
    ssum = torch.exp(soft - m[:, None]).sum(dim=-1)
    tl = soft.gather(1, tg.clamp(0, v - 1)[:, None])[:, 0]
    row_loss = torch.log(ssum) + m - tl
    row_loss = torch.where(ignored, torch.zeros_like(row_loss), row_loss)
    row_loss = torch.where(oob, torch.full_like(row_loss, float("nan")), row_loss)
    valid = (~ignored).to(torch.float32)
    count = valid.sum()
    inv = (1.0 / count) if count > 0 else torch.tensor(0.0)
    loss = row_loss.sum() * inv if count > 0 else torch.tensor(float("nan"))
    return {"loss": loss.to(torch.float32), "soft": soft, "row_max": m, "row_inv_sum": 1.0 / ssum, "row_loss": row_loss,
            "inv_valid": torch.as_tensor(inv, dtype=torch.float32), "ignored": ignored | oob}


def lm_cross_entropy_dlogits(targets, saved, grad_loss: float, cap: float, dtype: str = "f16"):
    """dlogits = (p - onehot) * max(0, 1 - (soft/cap)^2) * grad * inv_valid stored in the storage
    dtype (metal_lm_cross_entropy.metal:254-311); zero for rows without a usable target."""
    soft = saved["soft"]
    tg = targets.to(torch.int64)
    p = torch.exp(soft - saved["row_max"][:, None]) * saved["row_inv_sum"][:, None]
    onehot = torch.zeros_like(p)
    okrows = ~saved["ignored"]
    onehot[okrows, tg[okrows]] = 1.0
    g = p - onehot
    if cap > 0.0:
        y = soft * float(np.float32(1.0) / np.float32(cap))
        g = g * torch.clamp(1.0 - y * y, min=0.0)
    seed = float(np.float32(grad_loss)) * float(saved["inv_valid"])
    g = rnd(g * seed, dtype)
    g[saved["ignored"]] = 0.0
    return g


def lm_cross_entropy_backward(hidden, weight, bias, targets, saved, grad_loss: float, cap: float, dtype: str = "f16"):
    """dlogits (lm_cross_entropy_dlogits), then dh = dlogits w, dW = dlogits^T h, db = sum_rows dlogits
    (core_lm_cross_entropy.c:876-974)."""
    g = lm_cross_entropy_dlogits(targets, saved, grad_loss, cap, dtype)
    dh = rnd(g @ weight, dtype)
    dw = rnd(g.t() @ hidden, dtype)
    db = rnd(g.sum(dim=0), dtype) if bias is not None else None
    return dh, dw, db


# --------------------------------------------------------------------------- AMP / clip / AdamW
def amp_begin_step(state: dict, cfg: dict) -> None:
    """metal_amp.metal:59-69."""
    s = np.float32(min(max(state["scale"], cfg["min_scale"]), cfg["max_scale"]))
    state["scale"], state["inv_scale"], state["found_inf"] = s, np.float32(1.0) / s, 0


def amp_finish_step(state: dict, cfg: dict) -> None:
    """metal_amp.metal:71-95: back off on overflow, grow after growth_interval clean steps."""
    found = state["found_inf"] != 0
    s, tracker = np.float32(state["scale"]), state["growth_tracker"]
    state["last_found_inf"] = 1 if found else 0
    if found:
        s, tracker = max(np.float32(s * np.float32(cfg["backoff_factor"])), np.float32(cfg["min_scale"])), 0
    else:
        tracker += 1
        if tracker >= cfg["growth_interval"]:
            s, tracker = min(np.float32(s * np.float32(cfg["growth_factor"])), np.float32(cfg["max_scale"])), 0
    state["scale"], state["inv_scale"], state["growth_tracker"] = np.float32(s), np.float32(1.0) / np.float32(s), tracker


def grad_clip_scale(grads: list, inv_scale: float, max_norm: float, eps: float = 1.0e-6):
    """norm = sqrt(sum (g * inv_scale)^2); clip = min(1, max_norm / (norm + eps)), 0 when the norm
    is not finite; returns (clip * inv_scale, norm, found_inf) (metal_adamw.metal:197-270)."""
    total = torch.zeros((), dtype=torch.float32)
    found = False
    for g in grads:
        gg = g.to(torch.float32) * float(np.float32(inv_scale))
        found = found or not bool(torch.isfinite(gg).all())
        total = total + (gg * gg).sum()
    norm = torch.sqrt(total)
    if not bool(torch.isfinite(norm)):
        clip = 0.0
    else:
        clip = float(np.float32(max_norm) / (np.float32(norm.item()) + np.float32(eps)))
        if not clip < 1.0:
            clip = 1.0
    return float(np.float32(clip) * np.float32(inv_scale)), float(norm), found


def adamw_step(p, g, m, v, state: dict, lr: float, beta1: float, beta2: float, eps: float, wd: float,
               grad_scale: float, bias_correction: bool = True):
    """One AdamW update on FP32 masters with the device-state bias correction
    (metal_adamw.metal:35-52,83-179): returns (p_new, m_new, v_new); state holds beta powers."""
    f = np.float32
    b1p, b2p = f(state["beta1_power"]) * f(beta1), f(state["beta2_power"]) * f(beta2)
    bc1 = f(1.0) - b1p if bias_correction else f(1.0)
    bc2 = f(1.0) - b2p if bias_correction else f(1.0)
    bc2s = np.sqrt(bc2, dtype=np.float32)
    step_scale, decay_scale, eps_scaled = f(lr) * bc2s / bc1, f(lr) * f(wd), f(eps) * bc2s
    gs = g.to(torch.float32) * float(f(grad_scale)) if grad_scale != 0.0 else torch.zeros_like(g)
    m_new = float(f(beta1)) * m + float(f(1.0) - f(beta1)) * gs
    v_new = float(f(beta2)) * v + (float(f(1.0) - f(beta2)) * gs) * gs
    denom = torch.sqrt(v_new) + float(eps_scaled)
    p_new = p - (float(step_scale) * m_new) / denom - float(decay_scale) * p
    state["beta1_power"], state["beta2_power"] = b1p, b2p
    return p_new, m_new, v_new
