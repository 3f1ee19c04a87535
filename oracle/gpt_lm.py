"""CPU oracle of the gpt_lm training step and KV-cache decode, assembled from oracle/ops.py.

TEST INFRASTRUCTURE ONLY (see oracle/ops.py). Follows examples/gpt_lm/gpt_lm_shared.c:602-823
(forward), the backward rules of the op capsules (src/ops/*/autograd_*.c), gradient
accumulation with a storage-dtype rounding after every add (src/autograd/autograd.c:577-685,
src/backends/metal/primitives/memory/metal_memory.metal:31) and the optimizer step of
src/optim/adamw.c:2163-2270. The timed CPU baseline of bench.py runs this step.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import ops

MASK64 = (1 << 64) - 1
DROPOUT_EMBED = 0x9E3779B97F4A7C15
DROPOUT_ATTN = 0xBF58476D1CE4E5B9
DROPOUT_MLP = 0x94D049BB133111EB


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return x ^ (x >> 31)


@dataclass
class OracleConfig:
    vocab_size: int
    context_length: int
    d_model: int
    n_layers: int
    n_heads: int
    head_dim: int
    mlp_hidden: int
    tied_lm_head: bool
    dropout_p: float
    logits_softcap: float
    sdpa_window: int
    rms_eps: float
    pad_token_id: int
    dtype: str
    dropout_seed: int
    rope_theta: float = 10000.0


@dataclass
class OracleTrainConfig:
    lr: float = 3.0e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1.0e-8
    weight_decay: float = 1.0e-4
    grad_clip_norm: float = 1.0
    amp: dict = field(default_factory=lambda: dict(init_scale=32768.0, growth_factor=2.0, backoff_factor=0.5,
                                                   min_scale=1.0, max_scale=2147483648.0, growth_interval=2000))


def config_from(cfg) -> OracleConfig:
    """Build an OracleConfig from any object with the same attribute names (dtype code 1 = f16, 2 = bf16)."""
    dt = {1: "f16", 2: "bf16", 3: "f32"}.get(cfg.dtype, cfg.dtype)
    return OracleConfig(cfg.vocab_size, cfg.context_length, cfg.d_model, cfg.n_layers, cfg.n_heads, cfg.head_dim,
                        cfg.mlp_hidden, cfg.tied_lm_head, cfg.dropout_p, cfg.logits_softcap, cfg.sdpa_window,
                        cfg.rms_eps, cfg.pad_token_id, dt, cfg.dropout_seed, cfg.rope_theta)


def train_config_from(tc) -> OracleTrainConfig:
    a = tc.amp
    return OracleTrainConfig(tc.lr, tc.beta1, tc.beta2, tc.eps, tc.weight_decay, tc.grad_clip_norm,
                             dict(init_scale=a.init_scale, growth_factor=a.growth_factor, backoff_factor=a.backoff_factor,
                                  min_scale=a.min_scale, max_scale=a.max_scale, growth_interval=a.growth_interval))


class OracleGptLm:
    def __init__(self, cfg: OracleConfig, host_params: dict):
        self.cfg = cfg
        self.p = {k: torch.from_numpy(np.array(v, dtype=np.float32)) for k, v in host_params.items()}
        self.master = {k: v.clone() for k, v in self.p.items()}
        self.m = {k: torch.zeros_like(v) for k, v in self.p.items()}
        self.v = {k: torch.zeros_like(v) for k, v in self.p.items()}
        self.opt_state = {k: {"beta1_power": np.float32(1.0), "beta2_power": np.float32(1.0)} for k in self.p}
        self.amp = None
        self.training = True

    def _lm_w(self):
        return self.p["token_embedding"] if self.cfg.tied_lm_head else self.p["lm_head.weight"]

    def _lm_w_name(self):
        return "token_embedding" if self.cfg.tied_lm_head else "lm_head.weight"

    def _seed(self, site: int, layer: int, step: int) -> int:
        return splitmix64((self.cfg.dropout_seed ^ site ^ ((layer << 32) & MASK64) ^ step) & MASK64)

    # ------------------------------------------------------------------ forward + backward
    def loss_and_grads(self, input_ids, targets, positions, cu_seqlens, step: int, loss_scale: float = 1.0, need_grads: bool = True):
        c, p, dt = self.cfg, self.p, self.cfg.dtype
        ids = torch.from_numpy(np.asarray(input_ids, dtype=np.int32))
        tgt = torch.from_numpy(np.asarray(targets, dtype=np.int32))
        pos = torch.from_numpy(np.asarray(positions, dtype=np.int32))
        cu = np.asarray(cu_seqlens, dtype=np.int64)
        drop = self.training and c.dropout_p > 0.0
        tape = []
        x0 = ops.embedding_forward(p["token_embedding"], ids)
        emb_mask = None
        if drop:
            x, emb_mask = ops.dropout_forward(x0, c.dropout_p, splitmix64((c.dropout_seed ^ DROPOUT_EMBED ^ step) & MASK64), dt)
        else:
            x = x0
        for i in range(c.n_layers):
            pre = f"blocks.{i}."
            s = {"x": x}
            s["normed"], s["inv1"] = ops.rms_norm_forward(x, p[pre + "attn_norm_w"], c.rms_eps, dt)
            s["qkv"] = ops.linear_transposed_weight_forward(s["normed"], p[pre + "qkv_proj.weight"], p[pre + "qkv_proj.bias"], dt)
            s["q"], s["k"], s["v"] = ops.qkv_split_rope_forward(s["qkv"], pos, c.n_heads, c.head_dim, c.rope_theta, False, dt)
            attn, _ = ops.sdpa_varlen_forward(s["q"], s["k"], s["v"], cu, 0.0, True, c.sdpa_window, 0, dt)
            s["attn"] = attn.reshape(attn.shape[0], c.d_model)
            proj = ops.linear_transposed_weight_forward(s["attn"], p[pre + "attn_proj.weight"], p[pre + "attn_proj.bias"], dt)
            if drop:
                s["resid"], s["mask1"] = ops.dropout_add_forward(x, proj, c.dropout_p, self._seed(DROPOUT_ATTN, i, step), dt)
            else:
                s["resid"], s["mask1"] = ops.rnd(x + proj, dt), None
            s["normed2"], s["inv2"] = ops.rms_norm_forward(s["resid"], p[pre + "mlp_norm_w"], c.rms_eps, dt)
            s["up_gate"] = ops.linear_transposed_weight_forward(s["normed2"], p[pre + "up_gate.weight"], p[pre + "up_gate.bias"], dt)
            s["act"] = ops.swiglu_split_forward(s["up_gate"], dt)
            mlp = ops.linear_forward(s["act"], p[pre + "down_proj.weight"], p[pre + "down_proj.bias"], dt)
            if drop:
                x, s["mask2"] = ops.dropout_add_forward(s["resid"], mlp, c.dropout_p, self._seed(DROPOUT_MLP, i, step), dt)
            else:
                x, s["mask2"] = ops.rnd(s["resid"] + mlp, dt), None
            tape.append(s)
        final, inv_f = ops.rms_norm_forward(x, p["final_norm_w"], c.rms_eps, dt)
        ce = ops.lm_cross_entropy_forward(final, self._lm_w(), p["lm_head_bias"], tgt, c.logits_softcap, c.pad_token_id, dt)
        result = {"loss": float(ce["loss"])}
        if not need_grads:
            return result
        # ---- backward (reverse tape order; gradient accumulation rounds after every add) ----
        grads: dict[str, torch.Tensor] = {}

        def acc(name, g):
            grads[name] = g if name not in grads else ops.rnd(grads[name] + g, dt)

        dh, dw, db = ops.lm_cross_entropy_backward(final, self._lm_w(), p["lm_head_bias"], tgt, ce, loss_scale, c.logits_softcap, dt)
        acc(self._lm_w_name(), dw)
        acc("lm_head_bias", db)
        gx, gw = ops.rms_norm_backward(x, p["final_norm_w"], inv_f, dh, dt)
        acc("final_norm_w", gw)
        scale = float(np.float32(1.0) / (np.float32(1.0) - np.float32(c.dropout_p)))
        for i in reversed(range(c.n_layers)):
            pre = f"blocks.{i}."
            s = tape[i]
            # y = resid + dropout(mlp): x-branch gets the masked grad first, the residual adopts gx
            g_mlp = ops.dropout_backward_mask(s["mask2"], gx, scale, dt) if s["mask2"] is not None else gx
            g_resid = gx
            _, dwd, dbd = ops.linear_backward(s["act"], p[pre + "down_proj.weight"], g_mlp, dt)
            acc(pre + "down_proj.weight", dwd)
            acc(pre + "down_proj.bias", dbd)
            dact, _, _ = ops.linear_backward(s["act"], p[pre + "down_proj.weight"], g_mlp, dt)
            d_up = ops.swiglu_split_backward(s["up_gate"], dact, dt)
            dn2, dwu, dbu = ops.linear_transposed_weight_backward(s["normed2"], p[pre + "up_gate.weight"], d_up, dt)
            acc(pre + "up_gate.weight", dwu)
            acc(pre + "up_gate.bias", dbu)
            d_res2, gw2 = ops.rms_norm_backward(s["resid"], p[pre + "mlp_norm_w"], s["inv2"], dn2, dt)
            acc(pre + "mlp_norm_w", gw2)
            g_resid = ops.rnd(g_resid + d_res2, dt)
            g_proj = ops.dropout_backward_mask(s["mask1"], g_resid, scale, dt) if s["mask1"] is not None else g_resid
            d_attn, dwp, dbp = ops.linear_transposed_weight_backward(s["attn"], p[pre + "attn_proj.weight"], g_proj, dt)
            acc(pre + "attn_proj.weight", dwp)
            acc(pre + "attn_proj.bias", dbp)
            dq, dk, dv = ops.sdpa_varlen_backward(d_attn.reshape(s["q"].shape), s["q"], s["k"], s["v"], cu, 0.0, True, c.sdpa_window, 0, dt)
            dqkv = ops.qkv_split_rope_backward(dq, dk, dv, pos, c.rope_theta, False, dt)
            dn1, dwq, dbq = ops.linear_transposed_weight_backward(s["normed"], p[pre + "qkv_proj.weight"], dqkv, dt)
            acc(pre + "qkv_proj.weight", dwq)
            acc(pre + "qkv_proj.bias", dbq)
            d_x1, gw1 = ops.rms_norm_backward(s["x"], p[pre + "attn_norm_w"], s["inv1"], dn1, dt)
            acc(pre + "attn_norm_w", gw1)
            gx = ops.rnd(g_resid + d_x1, dt)
        if emb_mask is not None:
            gx = ops.dropout_backward_mask(emb_mask, gx, scale, dt)
        acc("token_embedding", ops.embedding_backward(gx, ids, c.vocab_size, dt))
        result["grads"] = grads
        return result

    # ------------------------------------------------------------------ full training step
    def train_step(self, input_ids, targets, positions, cu_seqlens, step: int, train: OracleTrainConfig, lr=None, wd_mask=None):
        if self.amp is None:
            a = train.amp
            s = np.float32(min(max(a["init_scale"], a["min_scale"]), a["max_scale"]))
            self.amp = {"scale": s, "inv_scale": np.float32(1.0) / s, "growth_tracker": 0, "found_inf": 0, "last_found_inf": 0}
        ops.amp_begin_step(self.amp, train.amp)
        res = self.loss_and_grads(input_ids, targets, positions, cu_seqlens, step, float(self.amp["scale"]))
        grads = res["grads"]
        names = [n for n in self.p if n in grads]
        gscale, norm, found = ops.grad_clip_scale([grads[n] for n in names], float(self.amp["inv_scale"]), train.grad_clip_norm)
        self.amp["found_inf"] = 1 if found else 0
        res["grad_norm"] = norm
        if not found:
            lr_now = train.lr if lr is None else lr
            for n in names:
                decay = 0.0 if (n.endswith("norm_w") or n.endswith("bias")) else train.weight_decay
                pn, mn, vn = ops.adamw_step(self.master[n], grads[n], self.m[n], self.v[n], self.opt_state[n], lr_now,
                                            train.beta1, train.beta2, train.eps, decay, gscale)
                self.master[n], self.m[n], self.v[n] = pn, mn, vn
                self.p[n] = ops.rnd(pn, self.cfg.dtype)
        ops.amp_finish_step(self.amp, train.amp)
        res["scale"] = float(self.amp["scale"])
        res["found_inf"] = found
        return res

    # ------------------------------------------------------------------ greedy KV-cache decode
    def _block_infer(self, i, x, q, k, v, attn):
        c, p, dt = self.cfg, self.p, self.cfg.dtype
        pre = f"blocks.{i}."
        proj = ops.linear_transposed_weight_forward(attn.reshape(attn.shape[0], c.d_model), p[pre + "attn_proj.weight"], p[pre + "attn_proj.bias"], dt)
        resid = ops.rnd(x + proj, dt)
        n2, _ = ops.rms_norm_forward(resid, p[pre + "mlp_norm_w"], c.rms_eps, dt)
        ug = ops.linear_transposed_weight_forward(n2, p[pre + "up_gate.weight"], p[pre + "up_gate.bias"], dt)
        mlp = ops.linear_forward(ops.swiglu_split_forward(ug, dt), p[pre + "down_proj.weight"], p[pre + "down_proj.bias"], dt)
        return ops.rnd(resid + mlp, dt)

    def greedy_generate(self, prompts: np.ndarray, new_tokens: int, capacity: int, return_logits: bool = False):
        c, p, dt = self.cfg, self.p, self.cfg.dtype
        b, plen = prompts.shape
        kc = [torch.zeros((b, capacity, c.n_heads, c.head_dim)) for _ in range(c.n_layers)]
        vc = [torch.zeros((b, capacity, c.n_heads, c.head_dim)) for _ in range(c.n_layers)]
        ids = torch.from_numpy(prompts.reshape(-1).astype(np.int32))
        pos = torch.from_numpy(np.tile(np.arange(plen, dtype=np.int32), b))
        cu = np.arange(b + 1, dtype=np.int64) * plen
        x = ops.embedding_forward(p["token_embedding"], ids)
        for i in range(c.n_layers):
            pre = f"blocks.{i}."
            n1, _ = ops.rms_norm_forward(x, p[pre + "attn_norm_w"], c.rms_eps, dt)
            qkv = ops.linear_transposed_weight_forward(n1, p[pre + "qkv_proj.weight"], p[pre + "qkv_proj.bias"], dt)
            q, k, v = ops.qkv_split_rope_forward(qkv, pos, c.n_heads, c.head_dim, c.rope_theta, False, dt)
            ops.kv_cache_append(kc[i], vc[i], k, v, np.zeros(b, dtype=np.int32), cu)
            attn, _ = ops.sdpa_varlen_forward(q, k, v, cu, 0.0, True, c.sdpa_window, 0, dt)
            x = self._block_infer(i, x, q, k, v, attn)
        last = x[torch.arange(b) * plen + plen - 1]
        fin, _ = ops.rms_norm_forward(last, p["final_norm_w"], c.rms_eps, dt)
        logits = ops.linear_transposed_weight_forward(fin, self._lm_w(), p["lm_head_bias"], dt)
        all_logits = [logits.clone()]
        out = np.zeros((b, new_tokens), dtype=np.int32)
        nxt = host_argmax(logits.numpy(), c.logits_softcap)
        for t in range(new_tokens):
            out[:, t] = nxt
            if t == new_tokens - 1:
                break
            cur = plen + t
            ids = torch.from_numpy(nxt.astype(np.int32))
            pos = torch.full((b,), cur, dtype=torch.int32)
            cpos = np.full(b, cur, dtype=np.int32)
            x = ops.embedding_forward(p["token_embedding"], ids)
            for i in range(c.n_layers):
                pre = f"blocks.{i}."
                n1, _ = ops.rms_norm_forward(x, p[pre + "attn_norm_w"], c.rms_eps, dt)
                qkv = ops.linear_transposed_weight_forward(n1, p[pre + "qkv_proj.weight"], p[pre + "qkv_proj.bias"], dt)
                q, k, v = ops.qkv_split_rope_forward(qkv, pos, c.n_heads, c.head_dim, c.rope_theta, False, dt)
                ops.kv_cache_append(kc[i], vc[i], k[:, None], v[:, None], cpos)
                attn = ops.sdpa_decode(q[:, None], kc[i], vc[i], cpos, 0.0, c.sdpa_window, 0, dt)[:, 0]
                x = self._block_infer(i, x, q, k, v, attn)
            fin, _ = ops.rms_norm_forward(x, p["final_norm_w"], c.rms_eps, dt)
            logits = ops.linear_transposed_weight_forward(fin, self._lm_w(), p["lm_head_bias"], dt)
            all_logits.append(logits.clone())
            nxt = host_argmax(logits.numpy(), c.logits_softcap)
        return (out, all_logits) if return_logits else out


def host_argmax(logits: np.ndarray, softcap: float) -> np.ndarray:
    """Soft cap on the host, then first-maximum argmax skipping non-finite values
    (examples/gpt_lm/gpt_lm_shared.c:1322,1388-1398)."""
    x = logits.astype(np.float32)
    if softcap > 0.0:
        x = np.float32(softcap) * np.tanh(x / np.float32(softcap))
    x = np.where(np.isfinite(x), x, -np.inf)
    return np.argmax(x, axis=1).astype(np.int32)
