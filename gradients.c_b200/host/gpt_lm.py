"""gpt_lm: the decoder-only transformer of the reference's examples/gpt_lm, expressed over the
op capsules of ops.py, with its training step and KV-cache prefill/decode.

Follows examples/gpt_lm/gpt_lm_shared.c: gpt_block_forward :602-749, gpt_lm_forward :751-823,
gpt_block_prefill_cached :825, gpt_block_decode_cached :961, dropout site seeds :724,747,788,
parameter init :196-218,296-344 (normal, std 0.02, residual projections 0.02/sqrt(2L), norms 1,
biases 0), weight-decay groups examples/gpt_lm/main.c:3374-3378, and the training step order
of src/train/trainer.c:75-223. Model dimensions are run-time values here (the reference fixes
them at compile time, gpt_lm_shared.h:10-28).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import abi, ops
from .abi import F16, BF16, F32, I32, U16, BackendError
from .optim import AdamW, AdamwConfig, AmpConfig, AmpScaler, gd_backward_amp
from .runtime import Context, Tensor

MASK64 = (1 << 64) - 1
GPT_DROPOUT_EMBED = 0x9E3779B97F4A7C15
GPT_DROPOUT_ATTN = 0xBF58476D1CE4E5B9
GPT_DROPOUT_MLP = 0x94D049BB133111EB
GPT_DEFAULT_SEED = 0x6750746C6D5EED00


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return x ^ (x >> 31)


@dataclass
class GptConfig:
    vocab_size: int = 2048
    context_length: int = 512
    d_model: int = 512
    n_layers: int = 3
    n_heads: int = 8
    head_dim: int = 64
    mlp_hidden: int = 1024          # reference: 2 * d_model (gpt_lm_shared.h:28)
    tied_lm_head: bool = True       # reference ties the LM head to the embedding (gpt_lm_shared.c:393-396)
    dropout_p: float = 0.05
    logits_softcap: float = 30.0
    sdpa_window: int = 256
    rms_eps: float = 1.0e-5
    pad_token_id: int = -1          # ignore_index passed to the loss
    dtype: int = F16
    dropout_seed: int = GPT_DEFAULT_SEED
    rope_theta: float = 10000.0

    @staticmethod
    def reference_default() -> "GptConfig":
        return GptConfig()

    @staticmethod
    def baseline() -> "GptConfig":
        """The benchmark configuration: SwiGLU hidden 1536, untied biased LM head, dropout 0.1,
        no sliding window."""
        return GptConfig(mlp_hidden=1536, tied_lm_head=False, dropout_p=0.1, sdpa_window=0)

    @staticmethod
    def scaled() -> "GptConfig":
        return GptConfig(vocab_size=32768, context_length=2048, d_model=2048, n_layers=24, n_heads=16, head_dim=128,
                         mlp_hidden=5632, tied_lm_head=False, dropout_p=0.1, sdpa_window=0, dtype=BF16)


def param_specs(cfg: GptConfig) -> list[tuple[str, tuple[int, ...], str]]:
    """(name, shape, kind) in registration order; kind is one of normal / residual / ones / zeros."""
    d, f = cfg.d_model, cfg.mlp_hidden
    specs = [("token_embedding", (cfg.vocab_size, d), "normal")]
    for i in range(cfg.n_layers):
        p = f"blocks.{i}."
        specs += [
            (p + "attn_norm_w", (d,), "ones"),
            (p + "qkv_proj.weight", (3 * d, d), "normal"), (p + "qkv_proj.bias", (3 * d,), "zeros"),
            (p + "attn_proj.weight", (d, d), "residual"), (p + "attn_proj.bias", (d,), "zeros"),
            (p + "mlp_norm_w", (d,), "ones"),
            (p + "up_gate.weight", (2 * f, d), "normal"), (p + "up_gate.bias", (2 * f,), "zeros"),
            (p + "down_proj.weight", (f, d), "residual"), (p + "down_proj.bias", (d,), "zeros"),
        ]
    specs.append(("final_norm_w", (d,), "ones"))
    if not cfg.tied_lm_head:
        specs.append(("lm_head.weight", (cfg.vocab_size, d), "normal"))
    specs.append(("lm_head_bias", (cfg.vocab_size,), "zeros"))
    return specs


def init_params(cfg: GptConfig, seed: int = 0, residual_scaled: bool = True) -> dict[str, np.ndarray]:
    """Host-side initial weights as float32 arrays already rounded to the storage dtype grid."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape, kind in param_specs(cfg):
        if kind == "ones":
            a = np.ones(shape, dtype=np.float32)
        elif kind == "zeros":
            a = np.zeros(shape, dtype=np.float32)
        else:
            std = 0.02 / math.sqrt(2.0 * cfg.n_layers) if (kind == "residual" and residual_scaled) else 0.02
            a = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
        out[name] = round_to_storage(a, cfg.dtype)
    return out


def round_to_storage(a: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F16:
        return a.astype(np.float16).astype(np.float32)
    if dtype == BF16:
        from .runtime import bf16_bits_from_f32, f32_from_bf16_bits
        return f32_from_bf16_bits(bf16_bits_from_f32(a)).reshape(a.shape)
    return a.astype(np.float32)


@dataclass
class Batch:
    """One packed training batch on the host: token ids, next-token targets (ignored rows hold
    pad_token_id or -1), positions restarting per segment, and cu_seqlens."""
    input_ids: np.ndarray
    targets: np.ndarray
    positions: np.ndarray
    cu_seqlens: np.ndarray
    real_tokens: int = 0

    @property
    def h2d_bytes(self) -> int:
        return int(self.input_ids.nbytes + self.targets.nbytes + self.positions.nbytes + self.cu_seqlens.nbytes)


def take_sequences(batch: Batch, indices: Sequence[int], pad_to: int = 0, context_length: int = 0) -> Batch:
    """The shard of a packed batch made of the given sequences (in the given order): same ids and targets, positions
    and cu_seqlens rebuilt, padding segments of the source dropped and, when pad_to > 0, appended anew as ignored rows."""
    cu = np.asarray(batch.cu_seqlens, dtype=np.int64)
    ids, tgt, pos, out_cu = [], [], [], [0]
    for i in indices:
        a, b = int(cu[i]), int(cu[i + 1])
        ids.append(np.asarray(batch.input_ids[a:b]))
        tgt.append(np.asarray(batch.targets[a:b]))
        pos.append(np.asarray(batch.positions[a:b]))
        out_cu.append(out_cu[-1] + (b - a))
    real = out_cu[-1]
    if pad_to > 0 and real % pad_to != 0:
        pad = pad_to - real % pad_to
        while pad > 0:
            n = min(pad, context_length or pad)
            ids.append(np.zeros(n, dtype=np.int32))
            tgt.append(np.full(n, -1, dtype=np.int32))
            pos.append(np.arange(n, dtype=np.int32))
            out_cu.append(out_cu[-1] + n)
            pad -= n
    return Batch(np.concatenate(ids).astype(np.int32), np.concatenate(tgt).astype(np.int32), np.concatenate(pos).astype(np.int32),
                 np.asarray(out_cu, dtype=np.int32), real)


@dataclass
class CompactBatch:
    """A batch of compact records as the reference stores them on disk (examples/gpt_lm/main.c:835-857): u16
    tokens [n_records, context_length + 1], the I32 lengths of the documents packed into each record, one list
    after another, and the index of each record's first length (record_offsets[n_records] = number of segments)."""
    tokens: np.ndarray
    segment_lengths: np.ndarray
    record_offsets: np.ndarray
    im_start_id: int = 1
    im_end_id: int = 2
    real_tokens: int = 0

    @property
    def h2d_bytes(self) -> int:
        return int(self.tokens.nbytes + self.segment_lengths.nbytes + self.record_offsets.nbytes)


def synthetic_compact_batch(cfg: GptConfig, n_records: int, seed: int, max_segments: int = 6) -> CompactBatch:
    """Records of context_length + 1 uniform token ids, each cut into 1..max_segments documents at random places."""
    rng = np.random.default_rng(seed)
    ctx = cfg.context_length
    tokens = rng.integers(0, cfg.vocab_size, size=(n_records, ctx + 1)).astype(np.uint16)
    lens, offs = [], [0]
    for _ in range(n_records):
        n = int(rng.integers(1, min(max_segments, ctx) + 1))
        cuts = np.sort(rng.choice(np.arange(1, ctx), size=n - 1, replace=False)) if n > 1 else np.zeros(0, dtype=np.int64)
        lens.extend(np.diff(np.concatenate([[0], cuts, [ctx]])).tolist())
        offs.append(len(lens))
    return CompactBatch(tokens, np.asarray(lens, dtype=np.int32), np.asarray(offs, dtype=np.int32), real_tokens=n_records * ctx)


def synthetic_batch(cfg: GptConfig, n_seqs: int, min_len: int, max_len: int, seed: int, pad_to: int = 0,
                    lengths: Optional[Sequence[int]] = None) -> Batch:
    """Packed sequences with lengths uniform in [min_len, max_len] and ids uniform over the
    vocabulary. The target of the last token of every sequence is ignored (-1). When pad_to > 0
    the stream is padded with one fully ignored segment up to a multiple of pad_to rows
    (the reference rejects token counts that are not a multiple of the context length,
    gpt_lm_shared.c:776). `lengths` overrides the drawn lengths (a data-parallel shard of a global batch)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(min_len, max_len + 1, size=n_seqs) if lengths is None else np.asarray(lengths, dtype=np.int64)
    ids, tgt, pos, cu = [], [], [], [0]
    for n in lens:
        n = int(n)
        s = rng.integers(0, cfg.vocab_size, size=n, dtype=np.int64).astype(np.int32)
        t = np.empty(n, dtype=np.int32)
        t[:-1] = s[1:]
        t[-1] = -1
        ids.append(s)
        tgt.append(t)
        pos.append(np.arange(n, dtype=np.int32))
        cu.append(cu[-1] + n)
    real = cu[-1]
    if pad_to > 0 and real % pad_to != 0:
        pad = pad_to - real % pad_to
        while pad > 0:  # padding segments never exceed the context length
            n = min(pad, cfg.context_length)
            ids.append(np.zeros(n, dtype=np.int32))
            tgt.append(np.full(n, -1, dtype=np.int32))
            pos.append(np.arange(n, dtype=np.int32))
            cu.append(cu[-1] + n)
            pad -= n
    return Batch(np.concatenate(ids), np.concatenate(tgt), np.concatenate(pos), np.asarray(cu, dtype=np.int32), real)


class GptLm:
    def __init__(self, ctx: Context, cfg: GptConfig, host_params: Optional[dict[str, np.ndarray]] = None, seed: int = 0):
        assert cfg.n_heads * cfg.head_dim == cfg.d_model
        self.ctx, self.cfg = ctx, cfg
        self.training = True
        host_params = host_params if host_params is not None else init_params(cfg, seed)
        self.params: dict[str, Tensor] = {}
        self.weight_decay_mask: dict[str, bool] = {}
        for name, shape, _ in param_specs(cfg):
            t = ctx.from_numpy(ctx.params, cfg.dtype, host_params[name].reshape(shape), name)
            t.requires_grad = True
            t.is_leaf = True
            self.params[name] = t
            self.weight_decay_mask[name] = not (name.endswith("norm_w") or name.endswith("bias"))
        self.k_cache: list[Tensor] = []
        self.v_cache: list[Tensor] = []

    # ---- parameters ----
    def param_list(self) -> list[Tensor]:
        return list(self.params.values())

    def lm_head_weight(self) -> Tensor:
        return self.params["token_embedding"] if self.cfg.tied_lm_head else self.params["lm_head.weight"]

    def n_params(self) -> int:
        return sum(t.count for t in self.params.values())

    def make_optimizer(self, config: AdamwConfig) -> AdamW:
        names = list(self.params.keys())
        wds = [config.weight_decay if self.weight_decay_mask[n] else 0.0 for n in names]
        return AdamW(self.ctx, [self.params[n] for n in names], config, wds)

    # ---- forward ----
    def _site_seed(self, site: int, layer: int, step: int) -> int:
        return splitmix64((self.cfg.dropout_seed ^ site ^ ((layer << 32) & MASK64) ^ step) & MASK64)

    def block_forward(self, i: int, x: Tensor, positions: Tensor, cu_seqlens: Tensor, step: int) -> Tensor:
        ctx, cfg, p = self.ctx, self.cfg, self.params
        pre = f"blocks.{i}."
        normed = ops.gd_rms_norm(ctx, x, p[pre + "attn_norm_w"], cfg.rms_eps)
        qkv = ops.gd_linear_transposed_weight(ctx, normed, p[pre + "qkv_proj.weight"], p[pre + "qkv_proj.bias"])
        q, k, v = ops.gd_qkv_split_rope(ctx, qkv, positions, cfg.n_heads, cfg.head_dim, cfg.rope_theta)
        attn = ops.gd_sdpa_varlen(ctx, q, k, v, cu_seqlens, causal=True, sliding_window=cfg.sdpa_window,
                                  max_seqlen=cfg.context_length)
        attn_flat = attn.reshape((attn.shape[0], cfg.d_model))
        attn_flat.requires_grad = attn.requires_grad
        if attn.requires_grad:
            def reshape_backward():
                if attn_flat.grad is not None:
                    ctx.accumulate_grad(attn, attn_flat.grad.reshape(attn.shape))
            ctx.record(reshape_backward)
        proj = ops.gd_linear_transposed_weight(ctx, attn_flat, p[pre + "attn_proj.weight"], p[pre + "attn_proj.bias"])
        resid = ops.gd_dropout_add(ctx, x, proj, cfg.dropout_p, self.training, self._site_seed(GPT_DROPOUT_ATTN, i, step))
        normed2 = ops.gd_rms_norm(ctx, resid, p[pre + "mlp_norm_w"], cfg.rms_eps)
        up_gate = ops.gd_linear_transposed_weight(ctx, normed2, p[pre + "up_gate.weight"], p[pre + "up_gate.bias"])
        mlp = ops.gd_swiglu_split_linear(ctx, up_gate, p[pre + "down_proj.weight"], p[pre + "down_proj.bias"])
        return ops.gd_dropout_add(ctx, resid, mlp, cfg.dropout_p, self.training, self._site_seed(GPT_DROPOUT_MLP, i, step))

    def forward(self, input_ids: Tensor, target_ids: Tensor, positions: Tensor, cu_seqlens: Tensor, step: int,
                shard_share: float = 1.0) -> Tensor:
        """gpt_lm_forward: returns the scalar F32 mean loss tensor (this shard's share of the global mean when
        shard_share < 1, see gd_lm_cross_entropy_softcapped_bias_ignore)."""
        ctx, cfg, p = self.ctx, self.cfg, self.params
        x = ops.gd_embedding(ctx, p["token_embedding"], input_ids)
        x = ops.gd_dropout(ctx, x, cfg.dropout_p, self.training, splitmix64((cfg.dropout_seed ^ GPT_DROPOUT_EMBED ^ step) & MASK64))
        for i in range(cfg.n_layers):
            x = self.block_forward(i, x, positions, cu_seqlens, step)
        final = ops.gd_rms_norm(ctx, x, p["final_norm_w"], cfg.rms_eps)
        return ops.gd_lm_cross_entropy_softcapped_bias_ignore(ctx, final, self.lm_head_weight(), p["lm_head_bias"], target_ids,
                                                              cfg.logits_softcap, cfg.pad_token_id, shard_share)

    def upload_batch(self, batch: Batch, stream_ordered: bool = False):
        """Places the batch in the data slot. `stream_ordered`: the arrays are page-locked and are copied behind
        the work already submitted, without a wait (they must stay unchanged until the step's fence completes)."""
        ctx = self.ctx
        if isinstance(batch, CompactBatch):
            return self.expand_compact_batch(batch, stream_ordered)[:4]
        if stream_ordered:
            out = []
            for a, name in ((batch.input_ids, "input_ids"), (batch.targets, "targets"), (batch.positions, "positions"), (batch.cu_seqlens, "cu_seqlens")):
                t = ctx.empty(ctx.data, I32, a.shape, name)
                t.write_async(a)
                out.append(t)
            return tuple(out)
        return (ctx.from_numpy(ctx.data, I32, batch.input_ids, "input_ids"),
                ctx.from_numpy(ctx.data, I32, batch.targets, "targets"),
                ctx.from_numpy(ctx.data, I32, batch.positions, "positions"),
                ctx.from_numpy(ctx.data, I32, batch.cu_seqlens, "cu_seqlens"))

    def expand_compact_batch(self, cb: CompactBatch, stream_ordered: bool = False, check: bool = True):
        """Copies the compact records into the data slot and expands them on the device into (input_ids, targets,
        positions, cu_seqlens, status). `check` reads the status word back (a host wait) and raises on input the
        reference's transform rejects (examples/gpt_lm/main.c:934-959)."""
        import ctypes as C
        ctx, cfg = self.ctx, self.cfg
        n_rec, n_seg = int(cb.tokens.shape[0]), int(cb.segment_lengths.size)
        assert cb.tokens.dtype == np.uint16 and cb.tokens.shape == (n_rec, cfg.context_length + 1)
        src = []
        for a, dt, name in ((cb.tokens.reshape(-1), U16, "compact.tokens"), (cb.segment_lengths, I32, "compact.segment_lengths"),
                            (cb.record_offsets, I32, "compact.record_offsets")):
            t = ctx.empty(ctx.data, dt, a.shape, name)
            if stream_ordered:
                t.write_async(a)
            else:
                t.write(a)
            src.append(t)
        n_tok = n_rec * cfg.context_length
        ids, tgt, pos = (ctx.empty(ctx.data, I32, (n_tok,), n) for n in ("input_ids", "targets", "positions"))
        cu = ctx.empty(ctx.data, I32, (n_seg + 1,), "cu_seqlens")
        status = ctx.empty(ctx.data, I32, (1,), "compact.status")
        b = abi.GptCompactBatch(ids.buffer, src[0].offset, src[1].offset, src[2].offset, ids.offset, tgt.offset, pos.offset, cu.offset,
                                status.offset, n_rec, n_seg, cfg.context_length, cfg.vocab_size, cfg.pad_token_id, cb.im_start_id, cb.im_end_id)
        ctx.check(ctx.lib.gdb200_gpt_compact_expand(ctx.backend, C.byref(b)), "gdb200_gpt_compact_expand")
        if check and not stream_ordered:
            flags = int(status.read()[0])
            if flags != 0:
                raise BackendError(abi.GD_ERR_INVALID_ARGUMENT, "gdb200_gpt_compact_expand", f"compact records rejected (flags {flags})")
        return ids, tgt, pos, cu, status

    # ---- KV-cache generation ----
    def alloc_kv_cache(self, batch: int, capacity: int) -> None:
        cfg, ctx = self.cfg, self.ctx
        self.k_cache = [ctx.zeros(ctx.state, cfg.dtype, (batch, capacity, cfg.n_heads, cfg.head_dim), f"k_cache.{i}") for i in range(cfg.n_layers)]
        self.v_cache = [ctx.zeros(ctx.state, cfg.dtype, (batch, capacity, cfg.n_heads, cfg.head_dim), f"v_cache.{i}") for i in range(cfg.n_layers)]

    def _mlp_infer(self, pre: str, resid: Tensor) -> Tensor:
        ctx, cfg, p = self.ctx, self.cfg, self.params
        normed2 = ops.gd_rms_norm(ctx, resid, p[pre + "mlp_norm_w"], cfg.rms_eps)
        up_gate = ops.gd_linear_transposed_weight(ctx, normed2, p[pre + "up_gate.weight"], p[pre + "up_gate.bias"])
        mlp = ops.gd_swiglu_split_linear(ctx, up_gate, p[pre + "down_proj.weight"], p[pre + "down_proj.bias"])
        return ops.gd_add(ctx, resid, mlp)

    def prefill_last_logits(self, input_ids: Tensor, positions: Tensor, cu_seqlens: Tensor, cache_pos: Tensor,
                            last_rows: np.ndarray) -> Tensor:
        """Packed prefill that fills the caches and returns logits [B, V] of the last row of each prompt
        (gpt_lm_shared.c:1117-1202)."""
        ctx, cfg, p = self.ctx, self.cfg, self.params
        prev = ctx.grad_enabled
        ctx.grad_enabled = False
        try:
            x = ops.gd_embedding(ctx, p["token_embedding"], input_ids)
            for i in range(cfg.n_layers):
                pre = f"blocks.{i}."
                normed = ops.gd_rms_norm(ctx, x, p[pre + "attn_norm_w"], cfg.rms_eps)
                qkv = ops.gd_linear_transposed_weight(ctx, normed, p[pre + "qkv_proj.weight"], p[pre + "qkv_proj.bias"])
                q, k, v = ops.gd_qkv_split_rope(ctx, qkv, positions, cfg.n_heads, cfg.head_dim, cfg.rope_theta)
                ops.gd_kv_cache_append_packed(ctx, self.k_cache[i], self.v_cache[i], cache_pos, cu_seqlens, k, v)
                attn = ops.gd_sdpa_varlen(ctx, q, k, v, cu_seqlens, causal=True, sliding_window=cfg.sdpa_window, max_seqlen=cfg.context_length)
                proj = ops.gd_linear_transposed_weight(ctx, attn.reshape((attn.shape[0], cfg.d_model)), p[pre + "attn_proj.weight"], p[pre + "attn_proj.bias"])
                resid = ops.gd_add(ctx, x, proj)
                x = self._mlp_infer(pre, resid)
            # gather the last row of each prompt: slice + concat_to_full per prompt
            b = len(last_rows)
            gathered = ctx.scratch_empty(cfg.dtype, (b, cfg.d_model), "last_rows")
            for j, r in enumerate(last_rows):
                args = abi.ConcatArgs(cfg.d_model, cfg.d_model, 1, b, j)
                src = x.rows(int(r), 1)
                ctx.check(ctx.lib.gd_backend_concat_to_full(ctx.backend, ops._tvp(src), ops._tvp(gathered), ops.byref(args)), "concat_to_full")
            final = ops.gd_rms_norm(ctx, gathered, p["final_norm_w"], cfg.rms_eps)
            return ops.gd_linear_transposed_weight(ctx, final, self.lm_head_weight(), p["lm_head_bias"])
        finally:
            ctx.grad_enabled = prev

    def decode_logits(self, input_ids: Tensor, positions: Tensor, cache_pos: Tensor) -> Tensor:
        """One decode step for B sequences: ids [B], positions [B], cache_pos [B] -> logits [B, V]
        (gpt_lm_shared.c:961-1115,1204-1246)."""
        ctx, cfg, p = self.ctx, self.cfg, self.params
        prev = ctx.grad_enabled
        ctx.grad_enabled = False
        try:
            b = input_ids.count
            x = ops.gd_embedding(ctx, p["token_embedding"], input_ids)
            for i in range(cfg.n_layers):
                pre = f"blocks.{i}."
                normed = ops.gd_rms_norm(ctx, x, p[pre + "attn_norm_w"], cfg.rms_eps)
                qkv = ops.gd_linear_transposed_weight(ctx, normed, p[pre + "qkv_proj.weight"], p[pre + "qkv_proj.bias"])
                q, k, v = ops.gd_qkv_split_rope(ctx, qkv, positions, cfg.n_heads, cfg.head_dim, cfg.rope_theta)
                shape4 = (b, 1, cfg.n_heads, cfg.head_dim)
                ops.gd_kv_cache_append_positions(ctx, self.k_cache[i], self.v_cache[i], cache_pos, k.reshape(shape4), v.reshape(shape4))
                attn = ops.gd_sdpa_decode_positions(ctx, q.reshape(shape4), self.k_cache[i], self.v_cache[i], cache_pos,
                                                    sliding_window=cfg.sdpa_window)
                proj = ops.gd_linear_transposed_weight(ctx, attn.reshape((b, cfg.d_model)), p[pre + "attn_proj.weight"], p[pre + "attn_proj.bias"])
                resid = ops.gd_add(ctx, x, proj)
                x = self._mlp_infer(pre, resid)
            final = ops.gd_rms_norm(ctx, x, p["final_norm_w"], cfg.rms_eps)
            return ops.gd_linear_transposed_weight(ctx, final, self.lm_head_weight(), p["lm_head_bias"])
        finally:
            ctx.grad_enabled = prev


@dataclass
class TrainConfig:
    lr: float = 3.0e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1.0e-8
    weight_decay: float = 1.0e-4
    grad_clip_norm: float = 1.0
    amp: AmpConfig = field(default_factory=AmpConfig)

    @staticmethod
    def baseline() -> "TrainConfig":
        return TrainConfig(weight_decay=0.1, amp=AmpConfig(init_scale=65536.0))


class Trainer:
    """gd_train_batch: begin_step -> loss_fn -> backward_amp -> optimizer step -> end_step."""

    def __init__(self, model: GptLm, cfg: TrainConfig, dp=None):
        self.model, self.cfg, self.ctx = model, cfg, model.ctx
        self.optimizer = model.make_optimizer(AdamwConfig(cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, True))
        self.scaler = AmpScaler(self.ctx, cfg.amp)
        self.global_step = 0
        self.dp = dp

    def train_batch(self, batch: Optional[Batch], lr: Optional[float] = None, device_batch=None, loss_out=None) -> Tensor:
        """One training step. `device_batch` = (ids, targets, positions, cu_seqlens) tensors that are
        already resident on the device; otherwise the host batch is uploaded into the data slot.
        `loss_out` (a page-locked FP32 array of one element) selects the pipelined form: the batch, which must be
        page-locked too, is copied in stream order, the loss is copied to `loss_out` in stream order, and nothing
        is waited for; the value is valid once the step's fence has completed (Context.wait_steps)."""
        ctx, model = self.ctx, self.model
        ctx.begin_step()
        self.optimizer.zero_grad()
        ids, tgt, pos, cu = device_batch if device_batch is not None else model.upload_batch(batch, loss_out is not None)
        # data parallel: the loss and its gradient are normalised by the valid rows of the GLOBAL batch
        share = self.dp.shard_share(batch, model.cfg.pad_token_id) if self.dp is not None else 1.0
        loss = model.forward(ids, tgt, pos, cu, self.global_step + 1, share)
        gd_backward_amp(ctx, loss, self.scaler)
        if self.dp is not None:
            self.dp.reduce_gradients(self.optimizer, loss)
        self.optimizer.step_amp_clip_lr(self.scaler, self.cfg.lr if lr is None else lr, self.cfg.grad_clip_norm)
        if loss_out is not None:
            loss.read_async(loss_out)
        ctx.end_step()
        self.global_step += 1
        return loss


class NativeTrainer(Trainer):
    """Same training step as Trainer, with the per-step call sequence issued by the library's
    native driver (gdb200_gpt_train_step) instead of the Python op capsules. State layout, kernels,
    rounding points and results are the same; only the host that enqueues the calls differs."""

    def __init__(self, model: GptLm, cfg: TrainConfig, dp=None):
        super().__init__(model, cfg, dp)
        import ctypes as C
        self._C = C
        mc, ctx, opt, sc = model.cfg, model.ctx, self.optimizer, self.scaler
        s = abi.GptSpec()
        s.params_buffer, s.state_buffer, s.scratch_buffer = ctx.params.buffer, ctx.state.buffer, ctx.scratch.buffer
        s.scratch_bytes = ctx.scratch.capacity
        s.vocab_size, s.context_length, s.d_model, s.n_layers = mc.vocab_size, mc.context_length, mc.d_model, mc.n_layers
        s.n_heads, s.head_dim, s.mlp_hidden, s.tied_lm_head = mc.n_heads, mc.head_dim, mc.mlp_hidden, 1 if mc.tied_lm_head else 0
        s.sdpa_window, s.pad_token_id, s.dtype = mc.sdpa_window, mc.pad_token_id, mc.dtype
        s.lm_ce_chunk = ops.lm_ce_chunk_classes(mc.vocab_size)
        s.n_params = len(opt.slots)
        s.dp_world = dp.world if dp is not None else 1
        s.dropout_p = mc.dropout_p if model.training else 0.0
        s.logits_softcap, s.rms_eps, s.rope_theta, s.dropout_seed = mc.logits_softcap, mc.rms_eps, mc.rope_theta, mc.dropout_seed
        s.adam_beta1, s.adam_beta2, s.adam_eps, s.grad_clip_norm = cfg.beta1, cfg.beta2, cfg.eps, cfg.grad_clip_norm
        a = cfg.amp
        s.amp_growth_factor, s.amp_backoff_factor, s.amp_min_scale, s.amp_max_scale = a.growth_factor, a.backoff_factor, a.min_scale, a.max_scale
        s.amp_growth_interval = a.growth_interval
        s.state_f32_offset, s.state_i32_offset = opt.state_f32.offset, opt.state_i32.offset
        s.partials_offset, s.clip_scale_offset = opt.partials.offset, opt.grad_clip_scale.offset
        s.amp_scale_offset, s.amp_flags_offset = sc.scale_state.offset, sc.flag_state.offset
        for i, slot in enumerate(opt.slots):
            assert slot.master is not None, "the native driver expects 16-bit parameters with FP32 masters"
            s.param_offset[i], s.param_count[i] = slot.param.offset, slot.param.count
            s.master_offset[i], s.m_offset[i], s.v_offset[i] = slot.master.offset, slot.m.offset, slot.v.offset
            s.weight_decay[i] = slot.weight_decay
        self.spec = s

    def train_batch(self, batch: Optional[Batch], lr: Optional[float] = None, device_batch=None, loss_out=None,
                    global_valid_rows: float = 0.0) -> Tensor:
        """`global_valid_rows` > 0: the batch is a shard of a global batch with that many valid target rows; loss and
        gradients are normalised by it (the loss returned is the shard's share of the global mean)."""
        C, ctx = self._C, self.ctx
        self.spec.global_valid_rows = float(global_valid_rows)
        ctx.begin_step()
        ids, tgt, pos, cu = device_batch if device_batch is not None else self.model.upload_batch(batch, loss_out is not None)
        assert ids.arena is tgt.arena is pos.arena is cu.arena
        b = abi.GptBatch(ids.buffer, ids.offset, tgt.offset, pos.offset, cu.offset, ids.count, cu.count)
        loss_off, used = C.c_size_t(), C.c_size_t()
        st = ctx.lib.gdb200_gpt_train_step(ctx.backend, C.byref(self.spec), C.byref(b), self.global_step + 1,
                                           self.cfg.lr if lr is None else lr, C.byref(loss_off), C.byref(used))
        ctx.check(st, "gdb200_gpt_train_step")
        ctx.scratch.top = used.value
        ctx.scratch.high_water = max(ctx.scratch.high_water, used.value)
        loss = Tensor(ctx, ctx.scratch, loss_off.value, F32, ())
        if loss_out is not None:
            loss.read_async(loss_out)
        ctx.end_step()
        self.global_step += 1
        return loss


def native_step_gradients(trainer: "NativeTrainer") -> dict[str, np.ndarray]:
    """Parameter gradients of the step the native driver enqueued last, read from the scratch arena before it is
    reused (float32, still multiplied by the loss scale of that step)."""
    import ctypes as C
    ctx, model = trainer.ctx, trainer.model
    names = list(model.params.keys())
    offs = (C.c_size_t * len(names))()
    n = ctx.lib.gdb200_gpt_train_step_grad_offsets(ctx.backend, offs, len(names))
    assert n == len(names), (n, len(names))
    ctx.flush()
    return {name: Tensor(ctx, ctx.scratch, int(offs[i]), model.cfg.dtype, model.params[name].shape).read_f32()
            for i, name in enumerate(names)}


def greedy_generate(model: GptLm, prompts: np.ndarray, new_tokens: int, capacity: int) -> np.ndarray:
    """Batched greedy KV-cache generation: packed prefill, then `new_tokens` decode steps with
    host argmax (first maximum wins, soft cap applied on the host as gpt_lm_shared.c:1322,1388-1398)."""
    ctx, cfg = model.ctx, model.cfg
    b, plen = prompts.shape
    model.alloc_kv_cache(b, capacity)
    out = np.zeros((b, new_tokens), dtype=np.int32)
    ctx.begin_step()
    ids = ctx.from_numpy(ctx.data, I32, prompts.reshape(-1).astype(np.int32))
    pos = ctx.from_numpy(ctx.data, I32, np.tile(np.arange(plen, dtype=np.int32), b))
    cu = ctx.from_numpy(ctx.data, I32, (np.arange(b + 1, dtype=np.int32) * plen))
    cpos = ctx.from_numpy(ctx.data, I32, np.zeros(b, dtype=np.int32))
    logits = model.prefill_last_logits(ids, pos, cu, cpos, np.arange(b) * plen + plen - 1)
    ctx.end_step()
    nxt = host_argmax(logits.read_f32(), cfg.logits_softcap)
    for t in range(new_tokens):
        out[:, t] = nxt
        if t == new_tokens - 1:
            break
        ctx.begin_step()
        cur = plen + t
        ids = ctx.from_numpy(ctx.data, I32, nxt.astype(np.int32))
        pos = ctx.from_numpy(ctx.data, I32, np.full(b, cur, dtype=np.int32))
        cpos = ctx.from_numpy(ctx.data, I32, np.full(b, cur, dtype=np.int32))
        logits = model.decode_logits(ids, pos, cpos)
        ctx.end_step()
        nxt = host_argmax(logits.read_f32(), cfg.logits_softcap)
    return out


def model_spec(model: GptLm) -> "abi.GptSpec":
    """gdb200_gpt_spec with the model fields and parameter locations only (what the decode driver reads)."""
    mc, ctx = model.cfg, model.ctx
    s = abi.GptSpec()
    s.params_buffer, s.state_buffer, s.scratch_buffer = ctx.params.buffer, ctx.state.buffer, ctx.scratch.buffer
    s.scratch_bytes = ctx.scratch.capacity
    s.vocab_size, s.context_length, s.d_model, s.n_layers = mc.vocab_size, mc.context_length, mc.d_model, mc.n_layers
    s.n_heads, s.head_dim, s.mlp_hidden, s.tied_lm_head = mc.n_heads, mc.head_dim, mc.mlp_hidden, 1 if mc.tied_lm_head else 0
    s.sdpa_window, s.pad_token_id, s.dtype = mc.sdpa_window, mc.pad_token_id, mc.dtype
    s.logits_softcap, s.rms_eps, s.rope_theta, s.dropout_seed = mc.logits_softcap, mc.rms_eps, mc.rope_theta, mc.dropout_seed
    plist = model.param_list()
    s.n_params, s.dp_world = len(plist), 1
    for i, t in enumerate(plist):
        s.param_offset[i], s.param_count[i] = t.offset, t.count
    return s


def device_argmax(ctx, logits: Tensor, softcap: float) -> Tensor:
    """gdb200_argmax_rows: I32 [rows] of the first maximum of softcap(logits) per row."""
    out = ctx.scratch_empty(I32, (logits.shape[0],), "argmax")
    lv, ov = logits.tv(), out.tv()
    ctx.check(ctx.lib.gdb200_argmax_rows(ctx.backend, lv, softcap, ov), "argmax_rows")
    return out


def greedy_generate_native(model: GptLm, prompts: np.ndarray, new_tokens: int, capacity: int, use_graph: bool = True,
                           timing: Optional[dict] = None) -> np.ndarray:
    """Same result as greedy_generate, with sampling and the id / position feedback on the device:
    packed prefill, device argmax of the prefill logits, then new_tokens - 1 decode steps enqueued
    by gdb200_gpt_decode_steps with no host round trip; the generated ids are read once at the end.
    `timing` (a dict) receives device milliseconds measured with events on the backend stream: "prefill_ms"
    (packed prefill + first argmax) and "decode_ms" (the new_tokens - 1 decode steps), and "decode_launches"."""
    import ctypes as C
    ctx, cfg = model.ctx, model.cfg
    b, plen = prompts.shape
    model.alloc_kv_cache(b, capacity)
    lib, be = ctx.lib, ctx.backend
    ctx.begin_step()
    ids = ctx.from_numpy(ctx.data, I32, prompts.reshape(-1).astype(np.int32))
    pos = ctx.from_numpy(ctx.data, I32, np.tile(np.arange(plen, dtype=np.int32), b))
    cu = ctx.from_numpy(ctx.data, I32, (np.arange(b + 1, dtype=np.int32) * plen))
    cpos = ctx.from_numpy(ctx.data, I32, np.zeros(b, dtype=np.int32))
    ev = [lib.gdb200_event_record(be)] if timing is not None else None
    logits = model.prefill_last_logits(ids, pos, cu, cpos, np.arange(b) * plen + plen - 1)
    first = device_argmax(ctx, logits, cfg.logits_softcap)
    if ev is not None:
        ev.append(lib.gdb200_event_record(be))
    ctx.end_step()
    # io words: tokens [b] = argmax of the prefill logits, positions [b] = prompt length,
    # out_tokens [new_tokens, b] with row 0 filled, step counter = 1 (one read-back per generation)
    first_ids = first.read().astype(np.int32)
    words = np.zeros(2 * b + new_tokens * b + 1, dtype=np.int32)
    words[:b], words[b:2 * b], words[2 * b:3 * b], words[-1] = first_ids, plen, first_ids, 1
    io = ctx.from_numpy(ctx.state, I32, words)
    d = abi.GptDecodeState()
    d.cache_buffer, d.io_buffer = ctx.state.buffer, ctx.state.buffer
    for i in range(cfg.n_layers):
        d.k_cache_offset[i], d.v_cache_offset[i] = model.k_cache[i].offset, model.v_cache[i].offset
    d.tokens_offset, d.positions_offset = io.offset, io.offset + 4 * b
    d.out_tokens_offset, d.step_counter_offset = io.offset + 8 * b, io.offset + 8 * b + 4 * new_tokens * b
    d.batch, d.capacity, d.max_steps = b, capacity, new_tokens
    ctx.begin_step()
    spec = model_spec(model)
    launches0 = ctx.launch_count()
    if ev is not None:
        ev.append(lib.gdb200_event_record(be))
    ctx.check(lib.gdb200_gpt_decode_steps(be, C.byref(spec), C.byref(d), new_tokens - 1, 1 if use_graph else 0, None), "gpt_decode_steps")
    if ev is not None:
        ev.append(lib.gdb200_event_record(be))
    ctx.end_step()
    ctx.flush()
    if ev is not None:
        timing["prefill_ms"] = float(lib.gdb200_event_elapsed_ms(ev[0], ev[1]))
        timing["decode_ms"] = float(lib.gdb200_event_elapsed_ms(ev[2], ev[3]))
        timing["decode_launches"] = int(ctx.launch_count() - launches0)
        for e in ev:
            lib.gdb200_event_destroy(e)
    flat = io.read()
    return flat[2 * b:2 * b + new_tokens * b].reshape(new_tokens, b).T.copy()


def host_argmax(logits: np.ndarray, softcap: float) -> np.ndarray:
    x = logits.astype(np.float32)
    if softcap > 0.0:
        x = np.float32(softcap) * np.tanh(x / np.float32(softcap))
    x = np.where(np.isfinite(x), x, -np.inf)
    return np.argmax(x, axis=1).astype(np.int32)  # numpy argmax returns the first maximum
