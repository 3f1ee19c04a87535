"""AdamW with FP32 master weights, device-side AMP loss scaling and global-norm clipping.

Mirrors the reference optimizer's host logic for the path gpt_lm uses
(src/optim/adamw.c: gd_amp_scaler_* :1099-1352, gd_backward_amp seed :1354-1395,
gd_optimizer_step_amp_clip_lr :2163-2270, device state layout :21-33,138-157;
src/optim/lr_scheduler.c:20-57). All arithmetic runs in gd_backend_* kernels; this file only
lays out state tensors and builds the descriptor arrays.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import abi
from .abi import F16, BF16, F32, I32
from .runtime import Context, Tensor

byref = C.byref
GRAD_CLIP_SCALE_EPS = 1.0e-6
NORM_BLOCK = 1024  # gradient elements per partial (src/optim/adamw/metal_adamw_types.h)


@dataclass
class AmpConfig:  # gd_amp_config_default, src/optim/adamw.c:1099-1110
    enabled: bool = True
    init_scale: float = 32768.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    min_scale: float = 1.0
    max_scale: float = 2147483648.0
    growth_interval: int = 2000


@dataclass
class AdamwConfig:  # gd_adamw_config_default, src/optim/adamw.c:1087-1097
    lr: float = 1.0e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1.0e-8
    weight_decay: float = 0.01
    bias_correction: bool = True


def gd_lr_scheduler_value(max_lr: float, min_lr: float, warmup_steps: int, total_steps: int, step: int) -> float:
    """Linear warm-up then cosine decay, evaluated in double (src/optim/lr_scheduler.c:20-57)."""
    if warmup_steps > 0 and step < warmup_steps:
        lr = max_lr * step / warmup_steps
    elif total_steps == warmup_steps:
        lr = min_lr
    else:
        progress = min(1.0, max(0, step - warmup_steps) / (total_steps - warmup_steps))
        lr = min_lr + 0.5 * (max_lr - min_lr) * (1.0 + math.cos(math.pi * progress))
    return float(np.float32(lr))


class AmpScaler:
    """Device-resident loss scale: scale_state F32[2] = {scale, 1/scale}, flag_state I32[3] =
    {growth_tracker, found_inf, last_found_inf}."""

    def __init__(self, ctx: Context, config: Optional[AmpConfig] = None):
        self.ctx, self.config = ctx, config or AmpConfig()
        cfg = self.config
        s = min(max(cfg.init_scale, cfg.min_scale), cfg.max_scale)
        self.scale_state = ctx.from_numpy(ctx.state, F32, np.array([s, 1.0 / s], dtype=np.float32), "amp_scale")
        self.flag_state = ctx.from_numpy(ctx.state, I32, np.zeros(3, dtype=np.int32), "amp_flags")
        self.step_begun = False
        d = abi.AmpStateDesc()
        d.scale_buffer, d.scale_offset = self.scale_state.buffer, self.scale_state.offset
        d.flags_buffer, d.flags_offset = self.flag_state.buffer, self.flag_state.offset
        d.growth_factor, d.backoff_factor = cfg.growth_factor, cfg.backoff_factor
        d.min_scale, d.max_scale, d.growth_interval = cfg.min_scale, cfg.max_scale, cfg.growth_interval
        self.desc = d

    def begin_step(self) -> None:
        if not self.step_begun:
            self.ctx.check(self.ctx.lib.gd_backend_amp_begin_step(self.ctx.backend, byref(self.desc)), "amp_begin_step")
            self.step_begun = True

    def finish_step(self) -> None:
        self.ctx.check(self.ctx.lib.gd_backend_amp_finish_step(self.ctx.backend, byref(self.desc)), "amp_finish_step")
        self.step_begun = False

    def fill_scale(self, dst: Tensor) -> None:
        self.begin_step()
        self.ctx.check(self.ctx.lib.gd_backend_amp_fill_scale(self.ctx.backend, dst.buffer, dst.offset, dst.count, dst.dtype,
                                                              self.scale_state.buffer, self.scale_state.offset), "amp_fill_scale")

    def sync(self) -> dict:
        s = self.scale_state.read()
        f = self.flag_state.read()
        return {"scale": float(s[0]), "inv_scale": float(s[1]), "growth_tracker": int(f[0]),
                "found_inf": int(f[1]), "last_found_inf": int(f[2])}


def gd_backward_amp(ctx: Context, loss: Tensor, scaler: Optional[AmpScaler]) -> None:
    """Seed d(loss) with the device loss scale (or 1) and walk the tape in reverse."""
    seed = ctx.scratch_empty(loss.dtype, loss.shape, "loss_grad")
    if scaler is not None and scaler.config.enabled:
        scaler.fill_scale(seed)
    else:
        one = {F32: 0x3F800000, F16: 0x3C00, BF16: 0x3F80}[loss.dtype]
        ctx.fill(seed, one)
    loss.grad = seed
    ctx.run_backward()


@dataclass
class ParamSlot:
    param: Tensor
    weight_decay: float
    lr_mult: float
    master: Optional[Tensor]
    m: Tensor
    v: Tensor


class AdamW:
    """gd_optimizer for AdamW: FP32 m/v (+ FP32 masters for 16-bit params) in the state arena and
    per-parameter device scalars [5][P] F32 (beta1^t, beta2^t, step_scale, decay_scale,
    eps_scaled) and I32 [P + 1] step counters."""

    F_BETA1, F_BETA2, F_STEP, F_DECAY, F_EPS = range(5)

    def __init__(self, ctx: Context, params: Sequence[Tensor], config: AdamwConfig, weight_decays: Optional[Sequence[float]] = None):
        self.ctx, self.config = ctx, config
        self.slots: list[ParamSlot] = []
        for i, p in enumerate(params):
            wd = config.weight_decay if weight_decays is None else weight_decays[i]
            master = None
            if p.dtype in (F16, BF16):
                master = ctx.empty(ctx.state, F32, p.shape, "master")
                master.write(p.read_f32())
            m = ctx.zeros(ctx.state, F32, p.shape, "adam_m")
            v = ctx.zeros(ctx.state, F32, p.shape, "adam_v")
            self.slots.append(ParamSlot(p, wd, 1.0, master, m, v))
        n = len(self.slots)
        f32 = np.zeros((5, n), dtype=np.float32)
        f32[self.F_BETA1] = 1.0
        f32[self.F_BETA2] = 1.0
        self.state_f32 = ctx.from_numpy(ctx.state, F32, f32, "optim_state_f32")
        self.state_i32 = ctx.from_numpy(ctx.state, I32, np.zeros(n + 1, dtype=np.int32), "optim_state_i32")
        self.partial_capacity = sum((s.param.count + NORM_BLOCK - 1) // NORM_BLOCK for s in self.slots)
        self.partials = ctx.zeros(ctx.state, F32, (max(1, self.partial_capacity),), "grad_norm_partials")
        self.grad_clip_scale = ctx.from_numpy(ctx.state, F32, np.array([1.0, 0.0], dtype=np.float32), "grad_clip_scale")
        self.n = n
        self._norm_descs = (abi.GradNormDesc * n)()
        self._adamw_descs = (abi.AdamwDesc * n)()

    def _f32_off(self, field: int, index: int) -> int:
        return self.state_f32.offset + (field * self.n + index) * 4

    def step_count(self) -> int:
        return int(self.state_i32.read()[self.n])

    def last_grad_norm(self) -> float:
        return float(self.grad_clip_scale.read()[1])

    def step_amp_clip_lr(self, scaler: AmpScaler, lr: float, max_grad_norm: float, inv_scale_override: Optional[Tensor] = None) -> None:
        """gd_optimizer_step_amp_clip_lr: unscale + global norm + clip factor in one pass over the
        gradients, then the AdamW update (skipped on overflow), then the scaler update."""
        ctx, lib = self.ctx, self.ctx.lib
        scaler.begin_step()
        inv_buf = scaler.scale_state.buffer
        inv_off = scaler.scale_state.offset + 4
        if inv_scale_override is not None:
            inv_buf, inv_off = inv_scale_override.buffer, inv_scale_override.offset
        found_buf, found_off = scaler.flag_state.buffer, scaler.flag_state.offset + 4
        count = 0
        partial_index = 0
        active = []
        for i, s in enumerate(self.slots):
            g = s.param.grad
            if g is None:
                continue
            groups = (s.param.count + NORM_BLOCK - 1) // NORM_BLOCK
            d = self._norm_descs[count]
            d.grad_buffer, d.grad_offset, d.count, d.grad_dtype = g.buffer, g.offset, g.count, g.dtype
            d.partial_buffer, d.partial_offset, d.partial_count = self.partials.buffer, self.partials.offset + partial_index * 4, groups
            d.grad_scale_buffer, d.grad_scale_offset = inv_buf, inv_off
            d.found_inf_buffer, d.found_inf_offset, d.has_found_inf = found_buf, found_off, 1
            partial_index += groups
            active.append(i)
            count += 1
        if count == 0:
            scaler.step_begun = False
            return
        ctx.check(lib.gd_backend_grad_clip_scale(ctx.backend, self._norm_descs, count, self.grad_clip_scale.buffer,
                                                 self.grad_clip_scale.offset, max_grad_norm, GRAD_CLIP_SCALE_EPS), "grad_clip_scale")
        cfg = self.config
        for j, i in enumerate(active):
            s = self.slots[i]
            g = s.param.grad
            d = self._adamw_descs[j]
            C.memset(byref(d), 0, C.sizeof(d))
            d.param_buffer, d.param_offset = s.param.buffer, s.param.offset
            if s.master is not None:
                d.master_buffer, d.master_offset, d.has_master = s.master.buffer, s.master.offset, 1
            d.grad_buffer, d.grad_offset = g.buffer, g.offset
            d.grad_scale_buffer, d.grad_scale_offset, d.has_grad_scale = self.grad_clip_scale.buffer, self.grad_clip_scale.offset, 1
            d.found_inf_buffer, d.found_inf_offset, d.has_found_inf = found_buf, found_off, 1
            d.m_buffer, d.m_offset, d.v_buffer, d.v_offset = s.m.buffer, s.m.offset, s.v.buffer, s.v.offset
            d.state_f32_buffer = self.state_f32.buffer
            d.beta1_power_offset, d.beta2_power_offset = self._f32_off(self.F_BETA1, i), self._f32_off(self.F_BETA2, i)
            d.step_scale_offset, d.decay_scale_offset = self._f32_off(self.F_STEP, i), self._f32_off(self.F_DECAY, i)
            d.eps_scaled_offset = self._f32_off(self.F_EPS, i)
            d.state_i32_buffer = self.state_i32.buffer
            d.param_step_offset = self.state_i32.offset + i * 4
            d.optimizer_step_offset = self.state_i32.offset + self.n * 4
            d.count, d.param_dtype, d.grad_dtype = s.param.count, s.param.dtype, g.dtype
            d.has_device_state, d.bias_correction = 1, 1 if cfg.bias_correction else 0
            d.update_optimizer_step = 1 if j == 0 else 0
            d.lr, d.beta1, d.beta2, d.eps, d.weight_decay = lr * s.lr_mult, cfg.beta1, cfg.beta2, cfg.eps, s.weight_decay
            d.bias_correction1 = d.bias_correction2 = 1.0
        ctx.check(lib.gd_backend_adamw_batch(ctx.backend, self._adamw_descs, count), "adamw_batch")
        scaler.finish_step()

    def zero_grad(self) -> None:
        for s in self.slots:
            s.param.grad = None
