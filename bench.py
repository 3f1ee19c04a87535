"""Benchmark of the gpt_lm hot path on B200 through the backend's C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload train|decode]

One "step" is one full gpt_lm training step (forward, backward with AMP, gradient clipping,
AdamW on FP32 masters) over one packed synthetic batch of the benchmark configuration:
vocab 2048, context 512, d_model 512, 3 layers, 8 heads x 64, SwiGLU hidden 1536, untied biased
LM head, dropout 0.1, logits soft cap 30; 64 sequences per GPU with lengths uniform in [64, 512],
padded with ignored rows to a multiple of 512 (padding is not counted as tokens).

Prints ONE JSON line (rank 0). `value` is tokens/s with the batches already resident in HBM;
`e2e` is the same metric with the per-step host->device copy of the batch from pinned host
memory and the device->host read of the loss inside the timed region. `roofline` describes the
dense-contraction kernels (the dominant ones), timed live with CUDA event pairs on the backend
stream; `cpu_baseline` times the CPU oracle on the host cores on a bounded sample.

--impl reference times the reference's CPU implementation of the path: the reference has no CPU
numeric backend (its Linux build links a null backend), so its PyTorch-CPU oracle style restated
in oracle/ is what runs, with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "gpt_lm_train_tokens_per_s"
UNIT = "tokens/s"
N_SEQS, MIN_LEN, MAX_LEN = 64, 64, 512
# mean DRAM bytes (read + write) per dense-contraction launch of the default train step, from an ncu capture of this
# same command (profiles/gemm_pair_train_step_dram.md): below the algorithmic 78.5 MB because outputs stay in L2
GEMM_DRAM_BYTES_PER_LAUNCH = 64.0e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="train", choices=["train", "decode", "linear", "sdpa", "timeline"],
                    help="timeline: per-kernel time of the running train step from CUPTI activity records (not a bench line)")
    ap.add_argument("--cpu-sample-seqs", type=int, default=8, help="sequences in the CPU-baseline sample batch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--host", default="native", choices=["native", "python"],
                    help="who enqueues the per-step backend calls: the library's native driver or the Python op capsules")
    ap.add_argument("--gemm-mode", type=int, default=0, help="0 auto, 1 portable kernel only, 2 tcgen05 required, 3 auto without the CTA-pair kernel")
    ap.add_argument("--model", default="baseline", choices=["baseline", "reference_default", "scaled"],
                    help="train workload: baseline = the benchmark configuration (default); reference_default = the reference's own "
                         "defaults (F1024, tied head, dropout 0.05, window 256); scaled = BF16 d2048 L24 H16x128 F5632 V32768 ctx2048, "
                         "32 sequences of U[256,2048] per GPU")
    ap.add_argument("--linear-shape", default="4096,512,1536", help="M,K,N of --workload linear (default: the C1 configuration)")
    ap.add_argument("--attention-mode", type=int, default=0, help="0 auto (tcgen05 forward when the shape allows), 1 mma.sync flash kernels only")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def model_flops_per_step(cfg, batch) -> float:
    """6 * N_mm * T for the contractions plus 14 * Dh * pairs * heads per layer for attention."""
    import numpy as np
    d, f, v, layers = cfg.d_model, cfg.mlp_hidden, cfg.vocab_size, cfg.n_layers
    n_mm = layers * (d * 3 * d + d * d + d * 2 * f + f * d) + v * d
    t = int(batch.input_ids.size)
    lens = np.diff(batch.cu_seqlens).astype(np.int64)
    if cfg.sdpa_window > 0:
        pairs = sum(int(sum(min(i + 1, cfg.sdpa_window) for i in range(int(n)))) for n in lens)
    else:
        pairs = int((lens * (lens + 1) // 2).sum())
    return 6.0 * n_mm * t + 14.0 * cfg.head_dim * pairs * cfg.n_heads * layers


# --------------------------------------------------------------------------------------- reference arm
def run_reference(args) -> None:
    """CPU arm: the oracle's training step on a bounded sample of the workload, all host threads."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    import numpy as np
    import torch
    import __graft_entry__ as graft
    from oracle import gpt_lm as OG
    pkg = graft.load_package()
    g = pkg.gpt_lm
    cfg, tc = g.GptConfig.baseline(), g.TrainConfig.baseline()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    hp = g.init_params(cfg, seed=0)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    otc = OG.train_config_from(tc)
    n_seqs = args.cpu_sample_seqs
    times, tokens = [], 0
    for step in range(args.warmup + args.steps):
        b = g.synthetic_batch(cfg, n_seqs, MIN_LEN, MAX_LEN, seed=1000 + step, pad_to=cfg.context_length)
        t0 = time.perf_counter()
        ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, step + 1, otc)
        dt = time.perf_counter() - t0
        if step >= args.warmup:
            times.append(dt)
            tokens += b.real_tokens
    total = sum(times)
    value = tokens / total
    sample = f"{n_seqs} of {N_SEQS} sequences per step (same length distribution), {args.steps} steps"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * total / max(1, len(times)), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "gpt_lm train step, vocab 2048 ctx 512 d512 L3 H8x64 F1536 untied, CPU oracle", "global_batch": n_seqs,
                   "seq_len": "U[64,512] packed"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline(g, cfg, tc, seqs: int) -> dict:
    import torch
    from oracle import gpt_lm as OG
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref = OG.OracleGptLm(OG.config_from(cfg), g.init_params(cfg, seed=0))
    otc = OG.train_config_from(tc)
    tokens, total = 0, 0.0
    for step in range(3):
        b = g.synthetic_batch(cfg, seqs, MIN_LEN, MAX_LEN, seed=2000 + step, pad_to=cfg.context_length)
        t0 = time.perf_counter()
        ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, step + 1, otc)
        dt = time.perf_counter() - t0
        if step >= 1:
            tokens += b.real_tokens
            total += dt
    return {"value": tokens / total, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"2 timed steps of {seqs} of {N_SEQS} sequences (lengths U[64,512]) after 1 warm-up, torch CPU threads = all cores"}


# --------------------------------------------------------------------------------------- B200 arm
def run_b200(args) -> None:
    rank, world, local = dist_env()
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with WORLD_SIZE={args.gpus} (got {world})")
    dist = None
    if world > 1:
        import torch  # loaded first so that both NCCL users bind the same libnccl
        import torch.distributed as dist
        os.environ.setdefault("GD_CUDA_DEVICE", str(local))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    import numpy as np
    import ctypes as C
    import __graft_entry__ as graft
    pkg = graft.load_package()
    g, abi = pkg.gpt_lm, pkg.abi
    n_seqs, min_len, max_len = N_SEQS, MIN_LEN, MAX_LEN
    if args.model == "scaled":
        cfg, tc = g.GptConfig.scaled(), g.TrainConfig.baseline()
        n_seqs, min_len, max_len = 32, 256, 2048
        ctx = pkg.runtime.Context(params_bytes=4 << 30, state_bytes=20 << 30, scratch_bytes=120 << 30, data_bytes=64 << 20)
    else:
        cfg = g.GptConfig.baseline() if args.model == "baseline" else g.GptConfig.reference_default()
        tc = g.TrainConfig.baseline() if args.model == "baseline" else g.TrainConfig()
        ctx = pkg.runtime.Context(params_bytes=256 << 20, state_bytes=1 << 30, scratch_bytes=10 << 30, data_bytes=64 << 20)
    lib = ctx.lib
    lib.gdb200_set_gemm_mode(ctx.backend, args.gemm_mode)
    lib.gdb200_set_attention_mode(ctx.backend, args.attention_mode)
    model = g.GptLm(ctx, cfg, g.init_params(cfg, seed=0))
    dp = None
    if world > 1:
        from gradients_c_b200.host import dp as dpmod
        dp = dpmod.DataParallel(ctx, model, rank, world, dist)
    trainer = (g.NativeTrainer if args.host == "native" else g.Trainer)(model, tc, dp=dp)

    total_steps = args.warmup + args.steps
    if world == 1:
        batches = [g.synthetic_batch(cfg, n_seqs, min_len, max_len, seed=10_000 + s, pad_to=cfg.context_length) for s in range(total_steps)]
    else:
        # the global batch of a step (n_seqs * world sequences, same length distribution) is drawn once on every rank
        # from the same seed and dealt out token-balanced, because a synchronous step runs at the pace of its heaviest rank
        from gradients_c_b200.host.dp import balanced_shards
        batches = []
        for s in range(total_steps):
            lens = np.random.default_rng(77_000 + s).integers(min_len, max_len + 1, size=n_seqs * world)
            mine = balanced_shards(lens, world)[rank]
            batches.append(g.synthetic_batch(cfg, n_seqs, min_len, max_len, seed=10_000 * (rank + 1) + s, pad_to=cfg.context_length,
                                             lengths=[int(lens[i]) for i in mine]))

    # end-to-end arm: the host batches live in page-locked memory
    for b in batches:
        b.input_ids, b.targets = ctx.pinned_copy(b.input_ids), ctx.pinned_copy(b.targets)
        b.positions, b.cu_seqlens = ctx.pinned_copy(b.positions), ctx.pinned_copy(b.cu_seqlens)

    loss_slots = [ctx.pinned_copy(np.zeros(1, dtype=np.float32)) for _ in range(2)]

    def barrier():
        ctx.flush()
        if dist is not None:
            dist.barrier()

    host_enqueue = [0.0]

    def timed_loop(e2e: bool):
        """Runs warm-up + K timed steps; returns (seconds, tokens, launches, last loss)."""
        staged = None
        if not e2e:
            # batches resident in HBM before the timed region: uploaded once into the state arena
            staged = []
            for b in batches:
                staged.append(tuple(ctx.from_numpy(ctx.state, abi.I32, a) for a in (b.input_ids, b.targets, b.positions, b.cu_seqlens)))
        loss_val = None
        # End-to-end loop: every step copies its batch from page-locked host memory and its loss back to the host,
        # both in stream order, and the host consumes the loss of step k while the device runs step k + 1 (one step
        # of run-ahead, as the reference's slot rings allow); all K copies and reads complete inside the timed region.
        ctx.run_ahead = 1 if e2e else 0

        def e2e_step(s):
            trainer.train_batch(batches[s], loss_out=loss_slots[s & 1])
            ctx.wait_steps(1)                      # step s - 1 is complete: its loss is on the host
            return float(loss_slots[(s - 1) & 1][0])

        for s in range(args.warmup):
            if e2e:
                loss_val = e2e_step(s)
            else:
                loss = trainer.train_batch(batches[s], device_batch=staged[s])
        barrier()
        launches0 = ctx.launch_count()
        ev0 = lib.gdb200_event_record(ctx.backend)
        t0 = time.perf_counter()
        tokens = 0
        for s in range(args.warmup, total_steps):
            if e2e:
                loss_val = e2e_step(s)
            else:
                loss = trainer.train_batch(batches[s], device_batch=staged[s])
            tokens += batches[s].real_tokens
        ev1 = lib.gdb200_event_record(ctx.backend)
        host_enqueue[0] = time.perf_counter() - t0
        barrier()
        if e2e:
            ctx.wait_steps(0)
            loss_val = float(loss_slots[(total_steps - 1) & 1][0])   # the last step's loss, read before the clock stops
        wall = time.perf_counter() - t0
        ctx.run_ahead = 0
        dev_ms = lib.gdb200_event_elapsed_ms(ev0, ev1)
        lib.gdb200_event_destroy(ev0)
        lib.gdb200_event_destroy(ev1)
        if loss_val is None:
            loss_val = float(loss.read()[()])
        # device time for the HBM-resident loop; wall time (which contains the copies and the
        # host-side read of the loss) for the end-to-end loop
        seconds = wall if e2e else dev_ms / 1000.0
        return seconds, tokens, ctx.launch_count() - launches0, loss_val

    sampler = ClockSampler(local)
    sampler.start()
    lib.gdb200_gemm_profile_enable(ctx.backend, 0)
    sec, tokens, launches, loss_val = timed_loop(e2e=False)
    clocks = sampler.stop()
    host_ms = 1000.0 * host_enqueue[0] / args.steps
    e_sec, e_tokens, _, _ = timed_loop(e2e=True)

    # roofline of the dominant kernels (dense contractions): a short separately instrumented run
    lib.gdb200_gemm_profile_enable(ctx.backend, 1)
    prof_steps = min(3, args.steps)
    for s in range(prof_steps):
        trainer.train_batch(batches[args.warmup + s])
    n_l, ms, fl, by = C.c_uint64(), C.c_double(), C.c_double(), C.c_double()
    lib.gdb200_gemm_profile_read(ctx.backend, C.byref(n_l), C.byref(ms), C.byref(fl), C.byref(by))
    lib.gdb200_gemm_profile_enable(ctx.backend, 0)
    peaks = measured_peaks()
    achieved_tf = fl.value / (ms.value * 1e-3) / 1e12 if ms.value > 0 else 0.0
    step_ms_prof = 1000.0 * sec / args.steps
    roofline = {"bound": "tensor", "achieved": achieved_tf, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved_tf / peaks["bf16_tflops_sustained"], "traffic": GEMM_DRAM_BYTES_PER_LAUNCH if args.model == "baseline" else None,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the 39 gemm_pair_kernel launches of one step "
                                  "(profiles/gemm_pair_train_step_dram.md); algorithmic bytes per launch = algorithmic_gb_per_step / launches_per_step",
                "peak_source": peaks["source"] + " (sustained)",
                "kernel": "dense contractions (matmul / matmul_nt / matmul_tn / linear)", "launches_per_step": n_l.value / prof_steps,
                "avg_launch_us": 1000.0 * ms.value / max(1, n_l.value), "share_of_step": (ms.value / prof_steps) / step_ms_prof,
                "algorithmic_gb_per_step": by.value / prof_steps / 1e9}

    # max over ranks of the timed durations, totals of tokens
    if dist is not None:
        import torch
        t = torch.tensor([sec, e_sec], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec, e_sec = float(t[0]), float(t[1])
        k = torch.tensor([tokens, e_tokens, launches], dtype=torch.float64)
        dist.all_reduce(k, op=dist.ReduceOp.SUM)
        tokens, e_tokens, launches = int(k[0]), int(k[1]), int(k[2])
    if rank == 0:
        flops = sum(model_flops_per_step(cfg, b) for b in batches[args.warmup:]) * 1.0
        out = {
            "metric": METRIC, "value": tokens / sec, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * sec / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if args.model == "scaled" else "f16", "data": "synthetic",
            "config": {"workload": f"gpt_lm train step ({args.model}), vocab {cfg.vocab_size} ctx {cfg.context_length} d{cfg.d_model} L{cfg.n_layers} "
                                   f"H{cfg.n_heads}x{cfg.head_dim} F{cfg.mlp_hidden} {'tied' if cfg.tied_lm_head else 'untied'} head, dropout {cfg.dropout_p}, "
                                   f"window {cfg.sdpa_window}, softcap {cfg.logits_softcap:g}, AdamW AMP clip",
                       "global_batch": n_seqs * world, "seq_len": f"U[{min_len},{max_len}] packed, padded to x{cfg.context_length}", "parallelism": f"dp{world}", "host": args.host,
                       "sharding": "one batch" if world == 1 else "global batch dealt out token-balanced (longest first to the lightest rank)",
                       "l2": "per-step working set (>2 GB of activations) exceeds the 126 MB L2; no explicit flush"},
            "e2e": {"value": e_tokens / e_sec, "unit": UNIT, "h2d_bytes_per_step": int(np.mean([b.h2d_bytes for b in batches])),
                    "d2h_bytes_per_step": 4,
                    "overlap": "copies are stream-ordered from / to page-locked memory; the host reads the loss of step k while step k+1 runs"},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "model_tflops": flops * world / sec / 1e12, "loss": loss_val, "host_enqueue_ms_per_step": host_ms,
        }
        if not args.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline(g, cfg, tc, args.cpu_sample_seqs)
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.destroy()


# --------------------------------------------------------------------------------------- kernel-level workloads
def _event_timed(ctx, fn, steps: int, warmup: int, flush_l2: bool = True) -> float:
    """Average device milliseconds of fn() over `steps` runs, each bracketed by its own CUDA event
    pair on the backend stream; L2 is flushed (untimed) before every run."""
    lib = ctx.lib
    for _ in range(warmup):
        fn()
    ctx.flush()
    total = 0.0
    for _ in range(steps):
        if flush_l2:
            ctx.check(lib.gdb200_flush_l2(ctx.backend), "flush_l2")
        e0 = lib.gdb200_event_record(ctx.backend)
        fn()
        e1 = lib.gdb200_event_record(ctx.backend)
        total += lib.gdb200_event_elapsed_ms(e0, e1)
        lib.gdb200_event_destroy(e0)
        lib.gdb200_event_destroy(e1)
    return total / steps


def run_linear(args) -> None:
    """Single F16 linear forward + backward: X[4096,512], W[1536,512] (transposed-weight layout),
    dY[4096,1536]; outputs Y, dX, dW, db."""
    import ctypes as C
    import numpy as np
    import __graft_entry__ as graft
    pkg = graft.load_package()
    abi = pkg.abi
    m, k, n = (int(v) for v in args.linear_shape.split(","))
    ctx = pkg.runtime.Context(params_bytes=max(64 << 20, 8 * (m * k + n * k + 2 * m * n)), state_bytes=64 << 20, scratch_bytes=256 << 20, data_bytes=8 << 20)
    lib = ctx.lib
    lib.gdb200_set_gemm_mode(ctx.backend, args.gemm_mode)
    rng = np.random.default_rng(0)
    x = ctx.from_numpy(ctx.params, abi.F16, rng.standard_normal((m, k)).astype(np.float32))
    w = ctx.from_numpy(ctx.params, abi.F16, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    dy = ctx.from_numpy(ctx.params, abi.F16, rng.standard_normal((m, n)).astype(np.float32))
    y, dx, dw, db = (ctx.empty(ctx.params, abi.F16, s) for s in ((m, n), (m, k), (n, k), (n,)))
    xv, wv, yv, dyv, dxv, dwv = x.mv(m, k), w.mv(n, k), y.mv(m, n), dy.mv(m, n), dx.mv(m, k), dw.mv(n, k)
    dbv = db.vv()

    def step():
        ctx.check(lib.gd_backend_matmul_nt(ctx.backend, C.byref(xv), C.byref(wv), C.byref(yv)), "y")
        ctx.check(lib.gd_backend_matmul(ctx.backend, C.byref(dyv), C.byref(wv), C.byref(dxv)), "dx")
        ctx.check(lib.gd_backend_matmul_tn(ctx.backend, C.byref(dyv), C.byref(xv), C.byref(dwv)), "dw")
        ctx.check(lib.gd_backend_reduce_rows(ctx.backend, C.byref(dyv), C.byref(dbv)), "db")

    l0 = ctx.launch_count()
    ms = _event_timed(ctx, step, args.steps, args.warmup)
    launches = (ctx.launch_count() - l0) // (args.steps + args.warmup) - 1
    peaks = measured_peaks()
    flops = 6.0 * m * n * k
    tf = flops / (ms * 1e-3) / 1e12
    print(json.dumps({"metric": "linear_fwd_bwd_ms", "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": ms, "higher_is_better": False, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": f"linear fwd+bwd X[{m},{k}] W[{n},{k}] dY[{m},{n}]", "l2": "flushed before every timed step"},
                      "gpu_launches": launches,
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                                   "traffic": None, "peak_source": peaks["source"] + " (burst)", "note": "includes reduce_rows and launch gaps"}}))
    ctx.destroy()


def run_sdpa(args) -> None:
    """Packed causal sdpa_varlen forward + backward, 8 heads x 64, 32768 tokens in sequences of
    length U[16,512], q/k/v produced by qkv_split_rope from a fused QKV[T,1536]."""
    import numpy as np
    import __graft_entry__ as graft
    pkg = graft.load_package()
    abi, ops = pkg.abi, pkg.ops
    rng = np.random.default_rng(0)
    lens, total = [], 32768
    while sum(lens) < total:
        lens.append(int(rng.integers(16, 513)))
    lens[-1] -= sum(lens) - total
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
    ctx = pkg.runtime.Context(params_bytes=512 << 20, state_bytes=64 << 20, scratch_bytes=1 << 30, data_bytes=8 << 20)
    qkv = ctx.from_numpy(ctx.params, abi.F16, rng.standard_normal((total, 1536)).astype(np.float32))
    go = ctx.from_numpy(ctx.params, abi.F16, rng.standard_normal((total, 8, 64)).astype(np.float32))
    cut, post = ctx.from_numpy(ctx.params, abi.I32, cu), ctx.from_numpy(ctx.params, abi.I32, pos)
    window = 0
    pairs = float(sum(n * (n + 1) // 2 for n in lens)) * 8
    results = {}
    for name in ("rope", "fwd", "fwd_bwd"):
        def step():
            ctx.begin_step()
            q, k, v = ops.gd_qkv_split_rope(ctx, qkv, post, 8, 64)
            if name != "rope":
                q.requires_grad = k.requires_grad = v.requires_grad = name == "fwd_bwd"
                out = ops.gd_sdpa_varlen(ctx, q, k, v, cut, causal=True, sliding_window=window, max_seqlen=512)
                if name == "fwd_bwd":
                    out.grad = go
                    ctx.run_backward()
            ctx.end_step()
        results[name] = _event_timed(ctx, step, args.steps, args.warmup)
    fwd_ms = results["fwd"] - results["rope"]
    bwd_ms = results["fwd_bwd"] - results["fwd"]
    peaks = measured_peaks()
    tf = 14.0 * 64 * pairs / ((fwd_ms + bwd_ms) * 1e-3) / 1e12
    print(json.dumps({"metric": "sdpa_varlen_fwd_bwd_ms", "value": fwd_ms + bwd_ms, "unit": "ms", "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": fwd_ms + bwd_ms, "higher_is_better": False, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "sdpa_varlen fwd+bwd H8 Dh64 T32768 lengths U[16,512] causal", "segments": len(lens),
                                 "l2": "flushed before every timed step"},
                      "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "qkv_split_rope_ms": results["rope"],
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                                   "traffic": None, "peak_source": peaks["source"] + " (burst)", "flops": "14*Dh*pairs (FlashAttention convention)"}}))
    ctx.destroy()


def run_decode(args) -> None:
    """KV-cache greedy decode: 64 prompts x 256 tokens, packed prefill, 256 decode steps, cache capacity 512."""
    import numpy as np
    import __graft_entry__ as graft
    pkg = graft.load_package()
    g = pkg.gpt_lm
    cfg = g.GptConfig.baseline()
    cfg.dropout_p = 0.0
    ctx = pkg.runtime.Context(params_bytes=256 << 20, state_bytes=1 << 30, scratch_bytes=2 << 30, data_bytes=16 << 20)
    model = g.GptLm(ctx, cfg, g.init_params(cfg, seed=0))
    model.training = False
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(64, 256)).astype(np.int32)
    new_tokens = 256
    native = args.host == "native"
    generate = (lambda p, n: g.greedy_generate_native(model, p, n, 512)) if native else (lambda p, n: g.greedy_generate(model, p, n, 512))
    generate(prompts[:, :32], 4)  # warm-up (kernel loading)
    l0 = ctx.launch_count()
    t0 = time.perf_counter()
    out = generate(prompts, new_tokens)
    ctx.flush()
    dt = time.perf_counter() - t0
    value = 64 * new_tokens / dt
    print(json.dumps({"metric": "gpt_lm_kv_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": new_tokens, "warmup": 1,
                      "ms_per_step": 1000.0 * dt / new_tokens, "higher_is_better": True, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "greedy KV decode, 64 prompts x 256, 256 new tokens, cache 512, prefill included",
                                 "host": "native: device argmax, ids / positions fed back on the device, decode step replayed as a CUDA graph" if native
                                 else "python: host argmax and three small uploads per step"},
                      "gpu_launches": ctx.launch_count() - l0, "checksum": int(out.astype(np.int64).sum())}))
    ctx.destroy()


def run_timeline(args) -> None:
    """Per-kernel time of the default train step as it runs (real cache state, programmatic dependent launch in effect):
    CUPTI activity records collected by torch.profiler around `--steps` steps (default 100 is capped at 8). Kernels are
    launched before their predecessor ends and then wait, so raw durations overlap; the time attributed to a kernel is the
    increment of the completion front, end(k) - max(end(k-1), start(k)), which sums to the step. Prints a markdown table."""
    import collections
    import re
    import torch
    from torch.profiler import ProfilerActivity, profile
    import __graft_entry__ as graft
    pkg = graft.load_package()
    g = pkg.gpt_lm
    cfg, tc = g.GptConfig.baseline(), g.TrainConfig.baseline()
    ctx = pkg.runtime.Context(params_bytes=256 << 20, state_bytes=1 << 30, scratch_bytes=10 << 30, data_bytes=64 << 20)
    trainer = g.NativeTrainer(g.GptLm(ctx, cfg, g.init_params(cfg, seed=0)), tc)
    steps, warm = min(args.steps, 8), max(args.warmup, 3)
    batches = [g.synthetic_batch(cfg, 64, 64, 512, seed=10_000 + s, pad_to=cfg.context_length) for s in range(warm + steps)]
    staged = [tuple(ctx.from_numpy(ctx.state, pkg.abi.I32, a) for a in (b.input_ids, b.targets, b.positions, b.cu_seqlens)) for b in batches]
    for s in range(warm):
        trainer.train_batch(batches[s], device_batch=staged[s])
    ctx.flush()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for s in range(warm, warm + steps):
            trainer.train_batch(batches[s], device_batch=staged[s])
        ctx.flush()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.end)
    agg = collections.defaultdict(lambda: [0, 0.0, 0.0])
    prev_end, t0, t1 = ev[0].time_range.start, ev[0].time_range.start, ev[-1].time_range.end
    for e in ev:
        name = re.sub(r"\(.*", "", e.name.replace("void ", "").replace("(anonymous namespace)::", "").replace("gdb_t5::", ""))
        a = agg[name]
        a[0] += 1
        a[1] += e.time_range.end - max(prev_end, e.time_range.start)
        a[2] += e.time_range.end - e.time_range.start
        prev_end = e.time_range.end
    tot = sum(v[1] for v in agg.values())
    print(f"span {(t1 - t0) / steps:.1f} us/step, attributed {tot / steps:.1f} us/step, {len(ev)} records over {steps} steps")
    print("| kernel | launches/step | us/step (completion increments) | share | avg us | avg raw duration us |")
    print("|---|---|---|---|---|---|")
    for name, (c, t, d) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"| {name[:64]} | {c / steps:.1f} | {t / steps:.1f} | {100 * t / tot:.1f}% | {t / c:.1f} | {d / c:.1f} |")
    ctx.destroy()


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "linear":
        run_linear(args)
    elif args.workload == "sdpa":
        run_sdpa(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "timeline":
        run_timeline(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
