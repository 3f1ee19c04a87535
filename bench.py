"""Benchmark of the gpt_lm hot path on B200 through the backend's C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--scaling weak|strong]
                    [--workload train|decode|linear|sdpa|c_host|timeline]

One "step" is one full gpt_lm training step (forward, backward with AMP, gradient clipping,
AdamW on FP32 masters) over one packed synthetic batch of the benchmark configuration:
vocab 2048, context 512, d_model 512, 3 layers, 8 heads x 64, SwiGLU hidden 1536, untied biased
LM head, dropout 0.1, logits soft cap 30; 64 sequences per GPU with lengths uniform in [64, 512]
(--scaling strong: 64 sequences in total, dealt out over the GPUs), padded with ignored rows to a
multiple of 512 (padding is not counted as tokens).

Prints ONE JSON line (rank 0). `value` is tokens/s with the batches already resident in HBM, over
exactly K steps timed with CUDA events; `e2e` is the same metric with the per-step host->device copy
of the batch from pinned host memory and the device->host read of the loss inside the timed region;
`spread` repeats the K-step loop ten times (median, min, max). `roofline` describes the
dense-contraction kernels (the dominant ones), timed live with CUDA event pairs on the backend
stream; `cpu_baseline` times the CPU oracle on the host cores on a bounded sample. On one GPU the
line also carries the other workloads the metric names, each measured in the same run: `decode`
(KV-cache greedy decode, 64 prompts x 256 tokens, 256 new tokens), `linear` (single F16 linear
forward + backward) and `sdpa` (packed causal attention forward + backward, T = 32768), and `c_host`
(the reference's own C host training its default model on this backend, when that binary is built).

--impl reference times the reference's CPU implementation of the path: the reference has no CPU
numeric backend (its Linux build links a null backend), so its PyTorch-CPU oracle style restated
in oracle/ is what runs, with all host threads, on the same 64-sequence batches.
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
SPREAD_REPEATS = 10


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="train", choices=["train", "decode", "linear", "sdpa", "c_host", "timeline"],
                    help="timeline: per-kernel time of the running train step from CUPTI activity records (not a bench line)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: 64 sequences per GPU; strong: a global batch of 64 sequences dealt out over the GPUs")
    ap.add_argument("--cpu-sample-seqs", type=int, default=N_SEQS, help="sequences per step of the CPU oracle (default: the full batch)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="train line only: skip the decode / linear / sdpa / c_host objects")
    ap.add_argument("--host", default="native", choices=["native", "python"],
                    help="who enqueues the per-step backend calls: the library's native driver or the Python op capsules")
    ap.add_argument("--gemm-mode", type=int, default=0, help="0 auto, 1 portable kernel only, 2 tcgen05 required, 3 auto without the CTA-pair kernel")
    ap.add_argument("--model", default="baseline", choices=["baseline", "reference_default", "scaled"],
                    help="train workload: baseline = the benchmark configuration (default); reference_default = the reference's own "
                         "defaults (F1024, tied head, dropout 0.05, window 256); scaled = BF16 d2048 L24 H16x128 F5632 V32768 ctx2048, "
                         "32 sequences of U[256,2048] per GPU")
    ap.add_argument("--linear-shape", default="4096,512,1536", help="M,K,N of --workload linear (default: the C1 configuration)")
    ap.add_argument("--decode-tokens", type=int, default=256, help="--workload decode: new tokens per prompt (default 256: positions 256..511; a small value makes a short run for profiling)")
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


def tensor_peak(peaks: dict, clocks: dict):
    """The tensor-core denominator that matches how the kernels were timed: the burst figure when the SM clock sampled
    during the timed region stayed within 5 % of its maximum (short, event-bracketed kernels), the sustained one when
    the clock had settled lower (a long step under the power cap)."""
    sm, mx = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
    if sm is not None and mx and sm < 0.95 * mx:
        return peaks["bf16_tflops_sustained"], f"{peaks['source']} (sustained: median SM clock {sm:.0f} of {mx:.0f} MHz)"
    return peaks["bf16_tflops"], f"{peaks['source']} (burst" + (f": median SM clock {sm:.0f} of {mx:.0f} MHz)" if sm is not None else ")")


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


def train_config_dict(cfg, model: str, n_seqs_global: int, min_len: int, max_len: int, world: int, scaling: str) -> dict:
    """The workload description both arms print (the B200 arm adds how it ran it)."""
    return {"workload": f"gpt_lm train step ({model}), vocab {cfg.vocab_size} ctx {cfg.context_length} d{cfg.d_model} L{cfg.n_layers} "
                        f"H{cfg.n_heads}x{cfg.head_dim} F{cfg.mlp_hidden} {'tied' if cfg.tied_lm_head else 'untied'} head, dropout {cfg.dropout_p}, "
                        f"window {cfg.sdpa_window}, softcap {cfg.logits_softcap:g}, AdamW AMP clip",
            "global_batch": n_seqs_global, "seq_len": f"U[{min_len},{max_len}] packed, padded to x{cfg.context_length}",
            "parallelism": f"dp{world}", "scaling": scaling}


def global_batch_seqs(world: int, scaling: str, per_gpu: int) -> int:
    return per_gpu if scaling == "strong" else per_gpu * world


# --------------------------------------------------------------------------------------- reference arm
def run_reference(args) -> None:
    """CPU arm: the oracle's training step on the same 64-sequence batches, all host threads. Under torchrun rank 0
    alone runs it (one process already uses every core); the line describes the same workload as the B200 arm."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
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
        b = g.synthetic_batch(cfg, n_seqs, MIN_LEN, MAX_LEN, seed=10_000 + step, pad_to=cfg.context_length)
        t0 = time.perf_counter()
        ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, step + 1, otc)
        dt = time.perf_counter() - t0
        if step >= args.warmup:
            times.append(dt)
            tokens += b.real_tokens
    total = sum(times)
    value = tokens / total
    gb = global_batch_seqs(args.gpus, args.scaling, N_SEQS)
    sample = (f"{n_seqs} sequences per step (the per-GPU batch of the B200 arm, same seeds and lengths), {args.steps} timed steps on one host; "
              f"tokens/s does not depend on how many such batches a {args.gpus}-GPU step holds")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * total / max(1, len(times)), "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": train_config_dict(cfg, "baseline", gb, MIN_LEN, MAX_LEN, args.gpus, args.scaling),
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
    tokens, total, timed = 0, 0.0, 0
    for step in range(4):
        b = g.synthetic_batch(cfg, seqs, MIN_LEN, MAX_LEN, seed=10_000 + step, pad_to=cfg.context_length)
        t0 = time.perf_counter()
        ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, step + 1, otc)
        dt = time.perf_counter() - t0
        if step >= 1:
            tokens += b.real_tokens
            total += dt
            timed += 1
    return {"value": tokens / total, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{timed} timed steps of {seqs} sequences (lengths U[64,512], the B200 arm's first batches) after 1 warm-up, torch CPU threads = all cores"}


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
    n_global = global_batch_seqs(world, args.scaling, n_seqs)
    if world == 1:
        batches = [g.synthetic_batch(cfg, n_seqs, min_len, max_len, seed=10_000 + s, pad_to=cfg.context_length) for s in range(total_steps)]
    else:
        # the global batch of a step (same length distribution) is drawn once on every rank from the same seed and dealt
        # out token-balanced, because a synchronous step runs at the pace of its heaviest rank
        from gradients_c_b200.host.dp import balanced_shards
        batches = []
        for s in range(total_steps):
            lens = np.random.default_rng(77_000 + s).integers(min_len, max_len + 1, size=n_global)
            mine = balanced_shards(lens, world)[rank]
            batches.append(g.synthetic_batch(cfg, len(mine), min_len, max_len, seed=10_000 * (rank + 1) + s, pad_to=cfg.context_length,
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

    host_issue = [0.0]
    staged = [tuple(ctx.from_numpy(ctx.state, abi.I32, a) for a in (b.input_ids, b.targets, b.positions, b.cu_seqlens)) for b in batches]

    def timed_loop(e2e: bool, with_warmup: bool = True):
        """Runs warm-up + K timed steps; returns (seconds, tokens, launches, last loss)."""
        loss_val = None
        # End-to-end loop: every step copies its batch from page-locked host memory and its loss back to the host,
        # both in stream order, and the host consumes the loss of step k while the device runs step k + 1 (one step
        # of run-ahead, as the reference's slot rings allow); all K copies and reads complete inside the timed region.
        ctx.run_ahead = 1 if e2e else 0

        def e2e_step(s):
            trainer.train_batch(batches[s], loss_out=loss_slots[s & 1])
            ctx.wait_steps(1)                      # step s - 1 is complete: its loss is on the host
            return float(loss_slots[(s - 1) & 1][0])

        for s in range(args.warmup if with_warmup else 0):
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
            if s == args.warmup:
                # the device was idle and the launch queue empty when this step was issued: pure host cost of one step
                host_issue[0] = time.perf_counter() - t0
            tokens += batches[s].real_tokens
        ev1 = lib.gdb200_event_record(ctx.backend)
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
    host_ms = 1000.0 * host_issue[0]
    # the same K-step loop repeated: how much one loop's figure moves from run to run
    repeat_ms = [1000.0 * timed_loop(e2e=False, with_warmup=False)[0] / args.steps for _ in range(SPREAD_REPEATS)]
    clocks = sampler.stop()
    e_sec, e_tokens, _, _ = timed_loop(e2e=True)

    # roofline of the dominant kernels (dense contractions): a short separately instrumented run
    lib.gdb200_gemm_profile_enable(ctx.backend, 1)
    prof_steps = min(3, args.steps)
    for s in range(prof_steps):
        trainer.train_batch(batches[args.warmup + s], device_batch=staged[args.warmup + s])
    n_l, ms, fl, by = C.c_uint64(), C.c_double(), C.c_double(), C.c_double()
    lib.gdb200_gemm_profile_read(ctx.backend, C.byref(n_l), C.byref(ms), C.byref(fl), C.byref(by))
    lib.gdb200_gemm_profile_enable(ctx.backend, 0)
    peaks = measured_peaks()
    peak_tf, peak_src = tensor_peak(peaks, clocks)
    achieved_tf = fl.value / (ms.value * 1e-3) / 1e12 if ms.value > 0 else 0.0
    step_ms_prof = 1000.0 * sec / args.steps
    roofline = {"bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved_tf / peak_tf,
                "traffic": None, "traffic_note": "DRAM bytes per launch are not measured by this run; the ncu capture of these kernels is summarised "
                                                 "under profiles/ (outputs of this size stay in the 126 MB L2, so DRAM traffic is below the algorithmic bytes)",
                "peak_source": peak_src,
                "kernel": "dense contractions (matmul / matmul_nt / matmul_tn / linear), each bracketed by its own CUDA event pair",
                "launches_per_step": n_l.value / prof_steps, "avg_launch_us": 1000.0 * ms.value / max(1, n_l.value),
                "share_of_step": (ms.value / prof_steps) / step_ms_prof, "algorithmic_gb_per_step": by.value / prof_steps / 1e9,
                "algorithmic_bytes_per_launch": by.value / max(1, n_l.value)}

    flops = float(sum(model_flops_per_step(cfg, b) for b in batches[args.warmup:]))
    # max over ranks of the timed durations, totals of tokens, launches and FLOPs
    if dist is not None:
        import torch
        t = torch.tensor([sec, e_sec] + repeat_ms, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec, e_sec, repeat_ms = float(t[0]), float(t[1]), [float(x) for x in t[2:]]
        k = torch.tensor([tokens, e_tokens, launches, flops], dtype=torch.float64)
        dist.all_reduce(k, op=dist.ReduceOp.SUM)
        tokens, e_tokens, launches, flops = int(k[0]), int(k[1]), int(k[2]), float(k[3])
    out = None
    if rank == 0:
        sm = clocks.get("sm_mhz")
        med = statistics.median(repeat_ms)
        conf = train_config_dict(cfg, args.model, n_global, min_len, max_len, world, args.scaling)
        conf.update({"host": args.host,
                     "sharding": "one batch" if world == 1 else "global batch dealt out token-balanced (longest first to the lightest rank)",
                     "loss_normaliser": "valid target rows of the global batch (one scalar all-reduce that overlaps the forward pass)" if world > 1 else "valid target rows",
                     "l2": "per-step working set (>2 GB of activations) exceeds the 126 MB L2; no explicit flush"})
        out = {
            "metric": METRIC, "value": tokens / sec, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * sec / args.steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "bf16" if args.model == "scaled" else "f16", "data": "synthetic", "config": conf,
            "e2e": {"value": e_tokens / e_sec, "unit": UNIT, "h2d_bytes_per_step": int(np.mean([b.h2d_bytes for b in batches])),
                    "d2h_bytes_per_step": 4,
                    "overlap": "copies are stream-ordered from / to page-locked memory; the host reads the loss of step k while step k+1 runs"},
            "spread": {"repeats": SPREAD_REPEATS, "steps_each": args.steps, "ms_per_step_median": med, "ms_per_step_min": min(repeat_ms),
                       "ms_per_step_max": max(repeat_ms), "ms_x_sm_mhz": med * sm if sm else None},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "model_tflops": flops / sec / 1e12, "loss": loss_val,
            "host_issue_ms_per_step": host_ms,
            "host_issue_note": "host time to issue the first timed step, on an idle device with an empty launch queue (later steps include waits for the device)",
        }
    ctx.destroy()
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(g, cfg, tc, args.cpu_sample_seqs)
        if not args.no_extras and args.model == "baseline":
            out["decode"] = measure_decode(args, with_cpu=not args.no_cpu_baseline)
            out["linear"] = measure_linear(args)
            out["sdpa"] = measure_sdpa(args)
            ch = measure_c_host(args)
            if ch is not None:
                out["c_host"] = ch
    if rank == 0:
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


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


def measure_linear(args) -> dict:
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
    bias = ctx.from_numpy(ctx.params, abi.F16, np.zeros(n, dtype=np.float32))
    y, dx, dw, db = (ctx.empty(ctx.params, abi.F16, s) for s in ((m, n), (m, k), (n, k), (n,)))
    xv, wv, yv, dyv, dxv, dwv = x.mv(m, k), w.mv(n, k), y.mv(m, n), dy.mv(m, n), dx.mv(m, k), dw.mv(n, k)
    dbv, bv = db.vv(), bias.vv()

    def step_reference_calls():
        # the reference's composition: matmul_nt, matmul, matmul_tn, reduce_rows
        ctx.check(lib.gd_backend_matmul_nt(ctx.backend, C.byref(xv), C.byref(wv), C.byref(yv)), "y")
        ctx.check(lib.gd_backend_matmul(ctx.backend, C.byref(dyv), C.byref(wv), C.byref(dxv)), "dx")
        ctx.check(lib.gd_backend_matmul_tn(ctx.backend, C.byref(dyv), C.byref(xv), C.byref(dwv)), "dw")
        ctx.check(lib.gd_backend_reduce_rows(ctx.backend, C.byref(dyv), C.byref(dbv)), "db")

    def step_fused_calls():
        # the additive entries the native step driver uses: bias in the GEMM epilogue, db from the dW pass
        ctx.check(lib.gdb200_matmul_nt_bias(ctx.backend, C.byref(xv), C.byref(wv), C.byref(bv), C.byref(yv)), "y + b")
        ctx.check(lib.gd_backend_matmul(ctx.backend, C.byref(dyv), C.byref(wv), C.byref(dxv)), "dx")
        ctx.check(lib.gdb200_matmul_tn_colsum(ctx.backend, C.byref(dyv), C.byref(xv), C.byref(dwv), C.byref(dbv)), "dw + db")

    out = {}
    for name, fn in (("reference_calls", step_reference_calls), ("fused_calls", step_fused_calls)):
        l0 = ctx.launch_count()
        ms = _event_timed(ctx, fn, args.steps, args.warmup)
        out[name] = (ms, (ctx.launch_count() - l0) // (args.steps + args.warmup) - 1)
    ctx.destroy()
    peaks = measured_peaks()
    flops = 6.0 * m * n * k
    ms = out["fused_calls"][0]
    tf = flops / (ms * 1e-3) / 1e12
    return {"metric": "linear_fwd_bwd_ms", "value": ms, "unit": "ms", "higher_is_better": False, "dtype": "f16",
            "config": {"workload": f"linear fwd+bwd X[{m},{k}] W[{n},{k}] dY[{m},{n}] (outputs Y, dX, dW, db)", "l2": "flushed before every timed step"},
            "gpu_launches_per_step": out["fused_calls"][1],
            "reference_call_sequence_ms": out["reference_calls"][0], "reference_call_sequence_launches": out["reference_calls"][1],
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                         "traffic": None, "peak_source": peaks["source"] + " (burst)",
                         "note": "6*M*N*K over the whole event-bracketed step: launch gaps and the bias-gradient column sums included"}}


def c2_case(seed: int = 0, total: int = 32768):
    import numpy as np
    rng = np.random.default_rng(seed)
    lens = []
    while sum(lens) < total:
        lens.append(int(rng.integers(16, 513)))
    lens[-1] -= sum(lens) - total
    return rng, lens


def measure_sdpa(args) -> dict:
    """Packed causal sdpa_varlen forward + backward, 8 heads x 64, 32768 tokens in sequences of
    length U[16,512], q/k/v produced by qkv_split_rope from a fused QKV[T,1536]."""
    import numpy as np
    import __graft_entry__ as graft
    pkg = graft.load_package()
    abi, ops = pkg.abi, pkg.ops
    total = 32768
    rng, lens = c2_case(0, total)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
    ctx = pkg.runtime.Context(params_bytes=512 << 20, state_bytes=64 << 20, scratch_bytes=1 << 30, data_bytes=8 << 20)
    ctx.lib.gdb200_set_attention_mode(ctx.backend, args.attention_mode)
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
    ctx.destroy()
    fwd_ms = results["fwd"] - results["rope"]
    bwd_ms = results["fwd_bwd"] - results["fwd"]
    peaks = measured_peaks()
    tf = 14.0 * 64 * pairs / ((fwd_ms + bwd_ms) * 1e-3) / 1e12
    el = total * 8 * 64
    fwd_bytes = 4.0 * el * 2 + 12.0 * total * 8            # q, k, v read, out written, statistics written
    bwd_bytes = 8.0 * el * 2 + 12.0 * total * 8            # q, k, v, out, dO read, dq, dk, dv written, statistics read
    gbs = (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
    return {"metric": "sdpa_varlen_fwd_bwd_ms", "value": fwd_ms + bwd_ms, "unit": "ms", "higher_is_better": False, "dtype": "f16",
            "config": {"workload": "sdpa_varlen fwd+bwd H8 Dh64 T32768 lengths U[16,512] causal", "segments": len(lens),
                       "l2": "flushed before every timed step"},
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "qkv_split_rope_ms": results["rope"],
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": peaks["source"],
                         "note": "algorithmic bytes: forward 4*T*H*Dh*2 + 12*T*H, backward 8*T*H*Dh*2 + 12*T*H; at these lengths the arithmetic intensity "
                                 "(about 100 FLOP/B) is below the ridge, so the byte roof binds",
                         "fwd_frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "bwd_frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "tensor_tflops": tf, "tensor_frac_of_burst": tf / peaks["bf16_tflops"], "flops": "14*Dh*pairs (FlashAttention convention)"}


def measure_decode(args, with_cpu: bool = True) -> dict:
    """KV-cache greedy decode: 64 prompts x 256 tokens, packed prefill, 256 new tokens, cache capacity 512."""
    import numpy as np
    import __graft_entry__ as graft
    pkg = graft.load_package()
    g = pkg.gpt_lm
    cfg = g.GptConfig.baseline()
    cfg.dropout_p = 0.0
    ctx = pkg.runtime.Context(params_bytes=256 << 20, state_bytes=1 << 30, scratch_bytes=2 << 30, data_bytes=16 << 20)
    hp = g.init_params(cfg, seed=0)
    model = g.GptLm(ctx, cfg, hp)
    model.training = False
    batch, plen, new_tokens, cap = 64, 256, max(4, int(getattr(args, "decode_tokens", 256))), 512
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(batch, plen)).astype(np.int32)
    native = args.host == "native"
    timing = {}
    if native:
        generate = lambda p, n, tm=None: g.greedy_generate_native(model, p, n, cap, timing=tm)
    else:
        generate = lambda p, n, tm=None: g.greedy_generate(model, p, n, cap)
    generate(prompts[:, :32], 4)  # warm-up (kernel loading)
    generate(prompts, new_tokens)
    ctx.flush()
    l0 = ctx.launch_count()
    t0 = time.perf_counter()
    out = generate(prompts, new_tokens, timing)          # uploads the prompts, downloads the generated ids
    ctx.flush()
    dt = time.perf_counter() - t0
    launches = ctx.launch_count() - l0
    ctx.destroy()
    peaks = measured_peaks()
    d, f, v, layers = cfg.d_model, cfg.mlp_hidden, cfg.vocab_size, cfg.n_layers
    n_mm = layers * (d * 3 * d + d * d + d * 2 * f + f * d) + v * d
    steps = new_tokens - 1
    # bytes one decode step must move: every weight once, and the live K and V rows of every sequence (positions plen .. plen + steps - 1)
    kv_rows = sum(plen + t + 1 for t in range(steps)) / steps
    bytes_per_step = 2.0 * n_mm + 2.0 * layers * batch * kv_rows * d * 2.0
    res = {"metric": "gpt_lm_kv_decode_tokens_per_s", "unit": "tokens/s", "higher_is_better": True, "dtype": "f16",
           "config": {"workload": f"greedy KV decode, {batch} prompts x {plen}, {new_tokens} new tokens, cache {cap}, gpt_lm baseline model",
                      "host": "native: all decode steps in one persistent cooperative kernel (grid barriers between the phases of a step), device argmax, ids / positions fed back on the device" if native
                      else "python: host argmax and three small uploads per step"},
           "checksum": int(out.astype(np.int64).sum()), "gpu_launches": launches}
    if native and timing:
        ms_step = timing["decode_ms"] / steps
        gbs = bytes_per_step / (ms_step * 1e-3) / 1e9
        res.update({"value": batch * steps / (timing["decode_ms"] * 1e-3), "ms_per_step": ms_step, "steps": steps,
                    "launches_per_step": timing["decode_launches"] / steps, "prefill_ms": timing["prefill_ms"],
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                                 "peak_source": peaks["source"], "algorithmic_bytes_per_step": bytes_per_step,
                                 "note": "weights once (2 B x 11.27 M) + live K / V of 64 sequences (mean over the timed positions)"}})
    else:
        res.update({"value": batch * new_tokens / dt, "ms_per_step": 1000.0 * dt / new_tokens, "steps": new_tokens})
    res["e2e"] = {"value": batch * new_tokens / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(prompts.nbytes // new_tokens),
                  "d2h_bytes_per_step": int(out.nbytes // new_tokens),
                  "note": "wall clock of the whole generation call: prompt upload, packed prefill, all decode steps, download of the generated ids"}
    if with_cpu:
        import torch
        from oracle import gpt_lm as OG
        torch.set_num_threads(os.cpu_count() or 1)
        ref = OG.OracleGptLm(OG.config_from(cfg), hp)
        sb, sn = 8, 9
        t0 = time.perf_counter()
        ref.greedy_generate(prompts[:sb], new_tokens=1, capacity=cap)
        t_prefill = time.perf_counter() - t0
        t0 = time.perf_counter()
        ref.greedy_generate(prompts[:sb], new_tokens=sn, capacity=cap)
        t_all = time.perf_counter() - t0
        per_step = max(t_all - t_prefill, 1e-9) / (sn - 1)
        res["cpu_baseline"] = {"value": sb / per_step, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"{sb} of {batch} prompts x {plen}, {sn - 1} decode steps after the prefill (prefill time measured separately and subtracted)"}
    return res


def measure_c_host(args):
    """The reference's own C host (gpt_lm_shared.c, tape, adamw.c inside gd_begin_step / gd_end_step) training its
    default model (F1024, tied head, window 256, dropout 0.05) on this backend, next to the native step driver on the
    same model and batches. None when the binary is not built (it needs the reference tree at build time)."""
    import tempfile
    import __graft_entry__ as graft
    pkg = graft.load_package()
    g, ch = pkg.gpt_lm, pkg.c_host
    if not os.path.exists(ch.BINARY):
        return None
    cfg, tc = g.GptConfig.reference_default(), g.TrainConfig()
    total = args.warmup + args.steps
    batches = [g.synthetic_batch(cfg, N_SEQS, MIN_LEN, MAX_LEN, seed=10_000 + s, pad_to=cfg.context_length) for s in range(total)]
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "batches.bin")
        ch.write_batches(path, batches)
        up = ch.run(path, steps=args.steps, warmup=args.warmup, feed="upload")
        hp = ch.run(path, steps=args.steps, warmup=args.warmup, feed="hostptr")
    ctx = pkg.runtime.Context(params_bytes=256 << 20, state_bytes=1 << 30, scratch_bytes=10 << 30, data_bytes=64 << 20)
    trainer = g.NativeTrainer(g.GptLm(ctx, cfg, g.init_params(cfg, seed=0)), tc)
    staged = [tuple(ctx.from_numpy(ctx.state, pkg.abi.I32, a) for a in (b.input_ids, b.targets, b.positions, b.cu_seqlens)) for b in batches]
    for s in range(args.warmup):
        trainer.train_batch(batches[s], device_batch=staged[s])
    ctx.flush()
    l0 = ctx.launch_count()
    e0 = ctx.lib.gdb200_event_record(ctx.backend)
    for s in range(args.warmup, total):
        trainer.train_batch(batches[s], device_batch=staged[s])
    e1 = ctx.lib.gdb200_event_record(ctx.backend)
    ctx.flush()
    native_ms = ctx.lib.gdb200_event_elapsed_ms(e0, e1) / args.steps
    native_launches = (ctx.launch_count() - l0) / args.steps
    ctx.destroy()
    tokens = sum(b.real_tokens for b in batches[args.warmup:])
    return {"metric": METRIC, "unit": UNIT, "value": up["tokens_per_s"], "ms_per_step": up["wall_ms_per_step"],
            "config": {"workload": "the reference's C host (examples/gpt_lm/gpt_lm_shared.c + tape + adamw.c), its default model (F1024, tied head, window 256, "
                                   "dropout 0.05), 64 sequences U[64,512] per step, batch placed with gd_tensor_write; wall clock, every step waits for the previous one "
                                   "(one scratch slot, gpt_lm_shared.c:175)"},
            "launches_per_step": up["launches_per_step"], "host_issue_ms_first_step": up["host_issue_ms_first_step"],
            "hostptr_feed": {"tokens_per_s": hp["tokens_per_s"], "ms_per_step": hp["wall_ms_per_step"],
                             "note": "batch written through the data slot's host pointer as the reference's loader threads do (managed memory: the pages migrate)"},
            "native_driver_same_model": {"tokens_per_s": tokens / (native_ms * 1e-3 * args.steps), "ms_per_step": native_ms, "launches_per_step": native_launches}}


def run_workload(args) -> None:
    """The single-workload modes print their object as one JSON line."""
    fn = {"linear": measure_linear, "sdpa": measure_sdpa, "decode": measure_decode, "c_host": measure_c_host}[args.workload]
    res = fn(args)
    if res is None:
        res = {"unavailable": "host_c/gpt_lm_synth is not built (it needs the reference tree at build time)"}
    res.update({"n_gpus": 1, "warmup": args.warmup, "data": "synthetic"})
    res.setdefault("steps", args.steps)
    print(json.dumps(res))


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
    elif args.workload in ("linear", "sdpa", "decode", "c_host"):
        run_workload(args)
    elif args.workload == "timeline":
        run_timeline(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
