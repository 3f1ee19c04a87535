"""The reference's C host on the B200 backend: build location, batch file format and runner for
host_c/gpt_lm_synth (the reference's gpt_lm_shared.c + tape + optimizer, linked against this library).

The binary is built by host_c/Makefile from the reference tree where it lies; it travels with the tree.
"""
from __future__ import annotations

import json
import os
import struct
import subprocess
from typing import Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
HOST_C_DIR = os.path.join(os.path.dirname(HERE), "host_c")
BINARY = os.path.join(HOST_C_DIR, "_build", "gpt_lm_synth")
BATCH_MAGIC = 0x47445342
REFERENCE_SEED = 0x6750746C6D5EED00        # GPT_DEFAULT_SEED, examples/gpt_lm/gpt_lm_shared.h:59
DROPOUT_SEED_SALT = 0xD00D1234             # gpt_lm_init: dropout_seed = splitmix64(seed ^ 0xd00d1234)


def reference_dir() -> Optional[str]:
    """The reference source tree: $GD_REFERENCE_DIR, else a directory `reference` beside the repository."""
    cand = os.environ.get("GD_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
    return cand if os.path.exists(os.path.join(cand, "src", "core", "backend.h")) else None


def build(jobs: int = 8) -> Optional[str]:
    """Builds host_c/_build/gpt_lm_synth when the reference tree is present; returns the binary's path if it exists."""
    ref = reference_dir()
    if ref is not None:
        res = subprocess.run(["make", "-C", HOST_C_DIR, f"REF={ref}", f"-j{jobs}"], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"host_c build failed:\n{res.stdout[-3000:]}\n{res.stderr[-3000:]}")
    return BINARY if os.path.exists(BINARY) else None


def write_batches(path: str, batches: Sequence) -> None:
    """Batch file read by gpt_lm_synth: int32 magic, count, then per batch n_tokens, n_cu, ids, targets, positions,
    cu_seqlens, real_tokens."""
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", BATCH_MAGIC, len(batches)))
        for b in batches:
            f.write(struct.pack("<ii", int(b.input_ids.size), int(b.cu_seqlens.size)))
            for a in (b.input_ids, b.targets, b.positions, b.cu_seqlens):
                f.write(np.ascontiguousarray(a, dtype="<i4").tobytes())
            f.write(struct.pack("<i", int(b.real_tokens)))


def read_params(path: str) -> dict[str, np.ndarray]:
    """Parameter dump of gpt_lm_synth --dump-params: name -> flat float32 array (values on the F16 grid)."""
    out = {}
    with open(path, "rb") as f:
        while True:
            head = f.read(4)
            if len(head) < 4:
                break
            (n,) = struct.unpack("<i", head)
            name = f.read(n).decode()
            (count,) = struct.unpack("<q", f.read(8))
            out[name] = np.frombuffer(f.read(4 * count), dtype="<f4").copy()
    return out


def run(batch_file: str, steps: int, warmup: int, *, layers: int = 3, feed: str = "hostptr", scratch_slots: int = 1, data_slots: int = 1,
        read_loss: bool = False, dump_params: Optional[str] = None, dropout: Optional[float] = None, env: Optional[dict] = None,
        timeout: float = 600.0) -> dict:
    if not os.path.exists(BINARY):
        raise FileNotFoundError(f"{BINARY} is not built (it needs the reference tree: make -C {HOST_C_DIR} REF=<tree>)")
    cmd = [BINARY, "--batches", batch_file, "--steps", str(steps), "--warmup", str(warmup), "--layers", str(layers), "--feed", feed,
           "--scratch-slots", str(scratch_slots), "--data-slots", str(data_slots)]
    if read_loss:
        cmd.append("--read-loss")
    if dump_params:
        cmd += ["--dump-params", dump_params]
    if dropout is not None:
        cmd += ["--dropout", repr(float(dropout))]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env={**os.environ, **(env or {})})
    if res.returncode != 0:
        raise RuntimeError(f"gpt_lm_synth failed (rc {res.returncode}):\n{res.stdout[-2000:]}\n{res.stderr[-2000:]}")
    return json.loads(res.stdout.strip().splitlines()[-1])
