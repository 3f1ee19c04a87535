"""Builds the oracle's native pieces with the committed Makefile: the plain-C restatement
(oracle/c/liboracle_int.so) always, and - when the reference tree is present - the reference's
own host code, the exported CPU references of its C tests and its C tests linked against the
B200 backend, all into oracle/_ref/ (never into history, never copied sources)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_dir() -> str:
    """The reference source tree: $GD_REFERENCE_DIR, else a directory `reference` beside the repository."""
    return os.environ.get("GD_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref: str = "", jobs: int = 8) -> None:
    ref = ref or reference_dir()
    targets = ["cref"]
    if os.path.exists(os.path.join(ref, "src", "core", "backend.h")):
        targets += ["ref", "tests_cuda"]
    res = subprocess.run(["make", "-C", HERE, f"REF={ref}", f"-j{jobs}", *targets], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"oracle build failed:\n{res.stdout[-4000:]}\n{res.stderr[-4000:]}")


if __name__ == "__main__":
    build()
