"""pytest configuration: the `gpu` marker, package loading by path, golden-fixture access."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU and the built backend library")


class Golden:
    """Loads tests/golden/<group>.npz and groups the flat keys `case/field` by case."""

    def __init__(self, group: str):
        path = os.path.join(ROOT, "tests", "golden", group + ".npz")
        data = np.load(path)
        self.cases: dict[str, dict[str, np.ndarray]] = {}
        for key in data.files:
            case, field = key.split("/", 1)
            self.cases.setdefault(case, {})[field] = data[key]

    def __getitem__(self, case: str) -> dict:
        return self.cases[case]

    def names(self, prefix: str = "") -> list[str]:
        return sorted(n for n in self.cases if n.startswith(prefix))


@pytest.fixture(scope="session")
def pkg():
    return graft.load_package()


@pytest.fixture(scope="session")
def gpu_ctx(pkg):
    """One backend context shared by the GPU tests (arenas sized for the test shapes)."""
    ctx = pkg.runtime.Context(params_bytes=128 << 20, state_bytes=256 << 20, scratch_bytes=1536 << 20, data_bytes=32 << 20)
    yield ctx
    ctx.destroy()


@pytest.fixture()
def step(gpu_ctx):
    """A fresh step scope: scratch and data arenas are reset before the test body."""
    gpu_ctx.begin_step()
    yield gpu_ctx
    gpu_ctx.end_step()
    gpu_ctx.flush()


def f16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)
