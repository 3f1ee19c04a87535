"""gradients.c B200 backend: a CUDA (sm_100a) implementation of the gradients.c backend ABI for
the gpt_lm training-step and KV-cache decode path, plus a thin host layer that mirrors the
reference's op capsules for tests and benchmarks.

The directory name contains a dot, so it is loaded by path (see __graft_entry__.load_package)
under the module name `gradients_c_b200`.
"""
from . import _build
from .host import abi, runtime, ops, optim, gpt_lm, dp, c_host  # noqa: F401

__all__ = ["_build", "abi", "runtime", "ops", "optim", "gpt_lm", "dp", "c_host"]
