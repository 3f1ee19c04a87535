"""GPU: the allocation-free embedding-gradient entry point against the regular one.

gdb200_embedding_backward_static is for callers that cannot allocate device memory (a runtime
whose arenas own all of it, or a foreign-function caller with raw pointers only): its FP32
accumulation table is a fixed array inside the library. It is called through the C ABI with raw
device pointers, twice in a row (the array keeps the previous call's sums and must be cleared by
each call), and compared with gd_backend_embedding_backward, which gets its scratch from the
caller. The file name makes pytest collect it last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import BF16, F16, F32, I32, TOL, abi, dev, host, pkg, rnd_np, storage_name
from oracle import ops as O

pytestmark = pytest.mark.gpu


def raw(ctx, t):
    return ctx.lib.gdb200_buffer_device_ptr(t.buffer, t.offset)


@pytest.mark.parametrize("dtype", [F16, BF16, F32])
def test_static_scratch_embedding_backward_matches_regular_entry(dtype):
    with pkg.runtime.Context(params_bytes=16 << 20, state_bytes=16 << 20, scratch_bytes=256 << 20, data_bytes=8 << 20) as ctx:
        lib = ctx.lib
        stream = lib.gdb200_stream(ctx.backend)
        vocab, dim = 2048, 512                      # exactly the maximum the static table holds
        assert vocab * dim == lib.gdb200_embedding_backward_static_max_elems()
        ctx.begin_step()
        for call, n_ids in enumerate((3000, 777)):  # second call must not see the first call's sums
            rng = np.random.default_rng(call)
            ids = rng.integers(0, vocab, size=n_ids).astype(np.int32)
            ids[::97] = -1
            g = rnd_np((rng.standard_normal((n_ids, dim)) * (1.0 + call)).astype(np.float32), dtype)
            gt, it = dev(ctx, g, dtype), dev(ctx, ids, I32)
            want_t = ctx.scratch_empty(dtype, (vocab, dim))
            scratch = ctx.scratch_empty(F32, (vocab, dim))
            args = abi.EmbeddingArgs(n_ids, vocab, dim)
            ctx.check(lib.gd_backend_embedding_backward(ctx.backend, C.byref(gt.tv()), C.byref(it.tv()), C.byref(want_t.tv()),
                                                        C.byref(scratch.tv()), C.byref(args)), "embedding_backward")
            got_t = ctx.scratch_empty(dtype, (vocab, dim))
            ctx.fill(got_t, {F16: 0x7E00, BF16: 0x7FC0, F32: 0x7FC00000}[dtype])   # NaN pattern: every element must be overwritten
            st = lib.gdb200_embedding_backward_static(stream, raw(ctx, gt), raw(ctx, it), raw(ctx, got_t), n_ids, vocab, dim, dtype)
            assert st == abi.GD_OK, lib.gdb200_embedding_backward_static_error()
            ctx.flush()
            got, want = host(got_t), host(want_t)
            assert np.isfinite(got).all()
            # both paths accumulate with FP32 atomics (order differs run to run), then round once
            np.testing.assert_allclose(got, want, atol=TOL[dtype]["atol"] * 4, rtol=TOL[dtype]["rtol"])
            # and against the CPU oracle's scatter-add
            oracle = O.embedding_backward(torch.from_numpy(g), torch.from_numpy(ids), vocab, storage_name(dtype)).numpy()
            np.testing.assert_allclose(got, oracle, atol=TOL[dtype]["atol"] * 4, rtol=TOL[dtype]["rtol"])
        # no ids at all: the table is still cleared and written, so the result is all zeros (the static array holds the last call's sums)
        ctx.fill(got_t, {F16: 0x7E00, BF16: 0x7FC0, F32: 0x7FC00000}[dtype])
        st = lib.gdb200_embedding_backward_static(stream, raw(ctx, gt), raw(ctx, it), raw(ctx, got_t), 0, vocab, dim, dtype)
        assert st == abi.GD_OK, lib.gdb200_embedding_backward_static_error()
        ctx.flush()
        assert not host(got_t).any()
        # beyond the maximum: refused with a message, nothing launched
        st = lib.gdb200_embedding_backward_static(stream, raw(ctx, gt), raw(ctx, it), raw(ctx, got_t), 1, vocab + 1, dim, dtype)
        assert st == abi.GD_ERR_INVALID_ARGUMENT
        assert b"exceeds" in lib.gdb200_embedding_backward_static_error()
        st = lib.gdb200_embedding_backward_static(stream, raw(ctx, gt), raw(ctx, it), raw(ctx, got_t), (1 << 64) - 1, 4, 4, dtype)
        assert st == abi.GD_ERR_INVALID_ARGUMENT
        ctx.end_step()
