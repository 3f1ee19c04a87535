"""GPU: MiniMax-M3 block-sparse attention entries (block selection, forward, backward) through the C ABI against the
golden vectors of the reference's own CPU references and against the oracle at larger sizes. Selected block indices
are compared exactly; attention outputs and gradients within one F16 rounding plus FP32 reassociation noise."""
import ctypes as C

import numpy as np
import pytest

from conftest import Golden, f16_bits_to_f32
from gpu_util import F16, F32, I32, abi, dev, host
from oracle import m3_sparse

pytestmark = pytest.mark.gpu
byref = C.byref
GOLD = Golden("ref_m3_sparse")


class SparseArgs(C.Structure):
    _fields_ = [("scale", C.c_float), ("block_size", C.c_uint32), ("topk", C.c_uint32), ("init_blocks", C.c_uint32),
                ("local_blocks", C.c_uint32), ("max_seqlen", C.c_uint32)]


def bind(lib):
    tv = C.POINTER(abi.TensorView)
    lib.gd_backend_minimax_m3_index_topk.argtypes = [C.c_void_p, tv, tv, tv, tv, C.POINTER(SparseArgs)]
    lib.gd_backend_minimax_m3_sparse_attention.argtypes = [C.c_void_p] + [tv] * 6 + [C.POINTER(SparseArgs)]
    lib.gd_backend_minimax_m3_sparse_attention_backward.argtypes = [C.c_void_p] + [tv] * 10 + [C.POINTER(SparseArgs)]
    for f in (lib.gd_backend_minimax_m3_index_topk, lib.gd_backend_minimax_m3_sparse_attention, lib.gd_backend_minimax_m3_sparse_attention_backward):
        f.restype = C.c_int


def run_all(ctx, q, k, v, go, iq, ik, cu, block, topk, init_b, local_b, scale, topk_override=None):
    lib = ctx.lib
    bind(lib)
    n, hq, dh = q.shape
    hkv = k.shape[1]
    args = SparseArgs(scale, block, topk, init_b, local_b, int(np.diff(cu).max()))
    dq_, dk_, dv_, dgo, diq, dik = (dev(ctx, a, F16) for a in (q, k, v, go, iq, ik))
    dcu = dev(ctx, np.asarray(cu, dtype=np.int32), I32)
    tk = ctx.scratch_empty(I32, (hkv, n, topk))
    ctx.check(lib.gd_backend_minimax_m3_index_topk(ctx.backend, byref(diq.tv()), byref(dik.tv()), byref(dcu.tv()), byref(tk.tv()), byref(args)), "topk")
    got_tk = tk.read()
    if topk_override is not None:
        tk = dev(ctx, topk_override, I32)
    out = ctx.scratch_empty(F16, (n, hq, dh))
    ctx.check(lib.gd_backend_minimax_m3_sparse_attention(ctx.backend, byref(dq_.tv()), byref(dk_.tv()), byref(dv_.tv()), byref(dcu.tv()), byref(tk.tv()),
                                                         byref(out.tv()), byref(args)), "fwd")
    gq, gk, gv = ctx.scratch_empty(F16, (n, hq, dh)), ctx.scratch_empty(F16, (n, hkv, dh)), ctx.scratch_empty(F16, (n, hkv, dh))
    stats = ctx.scratch_empty(F32, (n, hq, 3))
    ctx.check(lib.gd_backend_minimax_m3_sparse_attention_backward(ctx.backend, byref(dgo.tv()), byref(dq_.tv()), byref(dk_.tv()), byref(dv_.tv()),
                                                                  byref(dcu.tv()), byref(tk.tv()), byref(gq.tv()), byref(gk.tv()), byref(gv.tv()),
                                                                  byref(stats.tv()), byref(args)), "bwd")
    return got_tk, host(out), host(gq), host(gk), host(gv)


@pytest.mark.parametrize("name", GOLD.names())
def test_against_the_reference_tests_cpu_references(step, name):
    c = GOLD[name]
    block, topk, init_b, local_b = (int(x) for x in c["params"])
    q, k, v, go, iq, ik = (f16_bits_to_f32(c[x]) for x in ("q", "k", "v", "go", "iq", "ik"))
    tk, out, dq, dk, dv = run_all(step, q, k, v, go, iq, ik, c["cu"], block, topk, init_b, local_b, float(c["scale"]))
    np.testing.assert_array_equal(tk, c["topk"])
    np.testing.assert_allclose(out, c["out"], atol=2.5e-3, rtol=2e-3)               # the reference test's own bound
    for got, want in ((dq, c["dq"]), (dk, c["dk"]), (dv, c["dv"])):
        np.testing.assert_allclose(got, want, atol=3e-3, rtol=4e-3)


@pytest.mark.parametrize("lens,hq,hkv,dh,block,topk,init_b,local_b", [([300, 97, 512, 1], 4, 2, 64, 16, 8, 1, 2), ([129, 64], 2, 2, 32, 128, 16, 0, 1),
                                                                     ([200], 8, 1, 64, 8, 4, 2, 0)])
def test_against_the_oracle_at_model_sizes(step, lens, hq, hkv, dh, block, topk, init_b, local_b):
    rng = np.random.default_rng(len(lens) * 100 + dh)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    n = int(cu[-1])
    grid = lambda shape: (rng.integers(-8, 9, size=shape).astype(np.float32) / 8.0)      # exact index scores in FP32
    iq, ik = grid((n, hkv, dh)), grid((n, hkv, dh))
    f16 = lambda shape, s: (rng.standard_normal(shape) * s).astype(np.float16).astype(np.float32)
    q, k, v, go = f16((n, hq, dh), 0.7), f16((n, hkv, dh), 0.7), f16((n, hkv, dh), 1.0), f16((n, hq, dh), 1.0)
    scale = 1.0 / np.sqrt(dh)
    want_tk = m3_sparse.index_topk(iq, ik, cu, block, topk, init_b, local_b)
    tk, out, dq, dk, dv = run_all(step, q, k, v, go, iq, ik, cu, block, topk, init_b, local_b, scale)
    np.testing.assert_array_equal(tk, want_tk)
    np.testing.assert_allclose(out, m3_sparse.forward(q, k, v, cu, want_tk, block, scale), atol=2e-3, rtol=4e-3)
    wq, wk, wv = m3_sparse.backward(go, q, k, v, cu, want_tk, block, scale)
    for got, want, what in ((dq, wq, "dq"), (dk, wk, "dk"), (dv, wv, "dv")):
        np.testing.assert_allclose(got, want, atol=2e-3 * max(1.0, float(np.abs(want).max())), rtol=4e-3, err_msg=what)


def test_argument_errors(step):
    ctx = step
    bind(ctx.lib)
    q = dev(ctx, np.zeros((8, 2, 8), dtype=np.float32), F16)
    cu = dev(ctx, np.asarray([0, 8], dtype=np.int32), I32)
    tk = ctx.scratch_empty(I32, (2, 8, 2))
    ok = SparseArgs(1.0, 4, 2, 1, 1, 8)
    f = ctx.lib.gd_backend_minimax_m3_index_topk
    assert f(ctx.backend, byref(q.tv()), byref(q.tv()), byref(cu.tv()), byref(tk.tv()), byref(ok)) == abi.GD_OK
    for field, value in (("topk", 3), ("topk", 0), ("block_size", 0), ("block_size", 129), ("max_seqlen", 0)):
        bad = SparseArgs(1.0, 4, 2, 1, 1, 8)
        setattr(bad, field, value)
        assert f(ctx.backend, byref(q.tv()), byref(q.tv()), byref(cu.tv()), byref(tk.tv()), byref(bad)) == abi.GD_ERR_INVALID_ARGUMENT, field
    f32q = ctx.scratch_empty(F32, (8, 2, 8))
    assert f(ctx.backend, byref(f32q.tv()), byref(f32q.tv()), byref(cu.tv()), byref(tk.tv()), byref(ok)) == abi.GD_ERR_INVALID_ARGUMENT
    assert f(ctx.backend, byref(q.tv()), byref(q.tv()), byref(cu.tv()), byref(tk.tv()), None) == abi.GD_ERR_INVALID_ARGUMENT
