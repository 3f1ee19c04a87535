"""GPU parity of the entries off the gpt_lm path (mul / sub, sigmoid / tanh and their backward forms, the mul
backward fast paths, MSE / Huber, PoWLU, permute), called through the C ABI, against a plain PyTorch FP32 reference
of the same formula (src/ops/{mul,sub,sigmoid,tanh,mse,huber,powlu,permute}/metal_*.metal). Products, differences
and copies are bit-exact after the one rounding to the storage type; transcendental work is within gpu_util.TOL."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import BF16, F16, F32, I32, U8, abi, close, dev, host, rnd_np

pytestmark = pytest.mark.gpu
byref = C.byref


def rng(seed):
    return np.random.default_rng(seed)


def inputs(seed, shape, dtype, scale=1.0):
    return rnd_np((rng(seed).standard_normal(shape) * scale).astype(np.float32), dtype)


@pytest.mark.parametrize("dtype", [F16, BF16, F32])
@pytest.mark.parametrize("shape,bshape", [((300, 64), (300, 64)), ((37, 5, 24), (24,)), ((6, 7), (6, 1)), ((4, 3, 8), (3, 1))])
def test_mul_sub_broadcast(step, dtype, shape, bshape):
    ctx = step
    x, y = inputs(1, shape, dtype), inputs(2, bshape, dtype)
    for name, fn in (("mul", np.multiply), ("sub", np.subtract)):
        out = ctx.scratch_empty(dtype, shape)
        ctx.check(getattr(ctx.lib, "gd_backend_" + name)(ctx.backend, byref(dev(ctx, x, dtype).tv()), byref(dev(ctx, y, dtype).tv()),
                                                         byref(out.tv())), name)
        assert np.array_equal(host(out), rnd_np(fn(x, y).astype(np.float32), dtype)), name
    # the broadcast operand may also come first
    out = ctx.scratch_empty(dtype, shape)
    ctx.check(ctx.lib.gd_backend_sub(ctx.backend, byref(dev(ctx, y, dtype).tv()), byref(dev(ctx, x, dtype).tv()), byref(out.tv())), "sub")
    assert np.array_equal(host(out), rnd_np((y - x).astype(np.float32), dtype))


@pytest.mark.parametrize("dtype", [F16, BF16, F32])
@pytest.mark.parametrize("op", ["sigmoid", "tanh"])
def test_sigmoid_tanh_forward_and_both_backward_forms(step, dtype, op):
    ctx = step
    x = inputs(3, (257, 33), dtype, 3.0)
    x.reshape(-1)[:4] = [0.0, -30.0, 30.0, -0.0]
    g = inputs(4, (257, 33), dtype)
    tx = torch.from_numpy(x)
    y_ref = torch.sigmoid(tx) if op == "sigmoid" else torch.tanh(tx)
    lib = ctx.lib
    dx, dg = dev(ctx, x, dtype), dev(ctx, g, dtype)
    y = ctx.scratch_empty(dtype, x.shape)
    ctx.check(getattr(lib, f"gd_backend_{op}")(ctx.backend, byref(dx.tv()), byref(y.tv())), op)
    close(host(y), y_ref, dtype, what=op)
    grad_ref = torch.from_numpy(g) * (y_ref * (1 - y_ref) if op == "sigmoid" else 1 - y_ref * y_ref)
    gx = ctx.scratch_empty(dtype, x.shape)
    ctx.check(getattr(lib, f"gd_backend_{op}_backward")(ctx.backend, byref(dx.tv()), byref(dg.tv()), byref(gx.tv())), op + "_backward")
    close(host(gx), grad_ref, dtype, what=op + " backward")
    # from the saved (rounded) output: the same formula on the stored y
    ys = torch.from_numpy(host(y))
    want = torch.from_numpy(g) * (ys * (1 - ys) if op == "sigmoid" else 1 - ys * ys)
    gy = ctx.scratch_empty(dtype, x.shape)
    ctx.check(getattr(lib, f"gd_backend_{op}_backward_from_output")(ctx.backend, byref(y.tv()), byref(dg.tv()), byref(gy.tv())), op + "_from_output")
    close(host(gy), want, dtype, what=op + " backward from output")


@pytest.mark.parametrize("dtype", [F16, BF16])
def test_mul_backward_direct_and_reduce_suffix(step, dtype):
    ctx = step
    x, y, g = inputs(5, (40, 96), dtype), inputs(6, (40, 96), dtype), inputs(7, (40, 96), dtype)
    dx, dy, dg = dev(ctx, x, dtype), dev(ctx, y, dtype), dev(ctx, g, dtype)
    gx, gy = ctx.scratch_empty(dtype, x.shape), ctx.scratch_empty(dtype, x.shape)
    ctx.check(ctx.lib.gd_backend_mul_backward_direct(ctx.backend, byref(dx.tv()), byref(dy.tv()), byref(dg.tv()), byref(gx.tv()), byref(gy.tv())), "mbd")
    assert np.array_equal(host(gx), rnd_np(g * y, dtype)) and np.array_equal(host(gy), rnd_np(g * x, dtype))
    for rows, cols in ((40, 96), (700, 5), (3, 1280)):
        a, b = inputs(8, (rows, cols), dtype), inputs(9, (rows, cols), dtype)
        dst = ctx.scratch_empty(dtype, (cols,))
        ctx.check(ctx.lib.gd_backend_mul_reduce_suffix(ctx.backend, byref(dev(ctx, a, dtype).tv()), byref(dev(ctx, b, dtype).tv()), byref(dst.tv())), "mrs")
        close(host(dst), (a.astype(np.float64) * b).sum(axis=0).astype(np.float32), dtype, scale=np.sqrt(rows), what=f"reduce suffix {rows}x{cols}")
    f = ctx.scratch_empty(F32, (4, 4))
    assert ctx.lib.gd_backend_mul_backward_direct(ctx.backend, byref(f.tv()), byref(f.tv()), byref(f.tv()), byref(f.tv()), byref(f.tv())) == abi.GD_ERR_UNSUPPORTED


@pytest.mark.parametrize("dtype", [F16, BF16, F32])
@pytest.mark.parametrize("loss", ["mse", "huber"])
def test_mse_huber_forward_backward(step, dtype, loss):
    ctx = step
    n, chunk, scale, delta = 5000, 1024, 0.25, 0.75
    x, y = inputs(10, (n,), dtype, 1.5), inputs(11, (n,), dtype, 1.5)
    d = torch.from_numpy(x) - torch.from_numpy(y)
    if loss == "mse":
        val, grad = d * d, d
    else:
        val = torch.where(d.abs() <= delta, 0.5 * d * d, delta * (d.abs() - 0.5 * delta))
        grad = d.clamp(-delta, delta)
    chunks = (n + chunk - 1) // chunk
    want = np.array([float(val[c * chunk:(c + 1) * chunk].double().sum()) * scale for c in range(chunks)], dtype=np.float32)
    dx, dy = dev(ctx, x, dtype), dev(ctx, y, dtype)
    out = ctx.scratch_empty(F32, (chunks,))
    extra = (C.c_float(delta),) if loss == "huber" else ()
    ctx.check(getattr(ctx.lib, f"gd_backend_{loss}_forward")(ctx.backend, byref(dx.tv()), byref(dy.tv()), byref(out.tv()), chunk, scale, *extra), loss)
    np.testing.assert_allclose(host(out), want, rtol=2e-5)
    go = dev(ctx, np.array(1.5, dtype=np.float32), F32)
    gx, gy = ctx.scratch_empty(dtype, (n,)), ctx.scratch_empty(dtype, (n,))
    bwd = getattr(ctx.lib, f"gd_backend_{loss}_backward")
    ctx.check(bwd(ctx.backend, byref(dx.tv()), byref(dy.tv()), byref(go.tv()), byref(gx.tv()), byref(gy.tv()), scale, *extra), loss + "_backward")
    want_g = (grad * (1.5 * scale)).numpy()
    close(host(gx), want_g, dtype, what="grad_x")
    assert np.array_equal(host(gy), -host(gx))
    # either gradient alone; none at all is an error
    ctx.fill(gx, 0)
    ctx.check(bwd(ctx.backend, byref(dx.tv()), byref(dy.tv()), byref(go.tv()), byref(gx.tv()), None, scale, *extra), "x only")
    close(host(gx), want_g, dtype, what="grad_x only")
    assert bwd(ctx.backend, byref(dx.tv()), byref(dy.tv()), byref(go.tv()), None, None, scale, *extra) == abi.GD_ERR_INVALID_ARGUMENT
    bad = ctx.scratch_empty(F32, (chunks + 1,))
    fwd = getattr(ctx.lib, f"gd_backend_{loss}_forward")
    assert fwd(ctx.backend, byref(dx.tv()), byref(dy.tv()), byref(bad.tv()), chunk, scale, *extra) == abi.GD_ERR_INVALID_ARGUMENT


def powlu_ref(x1, x2, m):
    """out = x1 * gate(x2, m): gate = z * sigmoid(z) for z <= 0, z ** (m / (sqrt(z) + 1)) * sigmoid(z) for z > 0."""
    z = x2.clone().double().requires_grad_(True)
    zp = z.clamp_min(2.0 ** -24)
    gate = torch.where(z > 0, torch.exp(m / (zp.sqrt() + 1) * zp.log()) * torch.sigmoid(z), z * torch.sigmoid(z))
    return x1.double() * gate, gate, z


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("m", [2.0, 3.0])
def test_powlu_and_split_forward_backward(step, dtype, m):
    ctx = step
    rows, h = 37, 48
    x12 = inputs(12, (rows, 2 * h), dtype, 1.5)
    x12[0, h:h + 3] = [0.0, 1e-4, -4.0]
    x1, x2 = np.ascontiguousarray(x12[:, :h]), np.ascontiguousarray(x12[:, h:])
    g = inputs(13, (rows, h), dtype)
    out_ref, gate, z = powlu_ref(torch.from_numpy(x1), torch.from_numpy(x2), m)
    (dgate,) = torch.autograd.grad(gate.sum(), z)
    tg = torch.from_numpy(g).double()
    want_dx1, want_dx2 = (tg * gate).detach().float(), (tg * torch.from_numpy(x1).double() * dgate).float()
    lib = ctx.lib
    d1, d2, dg, d12 = dev(ctx, x1, dtype), dev(ctx, x2, dtype), dev(ctx, g, dtype), dev(ctx, x12, dtype)
    out = ctx.scratch_empty(dtype, (rows, h))
    ctx.check(lib.gd_backend_powlu_forward(ctx.backend, byref(d1.tv()), byref(d2.tv()), byref(out.tv()), m), "powlu")
    close(host(out), out_ref.detach().float(), dtype, scale=4.0, what="powlu")
    out_s = ctx.scratch_empty(dtype, (rows, h))
    ctx.check(lib.gd_backend_powlu_split_forward(ctx.backend, byref(d12.tv()), byref(out_s.tv()), m), "powlu_split")
    assert np.array_equal(host(out_s), host(out))
    g1, g2 = ctx.scratch_empty(dtype, (rows, h)), ctx.scratch_empty(dtype, (rows, h))
    ctx.check(lib.gd_backend_powlu_backward(ctx.backend, byref(d1.tv()), byref(d2.tv()), byref(dg.tv()), byref(g1.tv()), byref(g2.tv()), m), "powlu_bwd")
    close(host(g1), want_dx1, dtype, scale=4.0, what="dx1")
    close(host(g2), want_dx2, dtype, scale=8.0, what="dx2")
    g12 = ctx.scratch_empty(dtype, (rows, 2 * h))
    ctx.check(lib.gd_backend_powlu_split_backward(ctx.backend, byref(d12.tv()), byref(dg.tv()), byref(g12.tv()), m), "powlu_split_bwd")
    got12 = host(g12)
    assert np.array_equal(got12[:, :h], host(g1)) and np.array_equal(got12[:, h:], host(g2))
    only2 = ctx.scratch_empty(dtype, (rows, h))
    ctx.check(lib.gd_backend_powlu_backward(ctx.backend, byref(d1.tv()), byref(d2.tv()), byref(dg.tv()), None, byref(only2.tv()), m), "dx2 only")
    assert np.array_equal(host(only2), host(g2))


@pytest.mark.parametrize("dtype", [F16, F32, I32, U8, BF16])
@pytest.mark.parametrize("shape,axes", [((5, 7), (1, 0)), ((3, 4, 5), (2, 0, 1)), ((2, 3, 4, 8), (1, 0, 2, 3)), ((6, 2, 3, 5), (3, 1, 0, 2)),
                                        ((4, 9), (0, 1))])
def test_permute(step, dtype, shape, axes):
    ctx = step
    n = int(np.prod(shape))
    if dtype in (I32, U8):
        src = (rng(14).integers(0, 200, size=shape)).astype(np.int32 if dtype == I32 else np.uint8)
    else:
        src = inputs(14, shape, dtype)
    want = np.ascontiguousarray(np.transpose(src, axes))
    rank = len(shape)
    active = rank
    while active > 0 and axes[active - 1] == active - 1:
        active -= 1
    inner = int(np.prod(want.shape[active:])) if active < rank else 1
    args = abi.PermuteArgs(n, inner, rank, active, (C.c_uint32 * 8)(*axes), 0)
    ds = dev(ctx, src, dtype)
    dst = ctx.scratch_empty(dtype, want.shape)
    ctx.check(ctx.lib.gd_backend_permute(ctx.backend, byref(ds.tv()), byref(dst.tv()), byref(args)), "permute")
    got = host(dst) if dtype in (F16, F32, BF16) else dst.read()
    assert np.array_equal(got, want)
    bad = abi.PermuteArgs(n, inner, rank, active, (C.c_uint32 * 8)(*([0] * rank)), 0)
    if rank > 1:
        assert ctx.lib.gd_backend_permute(ctx.backend, byref(ds.tv()), byref(dst.tv()), byref(bad)) == abi.GD_ERR_INVALID_ARGUMENT
