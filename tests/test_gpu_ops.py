"""GPU parity: every backend entry on the gpt_lm path, called through the C ABI, against the CPU
oracle on the same seeded inputs. Integer / mask / copy work is bit-exact; floating-point work
is within gpu_util.TOL of the FP32 oracle."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from gpu_util import BF16, F16, F32, I32, U8, abi, close, dev, host, pkg, rnd_np, storage_name
from oracle import ops as O

pytestmark = pytest.mark.gpu
ops = pkg.ops
byref = C.byref


def rng(seed):
    return np.random.default_rng(seed)


def t32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


# ------------------------------------------------------------------ memory primitives
def test_fill_scale_accumulate_rand(step):
    ctx = step
    x = rnd_np(rng(0).standard_normal(1000 + 7).astype(np.float32), F16)
    y = rnd_np(rng(1).standard_normal(1000 + 7).astype(np.float32), F16)
    dx, dy = dev(ctx, x, F16), dev(ctx, y, F16)
    ctx.check(ctx.lib.gd_backend_accumulate(ctx.backend, dx.buffer, dx.offset, dy.buffer, dy.offset, dx.count, F16), "acc")
    assert np.array_equal(host(dx), rnd_np(x + y, F16))                      # one rounding per add: exact
    out = ctx.scratch_empty(F16, x.shape)
    ctx.check(ctx.lib.gd_backend_scale(ctx.backend, out.buffer, out.offset, dy.buffer, dy.offset, dy.count, F16, 0.375), "scale")
    assert np.array_equal(host(out), rnd_np(y * np.float32(0.375), F16))
    ctx.check(ctx.lib.gd_backend_scale(ctx.backend, out.buffer, out.offset, dy.buffer, dy.offset, dy.count, F16, 1.0), "scale1")
    assert np.array_equal(host(out), y)
    f = ctx.scratch_empty(F32, (33,))
    ctx.fill(f, 0xFF800000)
    assert np.all(np.isneginf(host(f)))
    r = ctx.scratch_empty(F32, (4096,))
    ctx.check(ctx.lib.gd_backend_rand_uniform(ctx.backend, r.buffer, r.offset, r.count, F32, 1234, -0.5, 1.5), "rand")
    assert np.array_equal(host(r), O.rand_uniform(4096, 1234, -0.5, 1.5))    # integer hash + FP32 affine: exact


@pytest.mark.parametrize("shape,bshape", [((64, 1536), (1536,)), ((5, 7), (7,)), ((3, 4, 6), (3, 4, 6)), ((3, 4, 6), (4, 1))])
def test_add_broadcast(step, shape, bshape):
    ctx = step
    x = rnd_np(rng(2).standard_normal(shape).astype(np.float32), F16)
    y = rnd_np(rng(3).standard_normal(bshape).astype(np.float32), F16)
    out = ctx.scratch_empty(F16, shape)
    ctx.check(ctx.lib.gd_backend_add(ctx.backend, byref(dev(ctx, x, F16).tv()), byref(dev(ctx, y, F16).tv()), byref(out.tv())), "add")
    assert np.array_equal(host(out), rnd_np(x + y, F16))


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype,dim", [(F16, 512), (F16, 12), (F32, 8), (BF16, 64)])
def test_embedding_forward_backward(step, dtype, dim):
    ctx = step
    vocab, n = 97, 301
    table = rnd_np(rng(4).standard_normal((vocab, dim)).astype(np.float32), dtype)
    ids = rng(5).integers(0, vocab, size=n).astype(np.int32)
    ids[[3, 50]] = [-1, vocab]                                               # invalid ids
    tt, it = dev(ctx, table, dtype), dev(ctx, ids, I32)
    tt.requires_grad = True
    out = ops.gd_embedding(ctx, tt, it)
    got = host(out)
    want = O.embedding_forward(t32(table), torch.from_numpy(ids)).numpy()
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(np.nan_to_num(got), np.nan_to_num(want))
    g = rnd_np(rng(6).standard_normal((n, dim)).astype(np.float32), dtype)
    out.grad = dev(ctx, g, dtype)
    ctx.run_backward()
    close(host(tt.grad), O.embedding_backward(t32(g), torch.from_numpy(ids), vocab, storage_name(dtype)), dtype, scale=4)


@pytest.mark.parametrize("dtype,dim,p", [(F16, 512, 0.1), (BF16, 64, 0.25), (F16, 24, 0.0), (F16, 12, 0.1)])
def test_embedding_dropout_and_first_norm_in_one_launch(step, dtype, dim, p):
    """gdb200_embedding_dropout_rms_norm against the three entries it stands for (embedding_forward, dropout_forward,
    rms_norm_forward_stats): x, mask and normed bit for bit, 1 / rms to FP32 rounding; ids outside the table give NaN rows."""
    ctx, lib = step, step.lib
    vocab, n, seed, eps = 97, 301, 0x0123456789ABCDEF, 1e-5
    table = rnd_np(rng(4).standard_normal((vocab, dim)).astype(np.float32), dtype)
    w = rnd_np((rng(5).standard_normal(dim) * 0.25 + 1).astype(np.float32), dtype)
    ids = rng(6).integers(0, vocab, size=n).astype(np.int32)
    ids[[3, 50]] = [-1, vocab]
    tt, it, wt = dev(ctx, table, dtype), dev(ctx, ids, I32), dev(ctx, w, dtype)
    x1, m1, y1, inv1 = ctx.scratch_empty(dtype, (n, dim)), ctx.scratch_empty(U8, (n, dim)), ctx.scratch_empty(dtype, (n, dim)), ctx.scratch_empty(F32, (n,))
    st = lib.gdb200_embedding_dropout_rms_norm(ctx.backend, byref(tt.tv()), byref(it.tv()), byref(wt.tv()), byref(x1.tv()), byref(m1.tv()), byref(y1.tv()),
                                               byref(inv1.tv()), eps, p, seed)
    if dim % 8:
        assert st == abi.GD_ERR_UNSUPPORTED
        return
    ctx.check(st, "embedding + dropout + rms_norm")
    e0, x0, m0, y0, inv0 = (ctx.scratch_empty(dtype, (n, dim)), ctx.scratch_empty(dtype, (n, dim)), ctx.scratch_empty(U8, (n, dim)),
                            ctx.scratch_empty(dtype, (n, dim)), ctx.scratch_empty(F32, (n,)))
    ea = abi.EmbeddingArgs(n, vocab, dim)
    ctx.check(lib.gd_backend_embedding_forward(ctx.backend, byref(tt.tv()), byref(it.tv()), byref(e0.tv()), byref(ea)), "embedding_forward")
    ctx.check(lib.gd_backend_dropout_forward(ctx.backend, byref(e0.tv()), byref(x0.tv()), byref(m0.tv()), p, seed), "dropout_forward")
    args = ops._rms_args(n, dim, eps)
    ctx.check(lib.gd_backend_rms_norm_forward_stats(ctx.backend, byref(x0.tv()), byref(wt.tv()), byref(y0.tv()), byref(inv0.tv()), byref(args)), "rms_norm_forward_stats")
    bits = lambda t: host(t).astype(np.float32).view(np.uint32)
    assert np.array_equal(host(m1), host(m0))
    assert np.array_equal(bits(x1), bits(x0)) and np.array_equal(bits(y1), bits(y0))
    ok = ~np.isnan(host(inv0))
    np.testing.assert_allclose(host(inv1)[ok], host(inv0)[ok], rtol=1e-6)
    assert np.isnan(host(x1)[3]).sum() + np.isnan(host(x1)[50]).sum() >= 1 and not np.isnan(host(x1)[4]).any()
    want = O.embedding_forward(t32(table), torch.from_numpy(ids))
    want_x, _ = O.dropout_forward(want.reshape(-1), p, seed, storage_name(dtype))
    assert np.array_equal(np.nan_to_num(host(x1).reshape(-1)), np.nan_to_num(want_x.numpy()))


# ------------------------------------------------------------------ dropout
@pytest.mark.parametrize("dtype,n,p,seed", [(F16, 4096 * 16, 0.1, 0x1234567890ABCDEF), (F16, 513, 0.2, 2**64 - 5), (F32, 1000, 0.35, 42)])
def test_dropout_family(step, dtype, n, p, seed):
    ctx = step
    x = rnd_np((rng(7).standard_normal(n) * 1.5).astype(np.float32), dtype)
    res = rnd_np(rng(8).standard_normal(n).astype(np.float32), dtype)
    xt = dev(ctx, x, dtype)
    xt.requires_grad = True
    y = ops.gd_dropout(ctx, xt, p, True, seed)
    want_y, want_mask = O.dropout_forward(t32(x), p, seed, storage_name(dtype))
    assert np.array_equal(host(y), want_y.numpy())                            # mask and values bit-exact
    g = rnd_np(rng(9).standard_normal(n).astype(np.float32), dtype)
    y.grad = dev(ctx, g, dtype)
    ctx.run_backward()
    assert np.array_equal(host(xt.grad), O.dropout_backward_mask(want_mask, t32(g), 1.0 / (1.0 - p), storage_name(dtype)).numpy())
    # recompute-from-seed backward
    dx = ctx.scratch_empty(dtype, (n,))
    ctx.check(ctx.lib.gd_backend_dropout_backward(ctx.backend, byref(dev(ctx, g, dtype).tv()), byref(dx.tv()), p, seed), "dropout_backward")
    assert np.array_equal(host(dx), host(xt.grad))
    if dtype == F16:
        rt, x2 = dev(ctx, res, dtype), dev(ctx, x, dtype)
        y2 = ops.gd_dropout_add(ctx, rt, x2, p, True, seed)
        want2, _ = O.dropout_add_forward(t32(res), t32(x), p, seed, "f16")
        assert np.array_equal(host(y2), want2.numpy())


# ------------------------------------------------------------------ rms_norm
@pytest.mark.parametrize("dtype,rows,cols", [(F16, 777, 512), (F16, 33, 24), (BF16, 130, 2048), (F32, 9, 17)])
def test_rms_norm(step, dtype, rows, cols):
    ctx = step
    x = rnd_np((rng(10).standard_normal((rows, cols)) * 0.5).astype(np.float32), dtype)
    w = rnd_np((rng(11).standard_normal(cols) * 0.25 + 1).astype(np.float32), dtype)
    g = rnd_np((rng(12).standard_normal((rows, cols)) * 0.25).astype(np.float32), dtype)
    xt, wt = dev(ctx, x, dtype), dev(ctx, w, dtype)
    xt.requires_grad = wt.requires_grad = True
    y = ops.gd_rms_norm(ctx, xt, wt, 1e-5)
    wy, winv = O.rms_norm_forward(t32(x), t32(w), 1e-5, storage_name(dtype))
    close(host(y), wy, dtype)
    y.grad = dev(ctx, g, dtype)
    ctx.run_backward()
    wdx, wdw = O.rms_norm_backward(t32(x), t32(w), winv, t32(g), storage_name(dtype))
    close(host(xt.grad), wdx, dtype)
    close(host(wt.grad), wdw, dtype, scale=8)
    # non-stats entries
    args = ops._rms_args(rows, cols, 1e-5)
    inv = ctx.scratch_empty(F32, (rows,))
    ctx.check(ctx.lib.gd_backend_rms_norm_inv(ctx.backend, byref(xt.tv()), byref(inv.tv()), byref(args)), "rms_inv")
    np.testing.assert_allclose(host(inv), winv.numpy(), rtol=2e-6)
    dx2 = ctx.scratch_empty(dtype, (rows, cols))
    ctx.check(ctx.lib.gd_backend_rms_norm_backward(ctx.backend, byref(xt.tv()), byref(wt.tv()), byref(dev(ctx, g, dtype).tv()), byref(dx2.tv()), byref(args)), "rms_bwd")
    close(host(dx2), wdx, dtype)


@pytest.mark.parametrize("dtype,rows,cols,accumulate", [(F16, 18432, 512, 0), (F16, 777, 512, 1), (BF16, 130, 256, 0), (F16, 9, 24, 1)])
def test_rms_norm_backward_with_weight_gradient_in_one_pass(step, dtype, rows, cols, accumulate):
    """gdb200_rms_norm_backward_with_weight against the two entries it stands for: grad_x bit for bit (also when it is
    accumulated into an existing gradient), grad_weight to FP32 summation order, both against the oracle."""
    ctx, lib = step, step.lib
    x = rnd_np((rng(20).standard_normal((rows, cols)) * 0.5).astype(np.float32), dtype)
    w = rnd_np((rng(21).standard_normal(cols) * 0.25 + 1).astype(np.float32), dtype)
    g = rnd_np((rng(22).standard_normal((rows, cols)) * 0.25).astype(np.float32), dtype)
    base = rnd_np((rng(23).standard_normal((rows, cols)) * 0.1).astype(np.float32), dtype)
    xt, wt, gt = dev(ctx, x, dtype), dev(ctx, w, dtype), dev(ctx, g, dtype)
    args = ops._rms_args(rows, cols, 1e-5)
    inv = ctx.scratch_empty(F32, (rows,))
    ctx.check(lib.gd_backend_rms_norm_inv(ctx.backend, byref(xt.tv()), byref(inv.tv()), byref(args)), "rms_inv")
    partial = ctx.scratch_empty(F32, (int(args.row_blocks), cols))
    # the two entries (+ accumulate)
    dx0, dw0 = ctx.scratch_empty(dtype, (rows, cols)), ctx.scratch_empty(dtype, (cols,))
    ctx.check(lib.gd_backend_rms_norm_backward_stats(ctx.backend, byref(xt.tv()), byref(wt.tv()), byref(inv.tv()), byref(gt.tv()), byref(dx0.tv()), byref(args)), "bwd")
    ctx.check(lib.gd_backend_rms_norm_weight_backward_stats(ctx.backend, byref(xt.tv()), byref(inv.tv()), byref(gt.tv()), byref(dw0.tv()), byref(partial.tv()), byref(args)), "wbwd")
    want_dx = host(dx0)
    if accumulate:
        acc0 = dev(ctx, base, dtype)
        ctx.check(lib.gd_backend_accumulate(ctx.backend, acc0.buffer, acc0.offset, dx0.buffer, dx0.offset, rows * cols, dtype), "accumulate")
        want_dx = host(acc0)
    # one pass
    dx1 = dev(ctx, base, dtype) if accumulate else ctx.scratch_empty(dtype, (rows, cols))
    dw1 = ctx.scratch_empty(dtype, (cols,))
    st = lib.gdb200_rms_norm_backward_with_weight(ctx.backend, byref(xt.tv()), byref(wt.tv()), byref(inv.tv()), byref(gt.tv()), byref(dx1.tv()),
                                                  accumulate, byref(dw1.tv()), byref(partial.tv()), byref(args))
    if cols > 512 or cols % 8:
        assert st == abi.GD_ERR_UNSUPPORTED
        return
    ctx.check(st, "rms backward + weight gradient")
    bits = np.uint16 if dtype != F32 else np.uint32
    assert np.array_equal(host(dx1).astype(np.float32).view(np.uint32), want_dx.astype(np.float32).view(np.uint32))
    winv = O.rms_norm_forward(t32(x), t32(w), 1e-5, storage_name(dtype))[1]
    wdx, wdw = O.rms_norm_backward(t32(x), t32(w), winv, t32(g), storage_name(dtype))
    if not accumulate:
        close(host(dx1), wdx, dtype)
    close(host(dw1), wdw, dtype, scale=8 * max(1.0, math.sqrt(rows / 777)))
    close(host(dw1), host(dw0), dtype, scale=2 * max(1.0, math.sqrt(rows / 777)))
    # the same launch with the dropout backward of its result as a second output: all three outputs bit for bit
    keep = (rng(24).random((rows, cols)) >= 0.1).astype(np.uint8)
    mt = dev(ctx, keep, U8)
    dx2 = dev(ctx, base, dtype) if accumulate else ctx.scratch_empty(dtype, (rows, cols))
    dw2, dropped2, dropped_want = ctx.scratch_empty(dtype, (cols,)), ctx.scratch_empty(dtype, (rows, cols)), ctx.scratch_empty(dtype, (rows, cols))
    colsum2, partial2 = ctx.scratch_empty(dtype, (cols,)), ctx.scratch_empty(F32, (2 * int(args.row_blocks), cols))
    scale = float(np.float32(1.0) / np.float32(0.9))
    ctx.check(lib.gdb200_rms_norm_backward_with_weight_dropout(ctx.backend, byref(xt.tv()), byref(wt.tv()), byref(inv.tv()), byref(gt.tv()), byref(dx2.tv()),
                                                               accumulate, byref(dw2.tv()), byref(partial2.tv()), byref(args), byref(mt.tv()),
                                                               byref(dropped2.tv()), scale, byref(colsum2.tv())), "rms backward + weight gradient + dropout backward")
    ctx.check(lib.gd_backend_dropout_backward_mask(ctx.backend, byref(mt.tv()), byref(dx1.tv()), byref(dropped_want.tv()), scale), "dropout backward")
    as_bits = lambda t: host(t).astype(np.float32).view(np.uint32)
    assert np.array_equal(as_bits(dx2), as_bits(dx1)) and np.array_equal(as_bits(dw2), as_bits(dw1))
    assert np.array_equal(as_bits(dropped2), as_bits(dropped_want))
    assert np.array_equal(host(dropped2)[keep == 0], np.zeros(int((keep == 0).sum()), dtype=np.float32))
    # its column sums: reduce_rows of the same tensor up to FP32 summation order, and the exact sum within the storage rounding
    colsum_want = ctx.scratch_empty(dtype, (cols,))
    gm, cv = dropped_want.mv(rows, cols), colsum_want.vv(0, cols)
    ctx.check(lib.gd_backend_reduce_rows(ctx.backend, byref(gm), byref(cv)), "reduce_rows")
    close(host(colsum2), host(colsum_want), dtype, scale=2 * max(1.0, math.sqrt(rows / 777)))
    close(host(colsum2), host(dropped_want).astype(np.float64).sum(axis=0), dtype, scale=2 * max(1.0, math.sqrt(rows / 777)))
    # without the column sums the same entry takes a null pointer
    ctx.check(lib.gdb200_rms_norm_backward_with_weight_dropout(ctx.backend, byref(xt.tv()), byref(wt.tv()), byref(inv.tv()), byref(gt.tv()),
                                                               byref((dev(ctx, base, dtype) if accumulate else ctx.scratch_empty(dtype, (rows, cols))).tv()),
                                                               accumulate, byref(dw2.tv()), byref(partial.tv()), byref(args), byref(mt.tv()),
                                                               byref(dropped2.tv()), scale, None), "without column sums")
    assert np.array_equal(as_bits(dropped2), as_bits(dropped_want))


# ------------------------------------------------------------------ GEMM family
GEMM_SHAPES = [(5, 3, 7), (64, 128, 96), (300, 512, 1536), (257, 520, 130),
               # decode-sized M: the K-split mma.sync kernel
               (64, 512, 1536), (33, 1536, 512), (1, 64, 16)]


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("m,k,n", GEMM_SHAPES)
def test_matmul_family(step, dtype, m, k, n):
    ctx, lib = step, step.lib
    sd = storage_name(dtype)
    a = rnd_np((rng(13).standard_normal((m, k)) * 0.5).astype(np.float32), dtype)
    b = rnd_np((rng(14).standard_normal((k, n)) * 0.5).astype(np.float32), dtype)
    bias = rnd_np(rng(15).standard_normal(n).astype(np.float32), dtype)
    want = t32(a) @ t32(b)
    sc = np.sqrt(k) / 4
    at, bt, btt, att = dev(ctx, a, dtype), dev(ctx, b, dtype), dev(ctx, b.T.copy(), dtype), dev(ctx, a.T.copy(), dtype)
    y = ctx.scratch_empty(dtype, (m, n))
    for name, fn, xv, wv in (("matmul", lib.gd_backend_matmul, at.mv(m, k), bt.mv(k, n)),
                             ("matmul_nt", lib.gd_backend_matmul_nt, at.mv(m, k), btt.mv(n, k)),
                             ("matmul_tn", lib.gd_backend_matmul_tn, att.mv(k, m), bt.mv(k, n))):
        ctx.fill(y, 0)
        yv = y.mv(m, n)
        ctx.check(fn(ctx.backend, byref(xv), byref(wv), byref(yv)), name)
        close(host(y), O.rnd(want, sd), dtype, scale=sc, what=name)
    bv, yv, xv, wv = dev(ctx, bias, dtype).vv(), y.mv(m, n), at.mv(m, k), bt.mv(k, n)
    ctx.check(lib.gd_backend_linear(ctx.backend, byref(xv), byref(wv), byref(bv), byref(yv)), "linear")
    close(host(y), O.linear_forward(t32(a), t32(b), t32(bias), sd), dtype, scale=sc, what="linear")
    red = ctx.scratch_empty(dtype, (k,))
    rv, xv = red.vv(), at.mv(m, k)
    ctx.check(lib.gd_backend_reduce_rows(ctx.backend, byref(xv), byref(rv)), "reduce_rows")
    close(host(red), O.rnd(t32(a).sum(dim=0), sd), dtype, scale=np.sqrt(m) / 2, what="reduce_rows")


def test_matmul_row_strided_views(step):
    """Weight chunks are passed as row-sliced views and outputs may be strided (LM-CE chunking)."""
    ctx, lib = step, step.lib
    m, k, n, n_total = 40, 64, 24, 80
    a = rnd_np(rng(16).standard_normal((m, k)).astype(np.float32), F16)
    w = rnd_np(rng(17).standard_normal((n_total, k)).astype(np.float32), F16)
    at, wt = dev(ctx, a, F16), dev(ctx, w, F16)
    y = ctx.zeros(ctx.scratch, F16, (m, n_total))
    xv, wv = at.mv(m, k), wt.mv(n, k, row_offset=32)
    yv = y.mv(m, n, row_bytes=n_total * 2)
    yv.offset += 32 * 2
    ctx.check(lib.gd_backend_matmul_nt(ctx.backend, byref(xv), byref(wv), byref(yv)), "matmul_nt strided")
    got = host(y)
    close(got[:, 32:32 + n], O.rnd(t32(a) @ t32(w[32:32 + n]).t()), F16, scale=2)
    assert np.all(got[:, :32] == 0) and np.all(got[:, 32 + n:] == 0)


def test_linear_capsules_autograd(step):
    ctx = step
    m, k, n = 96, 64, 48
    x = rnd_np(rng(18).standard_normal((m, k)).astype(np.float32), F16)
    wt_ = rnd_np((rng(19).standard_normal((n, k)) * 0.1).astype(np.float32), F16)
    w_ = rnd_np((rng(20).standard_normal((k, n)) * 0.1).astype(np.float32), F16)
    b = rnd_np(rng(21).standard_normal(n).astype(np.float32), F16)
    g = rnd_np(rng(22).standard_normal((m, n)).astype(np.float32), F16)
    for transposed in (True, False):
        xt, wt, bt = dev(ctx, x, F16), dev(ctx, wt_ if transposed else w_, F16), dev(ctx, b, F16)
        xt.requires_grad = wt.requires_grad = bt.requires_grad = True
        if transposed:
            y = ops.gd_linear_transposed_weight(ctx, xt, wt, bt)
            wy = O.linear_transposed_weight_forward(t32(x), t32(wt_), t32(b))
            wdx, wdw, wdb = O.linear_transposed_weight_backward(t32(x), t32(wt_), t32(g))
        else:
            y = ops.gd_linear(ctx, xt, wt, bt)
            wy = O.linear_forward(t32(x), t32(w_), t32(b))
            wdx, wdw, wdb = O.linear_backward(t32(x), t32(w_), t32(g))
        close(host(y), wy, F16, scale=2)
        y.grad = dev(ctx, g, F16)
        ctx.run_backward()
        close(host(xt.grad), wdx, F16, scale=2)
        close(host(wt.grad), wdw, F16, scale=8)
        close(host(bt.grad), wdb, F16, scale=8)


# ------------------------------------------------------------------ swiglu / rope
@pytest.mark.parametrize("dtype,rows,h", [(F16, 100, 1536), (F16, 7, 5), (BF16, 64, 256)])
def test_swiglu_split(step, dtype, rows, h):
    ctx = step
    x12 = rnd_np((rng(23).standard_normal((rows, 2 * h)) * 2).astype(np.float32), dtype)
    g = rnd_np(rng(24).standard_normal((rows, h)).astype(np.float32), dtype)
    xt = dev(ctx, x12, dtype)
    xt.requires_grad = True
    y = ops.gd_swiglu_split(ctx, xt)
    close(host(y), O.swiglu_split_forward(t32(x12), storage_name(dtype)), dtype, scale=2)
    y.grad = dev(ctx, g, dtype)
    ctx.run_backward()
    close(host(xt.grad), O.swiglu_split_backward(t32(x12), t32(g), storage_name(dtype)), dtype, scale=4)


@pytest.mark.parametrize("dtype,n,heads,dh,theta,inter", [(F16, 300, 8, 64, 10000.0, False), (F16, 17, 2, 8, 500.0, True),
                                                          (BF16, 50, 16, 128, 10000.0, False), (F16, 600, 4, 64, 10000.0, False)])
def test_qkv_split_rope(step, dtype, n, heads, dh, theta, inter):
    ctx = step
    qkv = rnd_np(rng(25).standard_normal((n, 3 * heads * dh)).astype(np.float32), dtype)
    pos = (np.arange(n) % 530).astype(np.int32)                               # crosses the 512-entry table
    qt, pt = dev(ctx, qkv, dtype), dev(ctx, pos, I32)
    qt.requires_grad = True
    q, k, v = ops.gd_qkv_split_rope(ctx, qt, pt, heads, dh, theta, inter)
    wq, wk, wv = O.qkv_split_rope_forward(t32(qkv), torch.from_numpy(pos), heads, dh, theta, inter, storage_name(dtype))
    close(host(q), wq, dtype, scale=2)
    close(host(k), wk, dtype, scale=2)
    assert np.array_equal(host(v), wv.numpy())                                # V is a bit copy
    gq, gk, gv = (rnd_np(rng(26 + i).standard_normal((n, heads, dh)).astype(np.float32), dtype) for i in range(3))
    q.grad, k.grad, v.grad = dev(ctx, gq, dtype), dev(ctx, gk, dtype), dev(ctx, gv, dtype)
    ctx.run_backward()
    close(host(qt.grad), O.qkv_split_rope_backward(t32(gq), t32(gk), t32(gv), torch.from_numpy(pos), theta, inter, storage_name(dtype)), dtype, scale=2)


# ------------------------------------------------------------------ attention
def make_cu(lengths):
    return np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)


ATTN_CASES = [
    # dtype, lengths, hq, hkv, dh, window, prefix
    (F16, [5, 1, 130, 64, 200], 8, 8, 64, 0, 0),
    (F16, [5, 1, 130, 64, 200], 8, 8, 64, 32, 0),
    (F16, [37, 300], 4, 2, 64, 256, 0),
    (F16, [2, 3], 2, 1, 4, 0, 0),
    (F16, [64, 96], 2, 1, 64, 8, 4),
    (BF16, [100, 129], 4, 4, 128, 0, 0),
    (F32, [9, 14], 2, 2, 16, 3, 0),
]


@pytest.mark.parametrize("dtype,lengths,hq,hkv,dh,window,prefix", ATTN_CASES)
def test_sdpa_varlen_forward_backward(step, dtype, lengths, hq, hkv, dh, window, prefix):
    ctx = step
    sd = storage_name(dtype)
    cu = make_cu(lengths)
    n = int(cu[-1])
    q = rnd_np(rng(30).standard_normal((n, hq, dh)).astype(np.float32), dtype)
    k = rnd_np(rng(31).standard_normal((n, hkv, dh)).astype(np.float32), dtype)
    v = rnd_np(rng(32).standard_normal((n, hkv, dh)).astype(np.float32), dtype)
    go = rnd_np(rng(33).standard_normal((n, hq, dh)).astype(np.float32), dtype)
    qt, kt, vt, cut = dev(ctx, q, dtype), dev(ctx, k, dtype), dev(ctx, v, dtype), dev(ctx, cu, I32)
    qt.requires_grad = kt.requires_grad = vt.requires_grad = True
    out = ops.gd_sdpa_varlen(ctx, qt, kt, vt, cut, causal=True, sliding_window=window, prefix_len=prefix, max_seqlen=max(lengths))
    want, _ = O.sdpa_varlen_forward(t32(q), t32(k), t32(v), cu, 0.0, True, window, prefix, sd)
    close(host(out), want, dtype, scale=2, what="forward")
    out.grad = dev(ctx, go, dtype)
    ctx.run_backward()
    wdq, wdk, wdv = O.sdpa_varlen_backward(t32(go), t32(q), t32(k), t32(v), cu, 0.0, True, window, prefix, sd)
    close(host(qt.grad), wdq, dtype, scale=4, what="dq")
    close(host(kt.grad), wdk, dtype, scale=6, what="dk")
    close(host(vt.grad), wdv, dtype, scale=6, what="dv")


@pytest.mark.parametrize("dtype,b,tq,tmax,hq,hkv,dh,window", [(F16, 5, 1, 512, 8, 8, 64, 256), (F16, 3, 2, 40, 4, 2, 64, 0),
                                                              (BF16, 2, 1, 300, 16, 16, 128, 0), (F16, 2, 3, 11, 2, 1, 8, 4)])
def test_kv_append_and_decode(step, dtype, b, tq, tmax, hq, hkv, dh, window):
    ctx = step
    sd = storage_name(dtype)
    kc = rnd_np(rng(40).standard_normal((b, tmax, hkv, dh)).astype(np.float32), dtype)
    vc = rnd_np(rng(41).standard_normal((b, tmax, hkv, dh)).astype(np.float32), dtype)
    kn = rnd_np(rng(42).standard_normal((b, tq, hkv, dh)).astype(np.float32), dtype)
    vn = rnd_np(rng(43).standard_normal((b, tq, hkv, dh)).astype(np.float32), dtype)
    q = rnd_np(rng(44).standard_normal((b, tq, hq, dh)).astype(np.float32), dtype)
    pos = rng(45).integers(0, tmax - tq + 1, size=b).astype(np.int32)
    pos[-1] = tmax - tq                                                       # last slot that still fits
    kct, vct, post = dev(ctx, kc, dtype), dev(ctx, vc, dtype), dev(ctx, pos, I32)
    ops.gd_kv_cache_append_positions(ctx, kct, vct, post, dev(ctx, kn, dtype), dev(ctx, vn, dtype))
    wk, wv = t32(kc).clone(), t32(vc).clone()
    O.kv_cache_append(wk, wv, t32(kn), t32(vn), pos)
    assert np.array_equal(host(kct), wk.numpy()) and np.array_equal(host(vct), wv.numpy())   # appended rows bit-exact
    out = ops.gd_sdpa_decode_positions(ctx, dev(ctx, q, dtype), kct, vct, post, sliding_window=window)
    close(host(out), O.sdpa_decode(t32(q), wk, wv, pos, 0.0, window, 0, sd), dtype, scale=2)


def test_kv_append_packed_and_overflow_rows_dropped(step):
    ctx = step
    b, tmax, h, dh = 3, 16, 2, 8
    lengths = [4, 9, 5]
    cu = make_cu(lengths)
    pos = np.array([0, 8, 3], dtype=np.int32)                                 # sequence 1 would cross the capacity: dropped
    kc = np.zeros((b, tmax, h, dh), dtype=np.float32)
    kn = rnd_np(rng(46).standard_normal((int(cu[-1]), h, dh)).astype(np.float32), F16)
    vn = rnd_np(rng(47).standard_normal((int(cu[-1]), h, dh)).astype(np.float32), F16)
    kct, vct = dev(ctx, kc, F16), dev(ctx, kc, F16)
    ops.gd_kv_cache_append_packed(ctx, kct, vct, dev(ctx, pos, I32), dev(ctx, cu, I32), dev(ctx, kn, F16), dev(ctx, vn, F16))
    wk, wv = t32(kc).clone(), t32(kc).clone()
    O.kv_cache_append(wk, wv, t32(kn), t32(vn), pos, cu)
    assert np.array_equal(host(kct), wk.numpy()) and np.array_equal(host(vct), wv.numpy())
    assert np.all(host(kct)[1] == 0)


# ------------------------------------------------------------------ LM cross entropy
@pytest.mark.parametrize("rows,dim,vocab,cap,chunk_env", [(200, 64, 2048, 30.0, None), (37, 32, 300, 0.0, None), (64, 32, 1000, 0.75, "256")])
def test_lm_cross_entropy(step, monkeypatch, rows, dim, vocab, cap, chunk_env):
    ctx = step
    if chunk_env:
        monkeypatch.setenv("GD_LM_CE_CHUNK_SIZE", chunk_env)
    h = rnd_np(rng(50).standard_normal((rows, dim)).astype(np.float32), F16)
    w = rnd_np((rng(51).standard_normal((vocab, dim)) * 0.3).astype(np.float32), F16)
    b = rnd_np((rng(52).standard_normal(vocab) * 0.1).astype(np.float32), F16)
    tg = rng(53).integers(0, vocab, size=rows).astype(np.int32)
    tg[::7] = -1
    tg[5] = 3                                                                 # equals ignore_index below
    ht, wt, bt, tt = dev(ctx, h, F16), dev(ctx, w, F16), dev(ctx, b, F16), dev(ctx, tg, I32)
    ht.requires_grad = wt.requires_grad = bt.requires_grad = True
    loss = ops.gd_lm_cross_entropy_softcapped_bias_ignore(ctx, ht, wt, bt, tt, cap, 3)
    saved = O.lm_cross_entropy_forward(t32(h), t32(w), t32(b), torch.from_numpy(tg), cap, 3)
    got = float(loss.read()[()])
    assert abs(got - float(saved["loss"])) <= 2e-3 * max(1.0, abs(float(saved["loss"])))
    seed = ctx.scratch_empty(F32, ())
    seed.write(np.array(64.0, dtype=np.float32))
    loss.grad = seed
    ctx.run_backward()
    dh, dw, db = O.lm_cross_entropy_backward(t32(h), t32(w), t32(b), torch.from_numpy(tg), saved, 64.0, cap)
    close(host(ht.grad), dh, F16, scale=4)
    close(host(wt.grad), dw, F16, scale=8)
    close(host(bt.grad), db, F16, scale=8)


@pytest.mark.parametrize("rows,vocab,cap,dtype", [(18432, 2048, 30.0, F16), (203, 2048, 30.0, F16), (37, 304, 0.0, F16), (64, 1000, 0.75, BF16), (21, 8192, 30.0, F16),
                                                  (50, 4096, 2.0, BF16), (16, 300, 30.0, F16), (9, 8200, 30.0, F16)])
def test_lm_cross_entropy_fused_rows(step, rows, vocab, cap, dtype):
    """gdb200_lm_cross_entropy_fused_rows (row losses and the logits gradient from one pass) against the oracle and against
    online update + finalize + backward chunk on the same logits; rows with an ignored or out-of-range target included."""
    ctx, lib = step, step.lib
    name = storage_name(dtype)
    lg = rnd_np((rng(54).standard_normal((rows, vocab)) * 3.0).astype(np.float32), dtype)
    b = rnd_np((rng(55).standard_normal(vocab) * 0.1).astype(np.float32), dtype)
    tg = rng(56).integers(0, vocab, size=rows).astype(np.int32)
    tg[::7] = -1
    tg[5] = 3                                                                 # equals ignore_index below
    tg[8] = vocab + 2                                                         # past the classes: NaN loss, zero gradient
    tg[2], tg[3] = 0, vocab - 1
    valid = float(np.count_nonzero((tg >= 0) & (tg != 3)))
    saved = O.lm_cross_entropy_from_logits(t32(lg), t32(b), torch.from_numpy(tg), cap, 3, name)
    want_g = O.lm_cross_entropy_dlogits(torch.from_numpy(tg), saved, 64.0, cap, name).numpy()
    assert abs(float(saved["inv_valid"]) * valid - 1.0) < 1e-6
    bt, tt = dev(ctx, b, dtype), dev(ctx, tg, I32)
    seed, counts = ctx.scratch_empty(F32, ()), ctx.scratch_empty(F32, (2,))
    seed.write(np.array(64.0, dtype=np.float32))
    counts.write(np.array([valid, valid], dtype=np.float32))
    # the three entries
    l0, rl0, rm0, rs0, rv0 = dev(ctx, lg, dtype), ctx.zeros(ctx.scratch, F32, (rows,)), ctx.scratch_empty(F32, (rows,)), ctx.zeros(ctx.scratch, F32, (rows,)), ctx.zeros(ctx.scratch, F32, (rows,))
    ctx.fill(rm0, 0xFF800000)
    inv0, loss0 = ctx.scratch_empty(F32, ()), ctx.scratch_empty(F32, ())
    ctx.check(lib.gd_backend_lm_cross_entropy_online_update(ctx.backend, byref(l0.tv()), byref(bt.tv()), byref(tt.tv()), byref(rl0.tv()), byref(rm0.tv()), byref(rs0.tv()), 0, vocab, cap), "update")
    ctx.check(lib.gd_backend_lm_cross_entropy_finalize(ctx.backend, byref(tt.tv()), byref(rl0.tv()), byref(rm0.tv()), byref(rs0.tv()), byref(rv0.tv()), vocab, 3), "finalize")
    ctx.check(lib.gd_backend_lm_cross_entropy_reduce_normalize(ctx.backend, byref(rl0.tv()), byref(rv0.tv()), byref(loss0.tv()), byref(inv0.tv())), "normalize")
    ctx.check(lib.gd_backend_lm_cross_entropy_backward_chunk(ctx.backend, byref(l0.tv()), byref(bt.tv()), byref(tt.tv()), byref(rm0.tv()), byref(rs0.tv()), byref(seed.tv()), byref(inv0.tv()),
                                                             byref(l0.tv()), 0, vocab, 1.0, cap, 3), "backward chunk")
    # one pass
    l1, rl1 = dev(ctx, lg, dtype), ctx.scratch_empty(F32, (rows,))
    st = lib.gdb200_lm_cross_entropy_fused_rows(ctx.backend, byref(l1.tv()), byref(bt.tv()), byref(tt.tv()), byref(seed.tv()), byref(counts.tv()), byref(rl1.tv()), 1.0, cap, 3)
    if vocab % 8 or vocab > 8192:
        assert st == abi.GD_ERR_UNSUPPORTED
        assert np.array_equal(host(l1), lg)                                   # declined: logits untouched
        return
    ctx.check(st, "fused rows")
    got_rl, want_rl = host(rl1), saved["row_loss"].numpy()
    assert np.array_equal(np.isnan(got_rl), np.isnan(want_rl)) and np.isnan(got_rl[8])
    ok = ~np.isnan(want_rl)
    np.testing.assert_allclose(got_rl[ok], want_rl[ok], rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(got_rl[ok], host(rl0)[ok], rtol=2e-6, atol=2e-6)
    assert np.all(got_rl[(tg < 0) | (tg == 3)] == 0.0)
    close(host(l1), want_g, dtype)
    # against the three entries: the same numbers up to the last storage bit of a few elements
    g0, g1 = host(l0).astype(np.float32), host(l1).astype(np.float32)
    ulp = 2.0 ** (-10 if dtype == F16 else -7)
    assert np.all(np.abs(g1 - g0) <= ulp * np.maximum(np.abs(g0), 2.0 ** -14) + 1e-12)
    # (a cap far below the logits saturates most classes: their slope 1 - tanh^2 is a difference of nearly equal numbers, which
    # the one-pass kernel forms from tanh and the reference's arithmetic from soft / cap, so more last bits differ there)
    assert np.mean(g1 != g0) < (1e-2 if cap == 0.0 or cap >= 2.0 else 0.1)
    assert not g1[(tg < 0) | (tg == 3) | (tg >= vocab)].any()


# ------------------------------------------------------------------ optimizer
def test_adamw_amp_clip_steps(step):
    """Three optimizer steps incl. an overflow step: parameters, masters and the scaler state follow the oracle."""
    ctx = step
    optim = pkg.optim
    shapes = [(300, 40), (40,), (1025,)]
    p0 = [rnd_np(rng(60 + i).standard_normal(s).astype(np.float32), F16) for i, s in enumerate(shapes)]
    params = []
    for a in p0:
        tns = dev(ctx, a, F16, ctx.params)
        tns.requires_grad = True
        params.append(tns)
    cfg = optim.AdamwConfig(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    opt = optim.AdamW(ctx, params, cfg, [0.1, 0.0, 0.1])
    scaler = optim.AmpScaler(ctx, optim.AmpConfig(init_scale=1024.0, growth_interval=2))
    master = [t32(a).clone() for a in p0]
    m = [torch.zeros_like(x) for x in master]
    v = [torch.zeros_like(x) for x in master]
    st = [{"beta1_power": np.float32(1), "beta2_power": np.float32(1)} for _ in master]
    amp = {"scale": np.float32(1024), "inv_scale": np.float32(1 / 1024), "growth_tracker": 0, "found_inf": 0, "last_found_inf": 0}
    acfg = dict(growth_factor=2.0, backoff_factor=0.5, min_scale=1.0, max_scale=2147483648.0, growth_interval=2)
    for it in range(4):
        grads = [rnd_np((rng(70 + it * 3 + i).standard_normal(s) * 1024 * 0.5).astype(np.float32), F16) for i, s in enumerate(shapes)]
        if it == 1:
            grads[2][7] = np.inf                                              # overflow: update skipped, scale backs off
        for prm, g in zip(params, grads):
            prm.grad = dev(ctx, g, F16)
        opt.step_amp_clip_lr(scaler, 1e-2, 1.0)
        O.amp_begin_step(amp, acfg)
        gscale, norm, found = O.grad_clip_scale([t32(g) for g in grads], float(amp["inv_scale"]), 1.0)
        amp["found_inf"] = int(found)
        if not found:
            for i in range(3):
                master[i], m[i], v[i] = O.adamw_step(master[i], t32(grads[i]), m[i], v[i], st[i], 1e-2, 0.9, 0.95, 1e-8,
                                                     [0.1, 0.0, 0.1][i], gscale)
        O.amp_finish_step(amp, acfg)
        s = scaler.sync()
        assert s["scale"] == float(amp["scale"]) and s["last_found_inf"] == amp["last_found_inf"] and s["growth_tracker"] == amp["growth_tracker"]
        if not found:
            assert abs(opt.last_grad_norm() - norm) <= 1e-4 * norm
        for i in range(3):
            np.testing.assert_allclose(opt.slots[i].master.read(), master[i].numpy(), rtol=2e-6, atol=1e-7)
            np.testing.assert_allclose(host(params[i]), O.rnd(master[i]).numpy(), rtol=1e-3, atol=1e-6)
    assert opt.step_count() == 3


def test_adamw_golden_bit_exact(step):
    """First AdamW step and the clip step of the reference's optimizer test, compared on F16 bits."""
    from conftest import Golden
    ctx, optim = step, pkg.optim
    g = Golden("ref_ctest_optim")
    c = g["adamw_first_step"]
    p = dev(ctx, c["p0"], F16, ctx.params)
    p.requires_grad = True
    opt = optim.AdamW(ctx, [p], optim.AdamwConfig(float(c["lr"]), float(c["beta1"]), float(c["beta2"]), float(c["eps"]), float(c["wd"])))
    scaler = optim.AmpScaler(ctx, optim.AmpConfig(init_scale=1.0))
    p.grad = dev(ctx, c["g0"], F32)
    opt.step_amp_clip_lr(scaler, float(c["lr"]), 1.0e9)
    assert np.array_equal(p.read().view(np.uint16), c["want_f16"])
    c = g["adamw_clip_step"]
    p = dev(ctx, c["p0"], F16, ctx.params)
    p.requires_grad = True
    opt = optim.AdamW(ctx, [p], optim.AdamwConfig(float(c["lr"]), 0.0, 0.0, 1.0, 0.0))
    p.grad = dev(ctx, c["g0"], F16)
    opt.step_amp_clip_lr(scaler, float(c["lr"]), float(c["max_norm"]))
    assert np.array_equal(p.read().view(np.uint16), c["want_f16"])
    assert abs(opt.last_grad_norm() - 5.0) < 1e-6


# ------------------------------------------------------------------ tcgen05 GEMM (required, no fallback)
TC_SHAPES = [
    # m, k, n : forward / dX shapes of the model and ragged edges
    (1024, 512, 1536), (1024, 512, 512), (1000, 512, 3072), (2048, 1536, 512), (640, 512, 2048),
    (300, 512, 1536), (128, 64, 64), (264, 200, 136), (4096, 512, 1536),
    # enough 256 x 256 tiles that resident CTA pairs take three units each (both accumulator buffers reused), ragged everywhere
    (8192, 512, 1536), (5000, 328, 776),
]


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("m,k,n", TC_SHAPES)
def test_tcgen05_gemm_all_layouts(step, dtype, m, k, n):
    ctx, lib = step, step.lib
    sd = storage_name(dtype)
    a = rnd_np((rng(80).standard_normal((m, k)) * 0.5).astype(np.float32), dtype)
    b = rnd_np((rng(81).standard_normal((k, n)) * 0.5).astype(np.float32), dtype)
    bias = rnd_np(rng(82).standard_normal(n).astype(np.float32), dtype)
    want = t32(a) @ t32(b)
    sc = np.sqrt(k) / 4
    at, bt, btt, att = dev(ctx, a, dtype), dev(ctx, b, dtype), dev(ctx, b.T.copy(), dtype), dev(ctx, a.T.copy(), dtype)
    y = ctx.scratch_empty(dtype, (m, n))
    old = lib.gdb200_set_gemm_mode(ctx.backend, 2)
    try:
        cases = [("matmul", lib.gd_backend_matmul, at.mv(m, k), bt.mv(k, n)), ("matmul_nt", lib.gd_backend_matmul_nt, at.mv(m, k), btt.mv(n, k))]
        if (m * 2) % 16 == 0:
            cases.append(("matmul_tn", lib.gd_backend_matmul_tn, att.mv(k, m), bt.mv(k, n)))
        for name, fn, xv, wv in cases:
            ctx.fill(y, 0)
            yv = y.mv(m, n)
            ctx.check(fn(ctx.backend, byref(xv), byref(wv), byref(yv)), name)
            close(host(y), O.rnd(want, sd), dtype, scale=sc, what=name)
        bv, yv, xv, wv = dev(ctx, bias, dtype).vv(), y.mv(m, n), at.mv(m, k), bt.mv(k, n)
        ctx.check(lib.gd_backend_linear(ctx.backend, byref(xv), byref(wv), byref(bv), byref(yv)), "linear")
        close(host(y), O.linear_forward(t32(a), t32(b), t32(bias), sd), dtype, scale=sc, what="linear")
        ctx.flush()
    finally:
        lib.gdb200_set_gemm_mode(ctx.backend, old)


@pytest.mark.parametrize("m,k,n", [(1536, 8192, 512), (512, 18432, 512), (3072, 4096, 512), (512, 9000, 1536)])
def test_tcgen05_gemm_split_k_weight_gradient(step, m, k, n):
    """dW = dY^T X: the contraction runs over the tokens, the output is small -> split-K path."""
    ctx, lib = step, step.lib
    dy = rnd_np((rng(83).standard_normal((k, m)) * 0.25).astype(np.float32), F16)   # stored [tokens, m]
    x = rnd_np((rng(84).standard_normal((k, n)) * 0.25).astype(np.float32), F16)    # stored [tokens, n]
    want = O.rnd(t32(dy).t() @ t32(x))
    dyt, xt = dev(ctx, dy, F16), dev(ctx, x, F16)
    y = ctx.scratch_empty(F16, (m, n))
    old = lib.gdb200_set_gemm_mode(ctx.backend, 2)
    try:
        xv, wv, yv = dyt.mv(k, m), xt.mv(k, n), y.mv(m, n)
        ctx.check(lib.gd_backend_matmul_tn(ctx.backend, byref(xv), byref(wv), byref(yv)), "matmul_tn split-k")
        close(host(y), want, F16, scale=np.sqrt(k) / 16, what="matmul_tn split-k")
        ctx.flush()
    finally:
        lib.gdb200_set_gemm_mode(ctx.backend, old)


@pytest.mark.parametrize("m,k,n", [(1536, 8192, 512), (512, 16384, 512), (3072, 4096, 512), (2048, 4096, 512), (300, 1000, 136), (64, 256, 64)])
def test_matmul_tn_colsum_equals_matmul_tn_plus_reduce_rows(step, m, k, n):
    """gdb200_matmul_tn_colsum: dW = dY^T X and db = colsum(dY) from one pass over dY (column sums by an extra MMA
    against a tile of ones); small / ragged shapes take the two-call path inside the entry."""
    ctx, lib = step, step.lib
    dy = rnd_np((rng(85).standard_normal((k, m)) * 0.25).astype(np.float32), F16)   # stored [tokens, m]
    x = rnd_np((rng(86).standard_normal((k, n)) * 0.25).astype(np.float32), F16)    # stored [tokens, n]
    dyt, xt = dev(ctx, dy, F16), dev(ctx, x, F16)
    y0, y1 = ctx.scratch_empty(F16, (m, n)), ctx.scratch_empty(F16, (m, n))
    b0, b1 = ctx.scratch_empty(F16, (m,)), ctx.scratch_empty(F16, (m,))
    xv, wv = dyt.mv(k, m), xt.mv(k, n)
    y0v, y1v, b0v, b1v = y0.mv(m, n), y1.mv(m, n), b0.vv(), b1.vv()
    ctx.check(lib.gd_backend_matmul_tn(ctx.backend, byref(xv), byref(wv), byref(y0v)), "matmul_tn")
    ctx.check(lib.gd_backend_reduce_rows(ctx.backend, byref(xv), byref(b0v)), "reduce_rows")
    ctx.check(lib.gdb200_matmul_tn_colsum(ctx.backend, byref(xv), byref(wv), byref(y1v), byref(b1v)), "matmul_tn_colsum")
    ctx.flush()
    want = O.rnd(t32(dy).t() @ t32(x))
    close(host(y1), want, F16, scale=np.sqrt(k) / 16, what="dW vs oracle")
    np.testing.assert_allclose(host(y1), host(y0), atol=1e-3 * np.sqrt(k) / 16, rtol=2e-3)
    want_b = O.rnd(t32(dy).sum(dim=0))
    close(host(b1), want_b, F16, scale=np.sqrt(k) / 8, what="db vs oracle")
    close(host(b1), host(b0), F16, scale=np.sqrt(k) / 8, what="db vs reduce_rows")


# ------------------------------------------------------------------ flash attention at benchmark-like shapes
@pytest.mark.parametrize("dtype,hq,hkv,dh,window,total", [(F16, 8, 8, 64, 0, 3000), (F16, 8, 8, 64, 256, 3000), (F16, 8, 2, 64, 100, 1500),
                                                          (BF16, 4, 4, 128, 0, 1200), (BF16, 4, 2, 128, 48, 700)])
def test_flash_attention_random_segments(step, dtype, hq, hkv, dh, window, total):
    """Lengths uniform in [16, 512] until `total` tokens, plus trailing rows outside any sequence."""
    ctx = step
    sd = storage_name(dtype)
    r = rng(90)
    lengths = []
    while sum(lengths) < total:
        lengths.append(int(r.integers(16, 513)))
    cu = make_cu(lengths)
    n = int(cu[-1]) + 37                                                      # 37 rows behind the last sequence
    q = rnd_np(r.standard_normal((n, hq, dh)).astype(np.float32), dtype)
    k = rnd_np(r.standard_normal((n, hkv, dh)).astype(np.float32), dtype)
    v = rnd_np(r.standard_normal((n, hkv, dh)).astype(np.float32), dtype)
    go = rnd_np(r.standard_normal((n, hq, dh)).astype(np.float32), dtype)
    qt, kt, vt, cut = dev(ctx, q, dtype), dev(ctx, k, dtype), dev(ctx, v, dtype), dev(ctx, cu, I32)
    qt.requires_grad = kt.requires_grad = vt.requires_grad = True
    out = ops.gd_sdpa_varlen(ctx, qt, kt, vt, cut, causal=True, sliding_window=window, max_seqlen=512)
    nv = int(cu[-1])
    want, _ = O.sdpa_varlen_forward(t32(q[:nv]), t32(k[:nv]), t32(v[:nv]), cu, 0.0, True, window, 0, sd)
    got = host(out)
    close(got[:nv], want, dtype, scale=2, what="forward")
    assert np.all(got[nv:] == 0)
    out.grad = dev(ctx, go, dtype)
    ctx.run_backward()
    wdq, wdk, wdv = O.sdpa_varlen_backward(t32(go[:nv]), t32(q[:nv]), t32(k[:nv]), t32(v[:nv]), cu, 0.0, True, window, 0, sd)
    close(host(qt.grad)[:nv], wdq, dtype, scale=4, what="dq")
    close(host(kt.grad)[:nv], wdk, dtype, scale=8, what="dk")
    close(host(vt.grad)[:nv], wdv, dtype, scale=8, what="dv")
    assert np.all(host(qt.grad)[nv:] == 0) and np.all(host(kt.grad)[nv:] == 0) and np.all(host(vt.grad)[nv:] == 0)


@pytest.mark.parametrize("dtype,hq,hkv,window", [(F16, 8, 8, 0), (F16, 8, 8, 256), (BF16, 4, 2, 100)])
def test_attention_tcgen05_forward_agrees_with_mma_sync_kernels(step, dtype, hq, hkv, window):
    """The tensor-memory forward (mode 0) and the mma.sync forward (mode 1) on the same packed batch:
    outputs within storage rounding of each other, statistics (row max, exp-sum) nearly equal."""
    ctx, lib = step, step.lib
    r = rng(92)
    lengths = []
    while sum(lengths) < 4000:
        lengths.append(int(r.integers(16, 513)))
    cu = make_cu(lengths)
    n, dh = int(cu[-1]) + 21, 64
    q, k, v = (rnd_np(r.standard_normal((n, h, dh)).astype(np.float32), dtype) for h in (hq, hkv, hkv))
    qt, kt, vt, cut = dev(ctx, q, dtype), dev(ctx, k, dtype), dev(ctx, v, dtype), dev(ctx, cu, I32)
    res = []
    for mode in (0, 1):
        old = lib.gdb200_set_attention_mode(ctx.backend, mode)
        try:
            out, stats = ctx.scratch_empty(dtype, (n, hq, dh)), ctx.scratch_empty(F32, (n, hq, 3))
            ctx.fill(out, 0x7E7E7E7E)
            ctx.fill(stats, 0)
            args = abi.SdpaVarlenArgs(0.125, 1, window, 0, 512, 0)
            ctx.check(lib.gd_backend_sdpa_varlen(ctx.backend, byref(qt.tv()), byref(kt.tv()), byref(vt.tv()), byref(cut.tv()), byref(out.tv()),
                                                 byref(stats.tv()), byref(args)), f"sdpa_varlen mode {mode}")
            ctx.flush()
            res.append((host(out), host(stats)))
        finally:
            lib.gdb200_set_attention_mode(ctx.backend, old)
    nv = int(cu[-1])
    want, _ = O.sdpa_varlen_forward(t32(q[:nv]), t32(k[:nv]), t32(v[:nv]), cu, 0.125, True, window, 0, storage_name(dtype))
    close(res[0][0][:nv], want, dtype, scale=2, what="tcgen05 forward vs oracle")
    close(res[0][0][:nv], res[1][0][:nv], dtype, scale=2, what="tcgen05 vs mma.sync")
    assert np.all(res[0][0][nv:] == 0)
    np.testing.assert_allclose(res[0][1][:nv, :, 0], res[1][1][:nv, :, 0], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(res[0][1][:nv, :, 1], res[1][1][:nv, :, 1], rtol=2e-3)


def test_flash_backward_without_forward_stats(step):
    """use_forward_stats = 0: the backward entry recomputes (max, sum) itself."""
    ctx = step
    lengths = [70, 200, 33]
    cu = make_cu(lengths)
    n, hq, dh = int(cu[-1]), 4, 64
    r = rng(91)
    q, k, v, go = (rnd_np(r.standard_normal((n, hq, dh)).astype(np.float32), F16) for _ in range(4))
    qt, kt, vt, gt, cut = dev(ctx, q, F16), dev(ctx, k, F16), dev(ctx, v, F16), dev(ctx, go, F16), dev(ctx, cu, I32)
    dq, dk, dv = (ctx.scratch_empty(F16, (n, hq, dh)) for _ in range(3))
    stats = ctx.scratch_empty(F32, (n, hq, 3))
    ctx.fill(stats, 0x7FC00000)
    args = abi.SdpaVarlenArgs(0.125, 1, 0, 0, 512, 0)
    ctx.check(ctx.lib.gd_backend_sdpa_varlen_backward(ctx.backend, byref(gt.tv()), byref(qt.tv()), byref(kt.tv()), byref(vt.tv()), byref(cut.tv()),
                                                      byref(dq.tv()), byref(dk.tv()), byref(dv.tv()), byref(stats.tv()), byref(args)), "bwd")
    wdq, wdk, wdv = O.sdpa_varlen_backward(t32(go), t32(q), t32(k), t32(v), cu, 0.125, True, 0, 0, "f16")
    close(host(dq), wdq, F16, scale=4)
    close(host(dk), wdk, F16, scale=8)
    close(host(dv), wdv, F16, scale=8)
    # and with no stats tensor at all
    ctx.check(ctx.lib.gd_backend_sdpa_varlen_backward(ctx.backend, byref(gt.tv()), byref(qt.tv()), byref(kt.tv()), byref(vt.tv()), byref(cut.tv()),
                                                      byref(dq.tv()), byref(dk.tv()), byref(dv.tv()), None, byref(args)), "bwd no stats")
    close(host(dq), wdq, F16, scale=4)


@pytest.mark.parametrize("m,k,n", [(1000, 512, 1536), (77, 40, 24), (4096, 1536, 512), (64, 512, 2048)])
def test_fused_matmul_nt_bias_is_bit_identical_to_two_calls(step, m, k, n):
    ctx = step
    x = rnd_np(rng(95).standard_normal((m, k)).astype(np.float32), F16)
    w = rnd_np((rng(96).standard_normal((n, k)) * 0.2).astype(np.float32), F16)
    b = rnd_np(rng(97).standard_normal(n).astype(np.float32), F16)
    outs = []
    for fuse in (True, False):
        ops.FUSE_BIAS_ADD = fuse
        try:
            outs.append(host(ops.gd_linear_transposed_weight(ctx, dev(ctx, x, F16), dev(ctx, w, F16), dev(ctx, b, F16))))
        finally:
            ops.FUSE_BIAS_ADD = True
    assert np.array_equal(outs[0], outs[1])
    close(outs[0], O.linear_transposed_weight_forward(t32(x), t32(w), t32(b)), F16, scale=np.sqrt(k) / 4)


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("m,k,f", [(64, 512, 1536), (1, 512, 1024), (37, 1536, 512), (8, 128, 8)])
def test_fused_linear_swiglu_is_bit_identical_to_two_calls(step, dtype, m, k, f):
    """Up / gate projection + gate of the decode step in one launch (64-row kernel) against
    gdb200_matmul_nt_bias + gd_backend_swiglu_split_forward; shapes it does not take answer UNSUPPORTED."""
    ctx = step
    x = rnd_np(rng(120).standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd_np((rng(121).standard_normal((2 * f, k)) * 0.1).astype(np.float32), dtype)
    b = rnd_np(rng(122).standard_normal(2 * f).astype(np.float32), dtype)
    dx, dw, db = dev(ctx, x, dtype), dev(ctx, w, dtype), dev(ctx, b, dtype)
    up_gate, act, fused = ctx.scratch_empty(dtype, (m, 2 * f)), ctx.scratch_empty(dtype, (m, f)), ctx.scratch_empty(dtype, (m, f))
    lib = ctx.lib
    bv = db.vv()
    xm, wm = dx.mv(m, k), dw.mv(2 * f, k)
    ugm, fm = up_gate.mv(m, 2 * f), fused.mv(m, f)
    ctx.check(lib.gdb200_matmul_nt_bias(ctx.backend, byref(xm), byref(wm), byref(bv), byref(ugm)), "nt_bias")
    ctx.check(lib.gd_backend_swiglu_split_forward(ctx.backend, byref(up_gate.tv()), byref(act.tv())), "swiglu")
    ctx.check(lib.gdb200_matmul_nt_bias_swiglu(ctx.backend, byref(xm), byref(wm), byref(bv), byref(fm)), "fused")
    assert np.array_equal(host(fused), host(act))
    big = ctx.scratch_empty(dtype, (65, k))
    out65 = ctx.scratch_empty(dtype, (65, f))
    assert lib.gdb200_matmul_nt_bias_swiglu(ctx.backend, byref(big.mv(65, k)), byref(wm), byref(bv), byref(out65.mv(65, f))) == abi.GD_ERR_UNSUPPORTED
    assert lib.gdb200_matmul_nt_bias_swiglu(ctx.backend, byref(xm), byref(wm), byref(bv), byref(ugm)) == abi.GD_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("dtype,lengths,hq,hkv,window", [(F16, [300, 17, 512, 64, 131], 8, 8, 0), (BF16, [257, 90], 4, 2, 0), (F16, [400, 200], 2, 2, 96)])
def test_sdpa_backward_with_forward_output_matches_the_two_pass_backward(step, dtype, lengths, hq, hkv, window):
    """gdb200_sdpa_varlen_backward_with_output (D from dO and the forward output, dQ accumulated in FP32 by the
    key-stationary kernel) against gd_backend_sdpa_varlen_backward on the same tensors, and both against the oracle."""
    ctx = step
    n, dh = sum(lengths), 64
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    q, k, v, go = (rnd_np(rng(130 + i).standard_normal((n, h, dh)).astype(np.float32) * s, dtype)
                   for i, (h, s) in enumerate(((hq, 0.5), (hkv, 0.5), (hkv, 1.0), (hq, 1.0))))
    grads = {}
    for with_out in (True, False):
        ops.SDPA_BACKWARD_WITH_OUTPUT = with_out
        try:
            qt, kt, vt = dev(ctx, q, dtype), dev(ctx, k, dtype), dev(ctx, v, dtype)
            qt.requires_grad = kt.requires_grad = vt.requires_grad = True
            out = ops.gd_sdpa_varlen(ctx, qt, kt, vt, dev(ctx, cu, I32), causal=True, sliding_window=window, max_seqlen=max(lengths))
            out.grad = dev(ctx, go, dtype)
            ctx.run_backward()
            grads[with_out] = (host(qt.grad), host(kt.grad), host(vt.grad))
        finally:
            ops.SDPA_BACKWARD_WITH_OUTPUT = True
    sd = storage_name(dtype)
    wdq, wdk, wdv = O.sdpa_varlen_backward(t32(go), t32(q), t32(k), t32(v), cu, 0.0, True, window, 0, sd)
    for i, (want, what, sc) in enumerate(((wdq, "dq", 4), (wdk, "dk", 6), (wdv, "dv", 6))):
        close(grads[True][i], want, dtype, scale=sc, what=what + " single pass")
        close(grads[False][i], want, dtype, scale=sc, what=what + " two passes")
    # dV does not depend on D; the two paths form P in different kernels (tensor-memory kernel: exp2 with 1/l folded
    # into the exponent; mma.sync kernel: exp2 times 1/l), so it agrees to the rounding of P, not bit for bit
    close(grads[True][2], grads[False][2], dtype, scale=2, what="dv single pass vs two passes")


@pytest.mark.parametrize("dtype,dh,lengths", [(F16, 64, [300, 17, 512, 64, 131]), (BF16, 64, [257, 90]), (F16, 128, [200, 56])])
def test_query_gradient_left_in_fp32_for_the_rope_backward(step, dtype, dh, lengths):
    """gdb200_sdpa_varlen_backward_with_output_q32 + gdb200_qkv_split_rope_backward_q32: where the one-pass attention backward
    runs (head_dim 64) the query gradient stays unrounded in the FP32 accumulator and the RoPE backward rounds it on load, bit
    for bit what rounding it first and calling the reference entry gives; elsewhere grad_q is written and the flag says so."""
    ctx, lib = step, step.lib
    n, h = sum(lengths), 4
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    q, k, v, go = (rnd_np(rng(140 + i).standard_normal((n, h, dh)).astype(np.float32) * s, dtype) for i, s in enumerate((0.5, 0.5, 1.0, 1.0)))
    pos = np.concatenate([np.arange(x) for x in lengths]).astype(np.int32)
    qt, kt, vt, got, cut, post = dev(ctx, q, dtype), dev(ctx, k, dtype), dev(ctx, v, dtype), dev(ctx, go, dtype), dev(ctx, cu, I32), dev(ctx, pos, I32)
    scale = 1.0 / math.sqrt(dh)
    stats, out = ctx.scratch_empty(F32, (n, h, 3)), ctx.scratch_empty(dtype, (n, h, dh))
    fargs = abi.SdpaVarlenArgs(scale, 1, 0, 0, max(lengths), 0)
    ctx.check(lib.gd_backend_sdpa_varlen(ctx.backend, byref(qt.tv()), byref(kt.tv()), byref(vt.tv()), byref(cut.tv()), byref(out.tv()), byref(stats.tv()), byref(fargs)), "sdpa_varlen")
    dq, dk, dv = (ctx.scratch_empty(dtype, (n, h, dh)) for _ in range(3))
    ctx.fill(dq, 0)
    acc = ctx.scratch_empty(F32, (n, h, dh))
    bargs = abi.SdpaVarlenArgs(scale, 1, 0, 0, max(lengths), 1)
    flag = C.c_int32(-1)
    ctx.check(lib.gdb200_sdpa_varlen_backward_with_output_q32(ctx.backend, byref(got.tv()), byref(qt.tv()), byref(kt.tv()), byref(vt.tv()), byref(cut.tv()),
                                                              byref(out.tv()), byref(dq.tv()), byref(dk.tv()), byref(dv.tv()), byref(stats.tv()), byref(acc.tv()),
                                                              byref(bargs), byref(flag)), "sdpa backward, query gradient in FP32")
    wdq, wdk, wdv = O.sdpa_varlen_backward(t32(go), t32(q), t32(k), t32(v), cu, scale, True, 0, 0, storage_name(dtype))
    close(host(dk), wdk, dtype, scale=6, what="dk")
    close(host(dv), wdv, dtype, scale=6, what="dv")
    rope = abi.RopeArgs(10000.0, dh, 0)
    dqkv = ctx.scratch_empty(dtype, (n, 3 * h * dh))
    if dh != 64:
        assert flag.value == 0                                           # the one-pass kernel does not take this head size
        close(host(dq), wdq, dtype, scale=4, what="dq")
        return
    assert flag.value == 1 and not host(dq).any()                        # grad_q untouched
    dq_rounded = rnd_np(host(acc), dtype)
    close(dq_rounded, wdq, dtype, scale=4, what="dq (rounded accumulator)")
    ctx.check(lib.gdb200_qkv_split_rope_backward_q32(ctx.backend, byref(acc.tv()), byref(dk.tv()), byref(dv.tv()), byref(post.tv()), byref(dqkv.tv()), h, dh, byref(rope)),
              "rope backward from the FP32 query gradient")
    want = ctx.scratch_empty(dtype, (n, 3 * h * dh))
    ctx.check(lib.gd_backend_qkv_split_rope_backward(ctx.backend, byref(dev(ctx, dq_rounded, dtype).tv()), byref(dk.tv()), byref(dv.tv()), byref(post.tv()), byref(want.tv()), h, dh,
                                                     byref(rope)), "rope backward, reference entry")
    assert np.array_equal(host(dqkv).view(np.uint32), host(want).view(np.uint32))


# ------------------------------------------------------------------ batched contractions (src/ops/matmul/core_matmul.c:47,54)
def _bview(t, batch_shape, rows, cols, strides_elems, es):
    v = abi.BatchedMatrixView()
    v.buffer, v.offset, v.rows, v.cols, v.row_bytes, v.dtype = t.buffer, t.offset, rows, cols, cols * es, t.dtype
    v.batch_rank = len(batch_shape)
    v.batch_count = int(np.prod(batch_shape))
    for d, (n, s) in enumerate(zip(batch_shape, strides_elems)):
        v.batch_shape[d], v.batch_strides[d] = n, s * es
    return v


@pytest.mark.parametrize("entry,ta,tb", [("batched_matmul", 0, 0), ("batched_matmul_nt", 0, 1), ("batched_matmul_tn", 1, 0)])
@pytest.mark.parametrize("case", ["plain", "broadcast_w", "rank2_nested", "rank2_strided", "small_fallback"])
def test_batched_matmul_against_oracle(step, entry, ta, tb, case):
    """x[..., M, K] w[..., K, N] with numpy-style broadcasting over the batch dimensions, against torch.matmul in FP32 rounded
    once. `plain` / `broadcast_w` / `rank2_nested` run as ONE launch with the batch as third grid dimension, `rank2_strided`
    (a permuted outer dimension) as one launch per outer index, `small_fallback` on the portable kernel per element."""
    ctx, lib, dtype, es = step, step.lib, F16, 2
    m, k, n = (200, 192, 136) if case != "small_fallback" else (24, 40, 16)
    ybs = {"plain": (5,), "broadcast_w": (4,), "rank2_nested": (2, 3), "rank2_strided": (2, 3), "small_fallback": (3,)}[case]
    xbs = ybs
    wbs = tuple(1 for _ in ybs) if case == "broadcast_w" else ybs
    r = rng(300 + len(case))
    xs, ws = ((k, m) if ta else (m, k)), ((n, k) if tb else (k, n))
    x = rnd_np(r.standard_normal(xbs + xs).astype(np.float32), dtype)
    w = rnd_np((r.standard_normal(wbs + ws) * 0.1).astype(np.float32), dtype)
    xt, wt = dev(ctx, x, dtype), dev(ctx, w, dtype)
    yt = ctx.scratch_empty(dtype, ybs + (m, n))

    def strides(bs, mat, permuted=False):
        st, acc = [], mat[0] * mat[1]
        for d in reversed(range(len(bs))):
            st.insert(0, 0 if bs[d] == 1 else acc)
            acc *= bs[d]
        return st

    xst, wst, yst = strides(xbs, xs), strides(wbs, ws), strides(ybs, (m, n))
    if case == "rank2_strided":
        # x is stored [3, 2, ...] and viewed as [2, 3, ...]: the outer pitch is not the inner extent times the inner pitch
        x = np.ascontiguousarray(np.transpose(x, (1, 0, 2, 3)))      # storage order [3, 2, ...]
        xt = dev(ctx, x, dtype)
        xst = [xs[0] * xs[1], 2 * xs[0] * xs[1]]                     # view dim 0 (size 2) steps one matrix, dim 1 (size 3) steps two
        x = np.transpose(x, (1, 0, 2, 3))                            # logical [2, 3, ...] for the oracle
    xv, wv, yv = _bview(xt, xbs, xs[0], xs[1], xst, es), _bview(wt, wbs, ws[0], ws[1], wst, es), _bview(yt, ybs, m, n, yst, es)
    launches0 = ctx.launch_count()
    ctx.check(getattr(lib, "gd_backend_" + entry)(ctx.backend, byref(xv), byref(wv), byref(yv)), entry)
    n_launch = ctx.launch_count() - launches0
    tx, tw = torch.from_numpy(x), torch.from_numpy(w)
    if ta:
        tx = tx.transpose(-1, -2)
    if tb:
        tw = tw.transpose(-1, -2)
    want = rnd_np(torch.matmul(tx, tw).numpy(), dtype)
    close(host(yt), want, dtype, scale=math.sqrt(k) / 4, what=f"{entry} {case}")
    expect = {"plain": 1, "broadcast_w": 1, "rank2_nested": 1, "rank2_strided": 2, "small_fallback": 3}[case]
    assert n_launch == expect, (case, n_launch)


@pytest.mark.parametrize("dtype,m,k,f", [(F16, 1024, 512, 1536), (BF16, 777, 256, 384), (F16, 300, 192, 128), (F16, 96, 128, 128)])
def test_up_gate_projection_with_swiglu_epilogue_is_bit_identical_to_the_three_calls(step, dtype, m, k, f):
    """gdb200_matmul_nt_bias_swiglu_both (x12 and act from one contraction, SwiGLU in the epilogue of the CTA-pair kernel; the
    last shape is below its 256-row minimum and takes the unfused calls) against gdb200_matmul_nt_bias followed by
    gd_backend_swiglu_split_forward bit for bit, and against the oracle."""
    ctx, lib = step, step.lib
    r = rng(410 + m)
    x = rnd_np(r.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd_np((r.standard_normal((2 * f, k)) * 0.05).astype(np.float32), dtype)
    b = rnd_np((r.standard_normal(2 * f) * 0.1).astype(np.float32), dtype)
    xt, wt, bt = dev(ctx, x, dtype), dev(ctx, w, dtype), dev(ctx, b, dtype)
    ug0, act0 = ctx.scratch_empty(dtype, (m, 2 * f)), ctx.scratch_empty(dtype, (m, f))
    ug1, act1 = ctx.scratch_empty(dtype, (m, 2 * f)), ctx.scratch_empty(dtype, (m, f))
    xm, wm, bv = xt.mv(m, k), wt.mv(2 * f, k), bt.vv()
    ctx.check(lib.gdb200_matmul_nt_bias(ctx.backend, byref(xm), byref(wm), byref(bv), byref(ug0.mv(m, 2 * f))), "matmul_nt_bias")
    ctx.check(lib.gd_backend_swiglu_split_forward(ctx.backend, byref(ug0.tv()), byref(act0.tv())), "swiglu_split_forward")
    ctx.check(lib.gdb200_matmul_nt_bias_swiglu_both(ctx.backend, byref(xm), byref(wm), byref(bv), byref(ug1.mv(m, 2 * f)), byref(act1.mv(m, f))), "fused")
    assert np.array_equal(ug1.read().view(np.uint16), ug0.read().view(np.uint16))
    assert np.array_equal(act1.read().view(np.uint16), act0.read().view(np.uint16))
    sd = storage_name(dtype)
    want_ug = O.linear_transposed_weight_forward(t32(x), t32(w), t32(b), sd)
    close(host(ug1), want_ug, dtype, scale=math.sqrt(k) / 4, what="up_gate")
    close(host(act1), O.swiglu_split_forward(torch.from_numpy(host(ug1)), sd), dtype, scale=2, what="act")


@pytest.mark.parametrize("dtype,m,k,f", [(F16, 1024, 512, 1536), (BF16, 777, 256, 384), (F16, 300, 192, 320)])
def test_down_projection_input_gradient_with_swiglu_backward_epilogue_is_bit_identical_to_the_two_calls(step, dtype, m, k, f):
    """gdb200_matmul_nt_swiglu_backward (d_up_gate from g, the down projection's weight and the saved up_gate in one launch)
    against gd_backend_matmul_nt into a scratch followed by gd_backend_swiglu_split_backward, bit for bit, and against the oracle."""
    ctx, lib = step, step.lib
    r = rng(510 + m)
    g = rnd_np(r.standard_normal((m, k)).astype(np.float32), dtype)
    w = rnd_np((r.standard_normal((f, k)) * 0.05).astype(np.float32), dtype)
    ug = rnd_np(r.standard_normal((m, 2 * f)).astype(np.float32), dtype)
    gt, wt, ugt = dev(ctx, g, dtype), dev(ctx, w, dtype), dev(ctx, ug, dtype)
    dact = ctx.scratch_empty(dtype, (m, f))
    d0, d1 = ctx.scratch_empty(dtype, (m, 2 * f)), ctx.scratch_empty(dtype, (m, 2 * f))
    gm, wm = gt.mv(m, k), wt.mv(f, k)
    ctx.check(lib.gd_backend_matmul_nt(ctx.backend, byref(gm), byref(wm), byref(dact.mv(m, f))), "matmul_nt")
    ctx.check(lib.gd_backend_swiglu_split_backward(ctx.backend, byref(ugt.tv()), byref(dact.tv()), byref(d0.tv())), "swiglu_split_backward")
    ctx.check(lib.gdb200_matmul_nt_swiglu_backward(ctx.backend, byref(gm), byref(wm), byref(ugt.mv(m, 2 * f)), byref(d1.mv(m, 2 * f))), "fused")
    assert np.array_equal(d1.read().view(np.uint16), d0.read().view(np.uint16))
    sd = storage_name(dtype)
    want_dact = O.rnd(t32(g) @ t32(w).t(), sd)
    close(host(d1), O.swiglu_split_backward(t32(ug), want_dact, sd), dtype, scale=math.sqrt(k) / 2, what="d_up_gate")
