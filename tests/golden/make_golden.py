"""Generates the committed golden fixtures under tests/golden/ from the REFERENCE's own code.

Run in a container that has the reference tree (see --ref for the default location) and after
`python -c "import __graft_entry__ as g; g.build()"` (which builds oracle/_ref/ref_harness.so):

    python tests/golden/make_golden.py [--ref <reference tree>]

Sources of truth (nothing is re-derived from this repository's oracle):
  * CPU reference functions that the reference's C tests carry (tests/test_sdpa_varlen.c:122-371,
    599-677; tests/test_lm_cross_entropy.c:141-296; tests/test_rope.c:67-103;
    tests/test_rms_norm.c:56-105), compiled from the reference tree into oracle/_ref/ref_harness.so,
    on the tests' own deterministic pattern inputs and case shapes.
  * The reference-side functions of the reference's PyTorch oracle scripts, imported from the
    reference tree: src/ops/rms_norm/{fwd,bwd}.py (make_inputs, reference), src/ops/dropout/fwd.py
    (case_input, dropout_mask, ref_dropout). src/ops/linear/{fwd,bwd}.py compute their reference
    inline in run_case (fwd.py:147-156, bwd.py:171-190); those lines are transcribed here.
  * The reference's compact-record transform (examples/gpt_lm/main.c:873-970), compiled from the reference
    tree into oracle/_ref/ref_compact.so, on seeded records (valid ones and ones it must reject).
  * The CPU references of tests/test_minimax_m3_sparse_attention.c:145-213,423-600 (block selection, forward and
    backward of the MiniMax-M3 sparse attention), from the same ref_harness.so, on the test's own pattern case and on
    seeded cases.
  * Closed-form expectations of tests/test_optim.c:197-211,228-229,293,313,363-372 and the
    schedule points of tests/test_optim.c:50-61.
The fixtures are small .npz files; tests/test_oracle_golden.py checks oracle/ against them on CPU
and tests/test_gpu_golden.py checks the CUDA backend against them on a B200.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import cref  # noqa: E402


def load_script(ref: str, rel: str, name: str):
    sys.path.insert(0, ref)
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref, rel))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def sdpa_cases(h: cref.RefHarness) -> dict:
    out = {}
    # (name, N, Hq, Hkv, Dh, cu, window, prefix): the shapes of tests/test_sdpa_varlen.c:373-597
    cases = [("n5_gqa_dh4", 5, 2, 1, 4, [0, 2, 5], 0, 0),
             ("n160_dh64_w8_p4", 160, 2, 1, 64, [0, 64, 160], 8, 4),
             ("n160_dh64_w8_p0", 160, 2, 1, 64, [0, 64, 160], 8, 0),
             ("n520_dh64_w32", 520, 1, 1, 64, [0, 520], 32, 0),
             ("n96_dh64_causal", 96, 4, 2, 64, [0, 17, 40, 96], 0, 0)]
    for name, n, hq, hkv, dh, cu, win, pre in cases:
        cu = np.asarray(cu, dtype=np.int32)
        q = h.fill_tokens(n * hq * dh, -0.2)
        k = h.fill_tokens(n * hkv * dh, 0.1)
        v = h.fill_tokens(n * hkv * dh, -0.05)
        go = h.fill_tokens(n * hq * dh, 0.02)
        scale = float(np.float32(1.0 / np.sqrt(np.float64(dh))))
        fwd = h.varlen_fwd(q, k, v, cu, hq, hkv, dh, scale, 1, win, pre)
        dq, dk, dv = h.varlen_bwd(go, q, k, v, cu, hq, hkv, dh, scale, 1, win, pre)
        out[name] = dict(q=q.reshape(n, hq, dh), k=k.reshape(n, hkv, dh), v=v.reshape(n, hkv, dh), go=go.reshape(n, hq, dh),
                         cu=cu, window=win, prefix=pre, scale=np.float32(scale), out=fwd, dq=dq, dk=dk, dv=dv)
    # decode (tests/test_sdpa_varlen.c:679-719 shape family): B1 Tq2 Tmax5 and a windowed Tq1 case
    for name, b, tq, tmax, hq, hkv, dh, pos, win, pre in [("decode_b1_tq2", 1, 2, 5, 2, 1, 4, 2, 0, 0),
                                                         ("decode_b2_tq1_w3", 2, 1, 9, 4, 2, 64, 6, 3, 0)]:
        q = h.fill_tokens(b * tq * hq * dh, -0.1)
        k = h.fill_tokens(b * tmax * hkv * dh, 0.07)
        v = h.fill_tokens(b * tmax * hkv * dh, -0.03)
        scale = float(np.float32(1.0 / np.sqrt(np.float64(dh))))
        o = h.decode(q, k, v, pos, b, tq, tmax, hq, hkv, dh, scale, win, pre)
        out[name] = dict(q=q.reshape(b, tq, hq, dh), k=k.reshape(b, tmax, hkv, dh), v=v.reshape(b, tmax, hkv, dh),
                         cache_pos=np.int32(pos), window=win, prefix=pre, scale=np.float32(scale), out=o)
    return out


def lmce_cases(h: cref.RefHarness) -> dict:
    out = {}
    base = np.array([3, 17, 31, 0, 8, 22], dtype=np.int32)
    ign = np.array([3, -1, 31, 0, -1, 22], dtype=np.int32)
    for name, targets, cap, bias in [("cap0_nobias", base, 0.0, False), ("cap075_bias", base, 0.75, True),
                                     ("cap30_bias_ignore", ign, 30.0, True), ("cap075_nobias_ignore", ign, 0.75, False)]:
        r = h.lmce_case(targets, cap, bias)
        out[name] = dict(hidden=r["hidden"], weight=r["weight"], bias=r["bias"], targets=targets, cap=np.float32(cap),
                         has_bias=np.int32(bias), loss=np.float32(r["loss"]), dh=r["dh"], dw=r["dw"], db=r["db"])
    return out


def rope_rms_cases(h: cref.RefHarness) -> dict:
    out = {}
    rng = np.random.default_rng(7)
    for name, shape, n_dims, inter in [("rope_half_full", (6, 2, 8), 8, False), ("rope_interleaved_tail", (5, 3, 10), 6, True),
                                       ("rope_dh64", (37, 2, 64), 64, False)]:
        x = rng.standard_normal(shape).astype(np.float32)
        pos = (np.arange(shape[0]) * 3 % 11).astype(np.int32)
        out[name] = dict(x=x, pos=pos, n_dims=np.int32(n_dims), interleaved=np.int32(inter), theta=np.float32(10000.0),
                         fwd=h.rope(x, pos, 10000.0, n_dims, inter, 1.0), bwd=h.rope(x, pos, 10000.0, n_dims, inter, -1.0))
    for name, rows, cols in [("rms_7x24", 7, 24), ("rms_33x512", 33, 512)]:
        x = (rng.standard_normal((rows, cols)) * 0.5).astype(np.float32)
        w = (rng.standard_normal(cols) * 0.25 + 1.0).astype(np.float32)
        g = (rng.standard_normal((rows, cols)) * 0.25).astype(np.float32)
        o, dx, dw = h.rms(x, w, g, 1.0e-5)
        out[name] = dict(x=x, w=w, g=g, eps=np.float32(1.0e-5), out=o, dx=dx, dw=dw)
    return out


def script_cases(ref: str) -> dict:
    out = {}
    fwd = load_script(ref, "src/ops/rms_norm/fwd.py", "ref_rms_fwd")
    bwd = load_script(ref, "src/ops/rms_norm/bwd.py", "ref_rms_bwd")
    for case in fwd.cases():
        x, w = fwd.make_inputs(case)
        out["py_rms_fwd_" + case.name] = dict(x=x.numpy(), w=w.numpy(), eps=np.float32(case.eps), is_f16=np.int32(case.dtype == "f16"),
                                              y=fwd.reference(case, x, w).numpy())
    for case in bwd.cases():
        x, w, g = bwd.make_inputs(case)
        dx, dw = bwd.reference(case, x, w, g)
        out["py_rms_bwd_" + case.name] = dict(x=x.numpy(), w=w.numpy(), g=g.numpy(), eps=np.float32(case.eps),
                                              is_f16=np.int32(case.dtype == "f16"), dx=dx.numpy(), dw=dw.numpy())
    dr = load_script(ref, "src/ops/dropout/fwd.py", "ref_dropout_fwd")
    for case in dr.make_cases():
        if not case.training:
            continue
        x = dr.case_input(case)
        y = dr.ref_dropout(x, case)
        mask = dr.dropout_mask(case.shape, case.p, case.seed).numpy().astype(np.uint8)
        out["py_dropout_" + case.name] = dict(x=x.float().numpy(), p=np.float32(case.p), seed=np.uint64(case.seed),
                                              is_f16=np.int32(case.dtype == "f16"), y=y.float().numpy(), mask=mask)
    # linear forward / backward: reference lines transcribed (src/ops/linear/fwd.py:147-156, bwd.py:171-190)
    for m, k, n, has_bias in [(4, 7, 6, True), (4, 7, 6, False), (64, 128, 96, True)]:
        seed = 3000 + m * 3 + k * 5 + n * 7 + (11 if has_bias else 0)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        x = (torch.randn(m, k, generator=gen, dtype=torch.float32) * 0.04).to(torch.float16)
        w = (torch.randn(k, n, generator=gen, dtype=torch.float32) * 0.04).to(torch.float16)
        b = (torch.randn(n, generator=gen, dtype=torch.float32) * 0.04).to(torch.float16)
        ref = x.float() @ w.float()
        if has_bias:
            ref = ref + b.float()
        ref = ref.to(torch.float16).float()
        gy = (torch.randn(m, n, generator=gen, dtype=torch.float32) * 0.04).to(torch.float16)
        dx = (gy.float() @ w.float().t()).to(torch.float16).float()
        dw = (x.float().t() @ gy.float()).to(torch.float16).float()
        db = gy.float().sum(dim=0).to(torch.float16).float()
        out[f"py_linear_m{m}k{k}n{n}_{'bias' if has_bias else 'nobias'}"] = dict(
            x=x.float().numpy(), w=w.float().numpy(), b=b.float().numpy(), has_bias=np.int32(has_bias), y=ref.numpy(),
            gy=gy.float().numpy(), dx=dx.numpy(), dw=dw.numpy(), db=db.numpy())
    return out


def optim_cases() -> dict:
    """Closed-form expectations restated from tests/test_optim.c (the test computes them inline)."""
    f = np.float32
    out = {}
    # first AdamW step (test_optim.c:197-211,228-229): p0 = {1,2,3}, g0 = {0.1,-0.2,0.3}
    p0, g0 = np.array([1, 2, 3], dtype=f), np.array([0.1, -0.2, 0.3], dtype=f)
    lr, eps, wd = f(1.0e-2), f(1.0e-8), f(0.1)
    m, v = g0, g0 * g0
    upd = m / (np.sqrt(v, dtype=f) + eps)
    out["adamw_first_step"] = dict(p0=p0, g0=g0, lr=lr, eps=eps, wd=wd, beta1=f(0.9), beta2=f(0.999),
                                   want_f16=(p0 - lr * (upd + wd * p0)).astype(np.float16).view(np.uint16))
    # clip case (test_optim.c:363-372): p0 = {1,2}, g0 = {3,4}, max_norm 0.5, lr 0.1, beta 0, eps 1, wd 0
    p0, g0 = np.array([1, 2], dtype=f), np.array([3, 4], dtype=f)
    clip = f(0.5) / (f(5.0) + f(1.0e-6))
    cg = g0 * clip
    want = p0 - f(0.1) * (cg / (np.abs(cg) + f(1.0)))
    out["adamw_clip_step"] = dict(p0=p0, g0=g0, max_norm=f(0.5), lr=f(0.1), want_f16=want.astype(np.float16).view(np.uint16),
                                  norm=f(5.0))
    # lr schedule points (test_optim.c:50-61): max 1e-3, min 1e-4, warmup 10, total 110
    steps = np.array([0, 5, 10, 60, 110, 500], dtype=np.int64)
    vals = []
    for s in steps:
        if s < 10:
            vals.append(1.0e-3 * s / 10)
        else:
            pr = min(1.0, (s - 10) / 100)
            vals.append(1.0e-4 + 0.5 * (1.0e-3 - 1.0e-4) * (1.0 + np.cos(np.pi * pr)))
    out["lr_schedule"] = dict(steps=steps, max_lr=f(1.0e-3), min_lr=f(1.0e-4), warmup=np.int64(10), total=np.int64(110),
                              values=np.array(vals, dtype=f))
    return out


def compact_cases() -> dict:
    """Seeded compact records through the reference transform: status and, when accepted, the three outputs."""
    rc = cref.RefCompact()
    rng = np.random.default_rng(20240)
    cases = {}

    def split(total: int, n: int) -> list:
        cuts = np.sort(rng.choice(np.arange(1, total), size=n - 1, replace=False)) if n > 1 else np.array([], dtype=np.int64)
        return np.diff(np.concatenate([[0], cuts, [total]])).astype(np.int32).tolist()

    def add(name, tokens, seg, ctx, vocab, pad, ims, ime):
        st, ids, pos, tgt = rc.transform(tokens, seg, ctx, vocab, pad, ims, ime)
        c = dict(tokens=np.asarray(tokens, dtype=np.uint16), segment_lengths=np.asarray(seg, dtype=np.int32),
                 params=np.asarray([ctx, vocab, pad, ims, ime], dtype=np.int32), status=np.int32(st))
        if st == 0:
            c.update(input_ids=ids, positions=pos, target_ids=tgt)
        cases[name] = c

    for k, (ctx, vocab, n_seg) in enumerate([(8, 16, 1), (8, 16, 3), (64, 320, 5), (64, 320, 64), (512, 2048, 1), (512, 2048, 7), (512, 2048, 40)]):
        add(f"valid{k}", rng.integers(0, vocab, size=ctx + 1), split(ctx, n_seg), ctx, vocab, 0, 1, 2)
    # the record ends on <|im_end|> and the extra token is <|im_start|>: the last target is masked (main.c:960-963)
    t = rng.integers(3, 320, size=65)
    t[63], t[64] = 2, 1
    add("tail_masked", t, split(64, 4), 64, 320, 0, 1, 2)
    t = t.copy()
    t[64] = 5
    add("tail_kept", t, split(64, 4), 64, 320, 0, 1, 2)
    # a document boundary right after an <|im_end|> inside the record
    add("pad_is_last_id", rng.integers(0, 320, size=65), split(64, 6), 64, 320, 319, 1, 2)
    # rejected inputs (main.c:934-959)
    bad = rng.integers(0, 320, size=65)
    bad[17] = 320
    add("bad_token", bad, split(64, 3), 64, 320, 0, 1, 2)
    bad = rng.integers(0, 320, size=65)
    bad[64] = 400
    add("bad_extra_token", bad, split(64, 3), 64, 320, 0, 1, 2)
    add("bad_zero_length", rng.integers(0, 320, size=65), [10, 0, 54], 64, 320, 0, 1, 2)
    add("bad_negative_length", rng.integers(0, 320, size=65), [70, -6], 64, 320, 0, 1, 2)
    add("bad_short", rng.integers(0, 320, size=65), [10, 20], 64, 320, 0, 1, 2)
    add("bad_long", rng.integers(0, 320, size=65), [40, 30], 64, 320, 0, 1, 2)
    return cases


def m3_cases(h: cref.RefHarness) -> dict:
    """MiniMax-M3 sparse attention: the reference test's pattern case and seeded ones (values on a 1/8 grid, so that
    index scores are exact in FP32 and FP64 alike and the selected blocks do not depend on the summation order)."""
    cases = {}

    def add(name, q, k, v, go, iq, ik, cu, block, topk, init_b, local_b, scale):
        bits = lambda a: np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)
        tk = h.m3_topk(bits(iq), bits(ik), cu, block, topk, init_b, local_b)
        out = h.m3_forward(bits(q), bits(k), bits(v), cu, tk, block, scale)
        dq, dk, dv = h.m3_backward(bits(go), bits(q), bits(k), bits(v), cu, tk, block, scale)
        cases[name] = dict(q=bits(q), k=bits(k), v=bits(v), go=bits(go), iq=bits(iq), ik=bits(ik), cu=np.asarray(cu, dtype=np.int32),
                           params=np.asarray([block, topk, init_b, local_b], dtype=np.int32), scale=np.float32(scale), topk=tk, out=out,
                           dq=dq, dk=dk, dv=dv)

    # the reference test's own case (test_sparse_fwd_bwd: N 6, H 2, Dh 4, cu {0, 3, 6}, block 2, topk 2, fill_tokens patterns)
    def pattern(count, base):
        return h.fill_tokens(count, base).view(np.float16).astype(np.float32)
    n, hh, dh = 6, 2, 4
    q, k, v, go = (pattern(n * hh * dh, b).reshape(n, hh, dh) for b in (-0.25, 0.125, -0.375, 0.0625))
    add("ctest_pattern", q, k, v, go, q, k, [0, 3, 6], 2, 2, 1, 1, 0.5)
    rng = np.random.default_rng(77)
    grid = lambda shape: rng.integers(-8, 9, size=shape).astype(np.float32) / 8.0
    for name, (lens, hq, hkv, dh, block, topk, init_b, local_b) in {
            "seeded_mha": ([13, 40, 7], 2, 2, 8, 4, 3, 1, 1),
            "seeded_gqa": ([9, 17, 6], 4, 2, 16, 4, 4, 1, 2),      # the test reference holds statistics of at most 128 (row, head) pairs
            "seeded_no_forced": ([50], 2, 1, 8, 4, 2, 0, 0)}.items():
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        n = int(cu[-1])
        add(name, grid((n, hq, dh)), grid((n, hkv, dh)), grid((n, hkv, dh)), grid((n, hq, dh)), grid((n, hkv, dh)), grid((n, hkv, dh)), cu,
            block, topk, init_b, local_b, 1.0 / np.sqrt(dh))
    return cases


def save(group: str, cases: dict) -> None:
    flat = {}
    for cname, fields in cases.items():
        for fname, val in fields.items():
            flat[f"{cname}/{fname}"] = np.asarray(val)
    path = os.path.join(HERE, group + ".npz")
    np.savez_compressed(path, **flat)
    print(f"{path}: {len(cases)} cases, {os.path.getsize(path)} bytes")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("GD_REFERENCE_DIR", ""), required=not os.environ.get("GD_REFERENCE_DIR"),
                    help="the reference source tree (or set GD_REFERENCE_DIR)")
    args = ap.parse_args()
    if not cref.harness_available():
        raise SystemExit("oracle/_ref/ref_harness.so is missing: run __graft_entry__.build() where the reference tree exists")
    h = cref.RefHarness()
    save("ref_ctest_sdpa", sdpa_cases(h))
    save("ref_ctest_lmce", lmce_cases(h))
    save("ref_ctest_rope_rms", rope_rms_cases(h))
    save("ref_py_scripts", script_cases(args.ref))
    save("ref_ctest_optim", optim_cases())
    save("ref_m3_sparse", m3_cases(h))
    if not cref.compact_available():
        raise SystemExit("oracle/_ref/ref_compact.so is missing: run __graft_entry__.build() where the reference tree exists")
    save("ref_compact_transform", compact_cases())


if __name__ == "__main__":
    main()
