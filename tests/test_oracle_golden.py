"""CPU: the oracle (oracle/ops.py, oracle/c) against the golden vectors produced from the
reference's own code (tests/golden/make_golden.py). This is what pins the oracle."""
import numpy as np
import pytest
import torch

from conftest import Golden, f16_bits_to_f32
from oracle import ops, cref, gpt_lm as ogpt


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


SDPA = Golden("ref_ctest_sdpa")


@pytest.mark.parametrize("name", [n for n in SDPA.names() if not n.startswith("decode")])
def test_sdpa_varlen_matches_reference_ctest(name):
    c = SDPA[name]
    q, k, v, go = (t(f16_bits_to_f32(c[x])) for x in ("q", "k", "v", "go"))
    out, _ = ops.sdpa_varlen_forward(q, k, v, c["cu"], float(c["scale"]), True, int(c["window"]), int(c["prefix"]), "f32")
    dq, dk, dv = ops.sdpa_varlen_backward(go, q, k, v, c["cu"], float(c["scale"]), True, int(c["window"]), int(c["prefix"]), "f32")
    # FP32 tolerance: torch's vectorised exp / sum paths depend on the run's memory alignment, which moves
    # results by up to about 1e-5 from run to run (seen on the N = 160 case)
    np.testing.assert_allclose(out.numpy(), c["out"], atol=3e-5, rtol=0)
    for got, want in ((dq, c["dq"]), (dk, c["dk"]), (dv, c["dv"])):
        np.testing.assert_allclose(got.numpy(), want, atol=5e-5, rtol=1e-5)


@pytest.mark.parametrize("name", SDPA.names("decode"))
def test_sdpa_decode_matches_reference_ctest(name):
    c = SDPA[name]
    q, k, v = (t(f16_bits_to_f32(c[x])) for x in ("q", "k", "v"))
    pos = np.full(q.shape[0], int(c["cache_pos"]), dtype=np.int32)
    out = ops.sdpa_decode(q, k, v, pos, float(c["scale"]), int(c["window"]), int(c["prefix"]), "f32")
    np.testing.assert_allclose(out.numpy(), c["out"], atol=2e-6, rtol=0)


LMCE = Golden("ref_ctest_lmce")


@pytest.mark.parametrize("name", LMCE.names())
def test_lm_cross_entropy_matches_reference_ctest(name):
    c = LMCE[name]
    h, w, b = t(f16_bits_to_f32(c["hidden"])), t(f16_bits_to_f32(c["weight"])), t(f16_bits_to_f32(c["bias"]))
    bias = b if int(c["has_bias"]) else None
    tg = torch.from_numpy(c["targets"])
    saved = ops.lm_cross_entropy_forward(h, w, bias, tg, float(c["cap"]), -1)
    assert abs(float(saved["loss"]) - float(c["loss"])) <= 2e-6
    dh, dw, db = ops.lm_cross_entropy_backward(h, w, bias, tg, saved, 1.0, float(c["cap"]))
    # the C oracle rounds dlogits, dh, dw, db to F16 exactly as the oracle does: allow 1 F16 ulp
    np.testing.assert_allclose(dh.numpy(), f16_bits_to_f32(c["dh"]), atol=2e-4, rtol=2e-3)
    np.testing.assert_allclose(dw.numpy(), f16_bits_to_f32(c["dw"]), atol=2e-4, rtol=2e-3)
    if bias is not None:
        np.testing.assert_allclose(db.numpy(), f16_bits_to_f32(c["db"]), atol=2e-4, rtol=2e-3)


RR = Golden("ref_ctest_rope_rms")


@pytest.mark.parametrize("name", RR.names("rope"))
def test_rope_matches_reference_ctest(name):
    c = RR[name]
    x, pos = t(c["x"]), torch.from_numpy(c["pos"])
    n_dims, inter = int(c["n_dims"]), bool(c["interleaved"])
    cos, sin = ops.rope_cos_sin(pos, n_dims, float(c["theta"]))
    for sign, want in ((1.0, c["fwd"]), (-1.0, c["bwd"])):
        got = x.clone()
        got[..., :n_dims] = ops._rotate(x[..., :n_dims], cos, sin * sign, inter) if not inter else ops._rotate(x[..., :n_dims], cos, sin * sign, True)
        np.testing.assert_allclose(got.numpy(), want, atol=3e-6, rtol=1e-5)


@pytest.mark.parametrize("name", RR.names("rms"))
def test_rms_norm_matches_reference_ctest(name):
    c = RR[name]
    x, w, g = t(c["x"]), t(c["w"]), t(c["g"])
    y, inv = ops.rms_norm_forward(x, w, float(c["eps"]), "f32")
    dx, dw = ops.rms_norm_backward(x, w, inv, g, "f32")
    np.testing.assert_allclose(y.numpy(), c["out"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(dx.numpy(), c["dx"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(dw.numpy(), c["dw"], atol=2e-5, rtol=1e-5)


PY = Golden("ref_py_scripts")


@pytest.mark.parametrize("name", PY.names("py_rms_fwd"))
def test_rms_forward_matches_reference_script(name):
    c = PY[name]
    dt = "f16" if int(c["is_f16"]) else "f32"
    y, _ = ops.rms_norm_forward(ops.rnd(t(c["x"]), dt), ops.rnd(t(c["w"]), dt), float(c["eps"]), dt)
    np.testing.assert_allclose(y.numpy(), c["y"], atol=1e-3 if dt == "f16" else 2e-6, rtol=1e-3 if dt == "f16" else 1e-5)


@pytest.mark.parametrize("name", PY.names("py_rms_bwd"))
def test_rms_backward_matches_reference_script(name):
    c = PY[name]
    dt = "f16" if int(c["is_f16"]) else "f32"
    x, w, g = (ops.rnd(t(c[k]), dt) for k in ("x", "w", "g"))
    _, inv = ops.rms_norm_forward(x, w, float(c["eps"]), dt)
    dx, dw = ops.rms_norm_backward(x, w, inv, g, dt)
    tol = dict(atol=1e-3, rtol=2e-3) if dt == "f16" else dict(atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(dx.numpy(), c["dx"], **tol)
    np.testing.assert_allclose(dw.numpy().reshape(c["dw"].shape), c["dw"], atol=4e-3 if dt == "f16" else 2e-5, rtol=2e-3)


@pytest.mark.parametrize("name", PY.names("py_dropout"))
def test_dropout_matches_reference_script(name):
    c = PY[name]
    dt = "f16" if int(c["is_f16"]) else "f32"
    y, mask = ops.dropout_forward(t(c["x"]), float(c["p"]), int(c["seed"]), dt)
    assert np.array_equal(mask.numpy().reshape(-1), c["mask"].reshape(-1))          # masks are bit-exact
    assert np.array_equal(y.numpy(), c["y"])                                          # and so are the values
    assert np.array_equal(cref.OracleInt().dropout_mask(c["x"].size, float(c["p"]), int(c["seed"])), c["mask"].reshape(-1))


@pytest.mark.parametrize("name", PY.names("py_linear"))
def test_linear_matches_reference_script(name):
    c = PY[name]
    x, w, b, gy = t(c["x"]), t(c["w"]), t(c["b"]), t(c["gy"])
    y = ops.linear_forward(x, w, b if int(c["has_bias"]) else None)
    assert np.array_equal(y.numpy(), c["y"])
    dx, dw, db = ops.linear_backward(x, w, gy)
    assert np.array_equal(dx.numpy(), c["dx"]) and np.array_equal(dw.numpy(), c["dw"]) and np.array_equal(db.numpy(), c["db"])


OPT = Golden("ref_ctest_optim")


def test_adamw_first_step_bit_exact():
    c = OPT["adamw_first_step"]
    st = {"beta1_power": np.float32(1.0), "beta2_power": np.float32(1.0)}
    p, _, _ = ops.adamw_step(t(c["p0"]), t(c["g0"]), torch.zeros(3), torch.zeros(3), st, float(c["lr"]), float(c["beta1"]),
                             float(c["beta2"]), float(c["eps"]), float(c["wd"]), 1.0)
    assert np.array_equal(p.numpy().astype(np.float16).view(np.uint16), c["want_f16"])


def test_adamw_clip_step_bit_exact():
    c = OPT["adamw_clip_step"]
    gscale, norm, found = ops.grad_clip_scale([t(c["g0"])], 1.0, float(c["max_norm"]))
    assert not found and abs(norm - float(c["norm"])) < 1e-6
    st = {"beta1_power": np.float32(1.0), "beta2_power": np.float32(1.0)}
    p, _, _ = ops.adamw_step(t(c["p0"]), t(c["g0"]), torch.zeros(2), torch.zeros(2), st, float(c["lr"]), 0.0, 0.0, 1.0, 0.0, gscale)
    assert np.array_equal(p.numpy().astype(np.float16).view(np.uint16), c["want_f16"])


def test_amp_growth_and_backoff():
    # tests/test_optim.c:293,313: scale 8 grows to 16 after growth_interval clean steps, backs off to 8 on overflow
    cfg = dict(growth_factor=2.0, backoff_factor=0.5, min_scale=1.0, max_scale=65536.0, growth_interval=1)
    st = {"scale": np.float32(8.0), "inv_scale": np.float32(0.125), "growth_tracker": 0, "found_inf": 0, "last_found_inf": 0}
    ops.amp_begin_step(st, cfg)
    ops.amp_finish_step(st, cfg)
    assert st["scale"] == 16.0
    ops.amp_begin_step(st, cfg)
    st["found_inf"] = 1
    ops.amp_finish_step(st, cfg)
    assert st["scale"] == 8.0 and st["last_found_inf"] == 1


def test_c_restatement_agrees_with_numpy_oracle():
    o = cref.OracleInt()
    for x in (0, 1, 0x9E3779B97F4A7C15, 2**64 - 1):
        assert o.splitmix64(x) == int(ops.splitmix64(np.array([x], dtype=np.uint64))[0]) == ogpt.splitmix64(x)
    for (i, j, ca, w, p) in [(3, 5, 1, 0, 0), (5, 3, 1, 2, 0), (5, 3, 1, 3, 0), (1, 3, 1, 0, 4), (6, 2, 1, 2, 4), (6, 5, 1, 2, 4), (2, 9, 0, 0, 0)]:
        assert bool(o.mask_allowed(i, j, ca, w, p)) == bool(ops.mask_allowed(np.array(i), np.array(j), bool(ca), w, p))
    assert o.argmax_first(np.array([np.nan, 1.0, 3.0, 3.0, np.inf], dtype=np.float32)) == 2
    assert o.argmax_first(np.array([np.nan, -np.inf, np.inf], dtype=np.float32)) == 0     # nothing finite: the reference's `best = 0`
