"""GPU parity of the whole gpt_lm path: training steps (loss, gradients, AMP state, updated
weights) and greedy KV-cache decode against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest

from gpu_util import F16, abi, host, pkg
from oracle import gpt_lm as OG
from oracle.cref import OracleInt

oracle_int = OracleInt()

pytestmark = pytest.mark.gpu
g = pkg.gpt_lm


def small_cfg(**kw):
    base = dict(vocab_size=320, context_length=64, d_model=128, n_layers=2, n_heads=2, head_dim=64, mlp_hidden=192,
                tied_lm_head=False, dropout_p=0.1, sdpa_window=0)
    base.update(kw)
    return g.GptConfig(**base)


@pytest.mark.parametrize("variant", ["baseline_untied", "reference_tied_window", "no_dropout"])
def test_train_steps_track_oracle(variant):
    cfg = {"baseline_untied": small_cfg(),
           "reference_tied_window": small_cfg(tied_lm_head=True, dropout_p=0.05, sdpa_window=16, mlp_hidden=256),
           "no_dropout": small_cfg(dropout_p=0.0)}[variant]
    tc = g.TrainConfig.baseline()
    host_params = g.init_params(cfg, seed=3)
    ref = OG.OracleGptLm(OG.config_from(cfg), host_params)
    otc = OG.train_config_from(tc)
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, host_params)
        trainer = g.Trainer(model, tc)
        for step in range(3):
            batch = g.synthetic_batch(cfg, n_seqs=5, min_len=4, max_len=64, seed=100 + step, pad_to=64)
            # gradients of step 0 are read before the optimizer consumes the scratch arena again
            ctx.begin_step()
            trainer.optimizer.zero_grad()
            ids, tgt, pos, cu = model.upload_batch(batch)
            loss = model.forward(ids, tgt, pos, cu, trainer.global_step + 1)
            pkg.optim.gd_backward_amp(ctx, loss, trainer.scaler)
            want = ref.train_step(batch.input_ids, batch.targets, batch.positions, batch.cu_seqlens, step + 1, otc)
            got_loss = float(loss.read()[()])
            # stated bound: relative loss error <= 2e-3 per step (F16 storage, FP32 accumulation)
            assert abs(got_loss - want["loss"]) <= 2e-3 * abs(want["loss"]), (step, got_loss, want["loss"])
            if step == 0:
                for name, prm in model.params.items():
                    gg, wg = host(prm.grad), want["grads"][name].numpy()
                    denom = np.abs(wg).max() + 1e-6
                    assert np.abs(gg.reshape(wg.shape) - wg).max() <= 2e-2 * denom, name
            trainer.optimizer.step_amp_clip_lr(trainer.scaler, tc.lr, tc.grad_clip_norm)
            ctx.end_step()
            trainer.global_step += 1
            s = trainer.scaler.sync()
            assert s["scale"] == want["scale"] and bool(s["last_found_inf"]) == want["found_inf"]
            assert abs(trainer.optimizer.last_grad_norm() - want["grad_norm"]) <= 2e-2 * want["grad_norm"]
        for name, prm in model.params.items():
            np.testing.assert_allclose(host(prm).reshape(-1), ref.p[name].numpy().reshape(-1), atol=2e-3, rtol=2e-2, err_msg=name)


def test_bf16_train_steps_track_oracle():
    """BF16 storage (the scaled configuration's dtype), head_dim 128: three steps of the native driver against the oracle
    with BF16 rounding points; loss within 1 %, same loss-scale trajectory, updated weights within BF16 tolerance."""
    cfg = small_cfg(dtype=abi.BF16, n_heads=1, head_dim=128, dropout_p=0.1)
    tc = g.TrainConfig.baseline()
    hp = g.init_params(cfg, seed=23)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    otc = OG.train_config_from(tc)
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, hp)
        trainer = g.NativeTrainer(model, tc)
        for step in range(3):
            b = g.synthetic_batch(cfg, n_seqs=5, min_len=4, max_len=64, seed=700 + step, pad_to=64)
            got = float(trainer.train_batch(b).read()[()])
            want = ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, step + 1, otc)
            assert abs(got - want["loss"]) <= 1e-2 * abs(want["loss"]), (step, got, want["loss"])
            s = trainer.scaler.sync()
            assert s["scale"] == want["scale"] and bool(s["last_found_inf"]) == want["found_inf"]
        for name, prm in model.params.items():
            np.testing.assert_allclose(host(prm).reshape(-1), ref.p[name].numpy().reshape(-1), atol=1.6e-2, rtol=3e-2, err_msg=name)


def test_fifty_seeded_steps_track_the_oracle_loss_and_scaler_trajectory():
    """Stated bound for the whole path: over 50 seeded steps (dropout masks identical by construction, learning rate
    3e-3 so that the loss really moves) the mean loss of every window of 10 steps stays within 2 % of the oracle's,
    every single step within 5 %, and the loss scale / overflow trajectory is identical."""
    cfg, tc = small_cfg(), g.TrainConfig.baseline()
    tc.lr = 3.0e-3
    hp = g.init_params(cfg, seed=17)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    otc = OG.train_config_from(tc)
    got, want, scales = [], [], []
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
        trainer = g.NativeTrainer(g.GptLm(ctx, cfg, hp), tc)
        for step in range(50):
            b = g.synthetic_batch(cfg, n_seqs=6, min_len=8, max_len=64, seed=500 + step % 5, pad_to=64)   # 5 batches, revisited
            got.append(float(trainer.train_batch(b).read()[()]))
            w = ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, step + 1, otc)
            want.append(w["loss"])
            s = trainer.scaler.sync()
            scales.append((s["scale"], bool(s["last_found_inf"]), w["scale"], w["found_inf"]))
    got, want = np.array(got), np.array(want)
    assert all(a == c and b == d for a, b, c, d in scales)
    assert np.all(np.abs(got - want) <= 0.05 * np.abs(want)), np.abs(got / want - 1).max()
    for k in range(0, 50, 10):
        assert abs(got[k:k + 10].mean() - want[k:k + 10].mean()) <= 0.02 * want[k:k + 10].mean()
    assert want[-5:].mean() < 0.9 * want[:5].mean()          # the run does learn something


def test_shards_normalised_by_the_global_row_count_add_up_to_the_union_batch():
    """The data-parallel loss normaliser without a second GPU: the two shards of a batch are stepped one after the other
    through the native driver with global_valid_rows = valid target rows of the whole batch; the sum of the two gradient
    sets and of the two loss shares must equal one step on the union batch (and the oracle's)."""
    cfg = small_cfg(dropout_p=0.0, d_model=128, mlp_hidden=256)
    tc = g.TrainConfig.baseline()
    hp = g.init_params(cfg, seed=41)
    union = g.synthetic_batch(cfg, 7, 5, 64, seed=77)
    shards = [g.take_sequences(union, idx, pad_to=64, context_length=64) for idx in ([0, 2, 4, 6], [1, 3, 5])]
    union_p = g.take_sequences(union, list(range(7)), pad_to=64, context_length=64)
    total_rows = float(np.count_nonzero(union.targets >= 0))

    def one_step(batch, rows):
        with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
            trainer = g.NativeTrainer(g.GptLm(ctx, cfg, hp), tc)
            loss = float(trainer.train_batch(batch, global_valid_rows=rows).read()[()])
            return loss, g.native_step_gradients(trainer)

    (l0, g0), (l1, g1) = one_step(shards[0], total_rows), one_step(shards[1], total_rows)
    lu, gu = one_step(union_p, 0.0)
    assert abs((l0 + l1) - lu) <= 1e-5 * abs(lu)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    want = ref.loss_and_grads(union.input_ids, union.targets, union.positions, union.cu_seqlens, 1, 65536.0)
    assert abs((l0 + l1) - want["loss"]) <= 2e-3 * abs(want["loss"])
    for name in gu:
        both, one, w = g0[name] + g1[name], gu[name], want["grads"][name].numpy().reshape(gu[name].shape)
        denom = np.abs(one).max() + 1e-6
        assert np.abs(both - one).max() <= 1e-2 * denom, name       # F16 roundings at differently scaled values
        assert np.abs(both - w).max() <= 2e-2 * (np.abs(w).max() + 1e-6), name


def test_trainer_train_batch_matches_manual_sequence():
    cfg = small_cfg()
    hp = g.init_params(cfg, seed=5)
    batch = g.synthetic_batch(cfg, n_seqs=4, min_len=8, max_len=64, seed=9, pad_to=64)
    losses = []
    for _ in range(2):
        with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
            trainer = g.Trainer(g.GptLm(ctx, cfg, hp), g.TrainConfig.baseline())
            l1 = float(trainer.train_batch(batch).read()[()])
            l2 = float(trainer.train_batch(batch).read()[()])
            losses.append((l1, l2))
    assert losses[0] == losses[1]            # same seeds, same kernels: bit-identical across runs (no atomics on this path except embedding scatter)
    assert losses[0][1] < losses[0][0]       # the second step on the same batch has a lower loss


def test_greedy_decode_matches_oracle():
    cfg = small_cfg(dropout_p=0.0, tied_lm_head=True, sdpa_window=24)
    hp = g.init_params(cfg, seed=11, residual_scaled=False)
    prompts = np.random.default_rng(3).integers(0, cfg.vocab_size, size=(4, 12)).astype(np.int32)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    want_tokens, want_logits = ref.greedy_generate(prompts, new_tokens=10, capacity=32, return_logits=True)
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, hp)
        model.training = False
        got = g.greedy_generate(model, prompts, new_tokens=10, capacity=32)
    # argmax is integer-exact given equal logits; with F16 logits two candidates can tie within
    # rounding, so a mismatch is only accepted where the oracle's top-2 margin is below 2 F16 ulps.
    for b in range(prompts.shape[0]):
        for t in range(10):
            if got[b, t] != want_tokens[b, t]:
                lg = want_logits[t][b].numpy()
                top2 = np.sort(lg)[-2:]
                assert top2[1] - top2[0] <= 4e-3 * max(1.0, abs(top2[1])), (b, t, got[b, t], want_tokens[b, t])
                break


@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("mlp_hidden", [192, 256])
@pytest.mark.parametrize("batch,window", [(4, 24), (64, 0)])
def test_native_decode_feeds_back_on_the_device_and_matches_the_host_loop(batch, window, mlp_hidden, use_graph):
    """gdb200_gpt_decode_steps (device argmax, ids / positions kept on the device) generates exactly the ids of the
    per-step host loop: same arithmetic, same logits, same tie rule. use_graph = False enqueues one launch per
    operation; with use_graph the run is ONE persistent kernel when the shapes allow (mlp_hidden 256: 13 steps in one
    launch after the memset of its barrier words), else a replayed CUDA graph of the per-operation launches (192)."""
    cfg = small_cfg(dropout_p=0.0, tied_lm_head=(batch == 4), sdpa_window=window, mlp_hidden=mlp_hidden)
    hp = g.init_params(cfg, seed=12, residual_scaled=False)
    prompts = np.random.default_rng(5).integers(0, cfg.vocab_size, size=(batch, 9)).astype(np.int32)
    timing = {}
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=256 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, hp)
        model.training = False
        want = g.greedy_generate(model, prompts, new_tokens=14, capacity=32)
        got = g.greedy_generate_native(model, prompts, new_tokens=14, capacity=32, use_graph=use_graph, timing=timing)
    assert np.array_equal(got, want)
    if use_graph and mlp_hidden == 256:
        assert timing["decode_launches"] <= 2, timing
    else:
        assert timing["decode_launches"] >= 13, timing


def test_persistent_decode_kernel_past_the_cache_capacity_and_bf16():
    """The persistent decode kernel with rows whose position runs past the cache capacity (the append is dropped and
    attention reads the live part only, as the per-operation path does), in BF16."""
    cfg = small_cfg(dropout_p=0.0, mlp_hidden=256, dtype=abi.BF16)
    hp = g.init_params(cfg, seed=3, residual_scaled=False)
    prompts = np.random.default_rng(6).integers(0, cfg.vocab_size, size=(8, 9)).astype(np.int32)
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=256 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, hp)
        model.training = False
        want = g.greedy_generate(model, prompts, new_tokens=12, capacity=16)     # positions 9 .. 19 against 16 slots
        got = g.greedy_generate_native(model, prompts, new_tokens=12, capacity=16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("d_model,n_heads,mlp_hidden,vocab,batch,window,tied", [
    (256, 4, 512, 1024, 64, 0, False),     # 2 heads x 8 key ranges per CTA, two K chunks of 256 in the down projection
    (256, 4, 384, 512, 7, 12, True),       # odd batch: 1 head x 16 key ranges, K chunks of 128, sliding window, tied head
    (512, 8, 1024, 2048, 33, 0, True),     # the reference-default widths at a batch that leaves rows of the 64-row tile empty
])
def test_persistent_decode_kernel_shapes(d_model, n_heads, mlp_hidden, vocab, batch, window, tied):
    """The persistent decode kernel on other partitions of its work (heads per CTA, key ranges, K chunks, unit counts above
    and below the number of CTAs): the ids equal the per-operation host loop's, in one launch."""
    cfg = small_cfg(dropout_p=0.0, d_model=d_model, n_heads=n_heads, mlp_hidden=mlp_hidden, vocab_size=vocab, tied_lm_head=tied,
                    sdpa_window=window, n_layers=2)
    hp = g.init_params(cfg, seed=21, residual_scaled=False)
    prompts = np.random.default_rng(9).integers(0, cfg.vocab_size, size=(batch, 11)).astype(np.int32)
    timing = {}
    with pkg.runtime.Context(params_bytes=128 << 20, state_bytes=512 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, hp)
        model.training = False
        want = g.greedy_generate(model, prompts, new_tokens=12, capacity=48)
        got = g.greedy_generate_native(model, prompts, new_tokens=12, capacity=48, timing=timing)
    assert np.array_equal(got, want)
    assert timing["decode_launches"] <= 2, timing


def test_device_argmax_first_maximum_softcap_and_non_finite():
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((37, 2048)) * 3).astype(np.float16)
    x[0, 5] = x[0, 900] = np.float16(40.0)         # tie: the first index wins
    x[1, :] = np.float16(-np.inf)                   # nothing finite: index 0
    x[2, 7] = np.float16(np.nan)
    x[2, 8] = np.float16(np.inf)                    # +inf: non-finite without a cap, cap * tanh(inf) = cap with one
    x[3, 2047] = np.float16(60000.0)                # the last class
    x[4, :] = np.float16(1.0)                       # all equal
    with pkg.runtime.Context(params_bytes=16 << 20, state_bytes=16 << 20, scratch_bytes=64 << 20) as ctx:
        for cap in (0.0, 30.0):
            ctx.begin_step()
            t = ctx.from_numpy(ctx.scratch, abi.F16, x.astype(np.float32))
            got = g.device_argmax(ctx, t, cap).read()
            ctx.end_step()
            assert np.array_equal(got, g.host_argmax(x.astype(np.float32), cap)), cap
            # the C restatement of the reference's rule (soft cap applied first, as gpt_apply_logits_softcap does)
            capped = x.astype(np.float32)
            if cap > 0.0:
                capped = (np.float32(cap) * np.tanh(capped / np.float32(cap))).astype(np.float32)
            assert np.array_equal(got, np.array([oracle_int.argmax_first(row) for row in capped], dtype=np.int32)), cap
            assert got[0] == 5 and got[1] == 0 and got[4] == 0 and got[2] != 7 and (got[2] == 8) == (cap > 0.0)


@pytest.mark.parametrize("tied,chunk_env,extra", [(False, None, {}), (True, None, {}), (False, "128", {}),
                                                  (False, None, {"vocab_size": 324}),      # the one-pass cross entropy declines: three entries
                                                  (False, None, {"dropout_p": 0.0})])      # no dropout: none of the fused dropout outputs
def test_native_step_driver_matches_python_host(monkeypatch, tied, chunk_env, extra):
    """The library's native per-step driver and the Python op capsules enqueue the same calls (the driver through its fused
    entries where they take the shape): losses and updated parameters agree to within atomics noise (embedding scatter),
    and both track the oracle."""
    if chunk_env:
        monkeypatch.setenv("GD_LM_CE_CHUNK_SIZE", chunk_env)
    cfg = small_cfg(tied_lm_head=tied, sdpa_window=0 if not tied else 16, **extra)
    tc = g.TrainConfig.baseline()
    hp = g.init_params(cfg, seed=21)
    batches = [g.synthetic_batch(cfg, n_seqs=5, min_len=4, max_len=64, seed=300 + s, pad_to=64) for s in range(3)]
    results = {}
    for kind in ("python", "native"):
        with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
            model = g.GptLm(ctx, cfg, hp)
            trainer = (g.NativeTrainer if kind == "native" else g.Trainer)(model, tc)
            losses = [float(trainer.train_batch(b).read()[()]) for b in batches]
            results[kind] = (losses, {n: host(p) for n, p in model.params.items()}, trainer.scaler.sync(), trainer.optimizer.step_count())
    lp, ln = results["python"][0], results["native"][0]
    # first forward, identical inputs: the same kernels up to the loss, which the native driver takes from its one-pass
    # cross entropy when one chunk holds all classes (row maximum before the exponentials instead of an online merge)
    assert lp[0] == ln[0] if chunk_env else abs(lp[0] - ln[0]) <= 2e-6 * abs(lp[0])
    np.testing.assert_allclose(ln, lp, rtol=2e-4)
    for n in results["python"][1]:
        np.testing.assert_allclose(results["native"][1][n], results["python"][1][n], atol=2e-3, rtol=2e-2, err_msg=n)
    assert results["python"][2] == results["native"][2] and results["python"][3] == results["native"][3] == 3
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    otc = OG.train_config_from(tc)
    for s, b in enumerate(batches):
        want = ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, s + 1, otc)
        assert abs(ln[s] - want["loss"]) <= 2e-3 * abs(want["loss"])


@pytest.mark.parametrize("kind", ["python", "native"])
def test_pipelined_steps_match_synchronous_steps(kind):
    """Stream-ordered batch upload and loss download with one step of host run-ahead (the reference's slot rings,
    src/core/memory.c:701,1149-1208) give the same losses, parameters and scaler state as the synchronous form."""
    cfg = small_cfg()
    tc = g.TrainConfig.baseline()
    hp = g.init_params(cfg, seed=33)
    batches = [g.synthetic_batch(cfg, n_seqs=5, min_len=4, max_len=64, seed=500 + s, pad_to=64) for s in range(6)]
    results = {}
    for mode in ("sync", "pipelined"):
        with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
            model = g.GptLm(ctx, cfg, hp)
            trainer = (g.NativeTrainer if kind == "native" else g.Trainer)(model, tc)
            if mode == "sync":
                losses = [float(trainer.train_batch(b).read()[()]) for b in batches]
            else:
                ctx.run_ahead = 1
                slots = [ctx.pinned_copy(np.full(1, np.nan, dtype=np.float32)) for _ in range(2)]
                pinned = []
                for b in batches:
                    b.input_ids, b.targets = ctx.pinned_copy(b.input_ids), ctx.pinned_copy(b.targets)
                    b.positions, b.cu_seqlens = ctx.pinned_copy(b.positions), ctx.pinned_copy(b.cu_seqlens)
                    pinned.append(b)
                losses = []
                for s, b in enumerate(pinned):
                    trainer.train_batch(b, loss_out=slots[s & 1])
                    ctx.wait_steps(1)
                    if s > 0:
                        losses.append(float(slots[(s - 1) & 1][0]))
                ctx.wait_steps(0)
                losses.append(float(slots[(len(pinned) - 1) & 1][0]))
                ctx.run_ahead = 0
            results[mode] = (losses, {n: host(p) for n, p in model.params.items()}, trainer.scaler.sync(), trainer.optimizer.step_count())
    ls, lpipe = results["sync"][0], results["pipelined"][0]
    assert len(lpipe) == len(ls) == 6 and ls[0] == lpipe[0]
    np.testing.assert_allclose(lpipe, ls, rtol=2e-4)
    for n in results["sync"][1]:
        np.testing.assert_allclose(results["pipelined"][1][n], results["sync"][1][n], atol=2e-3, rtol=2e-2, err_msg=n)
    assert results["sync"][2] == results["pipelined"][2] and results["sync"][3] == results["pipelined"][3] == 6
