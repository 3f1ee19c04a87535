"""GPU: the reference's OWN C host (examples/gpt_lm/gpt_lm_shared.c, the tape of src/autograd/autograd.c,
gd_backward_amp, gd_optimizer_step_amp_clip_lr, inside gd_begin_step / gd_end_step) training its gpt_lm model on the
B200 backend, against the Python mirror of the same op capsules and against the CPU oracle on the same weights and
batches. The binary (host_c/gpt_lm_synth) is built from the reference tree where that is present and travels with
the repository; without it the tests are skipped."""
import os

import numpy as np
import pytest

from gpu_util import pkg
from oracle import gpt_lm as OG

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(pkg.c_host.BINARY), reason="host_c/gpt_lm_synth is not built")]
g, ch = pkg.gpt_lm, pkg.c_host


def reference_model_config(layers: int, dropout: float):
    cfg = g.GptConfig.reference_default()
    cfg.n_layers, cfg.dropout_p = layers, dropout
    cfg.dropout_seed = g.splitmix64(ch.REFERENCE_SEED ^ ch.DROPOUT_SEED_SALT)
    return cfg


@pytest.mark.parametrize("feed", ["hostptr", "upload"])
def test_reference_c_host_losses_equal_the_python_mirror_and_track_the_oracle(tmp_path, feed):
    """Three training steps of the reference's C host == three steps of the Python mirror (same backend calls, same
    weights: the C host's own initialisation is read back and loaded into the mirror) and within 2e-3 of the oracle.
    `hostptr` writes the batch through the data slot's host pointer as the reference's loader threads do, with the
    backend's default settings and the 128 MiB data slots of the reference's example."""
    layers, dropout = 2, 0.05
    cfg = reference_model_config(layers, dropout)
    batches = [g.synthetic_batch(cfg, 12, 16, 512, seed=900 + s, pad_to=cfg.context_length) for s in range(3)]
    bfile, pfile = str(tmp_path / "batches.bin"), str(tmp_path / "params.bin")
    ch.write_batches(bfile, batches)
    res = ch.run(bfile, steps=3, warmup=0, layers=layers, feed=feed, read_loss=True, dump_params=pfile, dropout=dropout)
    c_losses = np.array(res["losses"], dtype=np.float32)
    assert np.isfinite(c_losses).all() and res["launches_per_step"] > 50
    flat = ch.read_params(pfile)
    hp = {name: flat[name].reshape(shape) for name, shape, _ in g.param_specs(cfg)}
    assert abs(float(hp["token_embedding"].std()) - 0.02) < 2e-3 and np.all(hp["final_norm_w"] == 1.0)
    tc = g.TrainConfig()                                        # the reference's defaults: lr 3e-4, wd 1e-4, clip 1.0
    with pkg.runtime.Context(params_bytes=128 << 20, state_bytes=256 << 20, scratch_bytes=4 << 30, data_bytes=32 << 20) as ctx:
        trainer = g.Trainer(g.GptLm(ctx, cfg, hp), tc)
        py_losses = np.array([float(trainer.train_batch(b).read()[()]) for b in batches], dtype=np.float32)
    # same kernels in the same order; the embedding scatter sums with atomics, so later steps may differ in the last bits
    assert c_losses[0] == py_losses[0], (c_losses, py_losses)
    np.testing.assert_allclose(c_losses, py_losses, rtol=2e-5)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    otc = OG.train_config_from(tc)
    for s, b in enumerate(batches):
        want = ref.train_step(b.input_ids, b.targets, b.positions, b.cu_seqlens, s + 1, otc)["loss"]
        assert abs(c_losses[s] - want) <= 2e-3 * abs(want), (s, c_losses[s], want)
