"""GPU: the reference's own C tests (tests/*.c of the reference tree, compiled unchanged against
this backend into oracle/_ref/tests_cuda/ by oracle/Makefile) run as the drop-in check. The
binaries exist only where the reference tree was available at build time; on a box without them
the test reports that and skips."""
import os
import subprocess

import pytest

from oracle import cref

pytestmark = pytest.mark.gpu

# Tests of the reference that exercise the gpt_lm path or the runtime contract of the backend.
HOT_PATH = ["test_memory", "test_tensor", "test_transfer", "test_linear", "test_matmul_batched", "test_sdpa_varlen",
            "test_kv_cache_decode", "test_rms_norm", "test_embedding", "test_rope", "test_swiglu", "test_dropout_ops",
            "test_lm_cross_entropy", "test_optim", "test_autograd", "test_backward_null_outputs", "test_module",
            "test_module_io", "test_dataloader"]
# The rest of the reference's suite: data formats either side of the path and the ops of its other examples
# including the MiniMax-M3 sparse-attention test: all 39 tests of the reference run against this backend.
WIDER = ["test_ops", "test_binary_ops", "test_reduce_ops", "test_reshape", "test_concat", "test_split", "test_permute",
         "test_sigmoid_ops", "test_tanh_ops", "test_mse", "test_huber", "test_cross_entropy", "test_powlu", "test_powlu_split_linear",
         "test_dataset", "test_gdds", "test_gdds_varlen", "test_tokenizer", "test_metrics", "test_minimax_m3_sparse_attention"]


@pytest.mark.parametrize("name", HOT_PATH + WIDER)
def test_reference_ctest(name, tmp_path):
    exe = os.path.join(cref.TESTS_CUDA_DIR, name)
    if not os.path.exists(exe):
        pytest.skip("reference C tests were not built (no reference tree at build time)")
    # the reference runs its tests from the repository root and writes checkpoints under build/
    os.makedirs(tmp_path / "build", exist_ok=True)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300, cwd=tmp_path)
    out = (res.stdout + res.stderr).strip()
    assert res.returncode == 0, out[-2000:]
    assert "skipped" not in out.lower(), f"{name} skipped instead of running on the CUDA backend: {out[-500:]}"
