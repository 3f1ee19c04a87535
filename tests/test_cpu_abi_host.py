"""CPU: the C-ABI library loads and exports every declared symbol (no compute calls without a GPU),
struct layouts match the C header, and the host-side logic (batch packing, schedules, seeds,
parameter inventory, data-parallel sharding over gloo ranks) behaves as specified."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from conftest import Golden, ROOT, graft

pkg = graft.load_package()
abi, g, optim = pkg.abi, pkg.gpt_lm, pkg.optim
HEADER = os.path.join(ROOT, "include", "gd_backend_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(gd_backend_[a-z0-9_]+|gdb200_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = abi.load_library()
    names = declared_symbols()
    assert len([n for n in names if n.startswith("gd_backend_")]) == 109   # the reference's backend boundary
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/gd_backend_b200.h but not exported"


def test_struct_layouts_match_the_c_header(tmp_path):
    src = tmp_path / "sizes.c"
    structs = ["gd_backend_matrix_view", "gd_backend_batched_matrix_view", "gd_backend_vector_view", "gd_backend_tensor_view",
               "gd_backend_adamw_desc", "gd_backend_amp_state_desc", "gd_backend_amp_unscale_desc", "gd_backend_grad_norm_desc",
               "gd_backend_embedding_args", "gd_backend_rope_args", "gd_backend_rms_norm_args", "gd_backend_concat_args",
               "gd_backend_sdpa_varlen_args", "gd_backend_sdpa_decode_args", "gd_backend_kv_cache_append_args",
               "gdb200_gpt_spec", "gdb200_gpt_batch", "gdb200_gpt_compact_batch"]
    body = "\n".join(f'printf("%zu\\n", sizeof({s}));' for s in structs)
    src.write_text(f'#include <stdio.h>\n#include "{HEADER}"\nint main(void){{{body} return 0;}}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c11", str(src), "-o", str(exe)], check=True)
    sizes = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    py = [abi.MatrixView, abi.BatchedMatrixView, abi.VectorView, abi.TensorView, abi.AdamwDesc, abi.AmpStateDesc, abi.AmpUnscaleDesc,
          abi.GradNormDesc, abi.EmbeddingArgs, abi.RopeArgs, abi.RmsNormArgs, abi.ConcatArgs, abi.SdpaVarlenArgs, abi.SdpaDecodeArgs,
          abi.KvCacheAppendArgs, abi.GptSpec, abi.GptBatch, abi.GptCompactBatch]
    assert sizes == [C.sizeof(t) for t in py]


@pytest.mark.skipif(pkg.c_host.reference_dir() is None, reason="reference tree not present")
def test_struct_layouts_match_the_reference_header(tmp_path):
    fields = {"gd_backend_matrix_view": ["buffer", "offset", "rows", "cols", "row_bytes", "dtype"],
              "gd_backend_tensor_view": ["buffer", "offset", "count", "dtype", "rank", "shape", "strides"],
              "gd_backend_adamw_desc": ["param_buffer", "grad_scale_offset", "state_f32_buffer", "eps_scaled_offset", "count", "param_dtype", "lr", "bias_correction2"],
              "gd_backend_grad_norm_desc": ["grad_buffer", "partial_count", "found_inf_offset", "has_found_inf"],
              "gd_backend_rms_norm_args": ["rows", "eps", "wgrad_row_block"], "gd_backend_sdpa_varlen_args": ["scale", "max_seqlen", "use_forward_stats"]}
    lines = [f'printf("%zu %zu\\n", sizeof({s}), offsetof({s}, {f}));' for s, fs in fields.items() for f in fs]
    outs = []
    ref = pkg.c_host.reference_dir()
    for hdr, extra in ((HEADER, []), (f"{ref}/src/core/backend.h", [f"-I{ref}/include", f"-I{ref}/src"])):
        src = tmp_path / "off.c"
        src.write_text(f'#include <stdio.h>\n#include <stddef.h>\n#include "{hdr}"\nint main(void){{{chr(10).join(lines)} return 0;}}\n')
        exe = tmp_path / "off"
        subprocess.run(["gcc", "-std=gnu11", *extra, str(src), "-o", str(exe)], check=True)
        outs.append(subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout)
    assert outs[0] == outs[1]


def test_create_default_without_gpu_reports_unsupported():
    lib = abi.load_library()
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    be = C.c_void_p()
    assert lib.gd_backend_create_default(C.byref(be)) == abi.GD_ERR_UNSUPPORTED and not be.value
    assert lib.gd_backend_name(None) == b"cuda-b200" and lib.gd_backend_kind_query(None) == 2
    with pytest.raises(abi.BackendError):
        pkg.runtime.Context()


def test_parameter_inventory_matches_the_reference_model():
    ref = g.GptConfig.reference_default()
    n = sum(int(np.prod(s)) for _, s, _ in g.param_specs(ref))
    assert n == 8_932_352                                  # examples/gpt_lm/README.md:12 "about 8.93M"
    base = g.GptConfig.baseline()
    nb = sum(int(np.prod(s)) for _, s, _ in g.param_specs(base))
    assert 12_300_000 < nb < 12_400_000
    assert len(g.param_specs(base)) == 1 + 10 * 3 + 3 and len(g.param_specs(ref)) == 1 + 10 * 3 + 2


def test_synthetic_batch_packing():
    cfg = g.GptConfig.baseline()
    b = g.synthetic_batch(cfg, 64, 64, 512, seed=3, pad_to=512)
    lens = np.diff(b.cu_seqlens)
    assert b.input_ids.size % 512 == 0 and b.cu_seqlens[0] == 0 and b.cu_seqlens[-1] == b.input_ids.size
    assert lens[:64].min() >= 64 and lens.max() <= 512 and b.real_tokens == lens[:64].sum()
    for s0, s1 in zip(b.cu_seqlens[:64], b.cu_seqlens[1:65]):
        assert np.array_equal(b.positions[s0:s1], np.arange(s1 - s0))
        assert np.array_equal(b.targets[s0:s1 - 1], b.input_ids[s0 + 1:s1]) and b.targets[s1 - 1] == -1
    assert np.all(b.targets[b.real_tokens:] == -1)          # padding rows are ignored by the loss
    assert b.input_ids.min() >= 0 and b.input_ids.max() < cfg.vocab_size


def test_lr_schedule_points():
    c = Golden("ref_ctest_optim")["lr_schedule"]
    got = [optim.gd_lr_scheduler_value(float(c["max_lr"]), float(c["min_lr"]), int(c["warmup"]), int(c["total"]), int(s)) for s in c["steps"]]
    np.testing.assert_allclose(got, c["values"], rtol=1e-6)


def test_dropout_site_seeds_follow_the_reference_formula():
    from oracle import gpt_lm as OG
    cfg = g.GptConfig.baseline()
    m = object.__new__(g.GptLm)
    m.cfg = cfg
    for layer in (0, 2):
        for step in (1, 77):
            want = OG.splitmix64((cfg.dropout_seed ^ g.GPT_DROPOUT_ATTN ^ (layer << 32) ^ step) & g.MASK64)
            assert m._site_seed(g.GPT_DROPOUT_ATTN, layer, step) == want


def test_balanced_shards_even_counts_and_tokens():
    lens = np.random.default_rng(5).integers(64, 513, size=64 * 8)
    shards = pkg.dp.balanced_shards(lens, 8)
    assert sorted(i for sh in shards for i in sh) == list(range(64 * 8))
    assert all(len(sh) == 64 for sh in shards)
    tokens = [int(sum(lens[i] for i in sh)) for sh in shards]
    strided = [int(sum(lens[i] for i in sh)) for sh in pkg.dp.split_global_batch(64 * 8, 8)]
    assert max(tokens) - min(tokens) <= 64                       # within one short sequence of each other
    assert max(tokens) - min(tokens) < max(strided) - min(strided)
    assert pkg.dp.balanced_shards([5, 9, 1], 2) == [[1], [0, 2]]   # odd count: the first ranks take the extra one


def _dp_worker(rank, world, port, q):
    """One data-parallel rank on CPU: the oracle computes this rank's gradients on its shard with the loss normalised
    by the valid rows of the GLOBAL batch (DataParallel.shard_share, counts summed over gloo), the gradients and the loss
    shares are summed over the ranks, and the result must equal ONE oracle step on the union batch."""
    import torch
    import torch.distributed as dist
    from oracle import gpt_lm as OG
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = g.GptConfig(vocab_size=64, context_length=16, d_model=32, n_layers=1, n_heads=2, head_dim=16, mlp_hidden=32,
                      tied_lm_head=False, dropout_p=0.0, sdpa_window=0)
    hp = g.init_params(cfg, seed=1)
    union = g.synthetic_batch(cfg, 5, 3, 16, seed=50)              # five sequences of unequal length: uneven shards
    shards = pkg.dp.split_global_batch(5, world)
    mine = g.take_sequences(union, shards[rank])
    dp = pkg.dp.DataParallel(None, None, rank, world, dist, connect=False)
    share = dp.shard_share(mine, cfg.pad_token_id)
    ref = OG.OracleGptLm(OG.config_from(cfg), hp)
    r = ref.loss_and_grads(mine.input_ids, mine.targets, mine.positions, mine.cu_seqlens, 1, share)   # d(share * local mean)
    names = sorted(r["grads"])
    flat = torch.cat([r["grads"][k].reshape(-1) for k in names] + [torch.tensor([r["loss"] * share], dtype=torch.float32)])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)                   # no division by world: the shares already add up
    w = OG.OracleGptLm(OG.config_from(cfg), hp).loss_and_grads(union.input_ids, union.targets, union.positions, union.cu_seqlens, 1, 1.0)
    want = torch.cat([w["grads"][k].reshape(-1) for k in names] + [torch.tensor([w["loss"]], dtype=torch.float32)])
    valid = int(np.count_nonzero(mine.targets >= 0))
    q.put((rank, float((flat - want).abs().max() / want.abs().max()), shards, share, valid))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_global_mean_over_two_gloo_ranks_equals_the_union_batch():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=240) for _ in procs]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    total = sum(r[4] for r in res)
    for rank, err, shards, share, valid in res:
        assert err < 2e-3            # F16 rounding points sit at differently scaled values on the two sides
        assert shards == [[0, 2, 4], [1, 3]]
        assert abs(share - valid / total) < 1e-12 and 0.0 < share < 1.0
    assert abs(sum(r[3] for r in res) - 1.0) < 1e-12
