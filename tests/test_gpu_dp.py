"""GPU, two devices: NCCL gradient all-reduce through the gdb200_dp_* entries, and lock-step
parameters after data-parallel train steps (native and Python hosts). Skipped on a one-GPU box;
the rank logic itself is covered on CPU by the gloo test in test_cpu_abi_host.py."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _n_gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, port, host, q):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        os.environ["GD_CUDA_DEVICE"] = str(rank)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        import torch  # first, so that both NCCL users bind the same libnccl
        import torch.distributed as dist
        import __graft_entry__ as graft
        dist.init_process_group("gloo", rank=rank, world_size=world)
        pkg = graft.load_package()
        g, abi = pkg.gpt_lm, pkg.abi
        ctx = pkg.runtime.Context(params_bytes=64 << 20, state_bytes=256 << 20, scratch_bytes=2 << 30, data_bytes=16 << 20)
        cfg = g.GptConfig(vocab_size=512, context_length=128, d_model=128, n_layers=2, n_heads=2, head_dim=64, mlp_hidden=256,
                          tied_lm_head=False, dropout_p=0.1, sdpa_window=0)
        model = g.GptLm(ctx, cfg, g.init_params(cfg, seed=4))
        dp = pkg.dp.DataParallel(ctx, model, rank, world, dist)
        # 1. a known buffer: rank r holds (r + 1) * x, the sum is 3 * x on both ranks
        x = (np.arange(10_000, dtype=np.float32) % 97) / 8.0
        ctx.begin_step()
        t = ctx.from_numpy(ctx.scratch, abi.F16, x * (rank + 1))
        ctx.check(ctx.lib.gdb200_dp_all_reduce(ctx.backend, t.buffer, t.offset, t.count, t.dtype), "all_reduce")
        ctx.check(ctx.lib.gdb200_dp_join(ctx.backend), "join")
        ctx.flush()
        got = t.read().astype(np.float32)
        ctx.end_step()
        ok_sum = bool(np.array_equal(got, (x * 3).astype(np.float16).astype(np.float32)))
        # 2. three train steps on different shards: parameters stay identical across ranks
        trainer = (g.NativeTrainer if host == "native" else g.Trainer)(model, g.TrainConfig.baseline(), dp=dp)
        losses = []
        for s in range(3):
            b = g.synthetic_batch(cfg, 4, 16, 128, seed=100 * (rank + 1) + s, pad_to=cfg.context_length)
            losses.append(float(trainer.train_batch(b).read()[()]))
        ctx.flush()
        flat = np.concatenate([p.read().view(np.uint16).reshape(-1) for p in model.param_list()])
        mine = torch.from_numpy(flat.astype(np.int32))
        both = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        q.put((rank, ok_sum, bool(torch.equal(both[0], both[1])), losses, None))
        dist.barrier()
        ctx.destroy()
        dist.destroy_process_group()
    except Exception as e:  # reported to the parent instead of a silent non-zero exit
        import traceback
        q.put((rank, False, False, [], traceback.format_exc()))
        raise


@pytest.mark.skipif(_n_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("host", ["native", "python"])
def test_two_rank_all_reduce_and_lockstep_parameters(host):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 1000) + (0 if host == "native" else 1)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, host, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=120)
    for rank, ok_sum, same, losses, err in res:
        assert err is None, err
        assert ok_sum, f"rank {rank}: all-reduced buffer is not 3x"
        assert same, f"rank {rank}: parameters diverged across ranks"
        assert all(np.isfinite(l) for l in losses)
    for p in procs:
        assert p.exitcode == 0
