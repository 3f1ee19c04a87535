"""GPU, two devices: NCCL gradient all-reduce through the gdb200_dp_* entries, lock-step parameters after
data-parallel train steps (native and Python hosts), and parity of a two-rank step with a one-GPU step on the
union batch (global loss normaliser). Skipped on a one-GPU box; there the normaliser is covered by
test_gpu_gpt_lm.py (shards stepped one after the other) and the rank logic by the gloo test in test_cpu_abi_host.py."""
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
        # 3. one step on the two halves of a batch == one step of ONE rank on the whole batch (global loss normaliser):
        #    the reduced gradients and the reported loss are compared with a single-GPU step computed afterwards
        cfg2 = g.GptConfig(vocab_size=512, context_length=128, d_model=128, n_layers=2, n_heads=2, head_dim=64, mlp_hidden=256,
                           tied_lm_head=False, dropout_p=0.0, sdpa_window=0)
        hp2 = g.init_params(cfg2, seed=9)
        union = g.synthetic_batch(cfg2, 6, 16, 128, seed=321)
        half = g.take_sequences(union, [0, 2, 4] if rank == 0 else [1, 3, 5], pad_to=128, context_length=128)
        m2 = g.GptLm(ctx, cfg2, hp2)
        dp2 = pkg.dp.DataParallel(ctx, m2, rank, world, dist, connect=False)     # the communicator of step 2 is still attached
        t2 = (g.NativeTrainer if host == "native" else g.Trainer)(m2, g.TrainConfig.baseline(), dp=dp2)
        if host == "native":
            dp_loss = float(t2.train_batch(half).read()[()])
            dp_grads = g.native_step_gradients(t2)
        else:
            ctx.begin_step()
            t2.optimizer.zero_grad()
            ids, tgt, pos, cu = m2.upload_batch(half)
            share = dp2.shard_share(half, cfg2.pad_token_id)
            lt = m2.forward(ids, tgt, pos, cu, 1, share)
            pkg.optim.gd_backward_amp(ctx, lt, t2.scaler)
            dp2.reduce_gradients(t2.optimizer, lt)
            ctx.flush()
            dp_loss = float(lt.read()[()])
            dp_grads = {n: p.grad.read_f32() for n, p in m2.params.items()}
            ctx.end_step()
        dist.barrier()
        parity = None
        ctx1 = pkg.runtime.Context(params_bytes=64 << 20, state_bytes=256 << 20, scratch_bytes=2 << 30, data_bytes=16 << 20)
        t1 = g.NativeTrainer(g.GptLm(ctx1, cfg2, hp2), g.TrainConfig.baseline())
        whole = g.take_sequences(union, list(range(6)), pad_to=128, context_length=128)
        one_loss = float(t1.train_batch(whole).read()[()])
        one_grads = g.native_step_gradients(t1)
        worst = max(float(np.abs(dp_grads[n].reshape(one_grads[n].shape) - one_grads[n]).max() / (np.abs(one_grads[n]).max() + 1e-6)) for n in one_grads)
        parity = (dp_loss, one_loss, worst)
        ctx1.destroy()
        q.put((rank, ok_sum, bool(torch.equal(both[0], both[1])), losses, None, parity))
        dist.barrier()
        ctx.destroy()
        dist.destroy_process_group()
    except Exception as e:  # reported to the parent instead of a silent non-zero exit
        import traceback
        q.put((rank, False, False, [], traceback.format_exc(), None))
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
    try:
        res = [q.get(timeout=300) for _ in procs]
        for p in procs:
            p.join(timeout=120)
    finally:
        for p in procs:            # a rank that failed before a collective leaves its peer waiting inside it
            if p.is_alive():
                p.kill()
    for rank, ok_sum, same, losses, err, parity in res:
        assert err is None, err
        assert ok_sum, f"rank {rank}: all-reduced buffer is not 3x"
        assert same, f"rank {rank}: parameters diverged across ranks"
        assert all(np.isfinite(l) for l in losses)
        dp_loss, one_loss, worst = parity
        assert abs(dp_loss - one_loss) <= 1e-5 * abs(one_loss), (dp_loss, one_loss)     # every rank reports the global mean
        assert worst <= 1e-2, worst                                                     # reduced gradients == one-GPU gradients
    for p in procs:
        assert p.exitcode == 0
