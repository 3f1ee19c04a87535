"""CPU: failure detection of the data-parallel path, with the failures made on the host (nothing here needs or faults a
GPU): the polling loop behind gdb200_dp_join driven by stub callbacks (completion, a reported communicator error, a
timeout), and gloo ranks whose launcher disagrees with the process group, who leave between steps, or of whom one alone
overflows."""
import ctypes as C
import os
import time

import numpy as np
import pytest

from conftest import graft

pkg = graft.load_package()
abi, g = pkg.abi, pkg.gpt_lm
CB = C.CFUNCTYPE(C.c_int, C.c_void_p)


def wait_with(completed, failed, timeout_ms):
    lib = abi.load_library()
    reason = C.c_int32(-1)
    c1, c2 = CB(completed), CB(failed) if failed is not None else None
    st = lib.gdb200_dp_wait_with(C.cast(c1, C.c_void_p), C.cast(c2, C.c_void_p) if c2 is not None else None, None, timeout_ms, C.byref(reason))
    return st, reason.value


def test_join_wait_completes_reports_errors_and_times_out():
    polls = {"n": 0}

    def done_after_three(_):
        polls["n"] += 1
        return 1 if polls["n"] >= 3 else 0

    assert wait_with(done_after_three, lambda _: 0, 1000) == (abi.GD_OK, 0) and polls["n"] == 3
    # the communicator reports an asynchronous error: the wait ends at once, whatever the completion query says
    assert wait_with(lambda _: 0, lambda _: 1, 5000) == (abi.GD_ERR_INTERNAL, 1)
    # a peer that never joins: the wait gives up after the limit, not earlier and not much later
    t0 = time.perf_counter()
    st, reason = wait_with(lambda _: 0, lambda _: 0, 150)
    dt = time.perf_counter() - t0
    assert (st, reason) == (abi.GD_ERR_INTERNAL, 2) and 0.14 <= dt < 2.0
    assert wait_with(lambda _: 1, None, 10) == (abi.GD_OK, 0)


def _worker(rank, world, port, case, q):
    try:
        import torch
        import torch.distributed as dist
        from oracle import gpt_lm as OG
        from oracle import ops as O
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = None
        if case == "mismatch":
            # the launcher believes in three ranks, the process group has two: refused before anything is enqueued
            try:
                pkg.dp.DataParallel(None, None, rank, 3, dist, connect=False)
                out = "accepted"
            except ValueError as e:
                out = "refused: " + str(e)
        elif case == "leave":
            dp = pkg.dp.DataParallel(None, None, rank, world, dist, connect=False)
            steps = 0
            t = torch.ones(4)
            for step in range(3):
                dist.barrier()                     # the host-side point between two steps
                if rank == 1 and step == 1:
                    dp.announce_leave()            # leaves between steps, nothing in flight
                    dist.barrier()
                    break
                if step == 1:
                    dist.barrier()                 # rank 1 has announced by now
                try:
                    dp.check_peers()
                except pkg.dp.PeerLeft as e:
                    out = ("stopped", e.ranks, steps)
                    break
                dist.all_reduce(t)                 # the step's collective: never entered once a peer has left
                steps += 1
            if out is None:
                out = ("left", [], steps) if rank == 1 else ("ran", [], steps)
        elif case == "found_inf":
            cfg = g.GptConfig(vocab_size=64, context_length=16, d_model=32, n_layers=1, n_heads=2, head_dim=16, mlp_hidden=32,
                              tied_lm_head=False, dropout_p=0.0, sdpa_window=0)
            hp = g.init_params(cfg, seed=2)
            b = g.synthetic_batch(cfg, 2, 6, 16, seed=70 + rank)
            ref = OG.OracleGptLm(OG.config_from(cfg), hp)
            grads = ref.loss_and_grads(b.input_ids, b.targets, b.positions, b.cu_seqlens, 1, 65536.0)["grads"]
            names = sorted(grads)
            flat = torch.cat([grads[k].reshape(-1) for k in names])
            if rank == 1:
                flat[7] = float("inf")             # overflow on ONE rank only
            dist.all_reduce(flat)                  # the sum carries the overflow to every rank
            pieces, o = [], 0
            for k in names:
                n = grads[k].numel()
                pieces.append(flat[o:o + n].reshape(grads[k].shape))
                o += n
            _, _, found = O.grad_clip_scale(pieces, 1.0 / 65536.0, 1.0)
            out = bool(found)
        q.put((rank, out, None))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, None, traceback.format_exc()))
        raise


def _run(case):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 500) + {"mismatch": 0, "leave": 1, "found_inf": 2}[case] * 7
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = sorted(q.get(timeout=180) for _ in procs)
        for p in procs:
            p.join(timeout=60)
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    for rank, out, err in res:
        assert err is None, err
    return [out for _, out, _ in res]


def test_world_size_mismatch_is_refused_on_every_rank():
    outs = _run("mismatch")
    assert all(o.startswith("refused") and "does not match the process group" in o for o in outs), outs


def test_a_rank_that_leaves_between_steps_stops_its_peer_before_the_next_collective():
    r0, r1 = _run("leave")
    assert r1 == ("left", [], 1)                   # rank 1 ran one step, announced, left
    assert r0 == ("stopped", [1], 1)               # rank 0 ran that step, saw the announcement, entered no further collective


def test_overflow_on_one_rank_makes_every_rank_skip_the_update():
    assert _run("found_inf") == [True, True]
