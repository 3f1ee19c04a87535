"""GPU: the device-side expansion of compact GPT-LM records (gdb200_gpt_compact_expand) against the golden
vectors of the reference's transform and against the CPU oracle, bit-exact (integer work)."""
import ctypes as C

import numpy as np
import pytest

from conftest import Golden
from gpu_util import abi, pkg
from oracle import compact

pytestmark = pytest.mark.gpu
g = pkg.gpt_lm
GOLD = Golden("ref_compact_transform")


def run_expand(ctx, tokens, seg, offs, ctx_len, vocab, pad, ims, ime):
    """Raw call through the C ABI; returns (status flags, ids, targets, positions, cu_seqlens)."""
    tokens = np.ascontiguousarray(tokens, dtype=np.uint16).reshape(-1, ctx_len + 1)
    seg, offs = np.asarray(seg, dtype=np.int32), np.asarray(offs, dtype=np.int32)
    n_rec, n_seg = tokens.shape[0], seg.size
    ctx.begin_step()
    try:
        t_tok = ctx.from_numpy(ctx.data, abi.U16, tokens.reshape(-1))
        t_seg = ctx.from_numpy(ctx.data, abi.I32, seg)
        t_off = ctx.from_numpy(ctx.data, abi.I32, offs)
        ids, tgt, pos = (ctx.empty(ctx.data, abi.I32, (n_rec * ctx_len,)) for _ in range(3))
        cu = ctx.empty(ctx.data, abi.I32, (n_seg + 1,))
        status = ctx.empty(ctx.data, abi.I32, (1,))
        b = abi.GptCompactBatch(ids.buffer, t_tok.offset, t_seg.offset, t_off.offset, ids.offset, tgt.offset, pos.offset, cu.offset,
                                status.offset, n_rec, n_seg, ctx_len, vocab, pad, ims, ime)
        ctx.check(ctx.lib.gdb200_gpt_compact_expand(ctx.backend, C.byref(b)), "gdb200_gpt_compact_expand")
        out = (int(status.read()[0]), ids.read(), tgt.read(), pos.read(), cu.read())
    finally:
        ctx.end_step()
    return out


@pytest.mark.parametrize("name", GOLD.names())
def test_single_records_match_the_reference_transform(gpu_ctx, name):
    c = GOLD[name]
    ctx_len, vocab, pad, ims, ime = (int(x) for x in c["params"])
    seg = c["segment_lengths"]
    flags, ids, tgt, pos, cu = run_expand(gpu_ctx, c["tokens"], seg, [0, seg.size], ctx_len, vocab, pad, ims, ime)
    if int(c["status"]) != 0:
        assert flags != 0
        want = {"bad_token": abi.COMPACT_BAD_TOKEN, "bad_extra_token": abi.COMPACT_BAD_TOKEN, "bad_zero_length": abi.COMPACT_BAD_LENGTH,
                "bad_negative_length": abi.COMPACT_BAD_LENGTH, "bad_short": abi.COMPACT_BAD_COVER, "bad_long": abi.COMPACT_BAD_COVER}[name]
        assert flags & want
        return
    assert flags == 0
    np.testing.assert_array_equal(ids, c["input_ids"])
    np.testing.assert_array_equal(pos, c["positions"])
    np.testing.assert_array_equal(tgt, c["target_ids"])
    np.testing.assert_array_equal(cu, np.concatenate([[0], np.cumsum(seg)]))


@pytest.mark.parametrize("n_rec,ctx_len,vocab,max_seg", [(1, 4, 8, 4), (5, 64, 320, 7), (64, 512, 2048, 6), (3, 512, 65536, 512),
                                                         (700, 16, 100, 16), (256, 512, 2048, 12)])
def test_batches_match_the_oracle(gpu_ctx, n_rec, ctx_len, vocab, max_seg):
    cfg = g.GptConfig(vocab_size=vocab, context_length=ctx_len, d_model=128, n_layers=1, n_heads=2, head_dim=64, mlp_hidden=192)
    cb = g.synthetic_compact_batch(cfg, n_rec, seed=n_rec * 31 + ctx_len, max_segments=max_seg)
    cb.tokens[::3, ctx_len - 1], cb.tokens[::3, ctx_len] = 2 % vocab, 1 % vocab      # some records end on <|im_end|> <|im_start|>
    per_rec = [cb.segment_lengths[cb.record_offsets[r]:cb.record_offsets[r + 1]] for r in range(n_rec)]
    want = compact.expand_batch(cb.tokens, per_rec, ctx_len, vocab, 0, 1, 2)
    flags, ids, tgt, pos, cu = run_expand(gpu_ctx, cb.tokens, cb.segment_lengths, cb.record_offsets, ctx_len, vocab, 0, 1, 2)
    assert flags == 0
    for got, exp in zip((ids, tgt, pos, cu), want):
        np.testing.assert_array_equal(got, exp)
    # size-independent properties: positions restart exactly at cu_seqlens, every document end but a record's last is masked
    assert np.all(pos[cu[:-1]] == 0) and np.all(np.diff(pos)[np.setdiff1d(np.arange(1, pos.size), cu[:-1]) - 1] == 1)
    inner_ends = np.setdiff1d(cu[1:] - 1, np.arange(n_rec) * ctx_len + ctx_len - 1)
    assert np.all(tgt[inner_ends] == 0)


def test_a_record_whose_own_lengths_fall_short_is_rejected_even_if_the_batch_adds_up(gpu_ctx):
    """[10, 20] + [34, 64] covers 2 x 64 tokens in total, but neither record is covered by its own lengths: the
    reference rejects both records (examples/gpt_lm/main.c:946,957)."""
    rng = np.random.default_rng(3)
    tokens = rng.integers(0, 320, size=(2, 65)).astype(np.uint16)
    for r, seg in enumerate(([10, 20], [34, 64])):
        with pytest.raises(compact.InvalidRecord):
            compact.expand_record(tokens[r], seg, 64, 320, 0, 1, 2)
    flags, *_ = run_expand(gpu_ctx, tokens, [10, 20, 34, 64], [0, 2, 4], 64, 320, 0, 1, 2)
    assert flags & abi.COMPACT_BAD_COVER
    flags, *_ = run_expand(gpu_ctx, tokens, [10, 54, 34, 30], [0, 2, 4], 64, 320, 0, 1, 2)
    assert flags == 0
    flags, *_ = run_expand(gpu_ctx, tokens, [10, 54, 34, 30], [0, 3, 4], 64, 320, 0, 1, 2)     # offsets disagree with the lengths
    assert flags & abi.COMPACT_BAD_COVER


def test_configuration_errors_return_invalid_argument(gpu_ctx):
    ctx = gpu_ctx
    b = abi.GptCompactBatch(ctx.data.buffer, 0, 1024, 2048, 4096, 8192, 12288, 16384, 20480, 1, 1, 64, 320, 0, 1, 2)
    lib = ctx.lib
    assert lib.gdb200_gpt_compact_expand(ctx.backend, C.byref(b)) == abi.GD_OK
    ctx.flush()
    for field, value in (("pad_id", 320), ("pad_id", -1), ("vocab_size", 0), ("vocab_size", 70000), ("context_length", 0), ("im_end_id", -1),
                         ("n_records", 0), ("n_segments", 0), ("n_segments", 65), ("tokens_offset", 1), ("cu_seqlens_offset", 2),
                         ("input_ids_offset", ctx.data.capacity - 8)):
        bad = abi.GptCompactBatch.from_buffer_copy(b)
        setattr(bad, field, value)
        assert lib.gdb200_gpt_compact_expand(ctx.backend, C.byref(bad)) == abi.GD_ERR_INVALID_ARGUMENT, field
    assert lib.gdb200_gpt_compact_expand(ctx.backend, None) == abi.GD_ERR_INVALID_ARGUMENT


def test_training_on_compact_records_equals_training_on_the_expanded_batch():
    cfg = g.GptConfig(vocab_size=320, context_length=64, d_model=128, n_layers=2, n_heads=2, head_dim=64, mlp_hidden=192,
                      tied_lm_head=False, dropout_p=0.1, sdpa_window=0, pad_token_id=0)
    tc = g.TrainConfig.baseline()
    hp = g.init_params(cfg, seed=8)
    cbs = [g.synthetic_compact_batch(cfg, 4, seed=40 + s) for s in range(3)]
    losses = {}
    for form in ("compact", "expanded"):
        with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
            trainer = g.NativeTrainer(g.GptLm(ctx, cfg, hp), tc)
            out = []
            for cb in cbs:
                if form == "compact":
                    out.append(float(trainer.train_batch(cb).read()[()]))
                else:
                    per_rec = [cb.segment_lengths[cb.record_offsets[r]:cb.record_offsets[r + 1]] for r in range(4)]
                    ids, tgt, pos, cu = compact.expand_batch(cb.tokens, per_rec, 64, 320, cfg.pad_token_id, cb.im_start_id, cb.im_end_id)
                    out.append(float(trainer.train_batch(g.Batch(ids, tgt, pos, cu, real_tokens=ids.size)).read()[()]))
            losses[form] = out
    assert losses["compact"][0] == losses["expanded"][0]            # same kernels on the same device inputs
    np.testing.assert_allclose(losses["compact"], losses["expanded"], rtol=2e-4)
    # invalid records surface as the reference's status when the host asks for the check
    with pkg.runtime.Context(params_bytes=64 << 20, state_bytes=128 << 20, scratch_bytes=1 << 30) as ctx:
        model = g.GptLm(ctx, cfg, hp)
        bad = g.synthetic_compact_batch(cfg, 2, seed=1)
        bad.tokens[1, 7] = 999
        ctx.begin_step()
        with pytest.raises(abi.BackendError) as e:
            model.expand_compact_batch(bad)
        ctx.end_step()
        assert e.value.status == abi.GD_ERR_INVALID_ARGUMENT
