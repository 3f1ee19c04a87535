"""CPU: the oracle's compact-record expansion (oracle/compact.py) against the golden vectors produced by the
reference's own transform (examples/gpt_lm/main.c:873-970 through tests/golden/make_golden.py), and, where the
reference tree was available at build time, against that transform directly on seeded records."""
import numpy as np
import pytest

from conftest import Golden
from oracle import compact, cref

GOLD = Golden("ref_compact_transform")


@pytest.mark.parametrize("name", GOLD.names())
def test_expand_record_matches_reference_transform(name):
    c = GOLD[name]
    ctx, vocab, pad, ims, ime = (int(x) for x in c["params"])
    if int(c["status"]) != 0:
        assert int(c["status"]) == -1                      # GD_ERR_INVALID_ARGUMENT
        with pytest.raises(compact.InvalidRecord):
            compact.expand_record(c["tokens"], c["segment_lengths"], ctx, vocab, pad, ims, ime)
        return
    ids, pos, tgt = compact.expand_record(c["tokens"], c["segment_lengths"], ctx, vocab, pad, ims, ime)
    np.testing.assert_array_equal(ids, c["input_ids"])
    np.testing.assert_array_equal(pos, c["positions"])
    np.testing.assert_array_equal(tgt, c["target_ids"])


def test_golden_set_covers_accepts_rejects_and_the_masked_tail():
    names = GOLD.names()
    assert len([n for n in names if n.startswith("valid")]) == 7 and len([n for n in names if n.startswith("bad_")]) == 6
    masked, kept = GOLD["tail_masked"], GOLD["tail_kept"]
    assert masked["target_ids"][-1] == 0 and kept["target_ids"][-1] == 5


def test_expand_batch_concatenates_records_and_accumulates_cu_seqlens():
    rng = np.random.default_rng(5)
    tokens = rng.integers(0, 50, size=(3, 9)).astype(np.uint16)
    segs = [[8], [3, 5], [1, 1, 6]]
    ids, tgt, pos, cu = compact.expand_batch(tokens, segs, 8, 50, 0, 1, 2)
    np.testing.assert_array_equal(cu, [0, 8, 11, 16, 17, 18, 24])
    np.testing.assert_array_equal(ids, tokens[:, :8].reshape(-1))
    np.testing.assert_array_equal(pos, [0, 1, 2, 3, 4, 5, 6, 7, 0, 1, 2, 0, 1, 2, 3, 4, 0, 0, 0, 1, 2, 3, 4, 5])
    want = tokens[:, 1:].astype(np.int32).reshape(-1)
    for i in (10, 16, 17):                                 # the last token of a document that is followed by another one
        want[i] = 0
    for r in range(3):
        if tokens[r, 7] == 2 and tokens[r, 8] == 1:
            want[r * 8 + 7] = 0
    np.testing.assert_array_equal(tgt, want)
    with pytest.raises(compact.InvalidRecord):
        compact.expand_batch(tokens, [[8], [3, 4], [1, 1, 6]], 8, 50, 0, 1, 2)


@pytest.mark.skipif(not cref.compact_available(), reason="oracle/_ref/ref_compact.so needs the reference tree at build time")
def test_oracle_matches_the_compiled_reference_transform_on_seeded_records():
    rc = cref.RefCompact()
    rng = np.random.default_rng(99)
    for trial in range(200):
        ctx = int(rng.choice([4, 16, 64, 512]))
        vocab = int(rng.choice([8, 320, 2048, 65536]))
        tokens = rng.integers(0, vocab + (2 if trial % 7 == 0 and vocab < 65535 else 0), size=ctx + 1).astype(np.uint16)
        n = int(rng.integers(1, min(ctx, 9) + 1))
        cuts = np.sort(rng.choice(np.arange(1, ctx), size=n - 1, replace=False)) if n > 1 else np.zeros(0, dtype=np.int64)
        seg = np.diff(np.concatenate([[0], cuts, [ctx]])).astype(np.int32)
        if trial % 11 == 0:
            seg[int(rng.integers(0, n))] += int(rng.choice([-1, 1]))
        pad, ims, ime = int(rng.integers(0, min(vocab, 4))), 1, 2
        if trial % 5 == 0:
            tokens[ctx - 1], tokens[ctx] = ime % vocab, ims % vocab
        st, ids, pos, tgt = rc.transform(tokens, seg, ctx, vocab, pad, ims, ime)
        if st != 0:
            with pytest.raises(compact.InvalidRecord):
                compact.expand_record(tokens, seg, ctx, vocab, pad, ims, ime)
            continue
        got = compact.expand_record(tokens, seg, ctx, vocab, pad, ims, ime)
        np.testing.assert_array_equal(got[0], ids)
        np.testing.assert_array_equal(got[1], pos)
        np.testing.assert_array_equal(got[2], tgt)
