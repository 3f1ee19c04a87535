"""CPU: the oracle's MiniMax-M3 sparse attention (oracle/m3_sparse.py) against golden vectors produced by the CPU
references of the reference's own test (tests/test_minimax_m3_sparse_attention.c through tests/golden/make_golden.py)."""
import numpy as np
import pytest

from conftest import Golden, f16_bits_to_f32
from oracle import m3_sparse

GOLD = Golden("ref_m3_sparse")


@pytest.mark.parametrize("name", GOLD.names())
def test_block_selection_forward_backward_match_reference(name):
    c = GOLD[name]
    block, topk, init_b, local_b = (int(x) for x in c["params"])
    q, k, v, go, iq, ik = (f16_bits_to_f32(c[x]) for x in ("q", "k", "v", "go", "iq", "ik"))
    tk = m3_sparse.index_topk(iq, ik, c["cu"], block, topk, init_b, local_b)
    np.testing.assert_array_equal(tk, c["topk"])
    out = m3_sparse.forward(q, k, v, c["cu"], c["topk"], block, float(c["scale"]))
    np.testing.assert_allclose(out, c["out"], atol=2e-6, rtol=1e-5)
    dq, dk, dv = m3_sparse.backward(go, q, k, v, c["cu"], c["topk"], block, float(c["scale"]))
    for got, want in ((dq, c["dq"]), (dk, c["dk"]), (dv, c["dv"])):
        np.testing.assert_allclose(got, want, atol=1e-5, rtol=1e-4)


def test_selection_keeps_forced_blocks_and_pads_short_prefixes():
    c = GOLD["seeded_gqa"]
    block, topk, init_b, local_b = (int(x) for x in c["params"])
    tk, cu = c["topk"], c["cu"]
    for b in range(len(cu) - 1):
        for i in range(int(cu[b + 1] - cu[b])):
            valid = (i + block) // block
            row = tk[0, cu[b] + i]
            assert np.count_nonzero(row >= 0) == min(valid, topk)
            assert row[0] == 0                                        # the initial block always ranks first
            if valid > 1:
                assert valid - 1 in row                               # the query's own (local) block is kept
            assert len(set(row[row >= 0].tolist())) == np.count_nonzero(row >= 0)
