"""ctypes access to the oracle's native checkers. TEST INFRASTRUCTURE ONLY.

liboracle_int.so  : plain-C restatement of the integer / byte-exact pieces (oracle/c/oracle_int.c).
_ref/ref_harness.so: the CPU reference functions of the reference's own C tests, compiled from the
                     reference tree (only present where that tree was available at build time).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
INT_LIB = os.path.join(HERE, "c", "liboracle_int.so")
HARNESS_LIB = os.path.join(HERE, "_ref", "ref_harness.so")
COMPACT_LIB = os.path.join(HERE, "_ref", "ref_compact.so")
TESTS_CUDA_DIR = os.path.join(HERE, "_ref", "tests_cuda")


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class OracleInt:
    def __init__(self):
        self.lib = C.CDLL(INT_LIB)
        self.lib.oracle_splitmix64.restype = C.c_uint64
        self.lib.oracle_splitmix64.argtypes = [C.c_uint64]
        self.lib.oracle_dropout_threshold.restype = C.c_uint32
        self.lib.oracle_dropout_threshold.argtypes = [C.c_float]
        self.lib.oracle_dropout_mask.argtypes = [C.c_void_p, C.c_uint64, C.c_float, C.c_uint64]
        self.lib.oracle_mask_allowed.argtypes = [C.c_int] * 5
        self.lib.oracle_kv_append_packed.argtypes = [C.c_void_p] * 6 + [C.c_uint32] * 3
        self.lib.oracle_kv_append.argtypes = [C.c_void_p] * 5 + [C.c_int32] + [C.c_uint32] * 4
        self.lib.oracle_argmax_first.restype = C.c_int32
        self.lib.oracle_argmax_first.argtypes = [C.c_void_p, C.c_uint32]
        self.lib.oracle_embedding_rows.argtypes = [C.c_void_p] * 3 + [C.c_uint32] * 3

    def splitmix64(self, x: int) -> int:
        return int(self.lib.oracle_splitmix64(x & 0xFFFFFFFFFFFFFFFF))

    def dropout_mask(self, count: int, p: float, seed: int) -> np.ndarray:
        out = np.empty(count, dtype=np.uint8)
        self.lib.oracle_dropout_mask(_p(out), count, p, seed & 0xFFFFFFFFFFFFFFFF)
        return out

    def mask_allowed(self, i: int, j: int, causal: int, window: int, prefix: int) -> int:
        return int(self.lib.oracle_mask_allowed(i, j, causal, window, prefix))

    def kv_append_packed(self, kc, vc, kn, vn, pos, cu, row_bytes: int) -> None:
        self.lib.oracle_kv_append_packed(_p(kc), _p(vc), _p(kn), _p(vn), _p(pos), _p(cu), kc.shape[0], kc.shape[1], row_bytes)

    def kv_append(self, kc, vc, kn, vn, pos, scalar_pos: int, tnew: int, row_bytes: int) -> None:
        self.lib.oracle_kv_append(_p(kc), _p(vc), _p(kn), _p(vn), _p(pos) if pos is not None else None, scalar_pos,
                                  kc.shape[0], tnew, kc.shape[1], row_bytes)

    def argmax_first(self, logits: np.ndarray) -> int:
        a = np.ascontiguousarray(logits, dtype=np.float32)
        return int(self.lib.oracle_argmax_first(_p(a), a.size))

    def embedding_rows(self, table: np.ndarray, ids: np.ndarray) -> np.ndarray:
        out = np.empty((ids.size, table.shape[1]), dtype=np.uint16)
        self.lib.oracle_embedding_rows(_p(table), _p(ids), _p(out), ids.size, table.shape[0], table.shape[1])
        return out


def harness_available() -> bool:
    return os.path.exists(HARNESS_LIB)


def compact_available() -> bool:
    return os.path.exists(COMPACT_LIB)


class RefCompact:
    """The reference's own compact-record transform (examples/gpt_lm/main.c:873-970), see
    oracle/ref_harness/harness_compact.c."""

    def __init__(self):
        self.lib = C.CDLL(COMPACT_LIB)
        i32, vp = C.c_int32, C.c_void_p
        self.lib.gdref_compact_transform.restype = C.c_int
        self.lib.gdref_compact_transform.argtypes = [vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, vp]

    def transform(self, tokens: np.ndarray, segment_lengths, context_length: int, vocab_size: int, pad_id: int, im_start_id: int,
                  im_end_id: int):
        """Returns (status, input_ids, positions, target_ids); the arrays are None unless status is 0 (GD_OK)."""
        tok = np.ascontiguousarray(tokens, dtype=np.uint16)
        seg = np.ascontiguousarray(segment_lengths, dtype=np.int32)
        assert tok.size == context_length + 1
        ids, pos, tgt = (np.zeros(context_length, dtype=np.int32) for _ in range(3))
        st = int(self.lib.gdref_compact_transform(_p(tok), context_length, _p(seg), seg.size, vocab_size, pad_id, im_start_id, im_end_id,
                                                  _p(ids), _p(pos), _p(tgt)))
        return (st, ids, pos, tgt) if st == 0 else (st, None, None, None)


class RefHarness:
    """CPU references embedded in the reference's C tests (see oracle/ref_harness/*.c)."""

    def __init__(self):
        self.lib = C.CDLL(HARNESS_LIB)
        f, u32, i32 = C.c_float, C.c_uint32, C.c_int
        vp = C.c_void_p
        self.lib.gdref_allowed.argtypes = [i32] * 5
        self.lib.gdref_fill_tokens.argtypes = [vp, u32, f]
        self.lib.gdref_varlen_fwd.argtypes = [vp] * 4 + [u32] * 4 + [f, i32, i32, i32, vp]
        self.lib.gdref_varlen_bwd.argtypes = [vp] * 5 + [u32] * 4 + [f, i32, i32, i32, vp, vp, vp]
        self.lib.gdref_decode.argtypes = [vp] * 3 + [i32] + [u32] * 6 + [f, i32, i32, vp]
        self.lib.gdref_lmce_dims.argtypes = [vp] * 3
        self.lib.gdref_lmce_fill.argtypes = [vp] * 3
        self.lib.gdref_lmce_oracle.argtypes = [vp] * 4 + [f] + [vp] * 4
        self.lib.gdref_rope.argtypes = [vp] * 4 + [u32, f, C.c_int32, i32, f]
        self.lib.gdref_rms.argtypes = [vp] * 3 + [u32, u32, f, vp, vp, vp]
        if hasattr(self.lib, "gdref_m3_topk"):
            self.lib.gdref_m3_topk.argtypes = [vp] * 3 + [u32] * 7 + [vp]
            self.lib.gdref_m3_fwd.argtypes = [vp] * 5 + [u32] * 6 + [f, vp]
            self.lib.gdref_m3_bwd.argtypes = [vp] * 6 + [u32] * 6 + [f, vp, vp, vp]

    def fill_tokens(self, count: int, base: float) -> np.ndarray:
        out = np.empty(count, dtype=np.uint16)
        self.lib.gdref_fill_tokens(_p(out), count, base)
        return out

    def varlen_fwd(self, q, k, v, cu, hq, hkv, dh, scale, causal, window, prefix) -> np.ndarray:
        out = np.zeros(int(cu[-1]) * hq * dh, dtype=np.float32)
        self.lib.gdref_varlen_fwd(_p(q), _p(k), _p(v), _p(cu), len(cu) - 1, hq, hkv, dh, scale, causal, window, prefix, _p(out))
        return out.reshape(int(cu[-1]), hq, dh)

    def varlen_bwd(self, go, q, k, v, cu, hq, hkv, dh, scale, causal, window, prefix):
        n = int(cu[-1])
        dq = np.zeros(n * hq * dh, dtype=np.float32)
        dk = np.zeros(n * hkv * dh, dtype=np.float32)
        dv = np.zeros(n * hkv * dh, dtype=np.float32)
        self.lib.gdref_varlen_bwd(_p(go), _p(q), _p(k), _p(v), _p(cu), len(cu) - 1, hq, hkv, dh, scale, causal, window, prefix,
                                  _p(dq), _p(dk), _p(dv))
        return dq.reshape(n, hq, dh), dk.reshape(n, hkv, dh), dv.reshape(n, hkv, dh)

    def decode(self, q, k, v, cache_pos, b, tq, tmax, hq, hkv, dh, scale, window, prefix) -> np.ndarray:
        out = np.zeros(b * tq * hq * dh, dtype=np.float32)
        self.lib.gdref_decode(_p(q), _p(k), _p(v), cache_pos, b, tq, tmax, hq, hkv, dh, scale, window, prefix, _p(out))
        return out.reshape(b, tq, hq, dh)

    def lmce_case(self, targets: np.ndarray, cap: float, with_bias: bool):
        r, d, v = C.c_int(), C.c_int(), C.c_int()
        self.lib.gdref_lmce_dims(C.byref(r), C.byref(d), C.byref(v))
        rows, dim, vocab = r.value, d.value, v.value
        hidden = np.empty(rows * dim, dtype=np.uint16)
        weight = np.empty(vocab * dim, dtype=np.uint16)
        bias = np.empty(vocab, dtype=np.uint16)
        self.lib.gdref_lmce_fill(_p(hidden), _p(weight), _p(bias))
        loss = np.zeros(1, dtype=np.float32)
        dh = np.zeros(rows * dim, dtype=np.uint16)
        dw = np.zeros(vocab * dim, dtype=np.uint16)
        db = np.zeros(vocab, dtype=np.uint16)
        t = np.ascontiguousarray(targets, dtype=np.int32)
        assert t.size == rows
        self.lib.gdref_lmce_oracle(_p(hidden), _p(weight), _p(bias) if with_bias else None, _p(t), cap, _p(loss), _p(dh), _p(dw),
                                   _p(db) if with_bias else None)
        return dict(hidden=hidden.reshape(rows, dim), weight=weight.reshape(vocab, dim), bias=bias, loss=loss[0],
                    dh=dh.reshape(rows, dim), dw=dw.reshape(vocab, dim), db=db)

    def rope(self, x: np.ndarray, pos: np.ndarray, theta: float, n_dims: int, interleaved: bool, sin_sign: float) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros_like(x)
        shape = np.asarray(x.shape, dtype=np.int64)
        self.lib.gdref_rope(_p(x), _p(np.ascontiguousarray(pos, dtype=np.int32)), _p(out), _p(shape), x.ndim, theta, n_dims,
                            1 if interleaved else 0, sin_sign)
        return out

    def rms(self, x: np.ndarray, w: np.ndarray, g: np.ndarray, eps: float):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        out, dx, dw = np.zeros_like(x), np.zeros_like(x), np.zeros(cols, dtype=np.float32)
        self.lib.gdref_rms(_p(x), _p(np.ascontiguousarray(w, dtype=np.float32)), _p(np.ascontiguousarray(g, dtype=np.float32)),
                           rows, cols, eps, _p(out), _p(dx), _p(dw))
        return out, dx, dw

    # MiniMax-M3 sparse attention references of tests/test_minimax_m3_sparse_attention.c (F16 bit patterns in, FP32 out)
    def m3_topk(self, q_bits, k_bits, cu, block_size: int, topk: int, init_blocks: int, local_blocks: int) -> np.ndarray:
        n, h, dh = q_bits.shape
        out = np.zeros((h, n, topk), dtype=np.int32)
        cu = np.ascontiguousarray(cu, dtype=np.int32)
        self.lib.gdref_m3_topk(_p(np.ascontiguousarray(q_bits)), _p(np.ascontiguousarray(k_bits)), _p(cu), len(cu) - 1, h, dh, block_size, topk,
                               init_blocks, local_blocks, _p(out))
        return out

    def m3_forward(self, q_bits, k_bits, v_bits, cu, topk_idx, block_size: int, scale: float) -> np.ndarray:
        n, hq, dh = q_bits.shape
        out = np.zeros((n, hq, dh), dtype=np.float32)
        cu, tk = np.ascontiguousarray(cu, dtype=np.int32), np.ascontiguousarray(topk_idx, dtype=np.int32)
        self.lib.gdref_m3_fwd(_p(np.ascontiguousarray(q_bits)), _p(np.ascontiguousarray(k_bits)), _p(np.ascontiguousarray(v_bits)), _p(cu), _p(tk),
                              len(cu) - 1, hq, k_bits.shape[1], dh, block_size, tk.shape[2], scale, _p(out))
        return out

    def m3_backward(self, go_bits, q_bits, k_bits, v_bits, cu, topk_idx, block_size: int, scale: float):
        n, hq, dh = q_bits.shape
        hkv = k_bits.shape[1]
        dq = np.zeros((n, hq, dh), dtype=np.float32)
        dk, dv = np.zeros((n, hkv, dh), dtype=np.float32), np.zeros((n, hkv, dh), dtype=np.float32)
        cu, tk = np.ascontiguousarray(cu, dtype=np.int32), np.ascontiguousarray(topk_idx, dtype=np.int32)
        self.lib.gdref_m3_bwd(_p(np.ascontiguousarray(go_bits)), _p(np.ascontiguousarray(q_bits)), _p(np.ascontiguousarray(k_bits)),
                              _p(np.ascontiguousarray(v_bits)), _p(cu), _p(tk), len(cu) - 1, hq, hkv, dh, block_size, tk.shape[2], scale,
                              _p(dq), _p(dk), _p(dv))
        return dq, dk, dv
