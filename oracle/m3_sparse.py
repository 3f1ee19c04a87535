"""CPU restatement of the reference's MiniMax-M3 block-sparse attention. TEST INFRASTRUCTURE ONLY.

Follows src/ops/minimax_m3_index_topk/metal_minimax_m3_index_topk.metal:21-136 (block selection) and
src/ops/minimax_m3_sparse_attention/metal_minimax_m3_sparse_attention.metal:36-113 (forward), :263-363 (dQ and
statistics), :365-481 (dK / dV). Arithmetic in float64 on the given (already rounded) inputs.

Pinned against the CPU references that the reference's own test carries (tests/test_minimax_m3_sparse_attention.c:
145-213, 423-600, compiled into oracle/_ref/ref_harness.so) through tests/golden/ref_m3_sparse.npz.
"""
from __future__ import annotations

import numpy as np


def index_topk(q: np.ndarray, k: np.ndarray, cu: np.ndarray, block_size: int, topk: int, init_blocks: int, local_blocks: int) -> np.ndarray:
    """q, k: [N, H, Dh] index heads. Returns I32 [H, N, topk]: selected sequence-local block ids, -1 padded."""
    n, h, _ = q.shape
    q64, k64 = q.astype(np.float64), k.astype(np.float64)
    out = np.full((h, n, topk), -1, dtype=np.int32)
    for b in range(len(cu) - 1):
        start, t_len = int(cu[b]), int(cu[b + 1] - cu[b])
        for hh in range(h):
            scores = q64[start:start + t_len, hh] @ k64[start:start + t_len, hh].T          # [i, j]
            for i in range(t_len):
                valid = (i + block_size) // block_size
                local_start = max(0, valid - local_blocks)
                best_s, best_i = [-np.inf] * topk, [-1] * topk
                for blk in range(valid):
                    k0, k1 = blk * block_size, min(blk * block_size + block_size, t_len, i + 1)
                    s = scores[i, k0:k1].max() if k1 > k0 else -np.inf
                    if np.isnan(s):
                        s = -np.inf
                    if blk < init_blocks:
                        s = 1.0e30
                    if local_blocks > 0 and blk >= local_start:
                        s = 1.0e29
                    for slot in range(topk):
                        if s > best_s[slot]:                      # strict: an equal later block does not displace
                            best_s[slot + 1:] = best_s[slot:-1]
                            best_i[slot + 1:] = best_i[slot:-1]
                            best_s[slot], best_i[slot] = s, blk
                            break
                for t in range(topk):
                    out[hh, start + i, t] = best_i[t] if t < valid else -1
    return out


def _selected_keys(sel: np.ndarray, i: int, t_len: int, block_size: int) -> np.ndarray:
    keys = []
    for blk in sel:
        if blk >= 0:
            keys.extend(range(int(blk) * block_size, min(int(blk) * block_size + block_size, t_len, i + 1)))
    return np.asarray(keys, dtype=np.int64)


def forward(q, k, v, cu, topk_idx, block_size: int, scale: float) -> np.ndarray:
    """q [N, Hq, Dh], k / v [N, Hkv, Dh], topk_idx [Hkv, N, topk] -> out [N, Hq, Dh] (float64)."""
    n, hq, dh = q.shape
    group = hq // k.shape[1]
    q64, k64, v64 = q.astype(np.float64), k.astype(np.float64), v.astype(np.float64)
    out = np.zeros((n, hq, dh))
    for b in range(len(cu) - 1):
        start, t_len = int(cu[b]), int(cu[b + 1] - cu[b])
        for h in range(hq):
            hk = h // group
            for i in range(t_len):
                keys = _selected_keys(topk_idx[hk, start + i], i, t_len, block_size)
                if keys.size == 0:
                    continue
                s = (k64[start + keys, hk] @ q64[start + i, h]) * scale
                p = np.exp(s - s.max())
                out[start + i, h] = (p / p.sum()) @ v64[start + keys, hk]
    return out


def backward(go, q, k, v, cu, topk_idx, block_size: int, scale: float):
    """Returns (dq [N, Hq, Dh], dk, dv [N, Hkv, Dh]) in float64."""
    n, hq, dh = q.shape
    group = hq // k.shape[1]
    q64, k64, v64, g64 = (a.astype(np.float64) for a in (q, k, v, go))
    dq, dk, dv = np.zeros_like(q64), np.zeros_like(k64), np.zeros_like(v64)
    for b in range(len(cu) - 1):
        start, t_len = int(cu[b]), int(cu[b + 1] - cu[b])
        for h in range(hq):
            hk = h // group
            for i in range(t_len):
                keys = _selected_keys(topk_idx[hk, start + i], i, t_len, block_size)
                if keys.size == 0:
                    continue
                kk, vv = k64[start + keys, hk], v64[start + keys, hk]
                s = (kk @ q64[start + i, h]) * scale
                p = np.exp(s - s.max())
                p /= p.sum()
                dp = vv @ g64[start + i, h]
                ds = p * (dp - float(p @ dp))
                dq[start + i, h] = scale * (ds @ kk)
                np.add.at(dk[:, hk], start + keys, scale * ds[:, None] * q64[start + i, h][None, :])
                np.add.at(dv[:, hk], start + keys, p[:, None] * g64[start + i, h][None, :])
    return dq, dk, dv
