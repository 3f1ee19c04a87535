"""CPU restatement of the reference's compact GPT-LM record expansion. TEST INFRASTRUCTURE ONLY.

A compact record holds `context_length + 1` little-endian u16 tokens and the I32 lengths of the documents
("segments") packed into it. The reference expands one record on the host per sample
(examples/gpt_lm/main.c:873-970), and the packed-sequence collate then concatenates the records of a batch and
generates cu_seqlens as the running sum of all segment lengths (src/dataset/gdds_dataset.c:2191-2224).

Pinned against the reference's own transform (compiled from the reference tree into
oracle/_ref/ref_compact.so) through tests/golden/ref_compact_transform.npz.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np


class InvalidRecord(ValueError):
    """The reference returns GD_ERR_INVALID_ARGUMENT for this input."""


def expand_record(tokens: np.ndarray, segment_lengths: Sequence[int], context_length: int, vocab_size: int, pad_id: int,
                  im_start_id: int, im_end_id: int):
    """One record -> (input_ids, positions, target_ids), each I32 [context_length] (main.c:873-970)."""
    tokens = np.asarray(tokens, dtype=np.uint16)
    seg = [int(x) for x in segment_lengths]
    if (context_length <= 0 or vocab_size <= 0 or pad_id < 0 or pad_id >= vocab_size or im_start_id < 0 or im_end_id < 0
            or tokens.shape != (context_length + 1,) or len(seg) <= 0 or len(seg) > context_length):   # main.c:891-916
        raise InvalidRecord("configuration or field shapes")
    t32 = tokens.astype(np.int32)
    if np.any(t32 >= vocab_size):                                   # main.c:934-939 (token and next token)
        raise InvalidRecord("token id outside the vocabulary")
    input_ids = t32[:-1].copy()
    target_ids = t32[1:].copy()
    positions = np.zeros(context_length, dtype=np.int32)
    offset = 0
    for ln in seg:                                                  # main.c:943-956
        if ln <= 0 or ln > context_length - offset:
            raise InvalidRecord("segment length")
        positions[offset:offset + ln] = np.arange(ln, dtype=np.int32)
        offset += ln
        if offset < context_length:
            target_ids[offset - 1] = pad_id                         # the next token belongs to another document
    if offset != context_length:                                    # main.c:957-959
        raise InvalidRecord("segment lengths do not cover the record")
    if input_ids[-1] == im_end_id and target_ids[-1] == im_start_id:   # main.c:960-963
        target_ids[-1] = pad_id
    return input_ids, positions, target_ids


def expand_batch(tokens: np.ndarray, segment_lengths: Sequence[Sequence[int]], context_length: int, vocab_size: int, pad_id: int,
                 im_start_id: int, im_end_id: int):
    """Records [R, context_length + 1] + per-record segment lengths -> the packed batch the model consumes:
    (input_ids, target_ids, positions) I32 [R * context_length] and cu_seqlens I32 [S + 1]."""
    tokens = np.asarray(tokens, dtype=np.uint16)
    ids, pos, tgt, lens = [], [], [], []
    for r in range(tokens.shape[0]):
        i, p, t = expand_record(tokens[r], segment_lengths[r], context_length, vocab_size, pad_id, im_start_id, im_end_id)
        ids.append(i)
        pos.append(p)
        tgt.append(t)
        lens.extend(int(x) for x in segment_lengths[r])
    cu = np.zeros(len(lens) + 1, dtype=np.int64)
    np.cumsum(np.asarray(lens, dtype=np.int64), out=cu[1:])         # gdds_dataset.c:2214-2222
    if cu[-1] > np.iinfo(np.int32).max:
        raise InvalidRecord("cu_seqlens overflow")
    return (np.concatenate(ids).astype(np.int32), np.concatenate(tgt).astype(np.int32), np.concatenate(pos).astype(np.int32),
            cu.astype(np.int32))
