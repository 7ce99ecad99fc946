"""Collators.

``PackedCollator`` concatenates the samples of each bin into one row, emits ``position_ids`` that
restart at 0 for every sample and pads the row to a multiple of 64 (or to ``sequence_len``):
labels with -100, input ids with the pad token, and position ids with ``0,1,2,...`` so the pad tail
reads as one more document -- the layout of the reference's V2 collator
(src/axolotl/utils/collators/batching.py:61-102, 158-196). Document boundaries travel as
``cu_seqlens`` (host array) so the attention kernels need no mask.
"""
from __future__ import annotations

import numpy as np
import torch

IGNORE_INDEX = -100


def _pad_len(n, multiple, fixed=None):
    if fixed is not None:
        return max(fixed, n) if multiple is None else ((max(fixed, n) + multiple - 1) // multiple) * multiple
    if multiple is None:
        return n
    return ((n + multiple - 1) // multiple) * multiple


class PackedCollator:
    def __init__(self, pad_token_id=0, pad_to_multiple_of=64, sequence_len=None, pad_to_sequence_len=False):
        self.pad_token_id = pad_token_id
        self.multiple = pad_to_multiple_of
        self.fixed = sequence_len if pad_to_sequence_len else None

    def __call__(self, bins):
        """bins: list (rows) of lists of samples; a sample is a dict with input_ids / labels
        (and optionally position_ids)."""
        rows_ids, rows_lab, rows_pos, cu_rows = [], [], [], []
        for samples in bins:
            ids = np.concatenate([np.asarray(s["input_ids"], dtype=np.int64) for s in samples])
            lab = np.concatenate([np.asarray(s.get("labels", s["input_ids"]), dtype=np.int64) for s in samples])
            pos = np.concatenate([np.asarray(s["position_ids"], dtype=np.int64) if "position_ids" in s
                                  else np.arange(len(s["input_ids"]), dtype=np.int64) for s in samples])
            rows_ids.append(ids)
            rows_lab.append(lab)
            rows_pos.append(pos)
        width = max(_pad_len(len(r), self.multiple, self.fixed) for r in rows_ids)
        B = len(rows_ids)
        input_ids = np.full((B, width), self.pad_token_id, dtype=np.int64)
        labels = np.full((B, width), IGNORE_INDEX, dtype=np.int64)
        position_ids = np.zeros((B, width), dtype=np.int64)
        for b in range(B):
            n = len(rows_ids[b])
            input_ids[b, :n] = rows_ids[b]
            labels[b, :n] = rows_lab[b]
            position_ids[b, :n] = rows_pos[b]
            position_ids[b, n:] = np.arange(width - n)
        flat_pos = position_ids.reshape(-1)
        starts = flat_pos == 0
        starts[np.arange(B) * width] = True
        cu = np.concatenate([np.flatnonzero(starts), [B * width]]).astype(np.int32)
        return {
            "input_ids": torch.from_numpy(input_ids),
            "labels": torch.from_numpy(labels),
            "position_ids": torch.from_numpy(position_ids.astype(np.int32)),
            "cu_seqlens": cu,
            "num_tokens": int(sum(len(r) for r in rows_ids)),
        }


class PaddedCollator:
    """Unpacked batches: right-pad every sample to the longest one (multiple of 64); each row is one
    document followed by a pad document (reference: DataCollatorForSeq2Seq,
    src/axolotl/utils/collators/batching.py:11-125)."""

    def __init__(self, pad_token_id=0, pad_to_multiple_of=64):
        self.inner = PackedCollator(pad_token_id, pad_to_multiple_of)

    def __call__(self, samples):
        return self.inner([[s] for s in samples])
