"""Synthetic token datasets (no tokenizer, no download).

``synthetic_fixed`` mirrors the reference's ``_synthetic`` strategy
(src/axolotl/prompt_strategies/_synthetic.py:31-96): ``length`` rows of ``sequence_length`` uniform
ids in [min_input_id, max_input_id), labels == input ids. ``synthetic_varlen`` draws sample lengths
uniformly from a range and masks a leading fraction of each sample's labels, which is what the
benchmark configurations ask for.
"""
from __future__ import annotations

import numpy as np

IGNORE_INDEX = -100


class ListDataset:
    def __init__(self, rows):
        self.rows = rows

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]

    @property
    def lengths(self):
        return np.array([len(r["input_ids"]) for r in self.rows], dtype=np.int32)


def synthetic_fixed(length=1000, sequence_length=2048, min_input_id=100, max_input_id=32000, seed=None):
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(length):
        ids = rng.integers(min_input_id, max_input_id, size=sequence_length, dtype=np.int64)
        rows.append({"input_ids": ids, "labels": ids.copy(), "attention_mask": np.ones(sequence_length, dtype=np.int64)})
    return ListDataset(rows)


def synthetic_varlen(num_samples, min_len, max_len, vocab_lo=3, vocab_hi=32000, mask_prefix_frac=0.0, seed=0):
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(num_samples):
        n = int(rng.integers(min_len, max_len + 1))
        ids = rng.integers(vocab_lo, vocab_hi, size=n, dtype=np.int64)
        lab = ids.copy()
        k = int(n * mask_prefix_frac)
        if k:
            lab[:k] = IGNORE_INDEX
        rows.append({"input_ids": ids, "labels": lab, "position_ids": np.arange(n, dtype=np.int64), "length": n})
    return ListDataset(rows)
