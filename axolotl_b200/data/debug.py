"""Coloured token / label dumps for ``preprocess --debug`` (src/axolotl/utils/tokenization.py:10-120)."""
from __future__ import annotations


def print_samples(ds, cfg, n=3, tokenizer=None):
    if tokenizer is None and cfg.get("base_model"):
        try:
            from .tokenizer import load_tokenizer

            tokenizer = load_tokenizer(cfg)
        except Exception:
            tokenizer = None
    for i in range(min(n, len(ds))):
        row = ds[i]
        parts = []
        for t, l in zip(row["input_ids"].tolist(), row["labels"].tolist()):
            text = tokenizer.decode([t]) if tokenizer is not None else str(t)
            colour = "\033[32m" if l != -100 else "\033[31m"
            parts.append(f"{colour}{text}\033[0m({l}, {t})")
        print(" ".join(parts))
        print()
