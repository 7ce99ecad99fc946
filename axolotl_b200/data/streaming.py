"""Streaming (iterable) datasets: rows are read lazily, tokenised on the fly and packed into
``sequence_len`` rows from a bounded buffer, so a corpus never has to fit in memory or be
pre-tokenised. ``pretraining_dataset:`` entries and ``streaming: true`` SFT datasets both come
here; ``max_steps`` bounds the run.

Reference behaviour: src/axolotl/utils/data/streaming.py:20-304 (buffered tokenise + multipack
of an ``IterableDataset`` with ``pretrain_multipack_buffer_size`` rows per packing round and
per-document attention via position-id resets, ``pretrain_multipack_attn``).
"""
from __future__ import annotations

import json
import os

import numpy as np

from .collator import PackedCollator
from .packing import bins_from_assignment, pack_first_fit
from .strategies import load_strategy


def iter_raw_rows(ds_cfg: dict):
    """Lazily yields the rows of one configured source, cycling over its files once per call."""
    path = ds_cfg.get("path")
    files = ds_cfg.get("data_files")
    if isinstance(files, str):
        files = [files]
    cands = []
    if path and os.path.isfile(path):
        cands = [path]
    elif path and os.path.isdir(path):
        cands = [os.path.join(path, f) for f in files] if files else sorted(
            os.path.join(path, f) for f in os.listdir(path) if f.endswith((".json", ".jsonl", ".parquet", ".csv", ".txt")))
    elif files and all(os.path.exists(f) for f in files):
        cands = list(files)
    if not cands:
        try:
            import datasets

            d = datasets.load_dataset(path, name=ds_cfg.get("name"), split=ds_cfg.get("split") or "train",
                                      data_files=files, streaming=True)
            for r in d:
                yield dict(r)
            return
        except Exception as exc:
            raise FileNotFoundError(f"streaming dataset '{path}' is not local and could not be opened: {exc}") from exc
    for f in cands:
        ext = os.path.splitext(f)[1].lstrip(".")
        if ext in ("jsonl", "json"):
            with open(f) as fh:
                head = fh.read(1)
                fh.seek(0)
                if head == "[":
                    yield from json.load(fh)
                else:
                    for line in fh:
                        if line.strip():
                            yield json.loads(line)
        elif ext == "parquet":
            import pyarrow.parquet as pq

            pf = pq.ParquetFile(f)
            for batch in pf.iter_batches(batch_size=1024):
                yield from batch.to_pylist()
        elif ext == "csv":
            import csv

            with open(f, newline="") as fh:
                for r in csv.DictReader(fh):
                    yield dict(r)
        else:
            with open(f) as fh:
                for line in fh:
                    if line.strip():
                        yield {"text": line.rstrip("\n")}


class StreamingPackedBatches:
    """callable(epoch) -> iterator of collated micro-batches for one data-parallel rank.

    Rows are dealt round-robin to ranks (row i belongs to rank i % dp_size), tokenised by the
    dataset's prompt strategy (``pretrain`` by default: every token trained, EOS appended), collected
    until ``buffer_size`` samples are waiting, packed first-fit into ``sequence_len`` bins and emitted
    ``micro_batch_size`` bins at a time; leftovers carry over to the next round."""

    def __init__(self, cfg, datasets_cfg, tokenizer, dp_rank=0, dp_size=1):
        self.cfg, self.ds_cfgs, self.tok = cfg, [dict(d) for d in datasets_cfg], tokenizer
        self.rank, self.size = dp_rank, dp_size
        self.seq = cfg["sequence_len"]
        self.mbs = cfg.get("micro_batch_size") or 1
        self.buffer = cfg.get("pretrain_multipack_buffer_size") or cfg.get("streaming_multipack_buffer_size") or 10_000
        self.packing = cfg.get("sample_packing") is not False
        self.coll = PackedCollator(cfg.get("pad_token_id") or 0, cfg.get("pad_to_multiple_of") or 64, self.seq,
                                   bool(cfg.get("pad_to_sequence_len", True)))
        self.per_doc_attention = cfg.get("pretrain_multipack_attn", True) is not False
        self.seed = cfg.get("seed") or 42

    def _samples(self, epoch):
        i = 0
        for d in self.ds_cfgs:
            strat = load_strategy(d.get("type") or "pretrain", self.tok, self.cfg, d)
            skip = d.get("skip") or 0
            for n, row in enumerate(iter_raw_rows(d)):
                if n < skip:
                    continue
                mine = (i % self.size) == self.rank
                i += 1
                if not mine:
                    continue
                res = strat.tokenize(row)
                if res is None:
                    continue
                for s in (res if isinstance(res, list) else [res]):
                    if 0 < len(s["input_ids"]) <= self.seq:
                        yield s

    def _emit(self, buf, rng, final):
        """Packs the buffer; returns (batches, leftover samples)."""
        if not self.packing:
            n_full = len(buf) // self.mbs * self.mbs
            out = [self.coll([[s] for s in buf[i:i + self.mbs]]) for i in range(0, n_full, self.mbs)]
            return out, buf[n_full:]
        order = rng.permutation(len(buf))
        lens = np.array([len(buf[j]["input_ids"]) for j in order], dtype=np.int64)
        bin_of, n_bins = pack_first_fit(lens, self.seq)
        bins = bins_from_assignment(order, bin_of, n_bins)
        # keep the fullest bins; the emptiest ones wait for the next round unless the stream ended
        fill = [sum(len(buf[j]["input_ids"]) for j in b) for b in bins]
        keep = sorted(range(len(bins)), key=lambda k: -fill[k])
        n_emit = len(bins) if final else max((len(bins) * 9 // 10) // self.mbs * self.mbs, 0)
        n_emit = n_emit // self.mbs * self.mbs
        emit, hold = keep[:n_emit], keep[n_emit:]
        out = []
        for i in range(0, len(emit), self.mbs):
            rows = []
            for k in emit[i:i + self.mbs]:
                samples = [dict(buf[j]) for j in bins[k]]
                if not self.per_doc_attention:   # one long document per row: positions run on
                    off = 0
                    for s in samples:
                        s["position_ids"] = np.arange(off, off + len(s["input_ids"]))
                        off += len(s["input_ids"])
                rows.append(samples)
            out.append(self.coll(rows))
        left = [buf[j] for k in hold for j in bins[k]]
        return out, left

    def __call__(self, epoch=0):
        rng = np.random.default_rng(self.seed + epoch)
        buf = []
        for s in self._samples(epoch):
            buf.append(s)
            if len(buf) >= self.buffer:
                batches, buf = self._emit(buf, rng, final=False)
                yield from batches
        if buf:
            batches, _ = self._emit(buf, rng, final=True)
            yield from batches
