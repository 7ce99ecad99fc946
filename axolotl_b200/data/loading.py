"""Dataset pipeline: raw sources -> prompt strategy -> tokenised ragged arrays -> packing
pre-processing -> on-disk cache keyed by a hash of everything that influences the result.

Mirrors the behaviour of the reference pipeline (src/axolotl/utils/data/sft.py:47-514,
src/axolotl/utils/data/shared.py:403-726, src/axolotl/utils/trainer.py:92-376):
* per-dataset ``type`` -> strategy; shards; merge + shuffle (seeded); exact dedup;
* samples longer than ``sequence_len`` are dropped / truncated / raise (``excess_length_strategy``),
  samples shorter than ``min_sample_len`` and samples without trainable labels are dropped;
* ``position_ids`` = 0..len-1 and ``length`` are attached for packing; PoSE position skipping;
* validation split by ``val_set_size`` (fraction or count) with a seeded permutation;
* rank 0 prepares under a file lock, other ranks wait and load the cache.
Tokenised data is stored as flat ``int32`` arrays plus offsets (one ``.npz``), which the C++
packer and the collator consume without per-row Python objects.
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import dataclass

import numpy as np

from ..utils.logging import get_logger
from .strategies import IGNORE_INDEX, is_pretokenized, load_strategy
from .synthetic import synthetic_fixed, synthetic_varlen

LOG = get_logger(__name__)
DEFAULT_PREPARED_PATH = "last_run_prepared"


class TokenizedDataset:
    """Ragged token dataset: ``input_ids`` / ``labels`` (flat) + ``offsets`` [n+1]; optional flat
    ``position_ids``."""

    def __init__(self, input_ids, labels, offsets, position_ids=None):
        self.input_ids = np.asarray(input_ids, dtype=np.int32)
        self.labels = np.asarray(labels, dtype=np.int32)
        self.offsets = np.asarray(offsets, dtype=np.int64)
        self.position_ids = None if position_ids is None else np.asarray(position_ids, dtype=np.int32)

    @classmethod
    def from_rows(cls, rows):
        lens = [len(r["input_ids"]) for r in rows]
        off = np.zeros(len(rows) + 1, dtype=np.int64)
        np.cumsum(lens, out=off[1:])
        ids = np.concatenate([np.asarray(r["input_ids"], dtype=np.int32) for r in rows]) if rows else np.zeros(0, np.int32)
        lab = np.concatenate([np.asarray(r.get("labels", r["input_ids"]), dtype=np.int32) for r in rows]) if rows else np.zeros(0, np.int32)
        pos = None
        if rows and all("position_ids" in r for r in rows):
            pos = np.concatenate([np.asarray(r["position_ids"], dtype=np.int32) for r in rows])
        return cls(ids, lab, off, pos)

    def __len__(self):
        return len(self.offsets) - 1

    @property
    def lengths(self):
        return (self.offsets[1:] - self.offsets[:-1]).astype(np.int32)

    def __getitem__(self, i):
        a, b = self.offsets[i], self.offsets[i + 1]
        row = {"input_ids": self.input_ids[a:b].astype(np.int64), "labels": self.labels[a:b].astype(np.int64)}
        row["position_ids"] = (self.position_ids[a:b].astype(np.int64) if self.position_ids is not None
                               else np.arange(b - a, dtype=np.int64))
        row["length"] = int(b - a)
        return row

    def select(self, idx):
        idx = np.asarray(idx, dtype=np.int64)
        lens = self.lengths[idx]
        off = np.zeros(len(idx) + 1, dtype=np.int64)
        np.cumsum(lens, out=off[1:])
        take = np.concatenate([np.arange(self.offsets[i], self.offsets[i + 1]) for i in idx]) if len(idx) else np.zeros(0, np.int64)
        return TokenizedDataset(self.input_ids[take], self.labels[take], off,
                                None if self.position_ids is None else self.position_ids[take])

    def save(self, path):
        os.makedirs(path, exist_ok=True)
        arrs = dict(input_ids=self.input_ids, labels=self.labels, offsets=self.offsets)
        if self.position_ids is not None:
            arrs["position_ids"] = self.position_ids
        tmp = os.path.join(path, "data.tmp.npz")
        np.savez(tmp, **arrs)
        os.replace(tmp, os.path.join(path, "data.npz"))
        with open(os.path.join(path, "meta.json"), "w") as fh:
            json.dump({"num_rows": len(self), "num_tokens": int(self.offsets[-1]),
                       "num_trainable": int((self.labels != IGNORE_INDEX).sum())}, fh)

    @classmethod
    def load(cls, path):
        z = np.load(os.path.join(path, "data.npz"))
        return cls(z["input_ids"], z["labels"], z["offsets"], z["position_ids"] if "position_ids" in z else None)

    def total_tokens(self):
        return int(self.offsets[-1])

    def total_trainable(self):
        return int((self.labels != IGNORE_INDEX).sum())


@dataclass
class TrainDatasetMeta:
    train: TokenizedDataset | None
    eval: TokenizedDataset | None = None
    total_num_steps: int | None = None


# ---------------------------------------------------------------------------------- raw sources
def read_raw(ds_cfg: dict) -> list[dict]:
    """Rows of one configured dataset (local json/jsonl/parquet/csv/txt, HF ``save_to_disk`` dir,
    or the Hub through ``datasets`` when reachable)."""
    path = ds_cfg.get("path")
    files = ds_cfg.get("data_files")
    if isinstance(files, str):
        files = [files]
    ds_type = ds_cfg.get("ds_type")
    cands = []
    if path and os.path.isfile(path):
        cands = [path]
    elif path and os.path.isdir(path):
        if files:
            cands = [os.path.join(path, f) for f in files]
        elif os.path.exists(os.path.join(path, "dataset_info.json")) or os.path.exists(os.path.join(path, "state.json")):
            import datasets

            d = datasets.load_from_disk(path)
            if isinstance(d, datasets.DatasetDict):
                d = d[ds_cfg.get("split") or "train"]
            return [dict(r) for r in d]
        else:
            cands = sorted(os.path.join(path, f) for f in os.listdir(path)
                           if f.endswith((".json", ".jsonl", ".parquet", ".csv", ".txt")))
    elif files and all(os.path.exists(f) for f in files):
        cands = files
    if not cands:
        try:
            import datasets

            d = datasets.load_dataset(path, name=ds_cfg.get("name"), split=ds_cfg.get("split") or "train",
                                      data_files=files, revision=ds_cfg.get("revision"),
                                      trust_remote_code=ds_cfg.get("trust_remote_code") or None)
            return [dict(r) for r in d]
        except Exception as exc:
            raise FileNotFoundError(f"dataset '{path}' is not a local file/directory and could not be fetched: {exc}") from exc
    rows = []
    for f in cands:
        kind = ds_type or os.path.splitext(f)[1].lstrip(".")
        if kind in ("json", "jsonl"):
            with open(f) as fh:
                head = fh.read(1)
                fh.seek(0)
                if head == "[":
                    rows.extend(json.load(fh))
                else:
                    rows.extend(json.loads(line) for line in fh if line.strip())
        elif kind == "parquet":
            import pyarrow.parquet as pq

            rows.extend(pq.read_table(f).to_pylist())
        elif kind == "csv":
            import csv

            with open(f, newline="") as fh:
                rows.extend(dict(r) for r in csv.DictReader(fh))
        elif kind in ("txt", "text"):
            with open(f) as fh:
                rows.extend({"text": line.rstrip("\n")} for line in fh if line.strip())
        else:
            raise ValueError(f"unsupported dataset file type: {f}")
    return rows


def _shard(rows, ds_cfg):
    n = ds_cfg.get("shards")
    if n:
        idx = ds_cfg.get("shards_idx") or 0
        rows = rows[idx::n]
    return rows


def tokenize_dataset(ds_cfg, tokenizer, cfg) -> TokenizedDataset:
    t = ds_cfg.get("type")
    if t == "_synthetic":
        if ds_cfg.get("min_length") and ds_cfg.get("max_length"):
            d = synthetic_varlen(ds_cfg.get("length") or 1000, ds_cfg["min_length"], ds_cfg["max_length"],
                                 ds_cfg.get("min_input_id") or 100, ds_cfg.get("max_input_id") or 32000,
                                 ds_cfg.get("mask_prefix_fraction") or 0.0, ds_cfg.get("seed") or 0)
        else:
            d = synthetic_fixed(ds_cfg.get("length") or 1000, ds_cfg.get("sequence_length") or cfg["sequence_len"],
                                ds_cfg.get("min_input_id") or 100, ds_cfg.get("max_input_id") or 32000,
                                ds_cfg.get("seed"))
        return TokenizedDataset.from_rows(d.rows)
    rows = _shard(read_raw(ds_cfg), ds_cfg)
    if not rows:
        return TokenizedDataset.from_rows([])
    if t is None and is_pretokenized(rows[0].keys()):
        t = "pretokenized"
    strat = load_strategy(t, tokenizer, cfg, ds_cfg)
    out = []
    for r in rows:
        res = strat.tokenize(r)
        if res is None:
            continue
        out.extend(res if isinstance(res, list) else [res])
    return TokenizedDataset.from_rows(out)


# ---------------------------------------------------------------------------------- processing
def concat(dsets):
    dsets = [d for d in dsets if len(d)]
    if not dsets:
        return TokenizedDataset.from_rows([])
    off = [np.zeros(1, np.int64)]
    base = 0
    for d in dsets:
        off.append(d.offsets[1:] + base)
        base += d.offsets[-1]
    pos = None
    if all(d.position_ids is not None for d in dsets):
        pos = np.concatenate([d.position_ids for d in dsets])
    return TokenizedDataset(np.concatenate([d.input_ids for d in dsets]), np.concatenate([d.labels for d in dsets]),
                            np.concatenate(off), pos)


def deduplicate(d: TokenizedDataset) -> TokenizedDataset:
    seen, keep = set(), []
    for i in range(len(d)):
        a, b = d.offsets[i], d.offsets[i + 1]
        h = hashlib.sha1(d.input_ids[a:b].tobytes() + d.labels[a:b].tobytes()).digest()
        if h not in seen:
            seen.add(h)
            keep.append(i)
    if len(keep) != len(d):
        LOG.info("dedup: dropped %d duplicate samples", len(d) - len(keep))
    return d.select(keep)


def filter_lengths(d: TokenizedDataset, sequence_len, min_len=None, strategy="drop") -> TokenizedDataset:
    lens = d.lengths
    min_len = min_len or 2
    too_long = lens > sequence_len
    if strategy == "raise" and too_long.any():
        raise ValueError(f"{int(too_long.sum())} samples exceed sequence_len={sequence_len} (excess_length_strategy: raise)")
    if strategy == "truncate" and too_long.any():
        rows = []
        for i in range(len(d)):
            r = d[i]
            rows.append({k: r[k][:sequence_len] for k in ("input_ids", "labels", "position_ids")})
        d = TokenizedDataset.from_rows(rows)
        lens = d.lengths
        too_long = lens > sequence_len
    keep = np.flatnonzero(~too_long & (lens >= min_len))
    if len(keep) != len(d):
        LOG.info("length filter: dropped %d of %d samples", len(d) - len(keep), len(d))
        d = d.select(keep)
    return d


def drop_untrainable(d: TokenizedDataset) -> TokenizedDataset:
    trainable = np.add.reduceat((d.labels != IGNORE_INDEX).astype(np.int64), d.offsets[:-1]) if len(d) else np.zeros(0)
    # reduceat on an empty trailing segment repeats the next value; lengths are >= 1 here
    keep = np.flatnonzero(trainable > 0)
    if len(keep) != len(d):
        LOG.info("dropped %d samples without trainable tokens", len(d) - len(keep))
        d = d.select(keep)
    return d


def add_position_ids(d: TokenizedDataset) -> TokenizedDataset:
    if d.position_ids is None:
        lens = d.lengths
        pos = np.arange(d.offsets[-1], dtype=np.int64) - np.repeat(d.offsets[:-1], lens)
        d.position_ids = pos.astype(np.int32)
    return d


def apply_pose(d: TokenizedDataset, max_context_len, num_chunks=2, split_on_token_ids=None, seed=0) -> TokenizedDataset:
    """PoSE: keep tokens, spread their position ids over [0, max_context_len) by inserting random
    skips between chunks (src/axolotl/utils/trainer.py:131-193)."""
    rng = np.random.default_rng(seed)
    pos = np.zeros(d.offsets[-1], dtype=np.int32)
    for i in range(len(d)):
        a, b = int(d.offsets[i]), int(d.offsets[i + 1])
        n = b - a
        budget = max(max_context_len - n, 0)
        if split_on_token_ids:
            cuts = [j for j in range(1, n) if int(d.input_ids[a + j]) in split_on_token_ids][: num_chunks - 1]
        else:
            cuts = sorted(rng.choice(np.arange(1, n), size=min(num_chunks - 1, max(n - 1, 0)), replace=False).tolist()) if n > 1 else []
        skips = sorted(rng.integers(0, budget + 1, size=len(cuts)).tolist())
        p = np.arange(n, dtype=np.int32)
        prev = 0
        for c, s in zip(cuts, skips):
            p[c:] += s - prev
            prev = s
        pos[a:b] = p
    d.position_ids = pos
    return d


def process_for_packing(d: TokenizedDataset, cfg) -> TokenizedDataset:
    d = filter_lengths(d, cfg["sequence_len"], cfg.get("min_sample_len"), cfg.get("excess_length_strategy") or "drop")
    d = drop_untrainable(d)
    if cfg.get("use_pose"):
        d = apply_pose(d, cfg.get("pose_max_context_len") or cfg["sequence_len"], cfg.get("pose_num_chunks") or 2,
                       cfg.get("pose_split_on_token_ids"), cfg.get("seed") or 0)
    else:
        d = add_position_ids(d)
    return d


def split_validation(d: TokenizedDataset, val_set_size, seed):
    n = len(d)
    n_val = int(val_set_size) if val_set_size >= 1 else int(round(n * val_set_size))
    n_val = min(max(n_val, 0), max(n - 1, 0))
    if n_val == 0:
        return d, None
    perm = np.random.default_rng(seed).permutation(n)
    return d.select(np.sort(perm[n_val:])), d.select(np.sort(perm[:n_val]))


# ---------------------------------------------------------------------------------- cache + entry
def dataset_hash(cfg, datasets_cfg, tokenizer_name) -> str:
    key = {
        "datasets": [{k: v for k, v in sorted(dict(d).items()) if v is not None} for d in datasets_cfg],
        "sequence_len": cfg.get("sequence_len"), "min_sample_len": cfg.get("min_sample_len"),
        "excess": cfg.get("excess_length_strategy"), "train_on_inputs": cfg.get("train_on_inputs"),
        "chat_template": cfg.get("chat_template"), "tokenizer": tokenizer_name, "dedup": cfg.get("dataset_exact_deduplication"),
        "pose": [cfg.get("use_pose"), cfg.get("pose_max_context_len"), cfg.get("pose_num_chunks")],
        "shuffle": [cfg.get("shuffle_merged_datasets"), cfg.get("seed")], "special_tokens": cfg.get("special_tokens"),
        "eot": cfg.get("eot_tokens"),
    }
    return hashlib.md5(json.dumps(key, sort_keys=True, default=str).encode()).hexdigest()


class FileLock:
    """Rank 0 prepares, others wait (src/axolotl/utils/data/lock.py:17-72)."""

    def __init__(self, path, timeout=3600):
        self.ready = os.path.join(path, ".ready")
        self.path, self.timeout = path, timeout

    def wait(self):
        t0 = time.time()
        while not os.path.exists(self.ready):
            if time.time() - t0 > self.timeout:
                raise TimeoutError(f"timed out waiting for {self.ready}")
            time.sleep(0.5)

    def done(self):
        os.makedirs(self.path, exist_ok=True)
        open(self.ready, "w").close()


def _prepare(datasets_cfg, tokenizer, cfg, split_name):
    parts = []
    for dc in datasets_cfg:
        d = tokenize_dataset(dict(dc), tokenizer, cfg)
        if cfg.get("shuffle_before_merging_datasets"):
            d = d.select(np.random.default_rng(cfg.get("seed") or 42).permutation(len(d)))
        parts.append(d)
    d = concat(parts)
    if cfg.get("dataset_exact_deduplication"):
        d = deduplicate(d)
    d = process_for_packing(d, cfg)
    if len(datasets_cfg) > 1 and cfg.get("shuffle_merged_datasets", True) and not cfg.get("curriculum_sampling"):
        d = d.select(np.random.default_rng(cfg.get("seed") or 42).permutation(len(d)))
    LOG.info("%s: %d samples, %d tokens (%d trainable)", split_name, len(d), d.total_tokens(), d.total_trainable())
    return d


def load_prepared(datasets_cfg, tokenizer, cfg, split_name="train") -> TokenizedDataset:
    tok_name = getattr(tokenizer, "name_or_path", "none") if tokenizer is not None else "none"
    h = dataset_hash(cfg, datasets_cfg, tok_name) + ("" if split_name == "train" else "_" + split_name)
    root = cfg.get("dataset_prepared_path") or DEFAULT_PREPARED_PATH
    path = os.path.join(root, h)
    rank = int(os.environ.get("RANK", "0"))
    lock = FileLock(path)
    if os.path.exists(os.path.join(path, "data.npz")) and os.path.exists(lock.ready) and not cfg.get("is_preprocess"):
        LOG.info("loading prepared dataset from %s", path)
        return TokenizedDataset.load(path)
    if rank != 0 and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        lock.wait()
        return TokenizedDataset.load(path)
    d = _prepare(datasets_cfg, tokenizer, cfg, split_name)
    if not cfg.get("skip_prepare_dataset"):
        d.save(path)
        lock.done()
        LOG.info("saved prepared dataset to %s", path)
    return d


def load_datasets(cfg, tokenizer=None, preprocess=False) -> TrainDatasetMeta:
    needs_tok = any((d.get("type") != "_synthetic") for d in (cfg.get("datasets") or []))
    if tokenizer is None and needs_tok:
        from .tokenizer import load_tokenizer

        tokenizer = load_tokenizer(cfg)
    train = load_prepared(cfg.get("datasets") or [], tokenizer, cfg, "train")
    ev = None
    if cfg.get("test_datasets"):
        ev = load_prepared(cfg["test_datasets"], tokenizer, cfg, "test")
    elif cfg.get("val_set_size"):
        train, ev = split_validation(train, cfg["val_set_size"], cfg.get("seed") or 42)
    meta = TrainDatasetMeta(train, ev, None)
    if not preprocess:
        meta.total_num_steps = calculate_total_num_steps(cfg, train)
    return meta


def calculate_total_num_steps(cfg, train: TokenizedDataset) -> int:
    """Packing: len(dataloader) * micro_batch_size // batch_size * epochs (minus ceil(epochs) when
    dropping the last batch); otherwise ceil(len * epochs / batch_size)
    (src/axolotl/utils/trainer.py:401-524)."""
    import math

    from .packing import MultipackBatchSampler, estimate_total_steps

    if cfg.get("max_steps"):
        return int(cfg["max_steps"])
    world = cfg.get("world_size") or 1
    dp = max(1, world // (cfg.get("context_parallel_size") or 1) // (cfg.get("tensor_parallel_size") or 1))
    epochs = cfg.get("num_epochs") or 1
    if cfg.get("sample_packing"):
        samp = MultipackBatchSampler(train.lengths, cfg["sequence_len"], cfg["micro_batch_size"],
                                     real_batches=bool(cfg.get("multipack_real_batches")),
                                     bin_size=cfg.get("sample_packing_bin_size") or 200,
                                     group_size=cfg.get("sample_packing_group_size") or 100_000,
                                     sequential=bool(cfg.get("sample_packing_sequentially")), seed=cfg.get("seed") or 42,
                                     world_size=dp)
        n = len(samp)
        cfg["sample_packing_eff_est"] = math.ceil(samp.efficiency() * 100) / 100
        return estimate_total_steps(n, cfg["micro_batch_size"], cfg["batch_size"] // dp, epochs,
                                    drop_last=bool(cfg.get("dataloader_drop_last", True)))
    return int(math.ceil(len(train) * epochs / max(cfg["batch_size"], 1)))
