"""Preference datasets and their packed collators.

A micro-batch of preference pairs becomes ONE varlen row: documents ``prompt+chosen_0,
prompt+rejected_0, prompt+chosen_1, ...`` back to back, position ids restarting per document,
labels (already shifted by one inside each document) set only on completion tokens, and a
``seq_ids`` vector naming the document of every token. No padding to the longest pair and no
second forward pass for the rejected half: the flash-varlen kernel keeps documents apart. The
reference instead pads chosen/rejected to a common length and concatenates them along the batch
dimension inside trl (selected in src/axolotl/core/builders/rl.py:40-250).
"""
from __future__ import annotations

import numpy as np
import torch

from ..data.loading import _shard, read_raw
from .strategies import load_preference_transform

IGNORE_INDEX = -100


def _encode(tokenizer, text, bos=False, eos=False):
    ids = list(tokenizer(text, add_special_tokens=False)["input_ids"])
    if bos and tokenizer.bos_token_id is not None and (not ids or ids[0] != tokenizer.bos_token_id):
        ids = [tokenizer.bos_token_id] + ids
    if eos and tokenizer.eos_token_id is not None and (not ids or ids[-1] != tokenizer.eos_token_id):
        ids = ids + [tokenizer.eos_token_id]
    return ids


def _truncate(prompt, completion, max_len, max_prompt_len):
    """Keep the END of an over-long prompt, then cut the completion to fit ``max_len``."""
    if max_prompt_len and len(prompt) > max_prompt_len:
        prompt = prompt[-max_prompt_len:]
    if max_len and len(prompt) + len(completion) > max_len:
        completion = completion[: max(max_len - len(prompt), 1)]
        if len(prompt) + len(completion) > max_len:
            prompt = prompt[-(max_len - len(completion)):]
    return prompt, completion


def tokenize_preference_rows(rows, tokenizer, rl, max_len=None, max_prompt_len=None):
    """rows with canonical string fields (or pre-tokenised ``*_input_ids``) -> list of records of
    int lists: pairwise {prompt, chosen, rejected}; kto {prompt, completion, label}."""
    out = []
    for r in rows:
        if "prompt_input_ids" in r:
            p = list(r["prompt_input_ids"])
        else:
            p = _encode(tokenizer, r["prompt"], bos=True)
        if rl == "kto":
            c = list(r["completion_input_ids"]) if "completion_input_ids" in r else _encode(tokenizer, r["completion"], eos=True)
            p2, c = _truncate(p, c, max_len, max_prompt_len)
            out.append({"prompt": p2, "completion": c, "label": bool(r.get("label", True))})
        else:
            ch = list(r["chosen_input_ids"]) if "chosen_input_ids" in r else _encode(tokenizer, r["chosen"], eos=True)
            rj = list(r["rejected_input_ids"]) if "rejected_input_ids" in r else _encode(tokenizer, r["rejected"], eos=True)
            pc, ch = _truncate(p, ch, max_len, max_prompt_len)
            pr, rj = _truncate(p, rj, max_len, max_prompt_len)
            rec = {"prompt": pc if len(pc) <= len(pr) else pr, "chosen": ch, "rejected": rj}
            if "margin" in r:
                rec["margin"] = float(r["margin"])
            out.append(rec)
    return out


def load_preference_dataset(cfg, tokenizer, split="train"):
    """Reads, transforms and tokenises every configured dataset of a preference run."""
    rl = cfg.get("rl")
    dsets = cfg.get("datasets" if split == "train" else "test_datasets") or []
    recs = []
    for i, d in enumerate(dsets):
        d = dict(d)
        if d.get("type") == "_synthetic_pref":
            recs.extend(synthetic_preference(d.get("length") or 64, d.get("prompt_len") or 16,
                                             d.get("completion_len") or 16, d.get("max_input_id") or 1000,
                                             kto=rl == "kto", seed=d.get("seed") or 0))
            continue
        fn = load_preference_transform(d.get("type"), rl, tokenizer, d)
        rows = [fn(dict(r)) for r in _shard(read_raw(d), d)]
        recs.extend(tokenize_preference_rows(rows, tokenizer, rl, cfg.get("sequence_len"),
                                             cfg.get("max_prompt_len")))
    return recs


def synthetic_preference(n, prompt_len, completion_len, vocab, kto=False, seed=0):
    """Random-token preference records whose 'chosen' completions are drawn from the low half of
    the vocabulary and 'rejected' from the high half, so that a model can actually learn the
    preference (used by tests and offline smoke runs)."""
    g = np.random.default_rng(seed)
    out = []
    half = vocab // 2
    for i in range(n):
        p = g.integers(3, vocab, prompt_len).tolist()
        lo = g.integers(3, half, completion_len).tolist()
        hi = g.integers(half, vocab, completion_len).tolist()
        if kto:
            good = bool(i % 2 == 0)
            out.append({"prompt": p, "completion": lo if good else hi, "label": good})
        else:
            out.append({"prompt": p, "chosen": lo, "rejected": hi})
    return out


class _DocPacker:
    """Accumulates documents of one packed row."""

    def __init__(self):
        self.ids, self.lab, self.pos, self.sid, self.cu = [], [], [], [], [0]

    def add(self, prompt, completion, completion_mask=None):
        """``completion_mask`` (0/1 per completion token): tokens the policy did not write (tool results an environment
        inserted between turns) stay in the context and are not targets."""
        doc = np.asarray(list(prompt) + list(completion), dtype=np.int64)
        lab = np.full(len(doc), IGNORE_INDEX, dtype=np.int64)
        # shifted labels: position t predicts token t+1; only completion tokens are targets
        lo = max(len(prompt) - 1, 0)
        lab[lo:len(doc) - 1] = doc[lo + 1:]
        if len(prompt) == 0:
            lab[:len(doc) - 1] = doc[1:]
        if completion_mask is not None and len(prompt) > 0:
            keep = np.asarray(list(completion_mask), dtype=bool)[: len(completion)]
            tgt = lab[len(prompt) - 1: len(prompt) - 1 + len(keep)]
            tgt[~keep] = IGNORE_INDEX
        k = len(self.cu) - 1
        self.ids.append(doc)
        self.lab.append(lab)
        self.pos.append(np.arange(len(doc), dtype=np.int32))
        self.sid.append(np.full(len(doc), k, dtype=np.int32))
        self.cu.append(self.cu[-1] + len(doc))
        return k

    def finish(self, pad_token_id, multiple, extra_aux=None, meta=None):
        ids, lab = np.concatenate(self.ids), np.concatenate(self.lab)
        pos, sid = np.concatenate(self.pos), np.concatenate(self.sid)
        n = len(ids)
        width = ((n + multiple - 1) // multiple) * multiple
        cu = list(self.cu)
        if width > n:
            pad = width - n
            ids = np.concatenate([ids, np.full(pad, pad_token_id, np.int64)])
            lab = np.concatenate([lab, np.full(pad, IGNORE_INDEX, np.int64)])
            pos = np.concatenate([pos, np.arange(pad, dtype=np.int32)])
            sid = np.concatenate([sid, np.full(pad, -1, np.int32)])
            cu.append(width)
        n_seq = len(self.cu) - 1
        aux = {"seq_ids": torch.from_numpy(sid)[None]}
        aux.update(extra_aux or {})
        m = {"n_seq": n_seq}
        m.update(meta or {})
        return {"input_ids": torch.from_numpy(ids)[None], "labels": torch.from_numpy(lab)[None],
                "position_ids": torch.from_numpy(pos)[None], "cu_seqlens": np.asarray(cu, dtype=np.int32),
                "labels_preshifted": True, "n_trainable": int((lab != IGNORE_INDEX).sum()), "n_tokens": int(n),
                "aux_tensors": aux, "meta": m}


class PairwiseCollator:
    """records -> one packed row with documents [c0, r0, c1, r1, ...]."""

    def __init__(self, pad_token_id=0, pad_to_multiple_of=64):
        self.pad, self.multiple = pad_token_id, pad_to_multiple_of

    def __call__(self, records):
        pk = _DocPacker()
        for r in records:
            pk.add(r["prompt"], r["chosen"])
            pk.add(r["prompt"], r["rejected"])
        aux = {}
        if any("margin" in r for r in records):
            aux["margin"] = torch.tensor([float(r.get("margin", 0.0)) for r in records])
        if all("ref_chosen_logp" in r for r in records):
            aux["ref_logps"] = torch.tensor([[r["ref_chosen_logp"], r["ref_rejected_logp"]] for r in records],
                                            dtype=torch.float32).reshape(-1)
        return pk.finish(self.pad, self.multiple, aux, {"n_pairs": len(records)})


class KTOCollator:
    """records -> documents [x_0 y_0, ..., x_{n-1} y_{n-1}, x_0 y_1, ..., x_{n-1} y_0]: the second
    half pairs every prompt with the NEXT record's completion and estimates the KL term."""

    def __init__(self, pad_token_id=0, pad_to_multiple_of=64):
        self.pad, self.multiple = pad_token_id, pad_to_multiple_of

    def __call__(self, records):
        pk = _DocPacker()
        n = len(records)
        for r in records:
            pk.add(r["prompt"], r["completion"])
        for i, r in enumerate(records):
            pk.add(r["prompt"], records[(i + 1) % n]["completion"])
        aux = {"is_desirable": torch.tensor([bool(r["label"]) for r in records])}
        return pk.finish(self.pad, self.multiple, aux, {"n_examples": n})


class PreferenceBatches:
    """Epoch iterator: shuffled records, ``micro_batch_size`` per collated row, sharded over the
    data-parallel ranks."""

    def __init__(self, records, collator, micro_batch_size, dp_rank=0, dp_size=1, seed=0, shuffle=True):
        self.records, self.collator, self.mbs = records, collator, micro_batch_size
        self.rank, self.size, self.seed, self.shuffle = dp_rank, dp_size, seed, shuffle

    def __len__(self):
        return len(self.records) // (self.mbs * self.size)

    def __call__(self, epoch):
        idx = np.arange(len(self.records))
        if self.shuffle:
            np.random.default_rng(self.seed + epoch).shuffle(idx)
        per = self.mbs * self.size
        for b in range(len(idx) // per):
            mine = idx[b * per + self.rank * self.mbs: b * per + (self.rank + 1) * self.mbs]
            yield self.collator([self.records[i] for i in mine])
