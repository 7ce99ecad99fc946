"""Stand-alone evaluation and text generation (src/axolotl/evaluate.py:68-151, cli/inference.py)."""
from __future__ import annotations

import math

import torch

from ..data.loading import load_datasets
from . import run as _run
from .trainer import count_trainable, to_device_batch


def _device(cfg):
    return torch.device("cuda", 0) if torch.cuda.is_available() and cfg.get("device") != "cpu" else torch.device("cpu")


def evaluate(cfg) -> dict:
    dev = _device(cfg)
    meta = load_datasets(cfg)
    ds = meta.eval if meta.eval is not None else meta.train
    model = _run.build_model(cfg, dev)
    _run.setup_adapter(cfg, model)
    model.eval()
    fn, _ = _run.make_batches_fn(cfg, ds, 0, 1, None, is_eval=True)
    tot, items = 0.0, 0
    for b in fn():
        d = to_device_batch(b, dev)
        n = max(count_trainable(b["labels"]), 1)
        out = model(d["input_ids"], d["position_ids"], d["labels"], attn_meta=d["attn_meta"], num_items=n)
        tot += float(out.loss.item()) * n
        items += n
    loss = tot / max(items, 1)
    return {"eval_loss": loss, "eval_ppl": math.exp(min(loss, 50)), "eval_samples": len(ds), "eval_tokens": items}


def generate_text(cfg, prompt: str, max_new_tokens=64, temperature=0.0) -> str:
    from ..data.tokenizer import load_tokenizer

    dev = _device(cfg)
    tok = load_tokenizer(cfg)
    model = _run.build_model(cfg, dev)
    _run.setup_adapter(cfg, model)
    ids = torch.tensor([tok(prompt)["input_ids"]], device=dev)
    out = model.generate(ids, max_new_tokens=max_new_tokens, temperature=temperature, eos_token_id=tok.eos_token_id)
    return tok.decode(out[0].tolist(), skip_special_tokens=True)
