"""Configuration normalisation: derived batch sizes, world-size scaling, dtype resolution,
save/eval cadence, model-family flags (rules of src/axolotl/utils/config/__init__.py:122-417)."""
from __future__ import annotations

import json
import os

import torch


def resolve_dtype(cfg):
    if cfg.get("bf16") == "auto" or cfg.get("bf16") is None:
        cfg["bf16"] = bool(torch.cuda.is_available()) or bool(cfg.get("bfloat16"))
    if cfg.get("tf32") == "auto":
        cfg["tf32"] = torch.cuda.is_available()
    if cfg.get("bf16") or cfg.get("bfloat16"):
        cfg["torch_dtype"] = "bfloat16"
    elif cfg.get("float32"):
        cfg["torch_dtype"] = "float32"
    else:
        cfg["torch_dtype"] = "float32" if not torch.cuda.is_available() else "bfloat16"
    return cfg


def normalize(cfg):
    g = cfg.get
    # ---- batch arithmetic (A.1)
    mbs = g("micro_batch_size") or 1
    cfg["micro_batch_size"] = mbs
    if g("gradient_accumulation_steps"):
        cfg["batch_size"] = g("batch_size") or mbs * g("gradient_accumulation_steps")
    elif g("batch_size"):
        cfg["gradient_accumulation_steps"] = max(1, g("batch_size") // mbs)
    else:
        cfg["gradient_accumulation_steps"] = 1
        cfg["batch_size"] = mbs
    if not g("eval_batch_size"):
        cfg["eval_batch_size"] = mbs
    world = int(os.environ.get("WORLD_SIZE", g("world_size") or 1))
    cfg["world_size"] = world
    cfg["local_rank"] = int(os.environ.get("LOCAL_RANK", g("local_rank") or 0))
    tp, cp = g("tensor_parallel_size") or 1, g("context_parallel_size") or 1
    if world > 1:
        # TP and CP ranks share a batch; EP ranks count as data parallel
        cfg["batch_size"] = cfg["batch_size"] * (world // cp // tp)
    # ---- dtype
    resolve_dtype(cfg)
    # ---- cadence
    n_ep = g("num_epochs") or 1
    if g("saves_per_epoch"):
        frac = 1.0 / (g("saves_per_epoch") * n_ep)
        if frac < 1.0:   # a ratio of 1 would checkpoint after every step: save at the end only instead
            cfg["save_steps"] = frac
            cfg["save_strategy"] = "steps"
    if g("evals_per_epoch") and (g("val_set_size") or g("test_datasets")):
        frac = 1.0 / (g("evals_per_epoch") * n_ep)
        if frac < 1.0:
            cfg["eval_steps"] = frac
            cfg["eval_strategy"] = "steps"
    if g("save_steps") and not g("save_strategy"):
        cfg["save_strategy"] = "steps"
    if g("eval_steps") and not g("eval_strategy"):
        cfg["eval_strategy"] = "steps"
    if g("save_total_limit") is None:
        cfg["save_total_limit"] = 4
    if g("val_set_size") in (None, 0, 0.0) and not g("test_datasets"):
        cfg["eval_strategy"] = "no"
        cfg["eval_steps"] = None
    # ---- model family flags
    mt = None
    src = g("base_model_config") or g("base_model")
    if src and os.path.isdir(src) and os.path.exists(os.path.join(src, "config.json")):
        with open(os.path.join(src, "config.json")) as fh:
            mt = json.load(fh).get("model_type")
    elif g("model_preset"):
        from ..models.config import PRESETS

        mt = PRESETS.get(g("model_preset"), {}).get("model_type")
    cfg["model_config_type"] = mt
    cfg["is_llama_derived_model"] = bool(g("is_llama_derived_model")) or mt == "llama"
    cfg["is_mistral_derived_model"] = bool(g("is_mistral_derived_model")) or mt in ("mistral", "mixtral")
    cfg["is_qwen_derived_model"] = bool(g("is_qwen_derived_model")) or (mt or "").startswith("qwen")
    # ---- defaults that depend on other keys
    if g("gradient_checkpointing") and g("gradient_checkpointing_kwargs") is None:
        cfg["gradient_checkpointing_kwargs"] = {"use_reentrant": False}
    if g("sample_packing") and g("multipack_real_batches") is None:
        cfg["multipack_real_batches"] = False
    if g("dataloader_drop_last") is None and g("sample_packing"):
        cfg["dataloader_drop_last"] = True
    if g("seed") is None:
        cfg["seed"] = 42
    if g("max_grad_norm") is None:
        cfg["max_grad_norm"] = 1.0
    return cfg
