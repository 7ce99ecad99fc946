"""Sparse fine-tuning: weights that are zero when training starts stay zero.

The reference delegates this to llm-compressor's session callbacks driven by a recipe with a
``ConstantPruningModifier`` (src/axolotl/integrations/llm_compressor/plugin.py:26-118). Here the
mask is applied to the gradient before the optimizer step: a masked entry has zero gradient, hence
zero AdamW moments and a zero update, and decoupled weight decay leaves a zero weight at zero, so
masking the gradient keeps the sparsity pattern exactly without touching the weights again.

YAML (same keys as the reference)::

    plugins: [axolotl.integrations.llm_compressor.LLMCompressorPlugin]
    llmcompressor:
      recipe:
        finetuning_stage:
          finetuning_modifiers:
            ConstantPruningModifier:
              targets: ["re:.*q_proj.weight", "re:.*down_proj.weight"]
      save_compressed: false
"""
from __future__ import annotations

import re

import torch
from pydantic import BaseModel

from ..train.trainer import Callback
from ..utils.logging import get_logger
from .base import BasePlugin

LOG = get_logger(__name__)


class CompressionArgs(BaseModel):
    recipe: dict | str | None = None
    save_compressed: bool | None = False


class LLMCompressorArgs(BaseModel):
    llmcompressor: CompressionArgs | None = None


def recipe_targets(recipe) -> list[str]:
    """Every ``targets`` entry found under a ``ConstantPruningModifier`` of the recipe (all
    2-D weights when the recipe names none)."""
    found = []

    def walk(node, inside):
        if isinstance(node, dict):
            for k, v in node.items():
                if k == "targets" and inside:
                    found.extend(v if isinstance(v, (list, tuple)) else [v])
                else:
                    walk(v, inside or k == "ConstantPruningModifier")
        elif isinstance(node, (list, tuple)):
            for v in node:
                walk(v, inside)

    if isinstance(recipe, str):
        import yaml

        recipe = yaml.safe_load(recipe) if "\n" in recipe or ":" in recipe else yaml.safe_load(open(recipe))
    walk(recipe or {}, False)
    return [str(t) for t in found]


def _target_matches(targets, name: str) -> bool:
    if not targets or "__ALL_PRUNABLE__" in targets or "__ALL__" in targets:
        return True
    for t in targets:
        if t.startswith("re:"):
            if re.match(t[3:], name):
                return True
        elif name == t or name.endswith("." + t) or name.endswith(t):
            return True
    return False


class SparsityMaskCallback(Callback):
    def __init__(self, targets):
        self.targets, self.masks = targets, []

    @torch.no_grad()
    def on_train_begin(self, trainer):
        # recipes name Hugging Face modules (q_proj ...); a fused projection is matched per row block
        fused = {}
        for name, m in trainer.model.fused_linears():
            parent = name.rsplit(".", 1)[0]
            fused[id(m.weight)] = [(f"model.{parent}.{sub}.weight",) + tuple(m.row_range(sub)) for sub in m.names]
        kept = total = 0
        for n, p in trainer.model.named_parameters():
            if not p.requires_grad or p.ndim < 2:
                continue
            mask = (p.detach() != 0)
            if id(p) in fused:
                hit = False
                for hf_name, r0, r1 in fused[id(p)]:
                    if _target_matches(self.targets, hf_name):
                        hit = True
                    else:
                        mask[r0:r1] = True
                if not hit:
                    continue
            elif not (_target_matches(self.targets, n) or _target_matches(self.targets, "model." + n)):
                continue
            if bool(mask.all()):
                continue
            self.masks.append((p, mask.to(torch.float32)))
            kept += int(mask.sum())
            total += mask.numel()
        if self.masks:
            LOG.info("sparse fine-tuning: %d tensors masked, %.1f%% of their weights are zero and stay zero",
                     len(self.masks), 100.0 * (1 - kept / max(total, 1)))
        else:
            LOG.warning("sparse fine-tuning: no trainable weight with zeros matched the recipe targets")

    @torch.no_grad()
    def on_pre_optimizer_step(self, trainer):
        trainer.opt.flat_grads()   # folds autograd-side gradients into the optimizer's buffers
        for p, mask in self.masks:
            g = getattr(p, "_axb_grad", None)
            if g is None:
                g = p.grad
            if g is not None:
                g.mul_(mask.to(g.dtype))

    def sparsity(self):
        z = sum(int((p == 0).sum()) for p, _ in self.masks)
        return z / max(1, sum(p.numel() for p, _ in self.masks))


class LLMCompressorPlugin(BasePlugin):
    def get_input_args(self):
        return LLMCompressorArgs

    def add_callbacks_post_trainer(self, cfg, trainer):
        block = cfg.get("llmcompressor") or {}
        return [SparsityMaskCallback(recipe_targets(block.get("recipe")))]
