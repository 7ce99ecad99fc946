"""Grokfast: low-pass (EMA) filtered gradients added back to the raw gradients before the
optimizer step (reference: src/axolotl/integrations/grokfast/__init__.py:16-36)."""
from __future__ import annotations

from pydantic import BaseModel

from ..train.trainer import Callback
from .base import BasePlugin


class GrokfastArgs(BaseModel):
    grokfast_alpha: float | None = 0.98
    grokfast_lamb: float | None = 2.0


class GrokfastCallback(Callback):
    def __init__(self, alpha, lamb):
        self.alpha, self.lamb, self.ema = alpha, lamb, None

    def on_pre_optimizer_step(self, trainer):
        grads = trainer.opt.flat_grads()
        if self.ema is None:
            self.ema = [g.clone() for g in grads]
        for e, g in zip(self.ema, grads):
            e.mul_(self.alpha).add_(g, alpha=1 - self.alpha)
            g.add_(e, alpha=self.lamb)


class GrokfastPlugin(BasePlugin):
    def get_input_args(self):
        return GrokfastArgs

    def add_callbacks_post_trainer(self, cfg, trainer):
        return [GrokfastCallback(cfg.get("grokfast_alpha") or 0.98, cfg.get("grokfast_lamb") or 2.0)]
