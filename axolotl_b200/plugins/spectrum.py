"""Spectrum: train only the top fraction of layers of each projection type ranked by a
signal-to-noise score of their weight spectrum, freeze the rest
(reference: src/axolotl/integrations/spectrum/__init__.py:55)."""
from __future__ import annotations

import re

import torch
from pydantic import BaseModel

from .base import BasePlugin


class SpectrumArgs(BaseModel):
    spectrum_top_fraction: float | None = 0.5
    spectrum_model_name: str | None = None


def snr_score(w: torch.Tensor) -> float:
    """Ratio of spectral energy above the Marchenko-Pastur edge to the energy below it."""
    s = torch.linalg.svdvals(w.float().cpu())
    n, m = w.shape
    sigma = s.median() / (1 + (min(n, m) / max(n, m)) ** 0.5)
    thresh = sigma * (1 + (min(n, m) / max(n, m)) ** 0.5)
    sig, noise = s[s >= thresh].sum(), s[s < thresh].sum()
    return float(sig / noise) if noise > 0 else float("inf")


class SpectrumPlugin(BasePlugin):
    def get_input_args(self):
        return SpectrumArgs

    def post_model_load(self, cfg, model):
        frac = cfg.get("spectrum_top_fraction") or 0.5
        by_kind = {}
        for name, m in model.fused_linears():
            for sub in m.names:
                kind = sub
                by_kind.setdefault(kind, []).append((snr_score(m.sub_weight(sub)), name, m))
        keep = set()
        for kind, items in by_kind.items():
            items.sort(key=lambda t: -t[0])
            for _, name, _ in items[: max(1, int(len(items) * frac))]:
                keep.add(name)
        for name, m in model.fused_linears():
            m.weight.requires_grad_(name in keep)
        cfg["unfrozen_parameters"] = [re.escape(n) + r"\.weight" for n in sorted(keep)]
