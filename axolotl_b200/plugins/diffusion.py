"""Masked-diffusion language-model fine-tuning (LLaDA-style) on packed documents.

Every document draws a noise level t ~ U(0, 1); its trainable tokens are replaced by the mask
token with probability p = (1 - eps) t + eps; the model sees the noisy row with BIDIRECTIONAL
attention inside each document (tile flag of the varlen attention kernel) and is trained to
recover the masked tokens, each term weighted by 1/p (importance weighting) and normalised by
the document's number of trainable tokens. As in the reference
(src/axolotl/integrations/diffusion/trainer.py:18-300, utils.py, generation.py:154-330), the
autoregressive head convention is kept: the logits at position i-1 predict token i.

Per-token losses come from the chunked lm-head + cross-entropy kernels
(``ops.functional.linear_token_logps``), so no [T, V] logits are kept. ``generate`` fills a
masked continuation by iterative unmasking of the most confident predictions.

YAML::

    plugins: [axolotl.integrations.diffusion.DiffusionPlugin]
    diffusion:
      mask_token_id: 128002
      eps: 1.0e-3
      importance_weighting: true
"""
from __future__ import annotations

from typing import Literal

import torch
from pydantic import BaseModel, Field, model_validator

from ..ops import functional as Fn
from ..train.trainer import Callback
from ..utils.logging import get_logger
from .base import BasePlugin

LOG = get_logger(__name__)


class DiffusionConfig(BaseModel):
    noise_schedule: Literal["linear", "cosine"] = "linear"
    min_mask_ratio: float = Field(default=0.1, ge=0.0, le=1.0)
    max_mask_ratio: float = Field(default=0.9, ge=0.0, le=1.0)
    num_diffusion_steps: int = Field(default=128, ge=1)
    eps: float = Field(default=1e-3, ge=0.0, le=1.0)
    importance_weighting: bool = True
    mask_token_id: int | None = None
    mask_token_str: str | None = None
    generate_samples: bool = True
    generation_interval: int = Field(default=100, ge=1)
    num_generation_samples: int = Field(default=3, ge=1)
    generation_steps: int = Field(default=128, ge=1)
    generation_temperature: float = Field(default=0.0, ge=0.0)
    generation_max_length: int = Field(default=100, ge=1)

    @model_validator(mode="after")
    def _ratios(self):
        if self.min_mask_ratio > self.max_mask_ratio:
            raise ValueError("min_mask_ratio must be <= max_mask_ratio")
        return self


class DiffusionArgs(BaseModel):
    diffusion: DiffusionConfig = Field(default_factory=DiffusionConfig)


def _doc_ids(cu_dev, T):
    """Document index of every token of the flattened row."""
    return torch.bucketize(torch.arange(T, device=cu_dev.device), cu_dev[1:].to(torch.long), right=True)


def forward_process(ids, labels, cu_dev, mask_token_id, eps, special_ids=(), generator=None):
    """(noisy ids, masked positions, per-token mask probability) for a flattened packed row.
    Only trainable tokens (label != -100) that are neither special tokens nor the first token of
    their document (nothing predicts it) can be masked."""
    T = ids.numel()
    flat, lab = ids.reshape(-1), labels.reshape(-1)
    doc = _doc_ids(cu_dev, T)
    n_docs = cu_dev.numel() - 1
    t = torch.rand(n_docs, device=flat.device, generator=generator)
    p_tok = ((1 - eps) * t + eps)[doc.clamp(max=n_docs - 1)]
    can = lab != -100
    for s in special_ids:
        can &= flat != s
    first = torch.zeros(T, dtype=torch.bool, device=flat.device)
    first[cu_dev[:-1].to(torch.long)] = True
    can &= ~first
    masked = (torch.rand(T, device=flat.device, generator=generator) < p_tok) & can
    noisy = torch.where(masked, torch.full_like(flat, mask_token_id), flat)
    return noisy.view(ids.shape), masked, p_tok, doc


class DiffusionObjective:
    """``compute_loss`` replacement: callable(model, device_batch, num_items) -> loss."""

    def __init__(self, dcfg: dict, special_ids=(), seed=0):
        self.c = dcfg
        self.special = tuple(int(s) for s in special_ids if s is not None)
        self.last_metrics = {}
        self.seed, self.gen = seed, None

    def __call__(self, model, b, n_items):
        c = self.c
        ids, lab = b["input_ids"], b["labels"]
        dev = ids.device
        meta = b["attn_meta"]
        if getattr(meta, "causal", True):      # same documents, bidirectional tiles
            meta = Fn.AttnMeta(meta.cu_seqlens_host, dev, causal=False)
            b["attn_meta"] = meta
        if self.gen is None or self.gen.device != dev:
            self.gen = torch.Generator(device=dev)
            self.gen.manual_seed(self.seed)
        noisy, masked, p_tok, doc = forward_process(ids, lab, meta.cu_seqlens, int(c["mask_token_id"]), float(c["eps"]),
                                                    self.special, self.gen)
        flat = ids.reshape(-1)
        # logits at i-1 predict token i: target row i-1 <- token i where i is masked
        tgt = torch.full_like(flat, -100)
        tgt[:-1] = torch.where(masked[1:], flat[1:], tgt[1:])
        out = model(noisy, b["position_ids"], attn_meta=meta, return_logits=False)
        h = out.hidden_states.reshape(-1, out.hidden_states.shape[-1])
        logp = Fn.linear_token_logps(h, model.output_weight(), tgt, chunk_rows=model.ce_chunk_rows)   # [T], 0 if ignored
        w = torch.zeros_like(logp)
        w[:-1] = (1.0 / p_tok[1:]) if c.get("importance_weighting", True) else 1.0
        n_docs = meta.cu_seqlens.numel() - 1
        ans = torch.zeros(n_docs, device=dev).index_add_(0, doc, (lab.reshape(-1) != -100).float()).clamp(min=1.0)
        doc_of_row = torch.cat([doc[1:], doc[-1:]])            # row i-1 scores token i's document
        per_doc = torch.zeros(n_docs, device=dev).index_add_(0, doc_of_row, -logp * w)
        loss = (per_doc / ans).mean()
        with torch.no_grad():
            n_masked = masked.sum()
            self.last_metrics = {
                "mask_ratio": float(masked.float().mean()), "num_masked_tokens": int(n_masked),
                "avg_p_mask": float((p_tok * masked).sum() / n_masked.clamp(min=1)),
                "ce_loss": float(-logp.sum() / n_masked.clamp(min=1)),
            }
        return loss / b.get("ga_steps", 1)


@torch.no_grad()
def generate(model, prompt_ids, max_new_tokens, mask_token_id, steps=128, temperature=0.0, generator=None):
    """Fills ``max_new_tokens`` masked positions after ``prompt_ids`` (1-D tensor) by iterative
    unmasking: every step predicts all masked positions with bidirectional attention and keeps the
    most confident 1/(steps - step) of them."""
    dev = model.embed_tokens.device
    L = prompt_ids.numel() + max_new_tokens
    seq = torch.full((L,), int(mask_token_id), dtype=torch.long, device=dev)
    seq[: prompt_ids.numel()] = prompt_ids.to(dev)
    pos = torch.arange(L, dtype=torch.int32, device=dev)[None]
    meta = Fn.AttnMeta([0, L], dev, causal=False)
    steps = max(1, min(steps, max_new_tokens))
    was_training = model.training
    model.eval()
    for step in range(steps):
        is_mask = seq == mask_token_id
        n_left = int(is_mask.sum())
        if n_left == 0:
            break
        logits = model(seq[None], pos, attn_meta=meta, return_logits=True).logits[0].float()
        logits = torch.cat([logits[:1], logits[:-1]], 0)        # row i now predicts token i
        logits[:, mask_token_id] = float("-inf")
        if temperature > 0:
            probs = torch.softmax(logits / temperature, -1)
            pred = torch.multinomial(probs, 1, generator=generator).squeeze(1)
            conf = probs.gather(1, pred[:, None]).squeeze(1)
        else:
            probs = torch.softmax(logits, -1)
            conf, pred = probs.max(-1)
        conf = torch.where(is_mask, conf, torch.full_like(conf, -1.0))
        k = n_left if step == steps - 1 else max(1, int(n_left / (steps - step)))
        top = conf.topk(k).indices
        seq[top] = pred[top]
    model.train(was_training)
    return seq


class DiffusionSampleCallback(Callback):
    def __init__(self, dcfg, tokenizer, prompts):
        self.c, self.tok, self.prompts = dcfg, tokenizer, prompts

    def on_step_end(self, trainer, logs):
        c = self.c
        if trainer.rank != 0 or trainer.global_step % int(c["generation_interval"]):
            return
        for p in self.prompts[: int(c["num_generation_samples"])]:
            out = generate(trainer.model, torch.as_tensor(p), int(c["generation_max_length"]), int(c["mask_token_id"]),
                           int(c["generation_steps"]), float(c["generation_temperature"]))
            text = self.tok.decode(out.tolist()) if self.tok is not None else str(out.tolist())
            LOG.info("diffusion sample @ step %d: %s", trainer.global_step, text)


class DiffusionPlugin(BasePlugin):
    def get_input_args(self):
        return DiffusionArgs

    def _cfg(self, cfg):
        d = dict(DiffusionConfig(**(cfg.get("diffusion") or {})).model_dump())
        if d["mask_token_id"] is None:
            raise ValueError("diffusion.mask_token_id is required (an id the tokenizer reserves for masking)")
        return d

    def compute_loss(self, cfg):
        if cfg.get("rl"):
            raise ValueError("the diffusion plugin trains SFT datasets; it cannot be combined with `rl`")
        if (cfg.get("context_parallel_size") or 1) > 1:
            raise ValueError("bidirectional attention is not available with context parallelism")
        special = [cfg.get(k) for k in ("bos_token_id", "eos_token_id", "pad_token_id")]
        return DiffusionObjective(self._cfg(cfg), special, int(cfg.get("seed") or 0))
