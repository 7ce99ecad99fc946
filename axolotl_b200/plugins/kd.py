"""Knowledge distillation from top-k teacher log-probabilities.

Every training position carries the teacher's K most likely next tokens and their log-probs
(``target_token_ids`` / ``target_logprobs`` [T, K], ``target_mask`` [T, K]); the loss is the
forward KL over those K tokens, ``sum_k p_t(k) (log p_t(k) - log p_s(k))``, averaged over
positions, mixed with the ordinary cross entropy:
``kd_alpha * KL + kd_ce_alpha * CE``. The student's log-normaliser is computed chunk by chunk
from lm-head GEMM tiles (``ce_chunk_rows`` rows at a time under activation recompute), so
[T, V] logits are never resident.

Reference: src/axolotl/integrations/kd/ (plugin + args), topk_logprob/forward_kl.py:23-150
(loss definition and chunked variant), collator.py (padding of the target tensors).
Config keys: ``kd_trainer``, ``kd_alpha``, ``kd_ce_alpha``, ``kd_temperature``,
``kd_zscore_base_temp`` is not applied. Dataset rows are pre-tokenised: ``input_ids``, ``labels``,
``target_token_ids``, ``target_logprobs`` and optionally ``target_mask``.
"""
from __future__ import annotations

import numpy as np
import torch
from pydantic import BaseModel

from ..ops.gemm import gemm
from .base import BasePlugin


class KDArgs(BaseModel):
    kd_trainer: bool | None = None
    kd_alpha: float | None = None
    kd_ce_alpha: float | None = None
    kd_temperature: float | None = None
    kd_top_k: int | None = None


class _DetachedGemmKL(torch.autograd.Function):
    """KL of one chunk with a hand-written backward: d/dlogits = (sum_k p_t) * softmax - scatter(p_t),
    pushed through the lm head by the tcgen05 GEMM (the frozen head gets no gradient)."""

    @staticmethod
    def forward(ctx, h, w, ids, t_logp, mask, temperature):
        logits = gemm(h, w, out_dtype=torch.float32) if h.is_cuda else (h @ w.to(h.dtype).t()).float()
        if temperature != 1.0:
            logits = logits / temperature
        lse = torch.logsumexp(logits, -1, keepdim=True)
        p_t = t_logp.exp() * mask
        s_logp = logits.gather(1, ids) - lse
        ctx.save_for_backward(h, w, ids, p_t)
        ctx.temperature = temperature
        return (p_t * (t_logp - s_logp)).sum()

    @staticmethod
    def backward(ctx, g):
        h, w, ids, p_t = ctx.saved_tensors
        logits = gemm(h, w, out_dtype=torch.float32) if h.is_cuda else (h @ w.to(h.dtype).t()).float()
        if ctx.temperature != 1.0:
            logits = logits / ctx.temperature
        d = torch.softmax(logits, -1) * p_t.sum(1, keepdim=True)
        d.scatter_add_(1, ids, -p_t)
        d = (d * (g / ctx.temperature)).to(h.dtype)
        dh = gemm(d, w, trans_b=True) if h.is_cuda else d @ w.to(h.dtype)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = (d.float().t() @ h.float()).to(w.dtype)
        return dh, dw, None, None, None, None


class KDObjective:
    """``compute_loss`` for the Trainer."""

    def __init__(self, cfg):
        self.alpha = cfg.get("kd_alpha") if cfg.get("kd_alpha") is not None else 1.0
        self.ce_alpha = cfg.get("kd_ce_alpha") or 0.0
        self.temperature = float(cfg.get("kd_temperature") or 1.0)
        self.last_metrics = {}

    def __call__(self, model, b, n_items):
        from ..ops.functional import linear_cross_entropy

        out = model(b["input_ids"], b["position_ids"], attn_meta=b["attn_meta"], return_logits=False)
        h = out.hidden_states.reshape(-1, out.hidden_states.shape[-1])
        W = model.output_weight()
        ids = b["target_token_ids"].reshape(h.shape[0], -1).long()
        t_logp = b["target_logprobs"].reshape(h.shape[0], -1).float()
        mask = b["target_mask"].reshape(h.shape[0], -1).float()
        n_pos = max(float(b.get("kd_positions_total", (mask.sum(1) > 0).sum().item())), 1.0)
        kl = h.new_zeros((), dtype=torch.float32)
        rows = model.ce_chunk_rows
        for r0 in range(0, h.shape[0], rows):
            sl = slice(r0, r0 + rows)
            if float(mask[sl].sum()) == 0.0:
                continue
            kl = kl + _DetachedGemmKL.apply(h[sl].contiguous(), W, ids[sl], t_logp[sl], mask[sl], self.temperature)
        kd = kl / n_pos * (self.temperature ** 2)
        loss = self.alpha * kd
        self.last_metrics = {"kd_loss": float(kd.detach())}
        if self.ce_alpha:
            lab = b["labels"].reshape(-1)
            if not b.get("labels_preshifted"):
                B, S = b["labels"].shape
                lab = torch.cat([b["labels"][:, 1:], b["labels"].new_full((B, 1), -100)], 1).reshape(-1)
            ce = linear_cross_entropy(h, W, lab, num_items=n_items, chunk_rows=rows)
            loss = loss + self.ce_alpha * ce
            self.last_metrics["ce_loss"] = float(ce.detach())
        return loss


class KDCollator:
    """Pads / packs pre-tokenised KD rows; the teacher tensors of position t describe token t+1
    (they are stored unshifted, aligned with ``labels``, and shifted here with the labels)."""

    def __init__(self, pad_token_id=0, pad_to_multiple_of=64, top_k=None):
        from ..data.collator import PackedCollator

        self.inner = PackedCollator(pad_token_id, pad_to_multiple_of)
        self.top_k = top_k

    def __call__(self, bins):
        if bins and not isinstance(bins[0], (list, tuple)):
            bins = [[s] for s in bins]
        base = self.inner(bins)
        B, S = base["input_ids"].shape
        K = self.top_k or max(len(s["target_token_ids"][0]) for row in bins for s in row if len(s["target_token_ids"]))
        tid = np.zeros((B, S, K), np.int64)
        tlp = np.full((B, S, K), -1e4, np.float32)
        msk = np.zeros((B, S, K), np.float32)
        for b, row in enumerate(bins):
            off = 0
            for s in row:
                n = len(s["input_ids"])
                ids = np.asarray(s["target_token_ids"], np.int64)[:, :K]
                lps = np.asarray(s["target_logprobs"], np.float32)[:, :K]
                m = np.asarray(s.get("target_mask", np.ones_like(ids)), np.float32)[:, :K]
                lab = np.asarray(s.get("labels", s["input_ids"]))
                m = m * (lab != -100)[:, None]
                # shift: position t predicts token t+1, inside the sample
                k = ids.shape[1]
                tid[b, off:off + n - 1, :k] = ids[1:n]
                tlp[b, off:off + n - 1, :k] = lps[1:n]
                msk[b, off:off + n - 1, :k] = m[1:n]
                off += n
        # renormalise the teacher distribution over its top-k support
        lse = np.log(np.exp(tlp.astype(np.float64)).sum(-1, keepdims=True).clip(min=1e-300))
        tlp = np.where(msk > 0, tlp - lse, tlp).astype(np.float32)
        base["aux_tensors"] = {"target_token_ids": torch.from_numpy(tid), "target_logprobs": torch.from_numpy(tlp),
                               "target_mask": torch.from_numpy(msk)}
        return base


class KDPlugin(BasePlugin):
    def get_input_args(self):
        return KDArgs

    def compute_loss(self, cfg):
        return KDObjective(cfg) if cfg.get("kd_trainer") else None

    def get_collator_cls_and_kwargs(self, cfg, is_eval=False):
        if not cfg.get("kd_trainer"):
            return None
        return KDCollator, {"pad_token_id": cfg.get("pad_token_id") or 0, "top_k": cfg.get("kd_top_k")}
