"""Sequence log-probabilities of packed documents in one forward pass."""
from __future__ import annotations

import torch

from ..models.layers import disable_adapters
from ..ops.functional import linear_token_logps


def token_logps(model, batch, entropy_out=None):
    """Per-token log-probs [T] (0 at ignored positions) of ``batch['labels']`` (pre-shifted) and the
    model output (for the MoE auxiliary loss). ``entropy_out`` [T] fp32 receives per-token entropies."""
    out = model(batch["input_ids"], batch["position_ids"], attn_meta=batch["attn_meta"], return_logits=False)
    h = out.hidden_states.reshape(-1, out.hidden_states.shape[-1])
    lab = batch["labels"].reshape(-1)
    return linear_token_logps(h, model.output_weight(), lab, chunk_rows=model.ce_chunk_rows,
                              entropy_out=entropy_out), out


def segment_sum(values, seq_ids, n_seq):
    """Sum of ``values`` [T] per document; tokens with seq_id < 0 (padding) are dropped."""
    keep = seq_ids >= 0
    out = torch.zeros(n_seq, dtype=values.dtype, device=values.device)
    return out.index_add_(0, seq_ids.clamp(min=0).long(), values * keep.to(values.dtype))


def sequence_logps(model, batch, average=False):
    """(per-document summed log-prob [n_seq], per-document trainable-token count [n_seq], output).
    ``average=True`` divides by the token count (IPO / SimPO / ORPO convention)."""
    tok, out = token_logps(model, batch)
    seq_ids = batch["seq_ids"].reshape(-1)
    n_seq = int(batch["n_seq"])
    valid = (batch["labels"].reshape(-1) != -100).float()
    sums = segment_sum(tok, seq_ids, n_seq)
    counts = segment_sum(valid, seq_ids, n_seq)
    if average:
        sums = sums / counts.clamp(min=1)
    return sums, counts, out


@torch.no_grad()
def reference_logps(model, batch, ref_model=None, average=False):
    """Log-probs under the reference policy: a separate frozen model if given, otherwise this model
    with its adapters switched off."""
    if ref_model is not None:
        was = ref_model.training
        ref_model.eval()
        s, _, _ = sequence_logps(ref_model, batch, average)
        ref_model.train(was)
        return s
    with disable_adapters():
        s, _, _ = sequence_logps(model, batch, average)
    return s
