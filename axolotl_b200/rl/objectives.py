"""``compute_loss`` objects for the Trainer: DPO/IPO, CPO/SimPO, ORPO, KTO, reward model, PRM.

Selection mirrors the reference's RL builder (src/axolotl/core/builders/rl.py:40-250:
``rl: dpo|ipo|orpo|kto|simpo`` plus ``reward_model`` / ``process_reward_model`` flags) and its
hyper-parameter names (``rl_beta``/``dpo_beta``, ``dpo_label_smoothing``, ``rpo_alpha``, ``orpo_alpha``,
``simpo_gamma``, ``cpo_alpha``, ``kto_desirable_weight``, ``kto_undesirable_weight``,
``dpo_loss_type``; src/axolotl/utils/schemas/config.py).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import losses as L
from .data import KTOCollator, PairwiseCollator
from .logps import reference_logps, segment_sum, sequence_logps


def _aux(model, out, loss, ga):
    coef = getattr(model.config, "router_aux_loss_coef", 0.0)
    if out is not None and out.aux_loss is not None and coef:
        loss = loss + (coef / ga) * out.aux_loss.to(loss.dtype)
    return loss


class Objective:
    """Base: keeps the detached metrics of the last micro-batch in ``last_metrics``."""

    needs_reference = False

    def __init__(self, cfg, ref_model=None, pad_token_id=0):
        self.cfg, self.ref_model = cfg, ref_model
        self.beta = cfg.get("rl_beta") or cfg.get("dpo_beta") or cfg.get("orpo_alpha") or 0.1
        self.last_metrics = {}
        self.pad_token_id = pad_token_id

    def collator(self):
        return PairwiseCollator(self.pad_token_id)

    def _done(self, loss, metrics, ga):
        self.last_metrics = {k: float(v) for k, v in metrics.items()}
        return loss / ga


class DPOObjective(Objective):
    needs_reference = True

    def __init__(self, cfg, ref_model=None, pad_token_id=0, loss_type=None):
        super().__init__(cfg, ref_model, pad_token_id)
        lt = loss_type or cfg.get("dpo_loss_type") or ("ipo" if cfg.get("rl") == "ipo" else "sigmoid")
        self.loss_type = lt[0] if isinstance(lt, (list, tuple)) else lt
        self.label_smoothing = cfg.get("dpo_label_smoothing") or 0.0
        self.rpo_alpha = cfg.get("rpo_alpha")
        self.average = self.loss_type == "ipo"

    def __call__(self, model, b, n_items):
        ga = b.get("ga_steps", 1)
        if "ref_logps" in b:
            ref = b["ref_logps"]
        else:
            ref = reference_logps(model, b, self.ref_model, average=self.average)
        pol, counts, out = sequence_logps(model, b, average=self.average)
        pc, pr, rc, rr = pol[0::2], pol[1::2], ref[0::2], ref[1::2]
        loss, m = L.dpo_loss(pc, pr, rc, rr, self.beta, self.loss_type, self.label_smoothing)
        if self.rpo_alpha:
            n = counts[0::2].clamp(min=1)
            nll = -((pc if self.average else pc / n)).mean()
            loss = loss + self.rpo_alpha * nll
            m["nll_loss"] = nll.detach()
        m["logps/chosen"], m["logps/rejected"] = pc.detach().mean(), pr.detach().mean()
        return self._done(_aux(model, out, loss, 1), m, ga)


class CPOObjective(Objective):
    """CPO and SimPO (``rl: simpo`` => loss_type simpo, length-averaged log-probs)."""

    def __init__(self, cfg, ref_model=None, pad_token_id=0):
        super().__init__(cfg, ref_model, pad_token_id)
        self.loss_type = "simpo" if cfg.get("rl") == "simpo" else (cfg.get("cpo_loss_type") or "sigmoid")
        self.cpo_alpha = cfg.get("cpo_alpha") if cfg.get("cpo_alpha") is not None else (0.0 if self.loss_type == "simpo" else 1.0)
        self.gamma = cfg.get("simpo_gamma") if cfg.get("simpo_gamma") is not None else 0.5
        self.label_smoothing = cfg.get("dpo_label_smoothing") or 0.0
        self.average = self.loss_type in ("simpo", "ipo")

    def __call__(self, model, b, n_items):
        ga = b.get("ga_steps", 1)
        pol, counts, out = sequence_logps(model, b, average=False)
        avg = pol / counts.clamp(min=1)
        use = avg if self.average else pol
        nll = -avg[0::2].mean()
        loss, m = L.cpo_loss(use[0::2], use[1::2], nll, self.beta, self.loss_type, self.label_smoothing,
                             self.cpo_alpha, self.gamma)
        return self._done(_aux(model, out, loss, 1), m, ga)


class ORPOObjective(Objective):
    def __call__(self, model, b, n_items):
        ga = b.get("ga_steps", 1)
        avg, _, out = sequence_logps(model, b, average=True)
        nll = -avg[0::2].mean()
        loss, m = L.orpo_loss(avg[0::2], avg[1::2], nll, self.beta)
        return self._done(_aux(model, out, loss, 1), m, ga)


class KTOObjective(Objective):
    needs_reference = True

    def __init__(self, cfg, ref_model=None, pad_token_id=0, dp_group=None):
        super().__init__(cfg, ref_model, pad_token_id)
        self.w_d = cfg.get("kto_desirable_weight") or 1.0
        self.w_u = cfg.get("kto_undesirable_weight") or 1.0
        self.dp_group = dp_group

    def collator(self):
        return KTOCollator(self.pad_token_id)

    def __call__(self, model, b, n_items):
        ga = b.get("ga_steps", 1)
        n = int(b["n_examples"])
        ref = reference_logps(model, b, self.ref_model)
        pol, _, out = sequence_logps(model, b)
        kl = (pol[n:].detach() - ref[n:]).mean()
        if dist.is_initialized() and dist.get_world_size(self.dp_group) > 1:
            dist.all_reduce(kl, group=self.dp_group)
            kl = kl / dist.get_world_size(self.dp_group)
        kl = kl.clamp(min=0)
        loss, m = L.kto_loss(pol[:n], ref[:n], b["is_desirable"].bool(), kl, self.beta, self.w_d, self.w_u)
        return self._done(_aux(model, out, loss, 1), m, ga)


# ------------------------------------------------------------------------------- scalar heads
def add_score_head(model, num_labels=1, seed=0):
    """Adds a trainable ``score`` projection [num_labels, hidden] (the sequence-classification head
    of HF ``*ForSequenceClassification`` / ``*ForTokenClassification`` models)."""
    if getattr(model, "score", None) is None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        w = torch.randn(num_labels, model.config.hidden_size, generator=g) * model.config.initializer_range
        model.score = torch.nn.Parameter(w.to(model.embed_tokens.device, torch.float32))
    return model.score


def _hidden(model, b):
    out = model(b["input_ids"], b["position_ids"], attn_meta=b["attn_meta"], return_logits=False)
    return out.hidden_states.reshape(-1, out.hidden_states.shape[-1]), out


class RewardObjective(Objective):
    """Bradley-Terry reward model: the score of a document is its last token's hidden state
    projected by ``score`` (reference: ``reward_model: true`` -> trl RewardTrainer,
    src/axolotl/core/trainers/trl.py)."""

    def __init__(self, cfg, ref_model=None, pad_token_id=0):
        super().__init__(cfg, ref_model, pad_token_id)
        self.center = cfg.get("center_rewards_coefficient")

    def __call__(self, model, b, n_items):
        ga = b.get("ga_steps", 1)
        h, out = _hidden(model, b)
        sid = b["seq_ids"].reshape(-1)
        n_seq = int(b["n_seq"])
        # last token of each document: the position where the next token belongs to another document
        nxt = torch.cat([sid[1:], sid.new_full((1,), -2)])
        last = (sid >= 0) & (nxt != sid)
        rows = h[last].float()                       # documents appear in order, one row each
        r = (rows @ model.score.float().t()).squeeze(-1)
        assert r.shape[0] == n_seq
        loss, m = L.bradley_terry_loss(r[0::2], r[1::2], b.get("margin"), self.center)
        return self._done(_aux(model, out, loss, 1), m, ga)


class PRMObjective(Objective):
    """Process reward model: two-class token classification at the labelled step ends (labels hold
    the class id there and -100 elsewhere; reference: ``process_reward_model: true`` -> trl
    PRMTrainer with the stepwise-supervised dataset type)."""

    def collator(self):
        from ..data.collator import PackedCollator

        inner = PackedCollator(self.pad_token_id)

        def collate(bins):
            out = inner(bins if bins and isinstance(bins[0], (list, tuple)) else [bins])
            out["labels_preshifted"] = True      # class labels sit on their own token, no shift
            out["n_trainable"] = int((out["labels"] != -100).sum())
            return out

        return collate

    def __call__(self, model, b, n_items):
        h, out = _hidden(model, b)
        lab = b["labels"].reshape(-1)
        keep = lab != -100
        logits = h[keep].float() @ model.score.float().t()
        loss = torch.nn.functional.cross_entropy(logits, lab[keep], reduction="sum") / max(n_items, 1)
        acc = (logits.argmax(-1) == lab[keep]).float().mean() if keep.any() else torch.zeros(())
        self.last_metrics = {"accuracy": float(acc)}
        return _aux(model, out, loss, b.get("ga_steps", 1))


def build_objective(cfg, ref_model=None, pad_token_id=0, dp_group=None):
    rl = cfg.get("rl")
    if cfg.get("reward_model"):
        return RewardObjective(cfg, ref_model, pad_token_id)
    if cfg.get("process_reward_model"):
        return PRMObjective(cfg, ref_model, pad_token_id)
    if rl in ("dpo", "ipo"):
        return DPOObjective(cfg, ref_model, pad_token_id)
    if rl in ("simpo", "cpo"):
        return CPOObjective(cfg, ref_model, pad_token_id)
    if rl == "orpo":
        return ORPOObjective(cfg, ref_model, pad_token_id)
    if rl == "kto":
        return KTOObjective(cfg, ref_model, pad_token_id, dp_group)
    raise ValueError(f"rl: {rl} has no preference objective (grpo/gdpo are built by rl.grpo)")


@torch.no_grad()
def precompute_reference_logps(model, records, collator, device, micro_batch_size=4, ref_model=None,
                               average=False):
    """Fills ``ref_chosen_logp`` / ``ref_rejected_logp`` on pairwise records
    (``precompute_ref_log_probs``): one pass with adapters off, so training steps skip the
    reference forward."""
    from ..train.trainer import to_device_batch

    for i in range(0, len(records), micro_batch_size):
        chunk = records[i:i + micro_batch_size]
        b = to_device_batch(collator(chunk), device)
        ref = reference_logps(model, b, ref_model, average=average).float().cpu()
        for j, r in enumerate(chunk):
            r["ref_chosen_logp"], r["ref_rejected_logp"] = float(ref[2 * j]), float(ref[2 * j + 1])
    return records
