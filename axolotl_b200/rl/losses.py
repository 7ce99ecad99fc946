"""Closed-form preference / policy-gradient losses on per-sequence (or per-token) log-probabilities.

Formulas follow the papers as implemented by the libraries the reference delegates to (trl's
DPO/CPO/ORPO/KTO/GRPO trainers, selected by ``rl:`` in the reference config,
src/axolotl/core/builders/rl.py:40-250 and src/axolotl/utils/schemas/enums.py:28-39).
All inputs are fp32 tensors on the training device; every function returns
``(loss, metrics dict of detached tensors)``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

DPO_LOSS_TYPES = ("sigmoid", "hinge", "ipo", "robust", "exo_pair", "nca_pair", "sppo_hard", "apo_zero", "apo_down")


def dpo_loss(pol_c, pol_r, ref_c, ref_r, beta=0.1, loss_type="sigmoid", label_smoothing=0.0):
    """pol_*/ref_*: [P] summed (or, for ipo, length-averaged) log-probs of chosen / rejected."""
    a = pol_c - ref_c            # chosen log-ratio
    b = pol_r - ref_r            # rejected log-ratio
    x = a - b
    ls = label_smoothing
    if loss_type == "sigmoid":
        losses = -F.logsigmoid(beta * x) * (1 - ls) - F.logsigmoid(-beta * x) * ls
    elif loss_type == "robust":
        losses = (-F.logsigmoid(beta * x) * (1 - ls) + F.logsigmoid(-beta * x) * ls) / (1 - 2 * ls)
    elif loss_type == "hinge":
        losses = torch.relu(1 - beta * x)
    elif loss_type == "ipo":
        losses = (x - 1 / (2 * beta)) ** 2
    elif loss_type == "exo_pair":
        eps = ls if ls > 0 else 1e-3
        px = torch.sigmoid(beta * x)
        losses = px * (F.logsigmoid(beta * x) - torch.log(torch.tensor(1 - eps))) + \
            (1 - px) * (F.logsigmoid(-beta * x) - torch.log(torch.tensor(eps)))
    elif loss_type == "nca_pair":
        losses = -F.logsigmoid(beta * a) - 0.5 * F.logsigmoid(-beta * a) - 0.5 * F.logsigmoid(-beta * b)
    elif loss_type == "sppo_hard":
        losses = (a - 0.5 / beta) ** 2 + (b + 0.5 / beta) ** 2
    elif loss_type == "apo_zero":
        losses = (1 - torch.sigmoid(beta * a)) + torch.sigmoid(beta * b)
    elif loss_type == "apo_down":
        losses = torch.sigmoid(beta * a) + (1 - torch.sigmoid(beta * (a - b)))
    else:
        raise ValueError(f"unknown dpo loss_type '{loss_type}' (known: {DPO_LOSS_TYPES})")
    rc, rr = (beta * a).detach(), (beta * b).detach()
    m = {"rewards/chosen": rc.mean(), "rewards/rejected": rr.mean(), "rewards/margins": (rc - rr).mean(),
         "rewards/accuracies": (rc > rr).float().mean()}
    return losses.mean(), m


def cpo_loss(pol_c, pol_r, nll_chosen, beta=0.1, loss_type="sigmoid", label_smoothing=0.0, cpo_alpha=1.0,
             simpo_gamma=0.5):
    """Reference-free contrastive preference loss; ``loss_type='simpo'`` expects length-averaged
    log-probs and subtracts the target margin gamma / beta."""
    x = pol_c - pol_r
    ls = label_smoothing
    if loss_type == "simpo":
        x = x - simpo_gamma / beta
        losses = -F.logsigmoid(beta * x) * (1 - ls) - F.logsigmoid(-beta * x) * ls
    elif loss_type == "sigmoid":
        losses = -F.logsigmoid(beta * x) * (1 - ls) - F.logsigmoid(-beta * x) * ls
    elif loss_type == "hinge":
        losses = torch.relu(1 - beta * x)
    elif loss_type == "ipo":
        losses = (x - 1 / (2 * beta)) ** 2
    else:
        raise ValueError(f"unknown cpo loss_type '{loss_type}'")
    loss = losses.mean() + cpo_alpha * nll_chosen
    rc, rr = (beta * pol_c).detach(), (beta * pol_r).detach()
    m = {"rewards/chosen": rc.mean(), "rewards/rejected": rr.mean(), "rewards/margins": (rc - rr).mean(),
         "rewards/accuracies": (rc > rr).float().mean(), "nll_loss": nll_chosen.detach()}
    return loss, m


def orpo_loss(avg_c, avg_r, nll_chosen, beta=0.1):
    """Odds-ratio preference optimisation: NLL on the chosen answer minus beta * log-sigmoid of the
    log odds ratio; ``avg_*`` are length-averaged log-probs (so exp() is a valid probability)."""
    log_odds = (avg_c - avg_r) - (torch.log1p(-torch.exp(avg_c).clamp(max=1 - 1e-7))
                                  - torch.log1p(-torch.exp(avg_r).clamp(max=1 - 1e-7)))
    ratio = F.logsigmoid(log_odds)
    loss = nll_chosen - beta * ratio.mean()
    rc, rr = (beta * avg_c).detach(), (beta * avg_r).detach()
    m = {"rewards/chosen": rc.mean(), "rewards/rejected": rr.mean(), "rewards/margins": (rc - rr).mean(),
         "rewards/accuracies": (rc > rr).float().mean(), "log_odds_ratio": ratio.detach().mean(),
         "log_odds_chosen": log_odds.detach().mean(), "nll_loss": nll_chosen.detach()}
    return loss, m


def kto_loss(pol, ref, is_desirable, kl, beta=0.1, desirable_weight=1.0, undesirable_weight=1.0):
    """pol/ref: [N] sequence log-probs of the completions; is_desirable: [N] bool; kl: scalar
    (detached, >= 0) estimate of KL(policy || reference) from mismatched prompt/completion pairs."""
    ratio = pol - ref
    des = 1 - torch.sigmoid(beta * (ratio - kl))
    und = 1 - torch.sigmoid(beta * (kl - ratio))
    w = torch.where(is_desirable, torch.full_like(ratio, desirable_weight), torch.full_like(ratio, undesirable_weight))
    losses = torch.where(is_desirable, des, und) * w
    r = (beta * ratio).detach()
    m = {"kl": kl.detach() if isinstance(kl, torch.Tensor) else torch.tensor(kl)}
    if is_desirable.any():
        m["rewards/chosen"] = r[is_desirable].mean()
    if (~is_desirable).any():
        m["rewards/rejected"] = r[~is_desirable].mean()
    return losses.mean(), m


def bradley_terry_loss(r_c, r_r, margin=None, center_rewards_coefficient=None):
    """Pairwise reward-model loss -log sigmoid(r_c - r_r - margin)."""
    x = r_c - r_r
    if margin is not None:
        x = x - margin
    loss = -F.logsigmoid(x).mean()
    if center_rewards_coefficient:
        loss = loss + center_rewards_coefficient * ((r_c + r_r) ** 2).mean()
    return loss, {"accuracy": (r_c > r_r).float().mean().detach(), "rewards/margins": x.detach().mean()}


def grpo_loss(tok_logp, old_logp, ref_logp, advantages, seq_ids, n_seq, mask, *, beta=0.0, epsilon=0.2,
              epsilon_high=None, loss_type="grpo", max_completion_length=None, delta=None,
              importance_sampling_level="token", num_items=None):
    """Clipped-surrogate group-relative policy optimisation on a packed stream.

    tok_logp [T] current log-probs (with grad); old_logp [T] log-probs of the sampling policy (or
    None => on-policy, ratio 1 with gradient); ref_logp [T] or None; advantages [n_seq];
    seq_ids [T] document index of every token; mask [T] bool (completion tokens).
    ``loss_type``: grpo (mean over tokens per sequence, then over sequences), bnpo (mean over all
    completion tokens of the batch), dr_grpo (sum / (n_seq * max_completion_length)), dapo (sum /
    ``num_items``, the completion tokens of the whole optimizer step).
    """
    eh = epsilon if epsilon_high is None else epsilon_high
    maskf = mask.float()
    sid = seq_ids.clamp(min=0).long()
    if old_logp is None:
        old_logp = tok_logp.detach()
    log_ratio = (tok_logp - old_logp) * maskf
    if importance_sampling_level == "sequence":      # GSPO: one ratio per sequence
        cnt = torch.zeros(n_seq, device=tok_logp.device).index_add_(0, sid, maskf).clamp(min=1)
        seq_lr = torch.zeros(n_seq, device=tok_logp.device).index_add_(0, sid, log_ratio) / cnt
        log_ratio = seq_lr[sid]
    ratio = torch.exp(log_ratio)
    adv = advantages[sid]
    r1 = ratio if delta is None else ratio.clamp(max=delta)
    per_tok = -torch.minimum(r1 * adv, ratio.clamp(1 - epsilon, 1 + eh) * adv)
    m = {}
    if beta and ref_logp is not None:
        d = (ref_logp - tok_logp) * maskf
        kl = torch.exp(d) - d - 1
        per_tok = per_tok + beta * kl
        m["kl"] = ((kl * maskf).sum() / maskf.sum().clamp(min=1)).detach()
    per_tok = per_tok * maskf
    if loss_type == "grpo":
        cnt = torch.zeros(n_seq, device=tok_logp.device).index_add_(0, sid, maskf).clamp(min=1)
        per_seq = torch.zeros(n_seq, device=tok_logp.device).index_add_(0, sid, per_tok) / cnt
        loss = per_seq.mean()
    elif loss_type == "bnpo":
        loss = per_tok.sum() / maskf.sum().clamp(min=1)
    elif loss_type == "dr_grpo":
        loss = per_tok.sum() / (n_seq * float(max_completion_length or 1))
    elif loss_type == "dapo":
        loss = per_tok.sum() / float(num_items or maskf.sum().clamp(min=1))
    else:
        raise ValueError(f"unknown grpo loss_type '{loss_type}'")
    clipped = ((ratio < 1 - epsilon) & (adv < 0)) | ((ratio > 1 + eh) & (adv > 0))
    m["clip_ratio"] = ((clipped.float() * maskf).sum() / maskf.sum().clamp(min=1)).detach()
    return loss, m


def group_advantages(rewards, group_size, scale_rewards="group", eps=1e-4):
    """rewards [G * group_size] -> advantages: reward minus the group mean, divided by the group
    (or batch) standard deviation unless ``scale_rewards`` is 'none'. 'rloo' uses the leave-one-out
    baseline instead (reward minus the mean of the OTHER samples of the group, unscaled)."""
    r = rewards.view(-1, group_size)
    if scale_rewards == "rloo" and group_size > 1:
        return (r - (r.sum(1, keepdim=True) - r) / (group_size - 1)).reshape(-1)
    adv = r - r.mean(1, keepdim=True)
    if scale_rewards in ("group", True):
        adv = adv / (r.std(1, keepdim=True, unbiased=True if group_size > 1 else False).nan_to_num(0.0) + eps)
    elif scale_rewards == "batch":
        adv = adv / (rewards.std().nan_to_num(0.0) + eps)
    return adv.reshape(-1)
