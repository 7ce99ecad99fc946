"""Optimizers and LR schedules.

``FlatAdamW`` keeps every trainable parameter of a group in one fp32 master buffer (gradients,
first and second moments likewise) so a step is: one squared-norm kernel + one fused
clip/AdamW/bf16-recast kernel per group, with no host synchronisation. Parameter groups follow
the reference's rules (src/axolotl/core/trainers/mixins/optimizer.py:22-105): weight decay on
matrices only, optional embedding LR, LoRA+ ratio for B matrices, named ``lr_groups``.
"""
from __future__ import annotations

import math
import re

import torch

from ..ops.optim import adamw_step_, grad_sumsq


def build_param_groups(named_params, *, weight_decay=0.0, embedding_lr=None, embedding_lr_scale=None,
                       loraplus_lr_ratio=None, loraplus_lr_embedding=None, lr_groups=None, lr=1e-4,
                       per_layer=False):
    """Returns a list of dicts {name, params: [(name, p)], lr_scale, weight_decay}. ``per_layer``
    gives every decoder layer its own groups (name suffix ``@layers.N``) so that layers can be
    switched on and off as units (LISA)."""
    import re as _re

    groups = {}

    def add(key, item, lr_scale, wd):
        if per_layer:
            m = _re.search(r"layers\.(\d+)\.", item[0])
            if m:
                key = f"{key}@layers.{m.group(1)}"
        g = groups.setdefault(key, {"name": key, "params": [], "lr_scale": lr_scale, "weight_decay": wd})
        g["params"].append(item)

    for n, p in named_params:
        if not p.requires_grad:
            continue
        is_embed = any(k in n for k in ("embed_tokens", "lm_head", "modules_to_save"))
        no_decay = p.dim() < 2 or n.endswith("bias") or "norm" in n
        matched = False
        for grp in lr_groups or []:
            if any(m in n for m in grp["modules"]):
                add(grp["name"], (n, p), grp["lr"] / lr, 0.0 if no_decay else weight_decay)
                matched = True
                break
        if matched:
            continue
        if is_embed and (embedding_lr is not None or embedding_lr_scale is not None):
            scale = embedding_lr / lr if embedding_lr is not None else embedding_lr_scale
            add("embeddings", (n, p), scale, 0.0)
        elif loraplus_lr_ratio and "lora_B" in n:
            add("lora_B", (n, p), loraplus_lr_ratio, weight_decay)
        elif no_decay:
            add("no_decay", (n, p), 1.0, 0.0)
        else:
            add("decay", (n, p), 1.0, weight_decay)
    return list(groups.values())


class FlatAdamW:
    def __init__(self, groups, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, max_grad_norm=0.0, alloc=None,
                 pad_multiple=8, moment_shard=None):
        self.lr, self.betas, self.eps, self.max_grad_norm = lr, betas, eps, max_grad_norm
        self.step_count = 0
        self.groups = []
        self.grad_scale = 1.0
        self.skip_zero_grad_once = False
        # (rank, world): the fused multi-GPU step updates only 1/world of every group on this rank,
        # so the AdamW moments are stored for that slice alone (ZeRO-1 style)
        self.moment_shard = moment_shard
        for g in groups:
            params = [(n, p) for n, p in g["params"] if p.requires_grad]
            if not params:
                continue
            # tensor-parallel replicated parameters first, sharded ones last: two contiguous ranges
            params.sort(key=lambda np_: bool(getattr(np_[1], "_tp_sharded", False)))
            dev = params[0][1].device
            total = sum(p.numel() for _, p in params)
            # 16-byte aligned slots so bf16 shadows stay usable as TMA / vector operands
            offs, off = [], 0
            for _, p in params:
                offs.append(off)
                off += (p.numel() + 7) // 8 * 8
            total = (off + pad_multiple - 1) // pad_multiple * pad_multiple
            # ZeRO-style: when the fused multi-GPU step owns the update and no parameter of the group is
            # fp32 (adapters keep fp32 masters as their storage), the fp32 master exists only for the slice
            # this rank updates; the bf16 copy every rank computes with stays complete.
            master_local = (moment_shard is not None and alloc is not None
                            and all(p.dtype == torch.bfloat16 for _, p in params))
            if master_local:
                mr, mw = moment_shard
                if total % (4 * mw):
                    raise ValueError("sharded masters need pad_multiple to be a multiple of 4 * world")
                master = torch.zeros(total // mw, dtype=torch.float32, device=dev)
                grad, shadow = alloc(total, torch.float32), alloc(total, torch.bfloat16)
            elif alloc is not None:  # e.g. peer-mapped symmetric memory for the fused multi-GPU step
                master, grad, shadow = alloc(total, torch.float32), alloc(total, torch.float32), alloc(total, torch.bfloat16)
            else:
                master = torch.zeros(total, dtype=torch.float32, device=dev)
                grad = torch.zeros(total, dtype=torch.float32, device=dev)
                shadow = torch.zeros(total, dtype=torch.bfloat16, device=dev)
            entries = []
            m_off = (total // moment_shard[1]) * moment_shard[0] if master_local else 0
            for (n, p), o in zip(params, offs):
                k = p.numel()
                if master_local:   # only the part of this parameter that falls into the local slice
                    a, b = max(o, m_off), min(o + k, m_off + master.numel())
                    if b > a:
                        master[a - m_off:b - m_off].copy_(p.detach().reshape(-1)[a - o:b - o].float())
                else:
                    master[o:o + k].copy_(p.detach().reshape(-1).float())
                shadow[o:o + k].copy_(p.detach().reshape(-1))
                gview = grad[o:o + k].view(p.shape)
                if p.dtype == torch.float32:
                    p.data = master[o:o + k].view(p.shape)
                    p.grad = gview
                elif p.dtype == torch.bfloat16:
                    p.data = shadow[o:o + k].view(p.shape)
                else:
                    raise TypeError(f"unsupported parameter dtype {p.dtype} for {n}")
                p._axb_grad = gview
                entries.append((n, p, o, k))
            tp_split = next((o for (n, p, o, k) in entries if getattr(p, "_tp_sharded", False)), total)
            if moment_shard is not None:
                mr, mw = moment_shard
                if total % (4 * mw):
                    raise ValueError("sharded moments need pad_multiple to be a multiple of 4 * world")
                m_len, m_lo = total // mw, (total // mw) * mr
            else:
                m_len, m_lo = total, 0
            self.groups.append({
                "m_lo": m_lo, "m_len": m_len, "master_local": master_local,
                "tp_split": tp_split,
                "name": g["name"], "lr_scale": g.get("lr_scale", 1.0), "weight_decay": g.get("weight_decay", 0.0),
                "master": master, "grad": grad, "shadow": shadow, "entries": entries,
                "exp_avg": torch.zeros(m_len, dtype=torch.float32, device=dev),
                "exp_avg_sq": torch.zeros(m_len, dtype=torch.float32, device=dev),
            })
        self._gnorm = None

    # ------------------------------------------------------------------
    def shadow_of(self, param):
        """bf16 shadow view matching ``param`` (used to bind LoRA GEMM operands)."""
        for g in self.groups:
            for n, p, o, k in g["entries"]:
                if p is param:
                    return g["shadow"][o:o + k].view(p.shape)
        return None

    @torch.no_grad()
    def reset_state(self, params, prune_ratio: float = 1.0):
        """Zeroes the AdamW moments of ``params`` (``prune_ratio`` < 1 keeps the largest-magnitude
        1 - ratio fraction, the magnitude pruning ReLoRA applies at every restart) and refreshes the
        bf16 shadows from the (possibly re-initialised) fp32 masters."""
        ids = {id(p) for p in params}
        for g in self.groups:
            for n, p, o, k in g["entries"]:
                if id(p) not in ids:
                    continue
                lo, hi = max(o, g["m_lo"]) - g["m_lo"], min(o + k, g["m_lo"] + g["m_len"]) - g["m_lo"]
                for key in ("exp_avg", "exp_avg_sq"):
                    if hi <= lo:
                        break
                    st = g[key][lo:hi]
                    k = hi - lo
                    if prune_ratio >= 1.0 or k < 2:
                        st.zero_()
                    else:
                        thr = st.abs().float().kthvalue(max(1, int(prune_ratio * k))).values
                        st.mul_((st.abs() > thr).to(st.dtype))
                if p.dtype == torch.float32 and not g.get("master_local"):
                    g["shadow"][o:o + k].copy_(g["master"][o:o + k])

    def bind_model_shadows(self, model):
        from ..models.layers import FusedLinear

        for m in model.modules():
            if isinstance(m, FusedLinear) and m.lora_A is not None and m.lora_A.is_cuda:
                a, b = self.shadow_of(m.lora_A), self.shadow_of(m.lora_B)
                if a is not None and b is not None:
                    m.lora_A16, m.lora_B16 = a, b

    def zero_grad(self):
        skip = self.skip_zero_grad_once
        self.skip_zero_grad_once = False
        for g in self.groups:
            if not skip:
                g["grad"].zero_()
            for _, p, _, _ in g["entries"]:
                if p.dtype != torch.float32:
                    p.grad = None

    def _fold_autograd_grads(self):
        for g in self.groups:
            for _, p, o, k in g["entries"]:
                if p.grad is not None and p.grad.data_ptr() != p._axb_grad.data_ptr():
                    p._axb_grad.add_(p.grad.float())
                    p.grad = None if p.dtype != torch.float32 else p._axb_grad
                elif p.dtype == torch.float32 and p.grad is None:
                    p.grad = p._axb_grad

    def flat_grads(self):
        self._fold_autograd_grads()
        return [g["grad"] for g in self.groups]

    def grad_norm_sq(self, extra_reduce=None):
        """Device scalar with the squared global gradient norm (before scaling/clipping)."""
        self._fold_autograd_grads()
        ss = None
        for g in self.groups:
            ss = grad_sumsq(g["grad"], ss)
        if extra_reduce is not None:
            ss = extra_reduce(ss)
        self._gnorm = ss
        return ss

    def set_active_layers(self, layers):
        """LISA: only the parameter groups of these decoder layers (and the groups outside any layer)
        are updated; the others keep weights AND moments untouched, like parameters without a
        gradient in a per-tensor optimizer. ``None`` re-activates everything."""
        keep = None if layers is None else {f"layers.{int(i)}" for i in layers}
        for g in self.groups:
            tag = g["name"].partition("@")[2]
            g["active"] = keep is None or not tag or tag in keep

    def step(self, lr=None, gnorm_sq=None):
        if self.moment_shard is not None:
            raise RuntimeError("this optimizer holds sharded moments: it is stepped by the fused parallel runtime")
        self.step_count += 1
        lr = self.lr if lr is None else lr
        if gnorm_sq is None and self.max_grad_norm and self.max_grad_norm > 0:
            gnorm_sq = self.grad_norm_sq()
        else:
            self._fold_autograd_grads()
        for g in self.groups:
            if not g.get("active", True):
                continue
            adamw_step_(g["master"], g["grad"], g["exp_avg"], g["exp_avg_sq"], step=self.step_count,
                        lr=lr * g["lr_scale"], beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                        weight_decay=g["weight_decay"], bf16_copy=g["shadow"], gnorm_sq=gnorm_sq,
                        max_norm=float(self.max_grad_norm or 0.0), grad_scale=self.grad_scale)
        return gnorm_sq

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self):
        return {"step": self.step_count, "lr": self.lr,
                "groups": [{"name": g["name"], "names": [e[0] for e in g["entries"]],
                            "exp_avg": g["exp_avg"].cpu(), "exp_avg_sq": g["exp_avg_sq"].cpu(),
                            "master": g["master"].cpu()} for g in self.groups]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, s in zip(self.groups, sd["groups"]):
            if [e[0] for e in g["entries"]] != s["names"]:
                raise ValueError(f"optimizer group '{g['name']}' does not match the checkpoint")
            g["exp_avg"].copy_(s["exp_avg"])
            g["exp_avg_sq"].copy_(s["exp_avg_sq"])
            g["master"].copy_(s["master"])
            if not g.get("master_local"):   # a local master slice cannot rebuild the complete bf16 copy
                g["shadow"].copy_(s["master"])


class TorchOptimizerAdapter:
    """Wraps any ``torch.optim`` optimizer behind the FlatAdamW interface (used for optimizers
    without a fused kernel: SGD, Adagrad, Adafactor-like user classes...)."""

    def __init__(self, opt, params, max_grad_norm=0.0, model=None):
        self.opt, self.params, self.max_grad_norm, self.model = opt, list(params), max_grad_norm, model
        self.step_count = 0
        self.grad_scale = 1.0
        self.lr = opt.param_groups[0]["lr"]
        self._base_lrs = [g["lr"] for g in opt.param_groups]

    moment_shard = None   # state lives inside the wrapped torch optimizer, never sharded by the fused runtime

    def zero_grad(self):
        self.opt.zero_grad(set_to_none=True)

    def flat_grads(self):
        return [p.grad for p in self.params if p.grad is not None]

    def grad_norm_sq(self, extra_reduce=None):
        ss = torch.zeros(1, dtype=torch.float32, device=self.params[0].device)
        for p in self.params:
            if p.grad is not None:
                ss += p.grad.float().pow(2).sum()
        return extra_reduce(ss) if extra_reduce is not None else ss

    def set_active_layers(self, layers):
        """LISA: only the parameter groups of these decoder layers (and the groups outside any layer)
        are updated; the others keep weights AND moments untouched, like parameters without a
        gradient in a per-tensor optimizer. ``None`` re-activates everything."""
        keep = None if layers is None else {f"layers.{int(i)}" for i in layers}
        for g in self.groups:
            tag = g["name"].partition("@")[2]
            g["active"] = keep is None or not tag or tag in keep

    def step(self, lr=None, gnorm_sq=None):
        self.step_count += 1
        if lr is not None:
            for g, b in zip(self.opt.param_groups, self._base_lrs):
                g["lr"] = lr * (b / self.lr if self.lr else 1.0)
        if self.grad_scale != 1.0:
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(self.grad_scale)
        if self.max_grad_norm and self.max_grad_norm > 0:
            if gnorm_sq is None:
                gnorm_sq = self.grad_norm_sq()
            coef = (self.max_grad_norm / (gnorm_sq.sqrt() * self.grad_scale + 1e-6)).clamp(max=1.0)
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(coef.to(p.grad.dtype))
        self.opt.step()
        if self.model is not None and hasattr(self.model, "refresh_lora_shadows"):
            self.model.refresh_lora_shadows()
        return gnorm_sq

    def state_dict(self):
        return {"step": self.step_count, "opt": self.opt.state_dict()}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.opt.load_state_dict(sd["opt"])


# ------------------------------------------------------------------------------ LR schedules
def _warmup(step, warmup):
    return float(step) / float(max(1, warmup))


def make_lr_lambda(kind: str, total_steps: int, warmup_steps: int = 0, *, min_lr_ratio: float = 0.0,
                   num_cycles: float = 0.5, constant_lr_ratio: float | None = None,
                   decay_steps: int | None = None, rex_max=1.0, rex_min=0.0):
    """Multiplier of the base LR at optimizer step ``step`` (0-based), mirroring the schedulers the
    reference exposes (HF cosine/linear/constant families, cosine_with_min_lr, quadratic-warmup
    cosine, rex, warmup-stable-decay; src/axolotl/utils/schedulers.py:12-358)."""
    kind = kind or "cosine"
    T, W = max(1, total_steps), warmup_steps

    def cosine(step):
        if step < W:
            return _warmup(step, W)
        prog = float(step - W) / float(max(1, T - W))
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * prog)))

    def cosine_min(step):
        if step < W:
            return _warmup(step, W)
        prog = min(1.0, float(step - W) / float(max(1, T - W)))
        return min_lr_ratio + (1 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * prog))

    def cosine_quadratic(step):
        if step < W:
            return _warmup(step, W) ** 2
        return cosine(step)

    def linear(step):
        if step < W:
            return _warmup(step, W)
        return max(0.0, float(T - step) / float(max(1, T - W)))

    def constant(step):
        return 1.0

    def constant_warmup(step):
        return _warmup(step, W) if step < W else 1.0

    def rex(step):
        if step < W:
            return _warmup(step, W)
        prog = float(step - W) / float(max(1, T - W))
        return rex_min + (rex_max - rex_min) * ((1 - prog) / (1 - prog / 2))

    def wsd(step):  # warmup - stable - decay
        d = decay_steps if decay_steps is not None else max(1, int(0.1 * T))
        if step < W:
            return _warmup(step, W)
        if step < T - d:
            return 1.0
        return max(min_lr_ratio, float(T - step) / float(d))

    def one_cycle(step):
        peak = max(1, int(0.3 * T))
        if step < peak:
            return 0.04 + (1 - 0.04) * 0.5 * (1 - math.cos(math.pi * step / peak))
        prog = (step - peak) / max(1, T - peak)
        return 1e-4 + (1 - 1e-4) * 0.5 * (1 + math.cos(math.pi * prog))

    def cosine_constant(step):  # cosine down to constant_lr_ratio over the first part, then flat
        ratio = constant_lr_ratio if constant_lr_ratio is not None else 0.1
        return max(ratio, cosine_min(step)) if min_lr_ratio else max(ratio, cosine(step))

    table = {
        "cosine": cosine, "cosine_with_restarts": cosine, "linear": linear, "constant": constant,
        "constant_with_warmup": constant_warmup, "cosine_with_min_lr": cosine_min,
        "cosine_with_quadratic_warmup": cosine_quadratic, "rex": rex, "warmup_stable_decay": wsd,
        "one_cycle": one_cycle, "cosine_min_lr": cosine_min, "constant_with_cosine": cosine_constant,
    }
    if kind not in table:
        raise ValueError(f"lr_scheduler '{kind}' is not supported (have: {sorted(table)})")
    return table[kind]


def jagged_restarts(base_lambda, restart_steps: int, warmup_steps: int = 10, anneal_steps: int = 1,
                    min_scale: float = 0.001):
    """Wraps a schedule with periodic restarts: after every ``restart_steps`` optimizer steps the LR
    is annealed to ``min_scale`` over ``anneal_steps`` and warmed up again over ``warmup_steps``
    (ReLoRA's saw-tooth; reference: JaggedLRRestartScheduler, src/axolotl/utils/schedulers.py)."""

    def f(step):
        base = base_lambda(step)
        if restart_steps <= 0 or step < restart_steps - anneal_steps:
            return base
        pos = step % restart_steps
        if pos < warmup_steps and step >= restart_steps:
            scale = min_scale + (1 - min_scale) * pos / max(1, warmup_steps)
        elif pos >= restart_steps - anneal_steps:
            scale = min_scale + (1 - min_scale) * (restart_steps - pos) / max(1, anneal_steps)
        else:
            scale = 1.0
        return base * scale

    return f


def default_warmup_steps(total_steps, warmup_steps=None, warmup_ratio=None):
    """explicit steps > ratio > min(3% of total, 100); a value of 1 is bumped to 2
    (src/axolotl/core/builders/base.py:235-258)."""
    if warmup_steps is not None:
        w = int(warmup_steps)
    elif warmup_ratio is not None:
        w = int(warmup_ratio * total_steps)
    else:
        w = min(int(0.03 * total_steps), 100)
    return 2 if w == 1 else w
