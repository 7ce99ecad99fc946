"""Sparse mixture-of-experts block (Qwen3-MoE / Mixtral routing) with per-expert LoRA.

Routing: softmax over experts -> top-k -> optional renormalisation; the load-balance auxiliary
loss follows the Switch/HF definition (E * sum_e f_e * P_e). Expert weights are stored fused as
``gate_up_proj`` [E, 2I, H] and ``down_proj`` [E, H, I] (HF v5 fused-expert layout) either in bf16
or frozen NVFP4 (packed nibbles + E4M3 block scales + fp32 per-tensor scale, see ops/nvfp4.py).
Expert LoRA uses the PEFT ``target_parameters`` layout: A [E*r, in] expert-major rows,
B [out, r*E] rank-major columns (reference: src/axolotl/integrations/expert_parallel/shard.py:279-303).

The local expert computation sorts tokens by expert and runs one grouped pass; with expert
parallelism the dispatch / combine is delegated to ``parallel.ep`` (installed as ``self.ep``).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Fn
from ..ops.lora import linear
from .config import ModelConfig
from .layers import adapters_enabled


def route_topk(router_logits, k, norm_topk_prob=True):
    """(weights [T,k] fp32, indices [T,k] int64, probs [T,E] fp32)."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, probs


def route_deepseek(router_logits, k, *, scoring="sigmoid", bias=None, n_group=1, topk_group=1, group_score="top2",
                   norm_topk_prob=True, scale=1.0):
    """DeepSeek-V2 / V3 routing. Scores are sigmoid (V3) or softmax (V2) of the router logits; with ``n_group`` > 1
    only the experts of the ``topk_group`` best groups compete (a group is rated by the sum of its two best
    biased scores in V3, by its best score in V2); ``bias`` (V3 ``e_score_correction_bias``) steers the CHOICE
    only, the mixing weights are the unbiased scores, optionally renormalised, times ``scale``."""
    lf = router_logits.float()
    scores = torch.sigmoid(lf) if scoring == "sigmoid" else torch.softmax(lf, -1)
    choice = scores + bias.float()[None] if bias is not None else scores
    T, E = scores.shape
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        rate = g.topk(2, dim=-1)[0].sum(-1) if group_score == "top2" else g.max(-1)[0]
        keep = torch.zeros_like(rate, dtype=torch.bool).scatter_(1, rate.topk(topk_group, dim=-1)[1], True)
        choice = choice.masked_fill(~keep[:, :, None].expand(T, n_group, E // n_group).reshape(T, E),
                                    0.0)
    idx = choice.topk(k, dim=-1)[1]
    w = scores.gather(1, idx)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scale, idx, scores


def load_balance_loss(probs, idx, num_experts):
    """E * sum_e (fraction of routed slots on e) * (mean router prob of e)."""
    T, k = idx.shape
    onehot = F.one_hot(idx, num_experts).float()          # [T, k, E]
    tokens_per_expert = onehot.mean(0)                     # [k, E]
    router_prob = probs.mean(0)                            # [E]
    return num_experts * (tokens_per_expert * router_prob[None]).sum()


class Experts(nn.Module):
    """E SwiGLU experts with fused weights and optional per-expert LoRA."""

    def __init__(self, num_experts, hidden, inter, act, dtype, device):
        super().__init__()
        self.E, self.H, self.I, self.act = num_experts, hidden, inter, act
        self.glu_limit = None      # clamped SwiGLU (config key ``swiglu_limit``)
        self.gate_up_proj = nn.Parameter(torch.empty(num_experts, 2 * inter, hidden, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(num_experts, hidden, inter, dtype=dtype, device=device))
        self.nvfp4 = None          # dict with packed tensors when the experts are frozen in NVFP4
        self.lora = None           # dict: gate_up_A [E*r,H], gate_up_B [2I,r*E], down_A [E*r,I], down_B [H,r*E]
        self.lora_r = 0
        self.scaling = 1.0
        self.expert_offset = 0     # first global expert id held locally (expert parallelism)
        self.gate_up_bias = None   # [E, 2I] / [E, H] per-expert biases (gpt-oss)
        self.down_bias = None

    def add_biases(self, dtype, device):
        self.gate_up_bias = nn.Parameter(torch.zeros(self.E, 2 * self.I, dtype=dtype, device=device))
        self.down_bias = nn.Parameter(torch.zeros(self.E, self.H, dtype=dtype, device=device))

    # ------------------------------------------------------------------ LoRA (PEFT target_parameters layout)
    def add_lora(self, r, alpha, use_rslora=False, dtype=torch.float32):
        dev = self.gate_up_proj.device if self.nvfp4 is None else self.nvfp4["gate_up"]["qdata"].device
        E, H, I = self.E, self.H, self.I
        if dev.type == "cuda" and r % 8:
            raise ValueError(f"lora_r={r}: the tensor-core path needs an adapter rank that is a multiple of 8")

        def mk_a(inp):
            a = torch.empty(E * r, inp, dtype=dtype, device=dev)
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
            return nn.Parameter(a)

        self.lora = nn.ParameterDict({
            "gate_up_A": mk_a(H), "gate_up_B": nn.Parameter(torch.zeros(2 * I, r * E, dtype=dtype, device=dev)),
            "down_A": mk_a(I), "down_B": nn.Parameter(torch.zeros(H, r * E, dtype=dtype, device=dev)),
        })
        self.lora_r = r
        self.scaling = alpha / math.sqrt(r) if use_rslora else alpha / r

    def expert_lora(self, which, e):
        """(A_e [r, in], B_e [out, r]) for local expert e."""
        r, E = self.lora_r, self.E
        A = self.lora[which + "_A"][e * r:(e + 1) * r]
        B = self.lora[which + "_B"].view(-1, r, E)[:, :, e]
        return A, B

    def expert_weight(self, which, e):
        if self.nvfp4 is not None:
            from ..ops.nvfp4 import dequantize_nvfp4

            q = self.nvfp4[which]
            return dequantize_nvfp4(q["qdata"][e], q["scale"][e], q["pts"][e])
        return (self.gate_up_proj if which == "gate_up" else self.down_proj)[e]

    # ------------------------------------------------------------------ compute
    def forward(self, x_sorted, counts):
        """x_sorted: tokens grouped by local expert ([M, H]); counts: python list of per-expert rows."""
        if x_sorted.is_cuda:
            from ..ops.grouped import grouped_experts_forward

            return grouped_experts_forward(self, x_sorted, counts)
        outs = []
        start = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            xe = x_sorted[start:start + n]
            start += n
            gu = linear(xe, self.expert_weight("gate_up", e))
            use_lora = self.lora is not None and adapters_enabled()
            if use_lora:
                A, B = self.expert_lora("gate_up", e)
                gu = gu + self.scaling * ((xe @ A.to(xe.dtype).t()) @ B.to(xe.dtype).t())
            if self.gate_up_bias is not None:
                gu = gu + self.gate_up_bias[e].to(gu.dtype)
            h = Fn.glu(gu, self.act, self.glu_limit)
            y = linear(h, self.expert_weight("down", e))
            if use_lora:
                A, B = self.expert_lora("down", e)
                y = y + self.scaling * ((h @ A.to(h.dtype).t()) @ B.to(h.dtype).t())
            if self.down_bias is not None:
                y = y + self.down_bias[e].to(y.dtype)
            outs.append(y)
        if not outs:
            return x_sorted.new_zeros((0, self.H))
        return torch.cat(outs, 0)


class _DenseRouterGrad(torch.autograd.Function):
    """Straight-through router gradient (DenseMixer): the forward value is zero, the backward pass
    hands every NON-selected expert e of token t the gradient <dy_t, O_e(x_t)> on its router
    probability, as if the layer output were the dense mixture sum_e p_e O_e(x). The selected experts
    get theirs through the sparse path. Costs one evaluation of every expert on every token in the
    backward pass (no expert or input gradient is taken through it)."""

    @staticmethod
    def forward(ctx, probs, x, idx, moe):
        ctx.moe, ctx.E = moe, probs.shape[1]
        ctx.save_for_backward(x, idx)
        return x.new_zeros(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x, idx = ctx.saved_tensors
        T, E = x.shape[0], ctx.E
        g = torch.zeros(T, E, dtype=torch.float32, device=x.device)
        dyf = dy.float()
        with torch.no_grad():
            for e in range(E):
                counts = [0] * E
                counts[e] = T
                g[:, e] = (dyf * ctx.moe.experts(x, counts).float()).sum(-1)
        sel = torch.zeros(T, E, dtype=torch.bool, device=x.device).scatter_(1, idx, True)
        return g.masked_fill(sel, 0.0), None, None, None


class SparseMoE(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.E, self.k = cfg.num_experts, cfg.num_experts_per_tok
        self.norm_topk_prob = cfg.norm_topk_prob
        self.gate = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden_size, dtype=dtype, device=device))
        self.experts = Experts(cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, cfg.hidden_act,
                               dtype, device)
        self.aux_coef = cfg.router_aux_loss_coef
        # Gemma 4: its router normalises and scales its own input and scales the chosen experts' weights
        self.gemma4 = cfg.model_type == "gemma4_text"
        if self.gemma4:
            self.router_eps = cfg.rms_norm_eps
            self.router_scale = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
            self.per_expert_scale = nn.Parameter(torch.ones(cfg.num_experts, dtype=dtype, device=device))
        self.ep = None  # parallel.ep.ExpertParallelGroup when experts are sharded across ranks
        self.dense_mixer = False   # DenseMixer plugin: straight-through router gradient over all experts
        # Qwen2-MoE: a dense "shared" expert runs on every token, scaled by a sigmoid gate
        self.shared_expert = None
        self.shared_expert_gate = None
        shared_I = (cfg.extra or {}).get("shared_expert_intermediate_size") if cfg.model_type in ("qwen2_moe", "qwen3_next", "qwen3_5_moe_text") else None
        if shared_I:
            from .transformer import MLP

            self.shared_expert = MLP(cfg.hidden_size, shared_I, cfg.hidden_act, False, dtype, device)
            self.shared_expert_gate = nn.Parameter(torch.empty(1, cfg.hidden_size, dtype=dtype, device=device))
        # Llama 4: the sigmoid of the chosen logit scales the expert's INPUT; one always-on shared expert
        self.input_scaled = cfg.model_type == "llama4_text"
        if self.input_scaled:
            from .transformer import MLP

            if self.k != 1:
                raise ValueError("Llama 4 routing scales the expert input, which is implemented for num_experts_per_tok = 1")
            self._llama4_shared = MLP(cfg.hidden_size, cfg.moe_intermediate_size, cfg.hidden_act, False, dtype, device)
        # Granite 4.0-H: the k best LOGITS are soft-maxed among themselves; one always-on shared MLP
        self.topk_softmax = cfg.model_type in ("granitemoe", "granitemoeshared", "granitemoehybrid")
        if self.topk_softmax:
            from .transformer import MLP

            shared = int((cfg.extra or {}).get("shared_intermediate_size") or 0) if cfg.model_type != "granitemoe" else 0
            self.shared_experts = MLP(cfg.hidden_size, shared, cfg.hidden_act, False, dtype, device, fused_names=True) \
                if shared else None
        # gpt-oss: router and experts carry biases; the k best LOGITS are chosen, then soft-maxed among themselves
        self.router_bias = None
        if cfg.model_type == "gpt_oss":
            self.router_bias = nn.Parameter(torch.zeros(cfg.num_experts, dtype=dtype, device=device))
            self.experts.add_biases(dtype, device)
        # DeepSeek-V2 / V3: grouped (sigmoid) routing, always-on shared experts, scaled mixing weights
        self.deepseek = None
        if not self.topk_softmax:
            self.shared_experts = None
        if self.input_scaled:
            self.shared_experts = self._llama4_shared
            del self._llama4_shared
        self.e_score_correction_bias = None
        if cfg.model_type in ("deepseek_v2", "deepseek_v3", "glm_moe_dsa", "glm4_moe", "minimax_m2", "hunyuan_v1_moe", "ernie4_5_moe", "mistral4", "lfm2_moe", "afmoe"):
            from .transformer import MLP

            ex = cfg.extra or {}
            v3 = cfg.model_type not in ("deepseek_v2", "hunyuan_v1_moe", "ernie4_5_moe")
            grouped = v3 or ex.get("topk_method") == "group_limited_greedy"
            soft = "softmax" if cfg.model_type in ("hunyuan_v1_moe", "ernie4_5_moe") else (ex.get("scoring_func") or "softmax")
            self.deepseek = dict(scoring="sigmoid" if v3 else soft,
                                 n_group=int(ex.get("n_group") or 1) if grouped else 1,
                                 topk_group=int(ex.get("topk_group") or 1), group_score="top2" if v3 else "max",
                                 norm_topk_prob=bool(cfg.norm_topk_prob), scale=float(ex.get("routed_scaling_factor") or 1.0))
            if cfg.model_type == "mistral4":      # softmax scores, groups rated by their two best, no selection bias
                self.deepseek.update(scoring="softmax", n_group=int(ex.get("n_group") or 1), group_score="top2")
            if (v3 and cfg.model_type not in ("mistral4", "lfm2_moe")) or cfg.model_type == "ernie4_5_moe" \
                    or (cfg.model_type == "lfm2_moe" and ex.get("use_expert_bias", True)):
                self.e_score_correction_bias = nn.Parameter(torch.zeros(cfg.num_experts, dtype=torch.float32, device=device),
                                                            requires_grad=False)
            n_shared = int(ex.get("n_shared_experts") or ex.get("moe_num_shared_experts") or 0)
            if cfg.model_type == "hunyuan_v1_moe":
                n_shared = 1
            if n_shared:
                self.shared_experts = MLP(cfg.hidden_size, cfg.moe_intermediate_size * n_shared, cfg.hidden_act, False,
                                          dtype, device)

    def _shared(self, x):
        g = self.shared_expert_gate
        if x.is_cuda:   # the tensor-core GEMM wants 16-byte output rows: pad the 1-row gate to 8 rows
            g8 = torch.cat([g, g.new_zeros(7, g.shape[1])], 0)
            gl = linear(x, g8)[:, :1]
        else:
            gl = linear(x, g)
        return torch.sigmoid(gl.float()).to(x.dtype) * self.shared_expert(x)

    def forward(self, x, router_x=None):
        y, aux = self._routed(x, router_x)
        if self.dense_mixer and self.training and torch.is_grad_enabled():
            if self.ep is not None:
                raise NotImplementedError("dense_mixer needs all experts on the rank (no expert parallelism)")
            y = y + _DenseRouterGrad.apply(self._last_probs, x.detach(), self._last_idx, self)
        if self.shared_expert is not None:
            y = y + self._shared(x)
        if self.shared_experts is not None:
            y = y + self.shared_experts(x)
        return y, aux

    def _routed(self, x, router_x=None):
        T, H = x.shape
        if self.gemma4:
            # the router reads the un-normed stream: RMS-normalise (no weight), scale per channel and by H^-1/2; softmax
            # over all experts, the k best renormalised, then a learned scale per chosen expert
            r = router_x.float()
            r = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + self.router_eps) * self.router_scale.float() * (H ** -0.5)
            probs = torch.softmax(r @ self.gate.float().t(), -1)
            w, idx = torch.topk(probs, self.k, dim=-1)
            w = (w / w.sum(-1, keepdim=True)) * self.per_expert_scale.float()[idx]
        elif self.deepseek is not None:
            logits = x.float() @ self.gate.float().t()       # HF keeps this router in fp32
            w, idx, probs = route_deepseek(logits, self.k, bias=self.e_score_correction_bias, **self.deepseek)
        elif self.input_scaled:
            logits = linear(x, self.gate).float()
            top, idx = torch.topk(logits, 1, dim=-1)
            x = (x.float() * torch.sigmoid(top)).to(x.dtype)        # the score goes in, the expert output comes back unweighted
            w, probs = torch.ones_like(top), torch.softmax(logits, -1)
        elif self.router_bias is not None or self.topk_softmax:
            logits = linear(x, self.gate).float()
            if self.router_bias is not None:
                logits = logits + self.router_bias.float()
            top, idx = torch.topk(logits, self.k, dim=-1)
            w, probs = torch.softmax(top, -1), torch.softmax(logits, -1)
        else:
            logits = linear(x, self.gate)
            w, idx, probs = route_topk(logits, self.k, self.norm_topk_prob)
        if self.dense_mixer:
            self._last_probs, self._last_idx = probs, idx
        aux = load_balance_loss(probs, idx, self.E) if self.training or self.aux_coef else None
        if self.ep is not None:
            y = self.ep.dispatch_compute_combine(self.experts, x, w, idx)
            return y, aux
        if x.is_cuda:
            from ..ops.grouped import moe_local_forward

            return moe_local_forward(self.experts, x, w, idx, self.E), aux
        # local: sort the T*k routed slots by expert
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = order // self.k
        counts = torch.bincount(flat_e, minlength=self.E).tolist()
        xs = x.index_select(0, tok)
        ys = self.experts(xs, counts)
        ws = w.reshape(-1).index_select(0, order).to(ys.dtype)
        y = torch.zeros_like(x)
        y.index_add_(0, tok, ys * ws[:, None])
        return y, aux
