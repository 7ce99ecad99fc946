"""Decoder-only causal LM (Llama / Mistral / Phi-3 / Qwen2 / Qwen3 / Qwen3-MoE / Mixtral block graph).

The model works on *packed token streams*: ``input_ids`` [B, S] is flattened to T = B*S tokens,
documents are delimited by resets of ``position_ids`` (and by row starts), attention is causal
inside each document (varlen flash attention kernel), and the loss is a chunked linear +
cross-entropy that never builds [T, V] logits. This is the layout the reference obtains from its
V2 collator + flash-attn varlen path (src/axolotl/utils/collators/batching.py:158-196,
src/axolotl/monkeypatch/utils.py:111-169) without the segment-id mask round trip.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..ops import functional as Fn
from ..ops.lora import glu_mlp, linear
from .config import ModelConfig
from .layers import FusedLinear, RMSNorm, adapters_enabled, make_norm

IGNORE_INDEX = -100


@dataclass
class CausalLMOutput:
    loss: torch.Tensor | None = None
    logits: torch.Tensor | None = None
    hidden_states: torch.Tensor | None = None
    aux_loss: torch.Tensor | None = None
    num_items: int = 0
    captured: dict | None = None


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, head_dim=None, kv_heads=None, k_eq_v=False):
        super().__init__()
        self.Hq, self.Hk, self.D = cfg.num_attention_heads, kv_heads or cfg.num_key_value_heads, head_dim or cfg.head_dim
        H = cfg.hidden_size
        self.k_eq_v = k_eq_v           # Gemma 4 global layers: values are the (un-normed, un-rotated) keys
        self.kv_store, self.kv_src = False, None      # Gemma 4 key / value sharing (set by the layer)
        if k_eq_v:
            self.qkv_proj = FusedLinear(H, [self.Hq * self.D, self.Hk * self.D], ["q_proj", "k_proj"], bias=cfg.attention_bias,
                                        dtype=dtype, device=device)
        elif cfg.model_type == "falcon":  # one projection in the checkpoint (its rows re-ordered to q | k | v on load)
            self.qkv_proj = FusedLinear(H, [(self.Hq + 2 * self.Hk) * self.D], ["query_key_value"], bias=cfg.attention_bias,
                                        dtype=dtype, device=device)
        elif cfg.model_type == "phi3":   # the checkpoint (and its adapters) name the fused projection itself
            self.qkv_proj = FusedLinear(H, [(self.Hq + 2 * self.Hk) * self.D], ["qkv_proj"], bias=cfg.attention_bias,
                                        dtype=dtype, device=device)
        else:
            self.qkv_proj = FusedLinear(H, [self.Hq * self.D, self.Hk * self.D, self.Hk * self.D],
                                        ["q_proj", "k_proj", "v_proj"], bias=cfg.attention_bias,
                                        dtype=dtype, device=device)
        o_bias = (cfg.attention_bias if cfg.model_type in ("gpt_oss", "olmo2", "olmo3", "starcoder2", "cohere", "cohere2", "nemotron", "phi", "falcon")
                  else bool((cfg.extra or {}).get("attention_out_bias")) if cfg.model_type == "seed_oss" else False)
        self.o_proj = FusedLinear(self.Hq * self.D, [H], ["o_proj"], bias=o_bias, dtype=dtype, device=device)
        # gpt-oss: one learned "sink" logit per head in every softmax denominator
        self.sinks = nn.Parameter(torch.zeros(self.Hq, dtype=dtype, device=device)) if cfg.model_type == "gpt_oss" else None
        # Qwen3-Next: the attention output is multiplied by sigmoid(gate(x)) before the output projection (the checkpoint
        # stores the gate rows inside q_proj, head by head; they are split off at load)
        self.out_gate = FusedLinear(H, [self.Hq * self.D], ["q_gate"], bias=cfg.attention_bias, dtype=dtype, device=device) \
            if cfg.model_type in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text") else None
        if cfg.model_type == "afmoe":      # Trinity: the same gate as a projection of its own
            self.out_gate = FusedLinear(H, [self.Hq * self.D], ["gate_proj"], dtype=dtype, device=device)
        off = cfg.norm_offset()
        self.q_norm = RMSNorm(self.D, cfg.rms_norm_eps, dtype, device, offset=off) if cfg.qk_norm else None
        self.k_norm = RMSNorm(self.D, cfg.rms_norm_eps, dtype, device, offset=off) if cfg.qk_norm else None
        self.clip_qkv = float((cfg.extra or {}).get("clip_qkv") or 0.0) if cfg.model_type == "olmo" else 0.0
        self.norm_after_rope = cfg.model_type in ("hunyuan_v1_dense", "hunyuan_v1_moe")   # HunYuan: per-head q / k norms act on the ROTATED vectors
        self.full_qk_norm = cfg.model_type in ("olmoe", "olmo2", "olmo3", "minimax_m2")   # OLMo family: q / k norms over ALL heads at once
        if self.full_qk_norm:
            self.q_norm = RMSNorm(self.Hq * self.D, cfg.rms_norm_eps, dtype, device)
            self.k_norm = RMSNorm(self.Hk * self.D, cfg.rms_norm_eps, dtype, device)
        self.eps = cfg.rms_norm_eps
        self.scale = cfg.multiplier("attention_multiplier")   # 1/sqrt(head_dim) except for Granite
        self.v_norm = cfg.model_type == "gemma4_text"         # Gemma 4: values are RMS-normalised per head (no learned scale)
        self.use_rope = True                                   # SmolLM3: some layers carry no position signal
        self.rot_dim = cfg.rope_dim() if cfg.rope_dim() < self.D else None   # partial rotary embedding (Phi-4-mini, Bamba)
        if cfg.model_type == "gemma4_text":      # its partial rotation is expressed by zero frequencies over the full width
            self.rot_dim = None
        self.window = cfg.sliding_window()                     # Mistral / Phi-3 ...: causal sliding window, 0 = none
        self.softcap = cfg.attn_softcap()                      # Gemma 2: scores -> cap * tanh(scores / cap)
        # Llama 4: unweighted per-head L2 norm of q / k on rotating layers; those layers attend inside chunks of
        # `attention_chunk_size` positions; position-free layers scale q by a slowly growing temperature
        ex = cfg.extra or {}
        self.llama4 = cfg.model_type == "llama4_text"
        self.chunk = 0
        self.temp = None
        if self.llama4:
            self.register_buffer("ones_d", torch.ones(self.D, dtype=dtype, device=device), persistent=False)
            self.l2_qk = bool(ex.get("use_qk_norm", True))
            self.temp = (float(ex.get("floor_scale") or 8192), float(ex.get("attn_scale") or 0.1)) if ex.get("attn_temperature_tuning", True) else None
        self.register_buffer("local_inv_freq", None, persistent=False)   # Gemma 3: sliding layers rotate with their own base
        # Ministral 3: queries grow with the position, 1 + beta * log(1 + floor(pos / original context))
        rp = ex.get("rope_parameters") or cfg.rope_scaling or {}
        self.q_pos_scale = (float(rp["llama_4_scaling_beta"]), float(rp.get("original_max_position_embeddings") or 1)) \
            if cfg.model_type == "ministral3" and rp.get("llama_4_scaling_beta") is not None else None

    def pre(self, x, positions, inv_freq, attn_scale):
        """Projections, q/k norms and rotary embedding: everything before the attention kernel."""
        qkv = self.qkv_proj(x)
        if self.k_eq_v:
            qkv = torch.cat([qkv, qkv[:, self.Hq * self.D:]], 1)
        if self.v_norm:
            T = qkv.shape[0]
            nqk = (self.Hq + self.Hk) * self.D
            v = qkv[:, nqk:].reshape(T * self.Hk, self.D).float()
            v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(qkv.dtype).reshape(T, self.Hk * self.D)
            qkv = torch.cat([qkv[:, :nqk], v], 1)
        if self.clip_qkv:
            qkv = qkv.clamp(-self.clip_qkv, self.clip_qkv)
        per_head_norm = self.q_norm is not None and not self.full_qk_norm
        if self.full_qk_norm:
            nq, nk = self.Hq * self.D, self.Hk * self.D
            q, _ = self.q_norm(qkv[..., :nq].contiguous())
            k, _ = self.k_norm(qkv[..., nq:nq + nk].contiguous())
            qkv = torch.cat([q, k, qkv[..., nq + nk:]], -1)
        if self.use_rope and per_head_norm and self.norm_after_rope:
            T = qkv.shape[0]
            nq, nk = self.Hq * self.D, self.Hk * self.D
            qkv = Fn.rope_qk_(qkv, positions, inv_freq, self.Hq, self.Hk, self.D, attn_scale, rot_dim=self.rot_dim)
            q = self.q_norm.plain(qkv[:, :nq].reshape(T * self.Hq, self.D)).reshape(T, nq)
            k = self.k_norm.plain(qkv[:, nq:nq + nk].reshape(T * self.Hk, self.D)).reshape(T, nk)
            return torch.cat([q, k, qkv[:, nq + nk:]], 1)
        if self.use_rope and per_head_norm and self.rot_dim is not None:
            # partial rotary embedding with q/k norms: the norms run on their own, then the first rot_dim dimensions rotate
            T = qkv.shape[0]
            nq, nk = self.Hq * self.D, self.Hk * self.D
            q = self.q_norm.plain(qkv[:, :nq].reshape(T * self.Hq, self.D)).reshape(T, nq)
            k = self.k_norm.plain(qkv[:, nq:nq + nk].reshape(T * self.Hk, self.D)).reshape(T, nk)
            qkv = torch.cat([q, k, qkv[:, nq + nk:]], 1)
            return Fn.rope_qk_(qkv, positions, inv_freq, self.Hq, self.Hk, self.D, attn_scale, rot_dim=self.rot_dim)
        if self.use_rope:
            if self.local_inv_freq is not None:
                inv_freq, attn_scale = self.local_inv_freq, 1.0
            if self.llama4 and self.l2_qk:       # the norm commutes with the rotation, so it runs in the same kernel
                qkv = Fn.rope_qk_(qkv, positions, inv_freq, self.Hq, self.Hk, self.D, attn_scale, self.ones_d, self.ones_d, self.eps)
            else:
                qkv = Fn.rope_qk_(qkv, positions, inv_freq, self.Hq, self.Hk, self.D, attn_scale,
                                  self.q_norm.effective_weight() if per_head_norm else None,
                                  self.k_norm.effective_weight() if per_head_norm else None, self.eps, rot_dim=self.rot_dim)
            if self.q_pos_scale is not None:
                beta, orig = self.q_pos_scale
                t = 1.0 + beta * torch.log1p(torch.floor(positions.float() / orig))
                nq = self.Hq * self.D
                qkv = torch.cat([(qkv[:, :nq].float() * t[:, None]).to(qkv.dtype), qkv[:, nq:]], 1)
        elif per_head_norm:                  # a position-free layer still normalises q / k per head (Trinity's global layers)
            T = qkv.shape[0]
            nq, nk = self.Hq * self.D, self.Hk * self.D
            q = self.q_norm.plain(qkv[:, :nq].reshape(T * self.Hq, self.D)).reshape(T, nq)
            k = self.k_norm.plain(qkv[:, nq:nq + nk].reshape(T * self.Hk, self.D)).reshape(T, nk)
            qkv = torch.cat([q, k, qkv[:, nq + nk:]], 1)
        elif self.llama4 and self.temp is not None:
            floor_scale, a = self.temp
            t = torch.log1p(torch.floor((positions.float() + 1.0) / floor_scale)) * a + 1.0
            nq = self.Hq * self.D
            qkv = torch.cat([(qkv[:, :nq].float() * t[:, None]).to(qkv.dtype), qkv[:, nq:]], 1)
        return qkv

    def core(self, qkv, meta):
        cache = getattr(meta, "kv_cache", None)
        if cache is not None:   # generation: keep the rotated k / v of every token
            return cache.attend(self.layer_idx, qkv, meta, self.Hq, self.Hk, self.D, self.scale, self.window)
        if self.chunk and getattr(meta, "causal", True):
            if getattr(meta, "cp", False):
                raise NotImplementedError("chunked attention is not available with context parallelism")
            meta = meta.chunked(self.chunk)
        if self.window and getattr(meta, "causal", True):
            if getattr(meta, "cp", False):
                raise NotImplementedError("sliding-window attention is not available with context parallelism")
            meta = meta.windowed(self.window)   # a no-op while no document exceeds the window
        return Fn.flash_varlen(qkv, meta, self.Hq, self.Hk, self.D, self.scale, softcap=self.softcap, sinks=self.sinks)

    def share_kv(self, qkv, meta):
        """Gemma 4's last layers attend the keys / values of the last earlier layer of their kind that still makes its own
        (after its norms and rotation); that layer leaves them on the batch's attention descriptor."""
        nq = self.Hq * self.D
        if self.kv_store:
            meta.shared_kv[self.layer_idx] = qkv[:, nq:]
        if self.kv_src is not None:
            qkv = torch.cat([qkv[:, :nq], meta.shared_kv[self.kv_src]], 1)
        return qkv

    def forward(self, x, positions, inv_freq, attn_scale, meta):
        qkv = self.pre(x, positions, inv_freq, attn_scale)
        if self.kv_store or self.kv_src is not None:
            qkv = self.share_kv(qkv, meta)
        a = self.core(qkv, meta)
        if self.out_gate is not None:
            a = (a.float() * torch.sigmoid(self.out_gate(x).float())).to(a.dtype)
        return self.o_proj(a)


class MLP(nn.Module):
    def __init__(self, hidden, inter, act, bias, dtype, device, fused_names=False):
        super().__init__()
        if fused_names:
            self.gate_up_proj = FusedLinear(hidden, [2 * inter], ["gate_up_proj"], bias=bias, dtype=dtype, device=device)
        else:
            self.gate_up_proj = FusedLinear(hidden, [inter, inter], ["gate_proj", "up_proj"], bias=bias,
                                            dtype=dtype, device=device)
        self.down_proj = FusedLinear(inter, [hidden], ["down_proj"], bias=bias, dtype=dtype, device=device)
        self.act = act
        self.glu_limit = None   # clamped SwiGLU (config key ``swiglu_limit``)
        self.tile_rows = None   # tiled MLP: rows per tile (None = whole sequence at once)
        self.gate_multiplier, self.down_multiplier = 1.0, 1.0   # Falcon-H1: scalars on the gate half and on the output

    def _mlp(self, x):
        if self.gate_multiplier != 1.0 or self.down_multiplier != 1.0:
            gu = self.gate_up_proj(x)
            inter = gu.shape[-1] // 2
            gu = torch.cat([gu[..., :inter] * self.gate_multiplier, gu[..., inter:]], -1)
            return self.down_proj(Fn.glu(gu, self.act, self.glu_limit)) * self.down_multiplier
        if x.is_cuda:   # one autograd node with the GLU folded into the GEMM epilogues, when it applies
            y = glu_mlp(x, self.gate_up_proj, self.down_proj, Fn._ACT_KIND[self.act], self.glu_limit, adapters_enabled())
            if y is not None:
                return y
        return self.down_proj(Fn.glu(self.gate_up_proj(x), self.act, self.glu_limit))

    def forward(self, x):
        """With ``tile_rows`` set, the token rows go through the MLP tile by tile and every tile's
        [rows, 2I] / [rows, I] intermediates are recomputed in the backward pass, so their peak size
        no longer grows with the sequence length (the reference's Tiled MLP for very long contexts,
        src/axolotl/monkeypatch/tiled_mlp/base.py:21-453)."""
        t = self.tile_rows
        if t is None or x.shape[0] <= t or not (self.training and torch.is_grad_enabled()):
            return self._mlp(x)
        outs = [checkpoint(self._mlp, x[i:i + t], use_reentrant=False) for i in range(0, x.shape[0], t)]
        return torch.cat(outs, 0)


class PlainMLP(nn.Module):
    """up -> activation -> down without a gate (Nemotron-H: squared ReLU; Apertus: xIELU with two learnable scalars per
    layer, alpha_p x^2 + beta x for x > 0 and alpha_n (expm1(min(x, eps)) - x) + beta x otherwise)."""

    def __init__(self, hidden, inter, act, bias, dtype, device):
        super().__init__()
        self.up_proj = FusedLinear(hidden, [inter], ["up_proj"], bias=bias, dtype=dtype, device=device)
        self.down_proj = FusedLinear(inter, [hidden], ["down_proj"], bias=bias, dtype=dtype, device=device)
        if act not in ("relu2", "relu", "gelu", "silu", "gelu_pytorch_tanh", "gelu_new", "xielu"):
            raise ValueError(f"activation '{act}' is not available for an ungated MLP")
        self.act = act
        if act == "xielu":       # stored through an inverse softplus, as the checkpoints do (alpha_p = 0.8, alpha_n = 0.8 - beta)
            self.xielu_beta, self.xielu_eps = 0.5, -1e-6
            self.alpha_p = nn.Parameter(torch.log(torch.expm1(torch.tensor([0.8]))).to(dtype=dtype, device=device))
            self.alpha_n = nn.Parameter(torch.log(torch.expm1(torch.tensor([0.8 - 0.5]))).to(dtype=dtype, device=device))

    def forward(self, x):
        u = self.up_proj(x)
        if self.act == "xielu":
            ap = torch.nn.functional.softplus(self.alpha_p.float())
            an = self.xielu_beta + torch.nn.functional.softplus(self.alpha_n.float())
            u = Fn.xielu(u, ap, an, self.xielu_beta, self.xielu_eps)
        elif self.act == "relu2":
            u = torch.relu(u).square()
        elif self.act == "relu":
            u = torch.relu(u)
        elif self.act == "gelu":
            u = torch.nn.functional.gelu(u)
        elif self.act in ("gelu_pytorch_tanh", "gelu_new"):
            u = torch.nn.functional.gelu(u, approximate="tanh")
        else:
            u = torch.nn.functional.silu(u)
        return self.down_proj(u)


class SingleBlockLayer(nn.Module):
    """norm -> ONE block (state-space mixer, attention or MLP) -> residual: the layer form of Nemotron-H, whose
    layer list interleaves the three kinds."""

    def __init__(self, cfg: ModelConfig, idx: int, dtype, device):
        super().__init__()
        self.kind = cfg.layer_kind(idx)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        ex = cfg.extra or {}
        if self.kind == "mamba":
            from .mamba import Mamba2Mixer

            self.mixer = Mamba2Mixer(cfg, dtype, device)
        elif self.kind == "attention":
            self.mixer = Attention(cfg, dtype, device)
            self.mixer.layer_idx = idx
            self.mixer.use_rope = cfg.uses_rope(idx)
            self.mixer.window = int(ex.get("sliding_window") or 0)
        else:
            self.mixer = PlainMLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act, cfg.mlp_bias, dtype, device)
        self.is_moe = False

    def forward(self, h, residual, positions, inv_freq, attn_scale, meta):
        x, residual = self.norm(h, residual)
        if self.kind == "mlp":
            return self.mixer(x), residual, None
        return self.mixer(x, positions, inv_freq, attn_scale, meta), residual, None


class ParallelHybridLayer(nn.Module):
    """Falcon-H1: a state-space mixer and an attention block read the SAME normalised input side by side, their
    outputs (each with its own scalar multiplier) are summed into the residual stream, then a gated MLP follows."""

    def __init__(self, cfg: ModelConfig, idx: int, dtype, device):
        super().__init__()
        from .mamba import Mamba2Mixer

        ex = cfg.extra or {}
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.mamba = Mamba2Mixer(cfg, dtype, device)
        self.self_attn = Attention(cfg, dtype, device)
        self.self_attn.layer_idx = idx
        self.self_attn.window = 0
        self.attention_in_multiplier = float(ex.get("attention_in_multiplier") or 1.0)
        self.attention_out_multiplier = float(ex.get("attention_out_multiplier") or 1.0)
        self.ssm_out_multiplier = float(ex.get("ssm_out_multiplier") or 1.0)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.mlp = MLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act, cfg.mlp_bias, dtype, device)
        gm, dm = ex.get("mlp_multipliers") or (1.0, 1.0)
        self.mlp.gate_multiplier, self.mlp.down_multiplier = float(gm), float(dm)
        self.is_moe = False

    def forward(self, h, residual, positions, inv_freq, attn_scale, meta):
        x, residual = self.input_layernorm(h, residual)
        m = self.mamba(x, positions, inv_freq, attn_scale, meta)
        xa = x * self.attention_in_multiplier if self.attention_in_multiplier != 1.0 else x
        a = self.self_attn(xa, positions, inv_freq, attn_scale, meta)
        mixed = m * self.ssm_out_multiplier + a * self.attention_out_multiplier
        x, residual = self.post_attention_layernorm(mixed, residual)
        return self.mlp(x), residual, None


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, dtype, device):
        super().__init__()
        off = cfg.norm_offset()
        self.input_layernorm = make_norm(cfg, cfg.hidden_size, dtype, device, offset=off)
        if cfg.model_type == "glm_moe_dsa":
            from .dsa import SparseMLAttention

            self.self_attn = SparseMLAttention(cfg, dtype, device)
        elif cfg.model_type in ("deepseek_v2", "deepseek_v3", "mistral4"):
            from .mla import MLAttention

            self.self_attn = MLAttention(cfg, dtype, device)
        elif cfg.layer_kind(idx) == "mamba":
            from .mamba import Mamba2Mixer

            self.self_attn = Mamba2Mixer(cfg, dtype, device)     # (kept under the same attribute: the layer's token mixer)
        elif cfg.layer_kind(idx) == "shortconv":
            from .shortconv import ShortConv

            self.self_attn = ShortConv(cfg, dtype, device)
        elif cfg.layer_kind(idx) == "deltanet":
            from .deltanet import GatedDeltaNet

            self.self_attn = GatedDeltaNet(cfg, dtype, device)
        elif cfg.model_type == "gemma4_text":
            wide = cfg.layer_head_dim(idx) != cfg.head_dim or cfg.layer_kv_heads(idx) != cfg.num_key_value_heads
            self.self_attn = Attention(cfg, dtype, device, head_dim=cfg.layer_head_dim(idx), kv_heads=cfg.layer_kv_heads(idx),
                                       k_eq_v=bool((cfg.extra or {}).get("attention_k_eq_v")) and cfg.sliding_window(idx) == 0)
            inv = cfg.layer_inv_freq(idx)
            self.self_attn.local_inv_freq = inv.to(device) if device is not None else inv
            del wide
            first_shared = cfg.num_hidden_layers - int((cfg.extra or {}).get("num_kv_shared_layers") or 0)
            if 0 < first_shared < cfg.num_hidden_layers:
                kinds = [cfg.sliding_window(i) == 0 for i in range(cfg.num_hidden_layers)]
                last_of_kind = {k: max(i for i in range(first_shared) if kinds[i] == k) for k in set(kinds[:first_shared])}
                if idx >= first_shared:
                    self.self_attn.kv_src = last_of_kind[kinds[idx]]
                else:
                    self.self_attn.kv_store = last_of_kind[kinds[idx]] == idx
        else:
            self.self_attn = Attention(cfg, dtype, device)
        self.self_attn.layer_idx = idx
        self.self_attn.use_rope = cfg.uses_rope(idx)
        self.self_attn.window = cfg.sliding_window(idx)
        if cfg.model_type == "llama4_text" and self.self_attn.use_rope:
            self.self_attn.chunk = int((cfg.extra or {}).get("attention_chunk_size") or 0)
        theta = cfg.local_rope_theta(idx)
        if theta is not None:
            D = cfg.head_dim
            inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
            self.self_attn.local_inv_freq = inv.to(device) if device is not None else inv
        self.residual_multiplier = cfg.multiplier("residual_multiplier")
        self.parallel_block = cfg.parallel_block()     # Cohere: one norm, attention and MLP side by side
        if not self.parallel_block:
            self.post_attention_layernorm = make_norm(cfg, cfg.hidden_size, dtype, device, offset=off)
        self.ln_mlp = None
        if cfg.model_type == "falcon" and self.parallel_block and (cfg.extra or {}).get("new_decoder_architecture") \
                and int((cfg.extra or {}).get("num_ln_in_parallel_attn") or 2) == 2:
            self.ln_mlp = make_norm(cfg, cfg.hidden_size, dtype, device, offset=off)
        # Gemma 2 / 3: post_attention_layernorm and post_feedforward_layernorm act on the BRANCH outputs,
        # pre_feedforward_layernorm takes the place the post-attention norm has elsewhere
        self.post_norm_only = cfg.post_norm_only()     # OLMo 2 / 3: branches read the stream itself, norms on their outputs
        if self.post_norm_only:
            del self.input_layernorm
            self.post_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.sandwich = cfg.sandwich_norms()
        if self.sandwich:
            self.pre_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, offset=off)
            self.post_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, offset=off)
        if cfg.is_moe_layer(idx):
            from .moe import SparseMoE

            self.mlp = SparseMoE(cfg, dtype, device)
        elif cfg.model_type == "llama4_text":          # dense layers have their own width
            self.mlp = MLP(cfg.hidden_size, int((cfg.extra or {}).get("dense_intermediate_size") or cfg.intermediate_size),
                           cfg.hidden_act, False, dtype, device)
        elif cfg.model_type in ("granitemoeshared", "granitemoehybrid"):     # dense variant: the "shared" MLP alone
            self.mlp = MLP(cfg.hidden_size, int((cfg.extra or {}).get("shared_intermediate_size") or cfg.intermediate_size),
                           cfg.hidden_act, False, dtype, device, fused_names=True)
        elif cfg.model_type in ("lfm2", "lfm2_moe"):   # its own width rule (two thirds, rounded up to a multiple)
            self.mlp = MLP(cfg.hidden_size, int((cfg.extra or {}).get("mlp_width") or cfg.intermediate_size), "silu", False,
                           dtype, device)
        elif cfg.model_type in ("arcee", "nemotron", "starcoder2", "apertus", "phi", "falcon"):      # up -> activation -> down, no gate
            self.mlp = PlainMLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act, cfg.mlp_bias, dtype, device)
        else:
            inter = cfg.intermediate_size
            if (cfg.model_type == "gemma4_text" and (cfg.extra or {}).get("use_double_wide_mlp")
                    and 0 < cfg.num_hidden_layers - int((cfg.extra or {}).get("num_kv_shared_layers") or 0) <= idx):
                inter *= 2           # the layers that make no keys / values of their own get an MLP twice as wide
            self.mlp = MLP(cfg.hidden_size, inter, cfg.hidden_act, cfg.mlp_bias, dtype, device,
                           fused_names=cfg.model_type in ("phi3", "glm", "glm4"))
        self.is_moe = cfg.is_moe_layer(idx)
        # Gemma 4: the layer output (stream included) is multiplied by a stored scalar
        self.layer_scalar = nn.Parameter(torch.ones(1, dtype=dtype, device=device), requires_grad=False) \
            if cfg.model_type == "gemma4_text" else None
        self.idx = idx
        self.ple_width, self.g4_moe = 0, None
        if cfg.model_type == "gemma4_text":
            ex = cfg.extra or {}
            self.ple_width = int(ex.get("hidden_size_per_layer_input") or 0)
            if self.ple_width:     # a gated read of this layer's slice of the per-layer input embeddings, after the MLP
                self.per_layer_input_gate = FusedLinear(cfg.hidden_size, [self.ple_width], ["per_layer_input_gate"], dtype=dtype, device=device)
                self.per_layer_projection = FusedLinear(self.ple_width, [cfg.hidden_size], ["per_layer_projection"], dtype=dtype, device=device)
                self.post_per_layer_input_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
            g4 = ex.get("g4_experts")
            if g4:                 # routed experts BESIDE the dense MLP, each branch with its own output norm
                import dataclasses

                from .moe import SparseMoE

                sub = dataclasses.replace(cfg, num_experts=g4["num_experts"], num_experts_per_tok=g4["top_k"],
                                          moe_intermediate_size=g4["intermediate"], router_aux_loss_coef=0.0)
                self.g4_moe = SparseMoE(sub, dtype, device)
                self.post_feedforward_layernorm_1 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
                self.post_feedforward_layernorm_2 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
                self.pre_feedforward_layernorm_2 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)

    def _stream(self, h, residual):
        """(input of the attention branch, residual stream)."""
        if self.post_norm_only:
            x = h if residual is None else h + residual
            return x, x
        return self.input_layernorm(h, residual)

    def _before_attention(self, h, residual, positions, inv_freq, attn_scale):
        x, residual = self._stream(h, residual)
        return self.self_attn.pre(x, positions, inv_freq, attn_scale), residual

    def _after_attention(self, a, residual):
        return self._mlp_half(self.self_attn.o_proj(a), residual)

    def _mlp_half(self, a, residual):
        """From the attention branch output to the layer output: (branch, residual stream, router aux)."""
        rm = self.residual_multiplier
        if rm != 1.0:
            a = a * rm
        if self.post_norm_only:
            x = residual + self.post_attention_layernorm.plain(a)
            return self.post_feedforward_layernorm.plain(self.mlp(x)), x, None
        if self.sandwich:
            a = self.post_attention_layernorm.plain(a)
            x, residual = self.pre_feedforward_layernorm(a, residual)
        else:
            x, residual = self.post_attention_layernorm(a, residual)
        y, aux = self.mlp(x) if self.is_moe else (self.mlp(x), None)
        if self.g4_moe is not None:
            y2, _ = self.g4_moe(self.pre_feedforward_layernorm_2.plain(residual), router_x=residual)
            y = self.post_feedforward_layernorm_1.plain(y) + self.post_feedforward_layernorm_2.plain(y2)
        if self.sandwich:
            y = self.post_feedforward_layernorm.plain(y)
        if rm != 1.0:
            y = y * rm
        if self.layer_scalar is not None:
            h = residual + y
            if self.ple_width:
                g = Fn.glu(torch.cat([self.per_layer_input_gate(h), self._ple.to(h.dtype)], -1), self.mlp.act)     # act(gate) * input
                h = h + self.post_per_layer_input_norm.plain(self.per_layer_projection(g))
            return h * self.layer_scalar.to(y.dtype), None, aux
        return y, residual, aux

    def forward_selective(self, h, residual, positions, inv_freq, attn_scale, meta):
        """Selective activation checkpointing: the attention kernel's inputs and result stay saved (it is the
        one part whose recomputation costs more than its activations), everything around it — norms,
        projections, rotary embedding, the MLP — is recomputed in the backward pass (the reference's
        ``selective_checkpointing: {save: [attention]}``, src/axolotl/monkeypatch/selective_checkpointing.py:167-330)."""
        if (not hasattr(self.self_attn, "core") or getattr(self.self_attn, "out_gate", None) is not None
                or getattr(self.self_attn, "indexer", None) is not None or self.parallel_block or self.ple_width):
            # state-space / linear-attention mixers have no attention result to keep (and a gated attention output
            # needs the layer input again)
            return checkpoint(self.forward, h, residual, positions, inv_freq, attn_scale, meta, use_reentrant=False)
        qkv, residual = checkpoint(self._before_attention, h, residual, positions, inv_freq, attn_scale, use_reentrant=False)
        if getattr(self.self_attn, "kv_store", False) or getattr(self.self_attn, "kv_src", None) is not None:
            qkv = self.self_attn.share_kv(qkv, meta)
        a = self.self_attn.core(qkv, meta)
        return checkpoint(self._after_attention, a, residual, use_reentrant=False)

    def forward(self, h, residual, positions, inv_freq, attn_scale, meta):
        if self.ple_width:
            self._ple = meta.per_layer_inputs[:, self.idx]
        x, residual = self._stream(h, residual)
        if self.parallel_block:
            xm = x if self.ln_mlp is None else self.ln_mlp.plain(residual)      # Falcon's larger models: a norm per branch
            return self.self_attn(x, positions, inv_freq, attn_scale, meta) + self.mlp(xm), residual, None
        return self._mlp_half(self.self_attn(x, positions, inv_freq, attn_scale, meta), residual)


class _FixedFeatures(nn.Module):
    """Stands in for the image front end during generation: the features of the prompt's images, computed once."""

    def __init__(self, front, feats):
        super().__init__()
        self.image_token_id, self.bidirectional_images = front.image_token_id, front.bidirectional_images
        self.tokens_per_image = front.tokens_per_image
        self.feats = feats

    def forward(self, _):
        return self.feats


class CausalLM(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.config = cfg
        self.dtype = dtype
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        layer_cls = {"nemotron_h": SingleBlockLayer, "falcon_h1": ParallelHybridLayer}.get(cfg.model_type, DecoderLayer)
        self.layers = nn.ModuleList([layer_cls(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = make_norm(cfg, cfg.hidden_size, dtype, device, offset=cfg.norm_offset())
        self.final_softcap = cfg.final_softcap()   # Gemma 2: logits -> cap * tanh(logits / cap)
        if cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        # Phi: the output projection has a bias. It rides along as one extra hidden column (a constant 1 in the
        # hidden states, the bias in the weight; padded to 8 columns for the GEMM), so that every consumer of
        # (hidden states, output weight) - the chunked cross-entropy, log-prob and distillation paths, generation -
        # sees it without knowing
        self.lm_head_bias = nn.Parameter(torch.zeros(cfg.vocab_size, dtype=dtype, device=device)) if cfg.model_type == "phi" else None
        self.vision = None       # LLaVA checkpoints: CLIP tower + projector feeding the image placeholder tokens
        if (cfg.extra or {}).get("vision_wrapper"):
            from .vision import VisionFrontEnd

            self.vision = VisionFrontEnd(cfg.extra["vision_wrapper"], cfg.hidden_size, dtype, device)
        # Gemma 4: a second embedding table gives every layer its own small input vector per token; it is mixed with a
        # projection of the (scaled) token embedding and read through a gate after each layer's MLP
        self.ple_width = int((cfg.extra or {}).get("hidden_size_per_layer_input") or 0) if cfg.model_type == "gemma4_text" else 0
        if self.ple_width:
            L, Dp = cfg.num_hidden_layers, self.ple_width
            self.embed_tokens_per_layer = nn.Parameter(torch.empty(int((cfg.extra or {}).get("vocab_size_per_layer_input") or cfg.vocab_size),
                                                                   L * Dp, dtype=dtype, device=device))
            self.per_layer_model_projection = FusedLinear(cfg.hidden_size, [L * Dp], ["per_layer_model_projection"], dtype=dtype, device=device)
            self.per_layer_projection_norm = RMSNorm(Dp, cfg.rms_norm_eps, dtype, device)
        inv, scale = cfg.rope_inv_freq()
        self.register_buffer("inv_freq", inv.to(device) if device is not None else inv, persistent=False)
        self.attn_scale = scale
        long = cfg.rope_inv_freq_long()      # Phi-3 longrope: second frequency set for long documents
        self.longrope_orig = long[1] if long is not None else 0
        self.register_buffer("inv_freq_long", (long[0].to(device) if device is not None else long[0]) if long is not None
                             else None, persistent=False)
        self.gradient_checkpointing = False
        self.ckpt_store = None        # activation_memory.HostStore / DiskStore: checkpointed layer inputs leave the device
        self.ckpt_selective = False   # keep the attention result, recompute the rest of every layer
        self.ce_chunk_rows = 2048
        self.hooks = None  # parallelism runtime may install per-layer pre/post hooks
        self.nvtx = bool(os.environ.get("AXB_NVTX"))   # NVTX range per decoder layer for timeline tools
        self.neftune_noise_alpha = None  # NEFTune: uniform noise on the embedding output while training
        # LoRA on the embedding: h = E[ids] + s * A^T[ids] @ B^T (PEFT's lora_embedding_A / lora_embedding_B)
        self.embed_lora_At = None   # [vocab, r]  (transposed lora_embedding_A, so that a lookup is a row gather)
        self.embed_lora_B = None    # [hidden, r]
        self.embed_lora_scaling = 1.0
        # trainable token rows (PEFT ``trainable_token_indices``): a few embedding rows train next to an adapter
        self.token_rows = None      # [n, hidden] replacement rows
        self.token_row_ids = None   # [n] vocabulary ids they replace
        self.register_buffer("token_remap", None, persistent=False)   # [vocab] -> row index or -1
        limit = (getattr(cfg, "extra", None) or {}).get("swiglu_limit")
        if limit:
            for m in self.modules():
                if hasattr(m, "glu_limit"):
                    m.glu_limit = float(limit)

    def add_embedding_lora(self, r, alpha, use_rslora=False, dtype=torch.float32):
        """PEFT init for embeddings: A zeros, B normal (the product starts at zero)."""
        dev = self.embed_tokens.device
        V, H = self.embed_tokens.shape
        self.embed_lora_At = nn.Parameter(torch.zeros(V, r, dtype=dtype, device=dev))
        self.embed_lora_B = nn.Parameter(torch.randn(H, r, dtype=dtype, device=dev))
        self.embed_lora_scaling = alpha / math.sqrt(r) if use_rslora else alpha / r

    def add_trainable_tokens(self, token_ids, dtype=torch.float32):
        """The listed embedding rows become a small trainable tensor (initialised to the current rows);
        every other row of the embedding stays frozen."""
        dev = self.embed_tokens.device
        ids = torch.as_tensor(sorted(set(int(t) for t in token_ids)), dtype=torch.long, device=dev)
        if ids.numel() == 0:
            return
        if int(ids.max()) >= self.embed_tokens.shape[0] or int(ids.min()) < 0:
            raise ValueError("trainable token index outside the vocabulary")
        self.token_row_ids = ids
        self.token_rows = nn.Parameter(self.embed_tokens.detach()[ids].to(dtype).clone())
        remap = torch.full((self.embed_tokens.shape[0],), -1, dtype=torch.long, device=dev)
        remap[ids] = torch.arange(ids.numel(), device=dev)
        self.token_remap = remap

    @torch.no_grad()
    def merge_trainable_tokens_(self):
        if self.token_rows is None:
            return
        self.embed_tokens[self.token_row_ids] = self.token_rows.to(self.embed_tokens.dtype)
        self.token_rows = self.token_row_ids = self.token_remap = None

    @torch.no_grad()
    def fix_untrained_tokens(self, token_ids=None, eps=1e-16):
        """Embedding (and lm_head) rows that were never trained -- all zeros in the checkpoint, or the ids
        given -- are set to the mean of the trained rows, so that new chat-template tokens do not start
        from a degenerate vector. Returns the number of rows changed."""
        n = 0
        for W in (self.embed_tokens, self.lm_head):
            if W is None:
                continue
            if token_ids is None or token_ids is True:
                bad = W.detach().abs().amax(1) <= eps
            else:
                bad = torch.zeros(W.shape[0], dtype=torch.bool, device=W.device)
                bad[torch.as_tensor(list(token_ids), dtype=torch.long, device=W.device)] = True
            if bool(bad.any()) and not bool(bad.all()):
                W[bad] = W.detach()[~bad].float().mean(0).to(W.dtype)
                n += int(bad.sum())
        return n

    @torch.no_grad()
    def merge_embedding_lora_(self):
        if self.embed_lora_At is None:
            return
        delta = self.embed_lora_scaling * (self.embed_lora_At.float() @ self.embed_lora_B.float().t())
        self.embed_tokens.copy_((self.embed_tokens.float() + delta).to(self.embed_tokens.dtype))
        self.embed_lora_At = self.embed_lora_B = None

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self, seed: int | None = 0):
        """N(0, initializer_range) on every matrix, ones on norms (HF `_init_weights` rule)."""
        std = self.config.initializer_range
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.embed_tokens.device)
            gen.manual_seed(seed)
        if self.vision is not None:
            self.vision.init_weights(std, seed or 0)
        for name, p in self.named_parameters():
            if "lora_" in name or name.startswith("vision."):
                continue
            if p.dim() >= 2:
                p.normal_(0.0, std, generator=gen)
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
        for m in self.modules():
            if isinstance(m, RMSNorm) and m.offset:
                m.weight.fill_(1.0 - m.offset)
            if isinstance(m, Attention) and m.sinks is not None:
                m.sinks.normal_(0.0, std, generator=gen)
            if type(m).__name__ == "GatedDeltaNet":
                m.A_log.uniform_(0.0, 2.5, generator=gen)
                m.conv_weight.normal_(0.0, 0.2, generator=gen)
                m.dt_bias.fill_(1.0)
                m.norm_weight.fill_(1.0)
            if type(m).__name__ == "Mamba2Mixer":
                m.A_log.copy_(torch.log(torch.arange(1, m.nh + 1, dtype=torch.float32, device=m.A_log.device)).to(m.A_log.dtype))
                m.conv_weight.normal_(0.0, 0.2, generator=gen)
        return self

    @torch.no_grad()
    def resize_token_embeddings(self, new_size: int, pad_to_multiple_of: int | None = None, mean_resizing: bool = True):
        """Grows (or shrinks) the vocabulary. New rows are initialised to the mean of the old embedding
        matrix (``mean_resizing``) or N(0, initializer_range); the size is rounded up to a multiple when
        asked (``resize_token_embeddings_to_32x``). Returns the new vocabulary size."""
        if pad_to_multiple_of:
            new_size = (new_size + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
        old = self.config.vocab_size
        if new_size == old:
            return old

        def grow(p):
            out = torch.empty(new_size, p.shape[1], dtype=p.dtype, device=p.device)
            n = min(old, new_size)
            out[:n].copy_(p[:n])
            if new_size > old:
                if mean_resizing:
                    out[old:] = p.float().mean(0, keepdim=True).to(p.dtype)
                else:
                    out[old:].normal_(0.0, self.config.initializer_range)
            return nn.Parameter(out, requires_grad=p.requires_grad)

        self.embed_tokens = grow(self.embed_tokens)
        if self.lm_head is not None:
            self.lm_head = grow(self.lm_head)
        self.config.vocab_size = new_size
        return new_size

    def output_weight(self):
        W = self.embed_tokens if self.lm_head is None else self.lm_head
        if self.lm_head_bias is not None:
            W = torch.cat([W, self.lm_head_bias[:, None].to(W.dtype), W.new_zeros(W.shape[0], 7)], 1)
        return W

    def enable_gradient_checkpointing(self, flag=True, offload=None, selective=False, offload_dir=None):
        """``offload``: None keeps checkpointed layer inputs on the device; True / "legacy" /
        "hidden_states" park them in pinned host memory, "disk" in files under ``offload_dir``.
        ``selective`` keeps the attention result and recomputes only the rest of each layer."""
        self.gradient_checkpointing = flag
        self.ckpt_selective = bool(selective) and flag
        if flag and offload:
            from ..train.activation_memory import make_store

            self.ckpt_store = make_store(offload, self.embed_tokens.device, offload_dir)
        else:
            self.ckpt_store = None

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids, position_ids=None, labels=None, attn_meta=None, num_items=None,
                return_logits=None, shift_labels=True, aux_scale=1.0, capture_hidden=None, pixel_values=None):
        """input_ids / position_ids / labels: [B, S] (or [T]). Returns CausalLMOutput.

        ``labels`` follow the HF convention (unshifted; the model shifts by one inside each row)
        unless ``shift_labels=False``. ``num_items`` is the loss denominator (trainable tokens of
        the whole optimizer step when gradients are accumulated); default = this batch's count.
        ``return_logits``: True / False, or None = only when no labels are given (False with no
        labels returns just the final hidden states, for objectives that score tokens themselves).
        ``aux_scale`` weights the router load-balance term (1 / accumulation steps, so that the
        term is a mean over micro-batches just as the token loss is a mean over tokens).
        ``capture_hidden``: indices in the HF ``hidden_states`` numbering (0 = embeddings, i = residual
        stream after layer i, last = after the final norm) returned as ``out.captured[i]`` [T, H].
        """
        cfg = self.config
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        B, S = input_ids.shape
        dev = self.embed_tokens.device
        if position_ids is None:
            position_ids = torch.arange(S, dtype=torch.int32).repeat(B, 1)
        if attn_meta is None:
            attn_meta = build_attn_meta(position_ids, dev)
        ids = input_ids.reshape(-1).to(dev, non_blocking=True)
        pos = position_ids.reshape(-1).to(device=dev, dtype=torch.int32, non_blocking=True)
        h = Fn.embedding(self.embed_tokens, ids)
        if self.embed_lora_At is not None and adapters_enabled():
            low = Fn.embedding(self.embed_lora_At.to(h.dtype), ids)                  # [T, r]
            h = h + self.embed_lora_scaling * linear(low, self.embed_lora_B.to(h.dtype))
        if self.token_rows is not None and adapters_enabled():
            j = self.token_remap[ids]
            hit = j >= 0
            h = torch.where(hit[:, None], self.token_rows.to(h.dtype)[j.clamp(min=0)], h)
        em = cfg.multiplier("embedding_multiplier")
        if em != 1.0:
            h = h * em
        if pixel_values is not None:        # image placeholder tokens take the projected patch features
            if self.vision is None:
                raise ValueError("pixel_values were given to a model without an image front end")
            from .vision import image_groups, merge_image_features

            h = merge_image_features(h, ids, self.vision(pixel_values), self.vision.image_token_id)
            if self.vision.bidirectional_images:
                attn_meta.image_groups = image_groups(ids, self.vision.image_token_id)
                attn_meta.image_group_span = self.vision.tokens_per_image
        if self.neftune_noise_alpha and self.training:
            # noise magnitude alpha / sqrt(L * d) with L the row length (NEFTune, as applied by the HF
            # trainer the reference builds on)
            mag = float(self.neftune_noise_alpha) / math.sqrt(S * h.shape[-1])
            h = h + (torch.rand_like(h) * 2 - 1) * mag
        if cfg.model_type == "gemma4_text":
            attn_meta.shared_kv = {}
        if self.ple_width:
            L, Dp = len(self.layers), self.ple_width
            tok = Fn.embedding(self.embed_tokens_per_layer, ids) * float(torch.tensor(Dp ** 0.5).to(self.embed_tokens_per_layer.dtype))
            proj = self.per_layer_model_projection(h) * (cfg.hidden_size ** -0.5)
            proj = self.per_layer_projection_norm.plain(proj.reshape(-1, Dp)).reshape(-1, L, Dp)
            attn_meta.per_layer_inputs = (proj + tok.reshape(-1, L, Dp).to(proj.dtype)) * (2.0 ** -0.5)
        inv_freq = self.inv_freq
        if self.longrope_orig and getattr(attn_meta, "max_len", 0) > self.longrope_orig:
            inv_freq = self.inv_freq_long
        residual = None
        aux_total = None
        captured = {} if capture_hidden is not None else None
        if captured is not None and 0 in capture_hidden:
            captured[0] = h
        hooks = self.hooks
        nvtx = self.nvtx and h.is_cuda
        for i, layer in enumerate(self.layers):
            if nvtx:
                torch.cuda.nvtx.range_push(f"layer{i}")
            if hooks is not None:
                hooks.pre_layer(i)
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                if self.ckpt_store is not None:
                    from ..train.activation_memory import offloaded_checkpoint

                    h, residual, aux = offloaded_checkpoint(layer, self.ckpt_store, (h, residual),
                                                            (pos, inv_freq, self.attn_scale, attn_meta))
                elif self.ckpt_selective and hasattr(layer, "forward_selective"):
                    h, residual, aux = layer.forward_selective(h, residual, pos, inv_freq, self.attn_scale, attn_meta)
                else:
                    h, residual, aux = checkpoint(layer, h, residual, pos, inv_freq, self.attn_scale,
                                                  attn_meta, use_reentrant=False)
            else:
                h, residual, aux = layer(h, residual, pos, inv_freq, self.attn_scale, attn_meta)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
            if captured is not None and (i + 1) in capture_hidden and i + 1 < len(self.layers):
                captured[i + 1] = h if residual is None else h + residual
            if hooks is not None:
                hooks.post_layer(i)
            if nvtx:
                torch.cuda.nvtx.range_pop()
        h, _ = self.norm(h, residual)
        ls = cfg.multiplier("logits_scaling")
        if ls != 1.0:
            h = h / ls          # logits = (h W^T) / logits_scaling, applied on the narrow side
        if self.lm_head_bias is not None:
            h = torch.cat([h, h.new_ones(h.shape[0], 1), h.new_zeros(h.shape[0], 7)], 1)
        out = CausalLMOutput(hidden_states=h.view(B, S, -1))
        if captured is not None:
            if len(self.layers) in capture_hidden:
                captured[len(self.layers)] = h
            out.captured = captured
        if aux_total is not None:
            out.aux_loss = aux_total / max(sum(l.is_moe for l in self.layers), 1)
        W = self.output_weight()
        if labels is not None:
            lab = labels.reshape(B, S)
            if shift_labels:
                lab = torch.cat([lab[:, 1:], torch.full((B, 1), IGNORE_INDEX, dtype=lab.dtype, device=lab.device)], 1)
            if num_items is None:
                num_items = int((lab != IGNORE_INDEX).sum().item())
            out.num_items = num_items
            lab = lab.reshape(-1).to(dev, non_blocking=True)
            loss = Fn.linear_cross_entropy(h, W, lab, num_items=num_items, chunk_rows=self.ce_chunk_rows,
                                           softcap=self.final_softcap)
            if out.aux_loss is not None and cfg.router_aux_loss_coef:
                loss = loss + (cfg.router_aux_loss_coef * aux_scale) * out.aux_loss.to(loss.dtype)
            out.loss = loss
        if return_logits or (return_logits is None and labels is None):
            logits = linear(h, W)
            if self.final_softcap:
                logits = (torch.tanh(logits.float() / self.final_softcap) * self.final_softcap).to(logits.dtype)
            out.logits = logits.view(B, S, -1)
        return out

    # ------------------------------------------------------------------ generation (greedy / sampling)
    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=32, temperature=0.0, top_p=1.0, eos_token_id=None, use_cache=True,
                 pixel_values=None):
        """Greedy / sampled continuation of one prompt; returns [1, prompt + new]. With ``use_cache``
        (default) every new token is one incremental step over a KV cache; without it the whole
        sequence is recomputed per token (kept as the oracle of the cached path). A prompt with images
        (``pixel_values``) takes the recomputing path: the image features enter through the embeddings of the prompt."""
        if pixel_values is not None:
            use_cache = False
            with torch.no_grad():        # the tower runs once; its features are merged on every pass
                feats = self.vision(pixel_values)
            vision, self.vision = self.vision, _FixedFeatures(self.vision, feats)
            try:
                return self.generate(input_ids, max_new_tokens, temperature, top_p, eos_token_id, False, None)
            finally:
                self.vision = vision
        from .registry import KV_CACHE, Unsupported, get_model_support

        sup = get_model_support(self.config.model_type)
        kernel_ok = (self.config.head_dim in (64, 128) and not self.config.attn_softcap()      # what the decode kernel takes
                     and not (sup is not None and isinstance(sup.capabilities.get(KV_CACHE), Unsupported)))
        if use_cache and kernel_ok and getattr(self.hooks, "supports_kv_cache", True) is not False:
            from .kv_cache import generate_cached

            prompt = input_ids.reshape(-1).tolist()
            new = generate_cached(self, [prompt], max_new_tokens, temperature, top_p, 0, eos_token_id)[0]
            return torch.tensor([prompt + new], dtype=torch.long, device=input_ids.device)
        was_training = self.training
        self.eval()
        ids = input_ids.reshape(1, -1).clone()
        for _ in range(max_new_tokens):
            out = self.forward(ids, return_logits=True, pixel_values=True if isinstance(self.vision, _FixedFeatures) else None)
            logits = out.logits[0, -1].float()
            if temperature and temperature > 0:
                probs = torch.softmax(logits / temperature, -1)
                if top_p < 1.0:
                    sp, si = probs.sort(descending=True)
                    keep = sp.cumsum(0) - sp < top_p
                    sp = sp * keep
                    probs = torch.zeros_like(probs).scatter_(0, si, sp / sp.sum())
                nxt = torch.multinomial(probs, 1)
            else:
                nxt = logits.argmax().reshape(1)
            ids = torch.cat([ids, nxt.reshape(1, 1).to(ids.device)], 1)
            if eos_token_id is not None and int(nxt) == eos_token_id:
                break
        self.train(was_training)
        return ids

    # ------------------------------------------------------------------ adapters
    def fused_linears(self):
        for name, m in self.named_modules():
            if isinstance(m, FusedLinear) or getattr(m, "tp", None) is not None and hasattr(m, "lora_blocks"):
                yield name, m

    def refresh_lora_shadows(self):
        from ..ops.grouped import bump_param_epoch

        bump_param_epoch()
        for _, m in self.fused_linears():
            m.refresh_shadows()
        for m in self.modules():
            if hasattr(m, "refresh_expert_shadows"):
                m.refresh_expert_shadows()


def build_attn_meta(position_ids, device, causal=True) -> Fn.AttnMeta:
    """cu_seqlens from position-id resets, with a forced boundary at every row start."""
    p = position_ids.detach().cpu().numpy() if isinstance(position_ids, torch.Tensor) else np.asarray(position_ids)
    if p.ndim == 1:
        p = p[None]
    B, S = p.shape
    flat = p.reshape(-1)
    is_start = flat == 0
    is_start[np.arange(B) * S] = True
    starts = np.flatnonzero(is_start)
    cu = np.concatenate([starts, [B * S]]).astype(np.int32)
    return Fn.AttnMeta(cu, device, causal)
