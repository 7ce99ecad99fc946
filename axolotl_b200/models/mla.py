"""Multi-head latent attention (DeepSeek-V2 / V3, GLM-5): queries and keys/values are produced through low-rank
bottlenecks with their own RMSNorms, every head has a 128-wide content part and shares one 64-wide rotary
part, values are 128 wide. The training graph expands k / v per head and runs the wide-head varlen attention
kernels (q/k width 192, v width 128, ``csrc/flash_wide.cu``).

The reference trains these models through HF's modelling code with its attention patches
(src/axolotl/loaders/model.py:560-640, src/axolotl/monkeypatch/attention/flash_attn_4.py:37-111).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as Fn
from .config import ModelConfig
from .layers import FusedLinear, RMSNorm


class MLAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ex = cfg.extra or {}
        H = cfg.hidden_size
        self.Hq = self.Hk = cfg.num_attention_heads
        self.d_nope, self.d_rope = int(ex["qk_nope_head_dim"]), int(ex["qk_rope_head_dim"])
        self.D, self.Dv = self.d_nope + self.d_rope, int(ex["v_head_dim"])
        self.q_lora_rank, self.kv_lora_rank = ex.get("q_lora_rank"), int(ex["kv_lora_rank"])
        eps = cfg.rms_norm_eps
        bias = bool(ex.get("attention_bias", False))
        if self.q_lora_rank:
            self.q_a_proj = FusedLinear(H, [self.q_lora_rank], ["q_a_proj"], bias=bias, dtype=dtype, device=device)
            self.q_a_layernorm = RMSNorm(self.q_lora_rank, eps, dtype, device)
            self.q_b_proj = FusedLinear(self.q_lora_rank, [self.Hq * self.D], ["q_b_proj"], dtype=dtype, device=device)
        else:
            self.q_proj = FusedLinear(H, [self.Hq * self.D], ["q_proj"], dtype=dtype, device=device)
        self.kv_a_proj_with_mqa = FusedLinear(H, [self.kv_lora_rank + self.d_rope], ["kv_a_proj_with_mqa"], bias=bias,
                                              dtype=dtype, device=device)
        self.kv_a_layernorm = RMSNorm(self.kv_lora_rank, eps, dtype, device)
        self.kv_b_proj = FusedLinear(self.kv_lora_rank, [self.Hq * (self.d_nope + self.Dv)], ["kv_b_proj"], dtype=dtype,
                                     device=device)
        self.o_proj = FusedLinear(self.Hq * self.Dv, [H], ["o_proj"], bias=bias, dtype=dtype, device=device)
        self.scale = self.D ** -0.5
        rs = cfg.rope_scaling or {}
        if rs.get("rope_type", rs.get("type")) == "yarn" and rs.get("mscale_all_dim") and cfg.model_type != "mistral4":
            m = 0.1 * float(rs["mscale_all_dim"]) * math.log(float(rs["factor"])) + 1.0 if float(rs["factor"]) > 1 else 1.0
            self.scale = self.scale * m * m
        # the checkpoints store the rotary part with interleaved (real, imaginary) pairs (V2 rotates complex numbers,
        # V3 carries ``rope_interleave``)
        self.interleave = bool(ex.get("rope_interleave", True))
        d = self.d_rope
        perm = torch.cat([torch.arange(0, d, 2), torch.arange(1, d, 2)])
        self.register_buffer("pe_perm", perm.to(device) if device is not None else perm, persistent=False)
        # Mistral 4: queries grow with the position, 1 + beta * log(1 + floor(pos / original context))
        rp = ex.get("rope_parameters") or cfg.rope_scaling or {}
        self.q_pos_scale = (float(rp["llama_4_scaling_beta"]), float(rp.get("original_max_position_embeddings") or 1)) \
            if cfg.model_type == "mistral4" and rp.get("llama_4_scaling_beta") is not None else None
        self.window, self.use_rope, self.softcap = 0, True, 0.0
        self.register_buffer("local_inv_freq", None, persistent=False)

    def _rot(self, t):
        """[..., d_rope] with interleaved pairs -> half-split layout the rotary kernel works on."""
        return t.index_select(-1, self.pe_perm) if self.interleave else t

    def pre(self, x, positions, inv_freq, attn_scale, q_resid=None):
        T = x.shape[0]
        Hq, dn, dr, Dv = self.Hq, self.d_nope, self.d_rope, self.Dv
        if self.q_lora_rank:
            q = self.q_b_proj(self.q_a_layernorm.plain(self.q_a_proj(x)) if q_resid is None else q_resid)
        else:
            q = self.q_proj(x)
        q = q.view(T, Hq, dn + dr)
        ckv = self.kv_a_proj_with_mqa(x)
        kv = self.kv_b_proj(self.kv_a_layernorm.plain(ckv[:, : self.kv_lora_rank].contiguous())).view(T, Hq, dn + Dv)
        # rotary part: Hq query heads + ONE shared key head, rotated in one fused buffer (a spare head keeps the
        # [T, (Hq + 2 Hk) * d] layout of the kernel)
        pe = torch.cat([self._rot(q[..., dn:]).reshape(T, Hq * dr), self._rot(ckv[:, self.kv_lora_rank:]),
                        x.new_zeros(T, dr)], 1)
        pe = Fn.rope_qk_(pe, positions, inv_freq, Hq, 1, dr, attn_scale)
        q_pe = pe[:, : Hq * dr].reshape(T, Hq, dr)
        k_pe = pe[:, Hq * dr:(Hq + 1) * dr].reshape(T, 1, dr).expand(T, Hq, dr)
        qf = torch.cat([q[..., :dn], q_pe], -1)
        if self.q_pos_scale is not None:
            beta, orig = self.q_pos_scale
            qf = (qf.float() * (1.0 + beta * torch.log1p(torch.floor(positions.float() / orig)))[:, None, None]).to(q.dtype)
        qf = qf.reshape(T, Hq * (dn + dr))
        kf = torch.cat([kv[..., :dn], k_pe], -1).reshape(T, Hq * (dn + dr))
        return torch.cat([qf, kf, kv[..., dn:].reshape(T, Hq * Dv)], 1)

    def core(self, qkv, meta):
        if getattr(meta, "kv_cache", None) is not None:
            raise NotImplementedError("KV-cache decoding is not available for latent attention; generate(use_cache=False)")
        return Fn.flash_varlen(qkv, meta, self.Hq, self.Hk, self.D, self.scale, Dv=self.Dv)

    def forward(self, x, positions, inv_freq, attn_scale, meta):
        return self.o_proj(self.core(self.pre(x, positions, inv_freq, attn_scale), meta))
