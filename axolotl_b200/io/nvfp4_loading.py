"""NVFP4 expert checkpoints: detection and fusing of per-expert tensors into [E, N, K/2] stacks.

Rules reproduced from the reference loader
(src/axolotl/integrations/kernels/libs/scattermoe_lora/nvfp4_moe_loading.py:95-243):
* NVFP4 = a uint8 weight accompanied by a group scale; key triplets are
  (weight, weight_scale, weight_scale_2) [modelopt: pts multiplies] or
  (weight_packed, weight_scale, weight_global_scale) [compressed-tensors: pts divides].
* gate and up are concatenated on N in that order; if their per-tensor scales differ the larger
  one is kept and each block scale is multiplied by its ratio (<= 1) before re-rounding to E4M3.
"""
from __future__ import annotations

import torch

_W_KEYS = ("weight", "weight_packed")


def is_nvfp4_parts(parts: dict) -> bool:
    has_u8 = any(k[2] in _W_KEYS and t.dtype == torch.uint8 for k, t in parts.items())
    has_scale = any(k[2] == "weight_scale" for k in parts)
    return has_u8 and has_scale


def _triplet(parts, e, sub):
    w = parts.get((e, sub, "weight"), parts.get((e, sub, "weight_packed")))
    s = parts[(e, sub, "weight_scale")]
    if (e, sub, "weight_scale_2") in parts:
        pts = parts[(e, sub, "weight_scale_2")].float().reshape(())
    else:
        pts = 1.0 / parts[(e, sub, "weight_global_scale")].float().reshape(())
    return w, s.to(torch.float8_e4m3fn) if s.dtype != torch.float8_e4m3fn else s, pts


def reconcile_scales(scales, ptss):
    """Common per-tensor scale = max; fold each ratio into the E4M3 block scales."""
    pmax = torch.stack([p.reshape(()) for p in ptss]).max()
    out = []
    for s, p in zip(scales, ptss):
        ratio = (p / pmax).item()
        out.append(s if ratio == 1.0 else (s.float() * ratio).to(torch.float8_e4m3fn))
    return out, pmax


def fuse_nvfp4_experts(parts: dict, num_experts: int, device="cpu") -> dict:
    gu_q, gu_s, gu_p, d_q, d_s, d_p = [], [], [], [], [], []
    for e in range(num_experts):
        gw, gs, gp = _triplet(parts, e, "gate_proj")
        uw, us, up = _triplet(parts, e, "up_proj")
        (gs2, us2), p = reconcile_scales([gs, us], [gp, up])
        gu_q.append(torch.cat([gw, uw], 0))
        gu_s.append(torch.cat([gs2.view(torch.uint8), us2.view(torch.uint8)], 0).view(torch.float8_e4m3fn))
        gu_p.append(p)
        dw, ds, dp = _triplet(parts, e, "down_proj")
        d_q.append(dw)
        d_s.append(ds)
        d_p.append(dp)

    def pack(q, s, p):
        return {"qdata": torch.stack(q).to(device),
                "scale": torch.stack([x.view(torch.uint8) for x in s]).view(torch.float8_e4m3fn).to(device),
                "pts": torch.stack([x.reshape(()) for x in p]).float().to(device)}

    return {"gate_up": pack(gu_q, gu_s, gu_p), "down": pack(d_q, d_s, d_p)}
