"""Quantised checkpoint weights in a LoRA merge: detect the storage format of a weight from its companion scale
tensors, expand it, and write the merged weight back IN THE SAME FORMAT so that the merged checkpoint loads exactly
like the base did.

Formats (scale tensor names are relative to the weight key ``K``):
  block_fp8   ``K`` e4m3 + ``K_scale_inv`` fp32, one scale per 128x128 block (any grid that divides the shape)
  mxfp8       ``K`` e4m3 + ``K_scale`` e8m0 bytes, one power-of-two scale per 32 elements of the last axis
  mxfp4       ``K`` packed E2M1 nibbles (low nibble = even element) + ``K_scale`` e8m0 bytes per 32 elements
  nvfp4       ``K`` packed E2M1 + ``K_scale`` e4m3 per 16 elements (+ ``K_scale_2`` fp32 per tensor)
NVFP4 re-quantisation has two scale modes: ``reuse`` keeps the base block scales and only re-rounds the codes (a
small LoRA delta then changes only the elements it pushes across a code boundary, instead of re-rounding every
element on a shifted grid), ``fresh`` recomputes the block scales from the merged weight (for adapters trained
against fake-quantised merged weights). ``simulate_nf4_roundtrip`` reproduces what a QLoRA adapter saw: the base
weight after NF4 quantise -> dequantise.

Behaviour of the reference's merge helpers (src/axolotl/cli/utils/lora_merge.py:140-198, 597-822, 1356-1513).
"""
from __future__ import annotations

import torch

E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
MX_BLOCK = 32
_E8M0 = getattr(torch, "float8_e8m0fnu", None)


def detect_format(key: str, w: torch.Tensor, shard: dict):
    """(format name, {suffix: scale tensor}) of checkpoint tensor ``key``, or (None, {}) for a plain weight."""
    si, sc, sc2 = shard.get(key + "_scale_inv"), shard.get(key + "_scale"), shard.get(key + "_scale_2")
    e8m0 = sc is not None and (sc.dtype == torch.uint8 or (_E8M0 is not None and sc.dtype == _E8M0))
    if w.dtype == torch.float8_e4m3fn and si is not None:
        return "block_fp8", {"_scale_inv": si}
    if w.dtype == torch.float8_e4m3fn and e8m0:
        return "mxfp8", {"_scale": sc}
    if w.dtype == torch.uint8 and sc is not None and sc.dtype == torch.float8_e4m3fn:
        return "nvfp4", ({"_scale": sc, "_scale_2": sc2} if sc2 is not None else {"_scale": sc})
    if w.dtype == torch.uint8 and e8m0:
        return "mxfp4", {"_scale": sc}
    return None, {}


def _unpack_e2m1(packed):
    lut = torch.tensor(E2M1, dtype=torch.float32, device=packed.device)
    pair = torch.stack([(packed & 0xF).long(), (packed >> 4).long()], -1)
    return lut[pair.reshape(*packed.shape[:-1], packed.shape[-1] * 2)]


def _pack_e2m1(codes):
    codes = codes.to(torch.uint8)
    return codes[..., 0::2] | (codes[..., 1::2] << 4)


def _nearest_e2m1(x):
    """Index of the nearest E2M1 value (ties to the even code, i.e. round-half-to-even on the grid)."""
    mag = x.abs()
    # decision boundaries between 0, .5, 1, 1.5, 2, 3, 4, 6; a tie goes to the neighbour with an even mantissa bit
    idx = ((mag > 0.25).long() + (mag >= 0.75).long() + (mag > 1.25).long() + (mag >= 1.75).long()
           + (mag > 2.5).long() + (mag >= 3.5).long() + (mag > 5.0).long())
    return idx + 8 * ((x < 0) & (idx > 0)).long()          # no negative zero


def _mx_scale(scale_bytes, K):
    s = torch.exp2(scale_bytes.view(torch.uint8).float() - 127.0)
    return s.repeat_interleave(MX_BLOCK, dim=-1)[..., :K]          # a ragged last block is trimmed


def dequantize(fmt: str, w: torch.Tensor, scales: dict, device="cpu") -> torch.Tensor:
    """fp32 expansion of a quantised weight."""
    w = w.to(device)
    if fmt == "block_fp8":
        s = scales["_scale_inv"].to(device).float()
        *lead, N, K = w.shape
        sr, sc = s.shape[-2:]
        if N % sr or K % sc:
            raise ValueError(f"block-fp8 weight {tuple(w.shape)} is not aligned to its {sr}x{sc} scale grid")
        bn, bk = N // sr, K // sc
        return (w.float().reshape(*lead, sr, bn, sc, bk) * s.reshape(*lead, sr, 1, sc, 1)).reshape(*lead, N, K)
    if fmt == "mxfp8":
        return w.float() * _mx_scale(scales["_scale"].to(device), w.shape[-1])
    if fmt == "mxfp4":
        v = _unpack_e2m1(w)
        return v * _mx_scale(scales["_scale"].to(device), v.shape[-1])
    if fmt == "nvfp4":
        v = _unpack_e2m1(w)
        s = scales["_scale"].to(device).float().repeat_interleave(16, dim=-1)[..., : v.shape[-1]]
        g = scales["_scale_2"].to(device).float().reshape(-1) if scales.get("_scale_2") is not None else None
        if g is not None:
            s = s * (g.reshape(-1, *([1] * (s.dim() - 1))) if g.numel() > 1 else g)
        return v * s
    raise ValueError(f"unknown quantisation format {fmt!r}")


def _quant_mx(w, to_fp4):
    *lead, N, K = w.shape
    if K % MX_BLOCK:
        raise ValueError(f"MX formats need the last axis ({K}) to be a multiple of {MX_BLOCK}")
    wb = w.reshape(*lead, N, K // MX_BLOCK, MX_BLOCK)
    amax = wb.abs().amax(-1).clamp_min(1e-12)
    exp = torch.floor(torch.log2(amax / 6.0)) if to_fp4 else torch.floor(torch.log2(amax)) - 8.0
    scaled = (wb / torch.exp2(exp)[..., None]).reshape(*lead, N, K)
    ebyte = (exp + 127.0).clamp_(0, 254).to(torch.uint8)
    if to_fp4:
        return _pack_e2m1(_nearest_e2m1(scaled.clamp(-6.0, 6.0))), ebyte
    return scaled.clamp_(-448, 448).to(torch.float8_e4m3fn), ebyte


def requantize(fmt: str, w: torch.Tensor, scales: dict, device="cpu", nvfp4_scale_mode="reuse") -> dict:
    """``{"": quantised weight, "_scale...": scale tensors}`` with the dtypes and shapes of the base's tensors."""
    w = w.to(device).float()
    if fmt == "block_fp8":
        si = scales["_scale_inv"]
        *lead, N, K = w.shape
        sr, sc = si.shape[-2:]
        bn, bk = N // sr, K // sc
        wb = w.reshape(*lead, sr, bn, sc, bk)
        scale_inv = wb.abs().amax(dim=(-3, -1), keepdim=True).clamp_min(1e-12) / 448.0
        q = (wb / scale_inv).clamp_(-448, 448).to(torch.float8_e4m3fn)
        return {"": q.reshape(*lead, N, K).cpu(), "_scale_inv": scale_inv.reshape(*lead, sr, sc).to(si.dtype).cpu()}
    if fmt in ("mxfp8", "mxfp4"):
        q, ebyte = _quant_mx(w, fmt == "mxfp4")
        return {"": q.cpu(), "_scale": ebyte.view(scales["_scale"].dtype).cpu()}
    if fmt == "nvfp4":
        sc2 = scales.get("_scale_2")
        g = sc2.to(device).float().reshape(-1) if sc2 is not None else torch.ones(1, device=device)
        gb = g.reshape(-1, *([1] * (w.dim() - 1))) if g.numel() > 1 else g
        *lead, N, K = w.shape
        wb = w.reshape(*lead, N, K // 16, 16)
        if nvfp4_scale_mode == "fresh":
            block = (wb.abs().amax(-1) / 6.0 / gb).clamp(max=448.0).to(torch.float8_e4m3fn)
        else:
            block = scales["_scale"].to(device)
        eff = (block.float() * gb).clamp_min(1e-30)[..., None]
        codes = _nearest_e2m1((wb / eff).clamp(-6.0, 6.0)).reshape(*lead, N, K)
        out = {"": _pack_e2m1(codes).cpu(), "_scale": block.to(scales["_scale"].dtype).cpu()}
        if sc2 is not None:
            out["_scale_2"] = sc2.cpu()
        return out
    raise ValueError(f"unknown quantisation format {fmt!r}")


def simulate_nf4_roundtrip(w: torch.Tensor, blocksize=64, double_quant=True) -> torch.Tensor:
    """The weight a QLoRA run trained against: NF4 quantise -> dequantise of ``w`` (same dtype and shape). Weights whose
    element count is not a multiple of the block size are returned unchanged (they were not quantised either)."""
    from ..ops.nf4 import dequantize_nf4, quantize_nf4

    if w.numel() % blocksize:
        return w
    q, st = quantize_nf4(w, blocksize=blocksize, double_quant=double_quant)
    return dequantize_nf4(q, st, dtype=torch.float32).reshape(w.shape).to(w.dtype)
