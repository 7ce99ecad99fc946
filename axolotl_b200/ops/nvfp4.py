"""NVFP4 (E2M1 values, 16-element blocks, E4M3 block scales, fp32 per-tensor scale).

Storage contract (identical to the checkpoint formats the reference reads,
src/axolotl/integrations/kernels/libs/scattermoe_lora/dequant_grouped.py:63-111):
  qdata  uint8 [..., N, K/2]   low nibble = even k, high nibble = odd k
  scale  float8_e4m3fn [..., N, K/16]
  pts    fp32 scalar per tensor (or per expert)
  value = codebook[nibble] * scale * pts
"""
from __future__ import annotations

import torch

from . import _lib

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_CODEBOOK = torch.tensor(list(E2M1_VALUES) + [-v for v in E2M1_VALUES], dtype=torch.float32)
_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32)
FP4_MAX = 6.0
E4M3_MAX = 448.0


def quantize_nvfp4(w: torch.Tensor, pts: torch.Tensor | None = None):
    """Quantise [..., N, K] (K % 16 == 0) -> (qdata, scale, pts). Round-to-nearest-even on the
    E2M1 grid; block scale = amax/6 rounded to E4M3 after division by the per-tensor scale."""
    wf = w.float()
    *lead, N, K = wf.shape
    if K % 16:
        raise ValueError("NVFP4 needs K to be a multiple of 16")
    if pts is None:
        amax = wf.abs().amax(dim=(-1, -2)) if lead else wf.abs().amax()
        pts = (amax / (FP4_MAX * E4M3_MAX)).clamp(min=1e-12)
    pts = pts.float()
    blocks = wf.reshape(*lead, N, K // 16, 16)
    pts_b = pts.reshape(*pts.shape, *([1] * (blocks.dim() - pts.dim())))
    bscale = (blocks.abs().amax(-1, keepdim=True) / FP4_MAX / pts_b).clamp(max=E4M3_MAX)
    bscale8 = bscale.to(torch.float8_e4m3fn)
    bs = bscale8.float() * pts_b
    x = torch.where(bs > 0, blocks / bs.clamp(min=1e-30), torch.zeros_like(blocks))
    mag = x.abs().clamp(max=FP4_MAX)
    code = torch.bucketize(mag, _BOUNDS.to(mag.device), right=False)
    # ties: bucketize(right=False) sends exact midpoints to the lower code; the grid's even codes
    # are 0,2,4,6 -> move midpoints whose lower code is odd up by one.
    mid = torch.isclose(mag, _BOUNDS.to(mag.device)[code.clamp(max=6)]) & (code < 7)
    code = torch.where(mid & (code % 2 == 1), code + 1, code).clamp(max=7)
    code = code | (((x < 0) & (code > 0)).to(code.dtype) << 3)   # no negative zero
    code = code.reshape(*lead, N, K).to(torch.uint8)
    qdata = code[..., 0::2] | (code[..., 1::2] << 4)
    return qdata.contiguous(), bscale8.squeeze(-1).contiguous(), pts


def dequantize_nvfp4(qdata, scale, pts, dtype=torch.bfloat16):
    """Inverse of quantize_nvfp4 for a single [N, K/2] tensor or a batch [..., N, K/2]."""
    if qdata.is_cuda and qdata.dim() == 2 and dtype == torch.bfloat16 and _has_kernel():
        return _dequant_cuda(qdata, scale, pts)
    cb = _CODEBOOK.to(qdata.device)
    lo = cb[(qdata & 0xF).long()]
    hi = cb[(qdata >> 4).long()]
    vals = torch.stack([lo, hi], -1).reshape(*qdata.shape[:-1], qdata.shape[-1] * 2)
    s = scale.float().repeat_interleave(16, dim=-1)
    p = torch.as_tensor(pts, dtype=torch.float32, device=qdata.device)
    p = p.reshape(*p.shape, *([1] * (vals.dim() - p.dim())))
    return (vals * s * p).to(dtype)


def _has_kernel():
    try:
        return hasattr(_lib.cuda_lib(), "axb_nvfp4_dequant")
    except Exception:
        return False


def _dequant_cuda(qdata, scale, pts):
    lib = _lib.cuda_lib()
    N, K2 = qdata.shape
    out = torch.empty((N, K2 * 2), dtype=torch.bfloat16, device=qdata.device)
    p = torch.as_tensor(pts, dtype=torch.float32, device=qdata.device).reshape(1)
    _lib.check_rc(lib.axb_nvfp4_dequant(qdata.data_ptr(), scale.data_ptr(), p.data_ptr(), out.data_ptr(),
                                        N, K2 * 2, _lib.stream_ptr()), "nvfp4_dequant")
    return out
