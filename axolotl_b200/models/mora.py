"""MoRA: high-rank updating with one square matrix per adapted projection.

LoRA spends its parameter budget on two thin matrices (rank r); MoRA (Jiang et al., 2024) spends
the same budget ``(in + out) * r`` on a square matrix ``M`` of side ``r_hat = sqrt((in + out) * r)``
and wraps it in parameter-free compress / decompress operators:

* ``sharing`` (type 1): the input is cut into chunks of ``r_hat`` columns that are summed,
  ``M`` is applied, and the result is tiled along the output columns.
* ``rope`` (type 6): the input is cut into ``in / r_hat`` chunks, each chunk gets a rotary position
  encoding of its chunk index (so that the shared ``M`` can tell chunks apart), ``M`` is applied to
  every chunk and the chunks are concatenated (tiled or truncated to the output width).

The reference exposes this as ``adapter: mora`` through a PEFT fork
(src/axolotl/integrations/mora/plugin.py:44-97, args.py:11-66); here the operators are part of the
model. ``M`` starts at zero, so training starts from the base model. On CUDA the ``M`` product runs
on the tcgen05 GEMM, which wants ``r_hat`` to be a multiple of 8 (the fork rounds to even).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..ops.lora import linear

SHARING, ROPE = 1, 6
_TYPE_IDS = {"sharing": SHARING, "rope": ROPE, 1: SHARING, 6: ROPE, "1": SHARING, "6": ROPE}


def mora_type_id(v) -> int:
    v = getattr(v, "value", v)
    if v not in _TYPE_IDS:
        raise ValueError("mora_type must be one of `sharing`, `rope`, 1, or 6")
    return _TYPE_IDS[v]


def mora_rank(in_features: int, out_features: int, r: int, multiple: int = 2) -> int:
    rh = int(math.sqrt((in_features + out_features) * r) + 0.5)
    return max(multiple, rh // multiple * multiple)


def _rope_tables(n_chunks, r_hat, device):
    inv = 1.0 / (10000 ** (torch.arange(0, r_hat, 2, device=device, dtype=torch.float32) / r_hat))
    ang = torch.arange(n_chunks, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], -1)
    return emb.cos(), emb.sin()


def _apply_M(z, M):
    """z [.., r_hat] @ M^T; M is the fp32 master (cast to the activation dtype on the way)."""
    if z.is_cuda:
        return linear(z.reshape(-1, z.shape[-1]).contiguous(), M.to(z.dtype), None).view(z.shape)
    return z @ M.to(z.dtype).t()


def mora_delta(x, M, out_features: int, kind: int):
    """The MoRA update ``decompress(M compress(x))`` for ``x`` [.., in] -> [.., out]."""
    in_f, rh = x.shape[-1], M.shape[0]
    lead = x.shape[:-1]
    n_chunks = -(-in_f // rh)
    pad = n_chunks * rh - in_f
    if pad:
        x = torch.cat([x, x[..., :pad]], -1)     # wrap-around padding, as in the paper's code
    z = x.reshape(*lead, n_chunks, rh)
    if kind == SHARING:
        y = _apply_M(z.sum(-2), M)                                   # [.., rh]
    else:
        cos, sin = _rope_tables(n_chunks, rh, x.device)
        rot = torch.cat([-z[..., rh // 2:], z[..., :rh // 2]], -1)
        z = (z.float() * cos + rot.float() * sin).to(x.dtype)
        y = _apply_M(z, M).reshape(*lead, n_chunks * rh)             # [.., n_chunks*rh]
    if y.shape[-1] < out_features:
        y = torch.cat([y] * (-(-out_features // y.shape[-1])), -1)
    return y[..., :out_features]


@torch.no_grad()
def mora_dense_delta(M, in_features: int, out_features: int, kind: int):
    """The [out, in] weight update that ``mora_delta`` amounts to (it is linear in x)."""
    eye = torch.eye(in_features, dtype=torch.float32, device=M.device)
    return mora_delta(eye, M.float(), out_features, kind).t().contiguous()
