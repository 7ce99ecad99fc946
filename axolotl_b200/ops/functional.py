"""Autograd-aware fused ops. CUDA tensors run the hand-written sm_100a kernels; CPU tensors run a
plain PyTorch implementation of the same math, which doubles as the numerical oracle in tests.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from . import _lib

IGNORE_INDEX = -100


# --------------------------------------------------------------------------------------- RMSNorm
def _rmsnorm_ref(h, w, eps, w_offset=0.0):
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    return (hf * rstd * (w.float() + w_offset)).to(h.dtype), rstd.squeeze(-1)


class _AddRMSNorm(torch.autograd.Function):
    """(x, residual) -> (y, h) with h = x + residual and y = rmsnorm(h) * (w + w_offset)."""

    @staticmethod
    def forward(ctx, x, residual, w, eps, w_offset):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        rows = x2.shape[0]
        ctx.has_res = residual is not None
        ctx.eps, ctx.w_offset = eps, w_offset
        if not x.is_cuda:
            h = x2 if residual is None else (x2.float() + residual.reshape(-1, H).float()).to(x.dtype)
            y, rstd = _rmsnorm_ref(h, w, eps, w_offset)
        else:
            lib = _lib.cuda_lib()
            x2 = x2.contiguous()
            r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
            y = torch.empty_like(x2)
            h = torch.empty_like(x2) if residual is not None else x2
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            _lib.check_rc(
                lib.axb_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(r2), w.data_ptr(), y.data_ptr(),
                                    h.data_ptr() if residual is not None else None, rstd.data_ptr(),
                                    rows, H, eps, w_offset, _lib.stream_ptr()),
                "rmsnorm_fwd")
        ctx.save_for_backward(h, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape), h.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        H = h.shape[-1]
        rows = h.shape[0]
        need_dw = ctx.needs_input_grad[2]
        if not h.is_cuda:
            hf, dyf = h.float(), dy.reshape(-1, H).float()
            wf = w.float() + ctx.w_offset
            xhat = hf * rstd[:, None]
            g = dyf * wf
            dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
            if dh is not None:
                dx = dx + dh.reshape(-1, H).float()
            dw = (dyf * xhat).sum(0).to(w.dtype) if need_dw else None
            dx = dx.to(h.dtype)
        else:
            lib = _lib.cuda_lib()
            dy2 = dy.reshape(-1, H).contiguous()
            dh2 = dh.reshape(-1, H).contiguous() if dh is not None else None
            dx = torch.empty_like(h)
            dwf = torch.zeros(H, dtype=torch.float32, device=h.device) if need_dw else None
            _lib.check_rc(
                lib.axb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                    _lib.ptr(dh2), dx.data_ptr(), _lib.ptr(dwf), rows, H,
                                    ctx.w_offset, _lib.stream_ptr()),
                "rmsnorm_bwd")
            dw = dwf.to(w.dtype) if need_dw else None
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_res else None), dw, None, None


def add_rmsnorm(x, residual, weight, eps=1e-6, w_offset=0.0):
    """Returns ``(rmsnorm(x + residual), x + residual)``; ``residual`` may be None."""
    return _AddRMSNorm.apply(x, residual, weight, eps, w_offset)


def rmsnorm(x, weight, eps=1e-6, w_offset=0.0):
    return _AddRMSNorm.apply(x, None, weight, eps, w_offset)[0]


# --------------------------------------------------------------------------------------- RoPE
def _rope_ref(x, pos, inv_freq, sign=1.0, attn_scale=1.0):
    # x: [T, H, D]
    ang = pos.float()[:, None] * inv_freq.float()[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :] * attn_scale
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, :] * attn_scale * sign
    half = x.shape[-1] // 2
    xf = x.float()
    rot = torch.cat([-xf[..., half:], xf[..., :half]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


class _RopeQK(torch.autograd.Function):
    """In-place rotary embedding (+ optional per-head q/k RMSNorm) on a fused qkv projection."""

    @staticmethod
    def forward(ctx, qkv, pos, inv_freq, Hq, Hk, D, attn_scale, qn_w, kn_w, eps):
        T = qkv.shape[0]
        ctx.dims = (Hq, Hk, D, attn_scale, eps)
        has_norm = qn_w is not None
        pre = None
        rstd = None
        if not qkv.is_cuda:
            qk = qkv[:, : (Hq + Hk) * D].reshape(T, Hq + Hk, D)
            if has_norm:
                pre = qk.clone()
                q, rq = _rmsnorm_ref(qk[:, :Hq], qn_w, eps)
                k, rk = _rmsnorm_ref(qk[:, Hq:], kn_w, eps)
                rstd = torch.cat([rq, rk], 1)
                qk = torch.cat([q, k], 1)
            out = _rope_ref(qk, pos, inv_freq, 1.0, attn_scale)
            qkv = torch.cat([out.reshape(T, -1), qkv[:, (Hq + Hk) * D:]], 1)
        else:
            lib = _lib.cuda_lib()
            if has_norm:
                pre = qkv[:, : (Hq + Hk) * D].clone()
                rstd = torch.empty(T * (Hq + Hk), dtype=torch.float32, device=qkv.device)
            _lib.check_rc(
                lib.axb_rope_qk(qkv.data_ptr(), pos.data_ptr(), inv_freq.data_ptr(), T, Hq, Hk, D,
                                qkv.stride(0), 1.0, attn_scale, _lib.ptr(qn_w), _lib.ptr(kn_w),
                                _lib.ptr(rstd), eps, _lib.stream_ptr()),
                "rope_qk")
            # The kernel rotated the buffer in place. Autograd is handed an alias of it as a fresh
            # output instead of a "dirty" input: the producer of qkv (the projection) does not keep its
            # output, so nothing else reads the pre-rotation values, and the in-place bookkeeping of
            # autograd (which copies the 100 MB buffer several times per layer) is avoided.
            qkv = qkv.detach()
        ctx.save_for_backward(pos, inv_freq, qn_w, kn_w, pre, rstd)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        pos, inv_freq, qn_w, kn_w, pre, rstd = ctx.saved_tensors
        Hq, Hk, D, attn_scale, eps = ctx.dims
        T = dqkv.shape[0]
        dqn = dkn = None
        if not dqkv.is_cuda:
            g = dqkv[:, : (Hq + Hk) * D].reshape(T, Hq + Hk, D)
            g = _rope_ref(g, pos, inv_freq, -1.0, attn_scale)
            if qn_w is not None:
                gf = g.float()
                xhat = pre.reshape(T, Hq + Hk, D).float() * rstd[:, :, None]
                wcat = torch.cat([qn_w.float().expand(Hq, D), kn_w.float().expand(Hk, D)], 0)[None]
                gw = gf * wcat
                dx = rstd[:, :, None] * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
                dqn = (gf[:, :Hq] * xhat[:, :Hq]).sum((0, 1)).to(qn_w.dtype)
                dkn = (gf[:, Hq:] * xhat[:, Hq:]).sum((0, 1)).to(kn_w.dtype)
                g = dx.to(dqkv.dtype)
            dqkv = torch.cat([g.reshape(T, -1), dqkv[:, (Hq + Hk) * D:]], 1)
        else:
            lib = _lib.cuda_lib()
            dqkv = dqkv.contiguous()
            need_dn = qn_w is not None and (ctx.needs_input_grad[7] or ctx.needs_input_grad[8])
            dqn_f = torch.zeros(D, dtype=torch.float32, device=dqkv.device) if need_dn else None
            dkn_f = torch.zeros(D, dtype=torch.float32, device=dqkv.device) if need_dn else None
            _lib.check_rc(
                lib.axb_rope_qk_bwd(dqkv.data_ptr(), _lib.ptr(pre), pos.data_ptr(),
                                    inv_freq.data_ptr(), T, Hq, Hk, D, dqkv.stride(0),
                                    pre.stride(0) if pre is not None else 0, attn_scale,
                                    _lib.ptr(qn_w), _lib.ptr(kn_w), _lib.ptr(rstd),
                                    _lib.ptr(dqn_f), _lib.ptr(dkn_f), _lib.stream_ptr()),
                "rope_qk_bwd")
            if need_dn:
                dqn, dkn = dqn_f.to(qn_w.dtype), dkn_f.to(kn_w.dtype)
        return dqkv, None, None, None, None, None, None, dqn, dkn, None


class _RopePartial(torch.autograd.Function):
    """Rotary embedding of the first ``rot`` dimensions of every q and k head (in place on CUDA); the rest of the head
    passes through. The backward pass is the inverse rotation of the gradient."""

    @staticmethod
    def _apply(qkv, pos, inv_freq, Hq, Hk, D, rot, attn_scale, sign):
        T = qkv.shape[0]
        if qkv.is_cuda:
            _lib.check_rc(_lib.cuda_lib().axb_rope_partial(qkv.data_ptr(), pos.data_ptr(), inv_freq.data_ptr(), T, Hq + Hk, D,
                                                           rot, qkv.stride(0), sign, attn_scale, _lib.stream_ptr()), "rope_partial")
            return qkv
        qk = qkv[:, : (Hq + Hk) * D].reshape(T, Hq + Hk, D)
        out = torch.cat([_rope_ref(qk[..., :rot], pos, inv_freq, sign, attn_scale), qk[..., rot:]], -1)
        return torch.cat([out.reshape(T, -1), qkv[:, (Hq + Hk) * D:]], 1)

    @staticmethod
    def forward(ctx, qkv, pos, inv_freq, Hq, Hk, D, rot, attn_scale):
        ctx.dims = (Hq, Hk, D, rot, attn_scale)
        ctx.save_for_backward(pos, inv_freq)
        out = _RopePartial._apply(qkv, pos, inv_freq, Hq, Hk, D, rot, attn_scale, 1.0)
        return out.detach() if qkv.is_cuda else out     # (alias handed out as a fresh tensor, as in _RopeQK)

    @staticmethod
    def backward(ctx, dqkv):
        pos, inv_freq = ctx.saved_tensors
        Hq, Hk, D, rot, attn_scale = ctx.dims
        g = _RopePartial._apply(dqkv.contiguous(), pos, inv_freq, Hq, Hk, D, rot, attn_scale, -1.0)
        return g, None, None, None, None, None, None, None


def rope_qk_(qkv, positions, inv_freq, Hq, Hk, D, attn_scale=1.0, q_norm_w=None, k_norm_w=None,
             eps=1e-6, rot_dim=None):
    """Rotates the q and k blocks of ``qkv`` [T, (Hq+2Hk)*D] (in place on CUDA). ``rot_dim`` < D: partial rotary
    embedding of the first ``rot_dim`` dimensions of each head (``inv_freq`` then has rot_dim / 2 entries)."""
    if rot_dim is not None and rot_dim < D:
        if q_norm_w is not None or k_norm_w is not None:
            raise NotImplementedError("partial rotary embedding together with the fused q/k norm")
        return _RopePartial.apply(qkv, positions, inv_freq, Hq, Hk, D, int(rot_dim), attn_scale)
    return _RopeQK.apply(qkv, positions, inv_freq, Hq, Hk, D, attn_scale, q_norm_w, k_norm_w, eps)


# --------------------------------------------------------------------------------------- GLU
_ACT_KIND = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu": 1, "gpt_oss_swiglu": 2}


def _act_ref(g, kind):
    if kind == 2:       # gpt-oss experts: g * sigmoid(1.702 g); the GLU multiplies by (up + 1)
        return g * torch.sigmoid(1.702 * g)
    return F.silu(g) if kind == 0 else F.gelu(g, approximate="tanh")


class _GLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, kind, limit, blocks=None):
        I = gu.shape[-1] // 2
        ctx.kind, ctx.limit = kind, float(limit or 0.0)
        ctx.blocks = blocks if gu.is_cuda else None
        ctx.save_for_backward(gu)
        if not gu.is_cuda:
            g, u = gu[..., :I].float(), gu[..., I:].float()
            if ctx.limit > 0:
                g, u = g.clamp(max=ctx.limit), u.clamp(-ctx.limit, ctx.limit)
            return (_act_ref(g, kind) * (u + 1.0 if kind == 2 else u)).to(gu.dtype)
        lib = _lib.cuda_lib()
        gu2 = gu.reshape(-1, 2 * I)
        h = torch.empty((gu2.shape[0], I), dtype=gu.dtype, device=gu.device)
        if ctx.blocks is not None:
            _lib.check_rc(lib.axb_glu_fwd_rows(gu2.data_ptr(), h.data_ptr(), gu2.shape[0], I, kind, ctx.limit,
                                               ctx.blocks.data_ptr(), _lib.stream_ptr()), "glu_fwd_rows")
        else:
            _lib.check_rc(lib.axb_glu_fwd(gu2.data_ptr(), h.data_ptr(), gu2.shape[0], I, kind, ctx.limit,
                                          _lib.stream_ptr()), "glu_fwd")
        return h.view(*gu.shape[:-1], I)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        I = gu.shape[-1] // 2
        L = ctx.limit
        if not gu.is_cuda:
            g_raw, u_raw = gu[..., :I].float(), gu[..., I:].float()
            gc = g_raw.clamp(max=L) if L > 0 else g_raw
            uc = u_raw.clamp(-L, L) if L > 0 else u_raw
            with torch.enable_grad():
                g = gc.detach().requires_grad_(True)
                a = _act_ref(g, ctx.kind)
                (da,) = torch.autograd.grad(a.sum(), g)
            dhf = dh.float()
            dg, du = dhf * (uc + 1.0 if ctx.kind == 2 else uc) * da, dhf * a.detach()
            if L > 0:
                dg = dg * (g_raw <= L)
                du = du * ((u_raw >= -L) & (u_raw <= L))
            return torch.cat([dg, du], -1).to(gu.dtype), None, None, None
        lib = _lib.cuda_lib()
        gu2 = gu.reshape(-1, 2 * I)
        dh2 = dh.reshape(-1, I).contiguous()
        dgu = torch.empty_like(gu2)
        if ctx.blocks is not None:
            _lib.check_rc(lib.axb_glu_bwd_rows(dh2.data_ptr(), gu2.data_ptr(), dgu.data_ptr(), gu2.shape[0], I, ctx.kind, L,
                                               ctx.blocks.data_ptr(), _lib.stream_ptr()), "glu_bwd_rows")
        else:
            _lib.check_rc(lib.axb_glu_bwd(dh2.data_ptr(), gu2.data_ptr(), dgu.data_ptr(), gu2.shape[0],
                                          I, ctx.kind, L, _lib.stream_ptr()), "glu_bwd")
        return dgu.view(gu.shape), None, None, None


def glu(gate_up, activation="silu", limit=None, blocks_in_use=None):
    """``act(gate) * up`` for a fused ``[.., 2I]`` (gate | up) projection. With ``limit`` the gate is
    clamped from above and the up branch to ``[-limit, limit]`` first (the clamped SwiGLU of the
    reference's grouped expert graph,
    src/axolotl/integrations/kernels/libs/scattermoe_lora/cutlass_fp4/swiglu.py:16-148)."""
    if blocks_in_use is not None:       # int32 device scalar: only the first blocks_in_use * 128 rows hold data
        return _GLU.apply(gate_up, _ACT_KIND[activation], limit, blocks_in_use)
    return _GLU.apply(gate_up, _ACT_KIND[activation], limit)


# --------------------------------------------------------------------------------------- gated RMSNorm
class _RMSNormGated(torch.autograd.Function):
    """y = (w + w_offset) * rmsnorm(x) * silu(g)."""

    @staticmethod
    def forward(ctx, x, g, w, eps, w_offset):
        H = x.shape[-1]
        x2, g2 = x.reshape(-1, H), g.reshape(-1, H)
        ctx.w_offset, ctx.shape = w_offset, x.shape
        if not x.is_cuda:
            n, rstd = _rmsnorm_ref(x2, w, eps, w_offset)
            y = (n.float() * F.silu(g2.float())).to(x.dtype)
        else:
            lib = _lib.cuda_lib()
            x2, g2 = x2.contiguous(), g2.contiguous()
            y = torch.empty_like(x2)
            rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
            _lib.check_rc(lib.axb_rmsnorm_gated_fwd(x2.data_ptr(), g2.data_ptr(), w.data_ptr(), y.data_ptr(),
                                                    rstd.data_ptr(), x2.shape[0], H, eps, w_offset,
                                                    _lib.stream_ptr()), "rmsnorm_gated_fwd")
        ctx.save_for_backward(x2, g2, w, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x, g, w, rstd = ctx.saved_tensors
        H = x.shape[-1]
        need_dw = ctx.needs_input_grad[2]
        if not x.is_cuda:
            dyf, xf, gf = dy.reshape(-1, H).float(), x.float(), g.float()
            wf = w.float() + ctx.w_offset
            sg = torch.sigmoid(gf)
            s = gf * sg
            xhat = xf * rstd[:, None]
            dn = dyf * s
            gw = dn * wf
            dx = rstd[:, None] * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
            dg = dyf * xhat * wf * sg * (1 + gf * (1 - sg))
            dw = (dn * xhat).sum(0).to(w.dtype) if need_dw else None
            return dx.to(x.dtype).view(ctx.shape), dg.to(g.dtype).view(ctx.shape), dw, None, None
        lib = _lib.cuda_lib()
        dy2 = dy.reshape(-1, H).contiguous()
        dx, dg = torch.empty_like(x), torch.empty_like(g)
        dwf = torch.zeros(H, dtype=torch.float32, device=x.device) if need_dw else None
        _lib.check_rc(lib.axb_rmsnorm_gated_bwd(dy2.data_ptr(), x.data_ptr(), g.data_ptr(), w.data_ptr(),
                                                rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), _lib.ptr(dwf),
                                                x.shape[0], H, ctx.w_offset, _lib.stream_ptr()),
                      "rmsnorm_gated_bwd")
        return dx.view(ctx.shape), dg.view(ctx.shape), (dwf.to(w.dtype) if need_dw else None), None, None


def rmsnorm_gated(x, gate, weight, eps=1e-6, w_offset=0.0):
    """``(weight + w_offset) * rmsnorm(x) * silu(gate)`` in one pass over the row (the output norm of
    gated linear-attention blocks; reference kernel: src/axolotl/kernels/rms_norm_gated.py:36-381)."""
    return _RMSNormGated.apply(x, gate, weight, eps, w_offset)


# --------------------------------------------------------------------------------------- entropy
@torch.no_grad()
def token_entropy(logits, temperature=1.0, return_lse=False):
    """Entropy of ``softmax(logits / temperature)`` per row of ``[.., V]`` logits in one online pass,
    without an fp32 softmax of the chunk (reference: src/axolotl/monkeypatch/trainer/utils.py:23-510).
    Not differentiable: the RL trainers only log it."""
    V = logits.shape[-1]
    z = logits.reshape(-1, V)
    if not z.is_cuda:
        lp = torch.log_softmax(z.float() / temperature, -1)
        ent = -(lp.exp() * lp).sum(-1)
        lse = torch.logsumexp(z.float() / temperature, -1)
    else:
        lib = _lib.cuda_lib()
        if z.dtype != torch.bfloat16 or z.stride(1) != 1 or z.stride(0) % 8:
            z = z.to(torch.bfloat16).contiguous()
            if V % 8:
                z = F.pad(z, (0, 8 - V % 8))[:, :V]   # keeps a 16-byte aligned row pitch
        ent = torch.empty(z.shape[0], dtype=torch.float32, device=z.device)
        lse = torch.empty_like(ent)
        _lib.check_rc(lib.axb_entropy(z.data_ptr(), ent.data_ptr(), lse.data_ptr(), z.shape[0], V, z.stride(0),
                                      1.0 / temperature, _lib.stream_ptr()), "entropy")
    ent, lse = ent.view(logits.shape[:-1]), lse.view(logits.shape[:-1])
    return (ent, lse) if return_lse else ent


# --------------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids):
        ctx.save_for_backward(ids)
        ctx.tshape = table.shape
        ctx.tdtype = table.dtype
        if not table.is_cuda:
            return F.embedding(ids, table)
        lib = _lib.cuda_lib()
        flat = ids.reshape(-1).contiguous()
        out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
        _lib.check_rc(lib.axb_embedding_fwd(table.data_ptr(), flat.data_ptr(), out.data_ptr(),
                                            flat.numel(), table.shape[1], table.shape[0],
                                            _lib.stream_ptr()), "embedding_fwd")
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None
        V, H = ctx.tshape
        if not dout.is_cuda:
            g = torch.zeros(V, H, dtype=torch.float32)
            g.index_add_(0, ids.reshape(-1), dout.reshape(-1, H).float())
            return g.to(ctx.tdtype), None
        lib = _lib.cuda_lib()
        g = torch.zeros(V, H, dtype=torch.float32, device=dout.device)
        d2 = dout.reshape(-1, H).contiguous()
        flat = ids.reshape(-1).contiguous()
        _lib.check_rc(lib.axb_embedding_bwd(d2.data_ptr(), flat.data_ptr(), g.data_ptr(),
                                            flat.numel(), H, V, _lib.stream_ptr()), "embedding_bwd")
        return g.to(ctx.tdtype), None


def embedding(table, ids):
    return _Embedding.apply(table, ids)


# --------------------------------------------------------------------------------------- attention
class AttnMeta:
    """Per-batch varlen metadata: cu_seqlens plus the tile tables of the attention kernels.

    Built once per packed row on the host (the collator knows the document boundaries) and
    reused by every layer's forward and backward.
    """

    def __init__(self, cu_seqlens, device, causal=True, window=None):
        cu = np.asarray(cu_seqlens, dtype=np.int32)
        self.cu_seqlens_host = cu
        self.causal = bool(causal)   # False: every token attends to its whole document
        self.window = int(window) if window else 0   # causal sliding window: token q sees (q - window, q]
        if self.window and not self.causal:
            raise ValueError("a sliding window applies to causal attention only")
        self.n_docs = len(cu) - 1
        self.total = int(cu[-1])
        self.max_len = int((cu[1:] - cu[:-1]).max()) if self.n_docs else 0
        self.device = torch.device(device)
        self.cu_seqlens = torch.from_numpy(cu.copy()).to(self.device)
        self.tiles_fwd = self.tiles_bwd = None
        self.n_tiles = 0
        if self.device.type == "cuda":
            host = _lib.host_lib()
            max_tiles = (self.total + 127) // 128 + self.n_docs
            bufs = []
            for heavy_first in (1, 0):
                buf = np.zeros((max_tiles, 4), dtype=np.int32)
                n = host.axb_build_attn_tiles(cu.ctypes.data, self.n_docs, 128, heavy_first,
                                              buf.ctypes.data, max_tiles)
                if not self.causal:
                    buf[:n, 3] |= 1    # tile flag bit 0: bidirectional document
                elif self.window:
                    buf[:n, 3] |= self.window << 1   # bits 1..: sliding window in tokens
                bufs.append(buf[:n])
            self.n_tiles = len(bufs[0])
            both = torch.from_numpy(np.concatenate(bufs, 0)).pin_memory()
            both = both.to(self.device, non_blocking=True)
            self.tiles_fwd, self.tiles_bwd = both[: self.n_tiles], both[self.n_tiles:]

    def windowed(self, window):
        """The same documents with a causal sliding window (cached: every layer of a model asks for it)."""
        if not window or window >= self.max_len:
            return self            # no document is longer than the window: plain causal attention is exact
        cache = self.__dict__.setdefault("_windowed", {})
        if window not in cache:
            cache[window] = AttnMeta(self.cu_seqlens_host, self.device, True, window)
        groups = getattr(self, "image_groups", None)
        if groups is not None:         # both directions inside an image hold on windowed layers too
            cache[window].image_groups, cache[window].image_group_span = groups, self.image_group_span
        return cache[window]

    def chunked(self, chunk):
        """The same token stream with every document cut at multiples of ``chunk`` positions: attention stays inside
        a chunk (Llama 4 local layers). Cached per chunk size."""
        if not chunk or chunk >= self.max_len:
            return self
        cache = self.__dict__.setdefault("_chunked", {})
        if chunk not in cache:
            cu = [0]
            for s0, e0 in zip(self.cu_seqlens_host[:-1], self.cu_seqlens_host[1:]):
                cu.extend(range(int(s0) + chunk, int(e0), chunk))
                cu.append(int(e0))
            cache[chunk] = AttnMeta(np.asarray(sorted(set(cu)), dtype=np.int32), self.device, self.causal)
        return cache[chunk]

    @staticmethod
    def from_position_ids(position_ids, device, causal=True):
        """Document starts are the positions where ``position_ids`` resets to 0."""
        p = position_ids.reshape(-1).cpu().numpy()
        starts = np.flatnonzero(p == 0)
        if len(starts) == 0 or starts[0] != 0:
            starts = np.concatenate([[0], starts])
        cu = np.concatenate([starts, [len(p)]]).astype(np.int32)
        return AttnMeta(cu, device, causal)


def _attn_ref(q, k, v, cu, scale, causal=True, window=0, softcap=0.0, sinks=None):
    # q [T,Hq,D], k [T,Hk,D], v [T,Hk,Dv]; per-document (causal or bidirectional) attention in fp32
    T, Hq, D = q.shape
    Hk = k.shape[1]
    rep = Hq // Hk
    out = torch.empty((T, Hq, v.shape[2]), dtype=q.dtype, device=q.device)
    for d in range(len(cu) - 1):
        s, e = int(cu[d]), int(cu[d + 1])
        qq = q[s:e].float().transpose(0, 1)
        kk = k[s:e].float().repeat_interleave(rep, 1).transpose(0, 1)
        vv = v[s:e].float().repeat_interleave(rep, 1).transpose(0, 1)
        sc = (qq @ kk.transpose(1, 2)) * scale
        if softcap:
            sc = torch.tanh(sc / softcap) * softcap
        if causal:
            mask = torch.ones(e - s, e - s, dtype=torch.bool, device=q.device).tril()
            if window:
                mask &= ~torch.ones(e - s, e - s, dtype=torch.bool, device=q.device).tril(-int(window))
            sc = sc.masked_fill(~mask, float("-inf"))
        if sinks is not None:    # one extra logit per head that takes probability mass and carries no value
            sk = sinks.float()[:, None, None].expand(Hq, e - s, 1)
            pr = torch.cat([sc, sk], -1).softmax(-1)[..., :-1]
        else:
            pr = sc.softmax(-1)
        out[s:e] = (pr @ vv).transpose(0, 1).to(q.dtype)
    return out


_LOG2E = 1.4426950408889634


def _apply_sinks(out, lse2, sinks, Hq):
    """Attention sinks as a rescale of the kernel's result: with one more logit ``sink_h`` in every softmax
    denominator, O' = O * exp(lse - lse') and lse' = logaddexp(lse, sink). Returns (O', lse' in the log2 domain)."""
    T = out.shape[0]
    s2 = sinks.float()[:, None] * _LOG2E
    lse_new = torch.logaddexp2(lse2, s2.expand_as(lse2))
    factor = torch.exp2(lse2 - lse_new)                         # [Hq, T]
    out = (out.view(T, Hq, -1).float() * factor.t()[:, :, None]).to(out.dtype).view(T, -1)
    return out, lse_new


class _FlashVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, meta, Hq, Hk, D, scale, sinks=None):
        T = qkv.shape[0]
        ctx.meta, ctx.dims = meta, (Hq, Hk, D, scale)
        if not qkv.is_cuda:
            raise RuntimeError("CPU tensors take the autograd reference path in flash_varlen()")
        lib = _lib.cuda_lib()
        out = torch.empty((T, Hq * D), dtype=qkv.dtype, device=qkv.device)
        lse2 = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
        _lib.check_rc(
            lib.axb_flash_varlen_fwd(qkv.data_ptr(), qkv.stride(0), T, Hq, Hk, D, 0, Hq * D,
                                     (Hq + Hk) * D, meta.tiles_fwd.data_ptr(), meta.n_tiles,
                                     out.data_ptr(), out.stride(0), lse2.data_ptr(), scale,
                                     _lib.status_word(qkv.device).data_ptr(), _lib.stream_ptr()),
            "flash_varlen_fwd")
        ctx.has_sinks = sinks is not None
        if sinks is not None:
            out, lse2 = _apply_sinks(out, lse2, sinks, Hq)
            ctx.save_for_backward(qkv, out, lse2, sinks)
        else:
            ctx.save_for_backward(qkv, out, lse2)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse2 = ctx.saved_tensors[:3]
        Hq, Hk, D, scale = ctx.dims
        meta = ctx.meta
        T = qkv.shape[0]
        lib = _lib.cuda_lib()
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dq_acc = torch.empty((T, Hq * D), dtype=torch.float32, device=qkv.device)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
        _lib.check_rc(
            lib.axb_flash_varlen_bwd(qkv.data_ptr(), qkv.stride(0), dout.data_ptr(),
                                     out.data_ptr(), out.stride(0), lse2.data_ptr(), T, Hq, Hk, D,
                                     0, Hq * D, (Hq + Hk) * D, meta.tiles_bwd.data_ptr(),
                                     meta.n_tiles, dqkv.data_ptr(), dqkv.stride(0),
                                     dq_acc.data_ptr(), delta.data_ptr(), scale,
                                     _lib.status_word(qkv.device).data_ptr(), _lib.stream_ptr()),
            "flash_varlen_bwd")
        dsinks = None
        if ctx.has_sinks:
            sinks = ctx.saved_tensors[3]
            if ctx.needs_input_grad[6]:
                # d sink_h = - sum_t p_sink[h, t] * <dO_t, O'_t>; the kernel left the row dot products in `delta`
                p_sink = torch.exp2(sinks.float()[:, None] * _LOG2E - lse2)
                dsinks = (-(p_sink * delta).sum(1)).to(sinks.dtype)
        return dqkv, None, None, None, None, None, dsinks


class _FlashWide(torch.autograd.Function):
    """Wide heads (q/k 256 with v 256, or q/k 192 with v 128) and tanh soft-capped scores: csrc/flash_wide.cu."""

    @staticmethod
    def forward(ctx, qkv, meta, Hq, Hk, D, Dv, scale, softcap):
        T = qkv.shape[0]
        ctx.meta, ctx.dims = meta, (Hq, Hk, D, Dv, scale, softcap)
        lib = _lib.cuda_lib()
        out = torch.empty((T, Hq * Dv), dtype=qkv.dtype, device=qkv.device)
        lse2 = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
        _lib.check_rc(
            lib.axb_flash_wide_fwd(qkv.data_ptr(), qkv.stride(0), T, Hq, Hk, D, Dv, 0, Hq * D, (Hq + Hk) * D,
                                   meta.tiles_fwd.data_ptr(), meta.n_tiles, out.data_ptr(), out.stride(0),
                                   lse2.data_ptr(), scale, float(softcap or 0.0),
                                   _lib.status_word(qkv.device).data_ptr(), _lib.stream_ptr()), "flash_wide_fwd")
        ctx.save_for_backward(qkv, out, lse2)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse2 = ctx.saved_tensors
        Hq, Hk, D, Dv, scale, softcap = ctx.dims
        meta = ctx.meta
        T = qkv.shape[0]
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dq_acc = torch.empty((T, Hq * D), dtype=torch.float32, device=qkv.device)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
        _lib.check_rc(
            _lib.cuda_lib().axb_flash_wide_bwd(
                qkv.data_ptr(), qkv.stride(0), dout.data_ptr(), out.data_ptr(), out.stride(0), lse2.data_ptr(), T, Hq,
                Hk, D, Dv, 0, Hq * D, (Hq + Hk) * D, meta.tiles_bwd.data_ptr(), meta.n_tiles, dqkv.data_ptr(),
                dqkv.stride(0), dq_acc.data_ptr(), delta.data_ptr(), scale, float(softcap or 0.0),
                _lib.status_word(qkv.device).data_ptr(), _lib.stream_ptr()), "flash_wide_bwd")
        return dqkv, None, None, None, None, None, None, None


WIDE_HEADS = ((256, 256), (192, 128))


_BLOCKED_WARNED = set()


def _attn_block(qb, kk, vv, q0, k0, scale, causal, window, softcap, gq=None, gk=None):
    """qb [B, Hk, rep, D] against kk [n, Hk, D] / vv [n, Hk, Dv]; q0 / k0: document positions of the first query / key.
    ``gq`` / ``gk``: image group of every query / key (-1 = text); members of one group see each other whatever the order."""
    sc = torch.einsum("bgrd,ngd->grbn", qb, kk).float() * scale
    if softcap:
        sc = torch.tanh(sc / softcap) * softcap
    if causal:
        qi = (q0 + torch.arange(qb.shape[0], device=qb.device))[:, None]
        ki = (k0 + torch.arange(kk.shape[0], device=qb.device))[None, :]
        keep = ki <= qi
        if window:
            keep &= ki > qi - window
        if gq is not None:
            keep |= (gq[:, None] == gk[None, :]) & (gq[:, None] >= 0)
        sc = sc.masked_fill(~keep, float("-inf"))
    return torch.einsum("grbn,ngd->bgrd", sc.softmax(-1).to(vv.dtype), vv)


def _blocked_attention(qkv, meta, Hq, Hk, D, Dv, scale, softcap, block=256, groups=None, group_span=0):
    """Head widths without a kernel of their own (e.g. 512): blocks of queries against their visible keys through
    library batched GEMMs, each block recomputed in the backward pass, so memory stays O(block x length) per head.
    Correct for every width; far from the tensor-core kernels in speed (said once per width on stderr)."""
    if groups is None and (D, Dv) not in _BLOCKED_WARNED:
        _BLOCKED_WARNED.add((D, Dv))
        import sys

        print(f"[axolotl_b200] attention head widths (q/k {D}, v {Dv}): no tcgen05 kernel for this layout, "
              f"running the blocked library path", file=sys.stderr)
    from torch.utils.checkpoint import checkpoint

    T = qkv.shape[0]
    rep = Hq // Hk
    q = qkv[:, : Hq * D].reshape(T, Hk, rep, D)
    k = qkv[:, Hq * D: (Hq + Hk) * D].reshape(T, Hk, D)
    v = qkv[:, (Hq + Hk) * D:].reshape(T, Hk, Dv)
    causal, window = getattr(meta, "causal", True), int(getattr(meta, "window", 0) or 0)
    cu = [int(c) for c in meta.cu_seqlens_host]
    outs = []
    need_grad = torch.is_grad_enabled() and qkv.requires_grad
    for s, e in zip(cu[:-1], cu[1:]):
        for b0 in range(s, e, block):
            b1 = min(b0 + block, e)
            k0 = max(s, b0 - window + 1) if (causal and window) else s
            k1 = b1 if causal else e
            args = (q[b0:b1], k[k0:k1], v[k0:k1], b0 - s, k0 - s, scale, causal, window, softcap)
            if groups is not None:      # an image may begin before the window or end after the block: widen by its length
                k0, k1 = max(s, k0 - group_span), min(e, k1 + group_span)
                args = (q[b0:b1], k[k0:k1], v[k0:k1], b0 - s, k0 - s, scale, causal, window, softcap, groups[b0:b1], groups[k0:k1])
            outs.append(checkpoint(_attn_block, *args, use_reentrant=False) if need_grad else _attn_block(*args))
    return torch.cat(outs, 0).reshape(T, Hq * Dv)


def flash_varlen(qkv, meta: AttnMeta, Hq, Hk, D, scale=None, Dv=None, softcap=0.0, sinks=None):
    """Attention inside each document of a packed row: causal, or bidirectional when the
    metadata was built with ``causal=False`` (masked-diffusion and encoder-style objectives).

    ``qkv`` is the fused projection [T, Hq*D + Hk*D + Hk*Dv] (q heads, then k heads, then v heads; ``Dv``
    defaults to ``D``). Returns [T, Hq * Dv]. Head widths 64 / 128 run the double-buffered kernels;
    (D, Dv) = (256, 256) or (192, 128), and any ``softcap`` (scores become softcap * tanh(scores / softcap))
    at those widths, run the wide kernels; every other width (e.g. 512) runs a blocked library path. ``sinks`` [Hq]: one learned logit per head joins every softmax
    denominator (gpt-oss); applied as a rescale of the kernel's output and log-sum-exp.
    """
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    Dv = D if Dv is None else Dv
    if getattr(meta, "image_groups", None) is not None:
        # Gemma 3 with images: causal attention plus both directions inside every image. The causal kernels cannot
        # express that mask; these batches take the blocked path (any device)
        if getattr(meta, "cp", False) or sinks is not None or getattr(meta, "kv_cache", None) is not None:
            raise NotImplementedError("bidirectional image attention runs without context parallelism, sinks and KV cache")
        return _blocked_attention(qkv, meta, Hq, Hk, D, Dv, scale, softcap, groups=meta.image_groups,
                                  group_span=int(meta.image_group_span))
    if sinks is not None and qkv.is_cuda and ((D, Dv) in WIDE_HEADS or getattr(meta, "cp", False)):
        raise NotImplementedError("attention sinks are available for head widths 64 / 128 without context parallelism")
    if qkv.is_cuda and ((D, Dv) in WIDE_HEADS):
        if getattr(meta, "cp", False):
            raise NotImplementedError("context parallelism is not available for head widths above 128")
        return _FlashWide.apply(qkv, meta, Hq, Hk, D, Dv, scale, softcap)
    if qkv.is_cuda and (softcap or Dv != D or D not in (64, 128)):
        if getattr(meta, "cp", False) or sinks is not None:
            raise NotImplementedError(
                f"attention head widths (q/k {D}, v {Dv}) with softcap={softcap}: the CUDA kernels take 64, 128, "
                f"(256, 256) and (192, 128); other widths run without context parallelism and sinks only")
        return _blocked_attention(qkv, meta, Hq, Hk, D, Dv, scale, softcap)
    if getattr(meta, "cp", False):
        from ..parallel.cp import flash_varlen_cp   # context parallelism is causal only, without a window

        return flash_varlen_cp(qkv, meta, Hq, Hk, D, scale)
    if qkv.is_cuda:
        return _FlashVarlen.apply(qkv, meta, Hq, Hk, D, scale, sinks)
    T = qkv.shape[0]
    q = qkv[:, : Hq * D].reshape(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hk) * D].reshape(T, Hk, D)
    v = qkv[:, (Hq + Hk) * D:].reshape(T, Hk, Dv)
    return _attn_ref(q, k, v, meta.cu_seqlens_host, scale, getattr(meta, "causal", True),
                     getattr(meta, "window", 0), softcap, sinks).reshape(T, Hq * Dv)


@torch.no_grad()
def decode_attention(qkv, k_cache, v_cache, lens, Hq, Hk, D, scale=None, window=0):
    """Attention of ONE new token per sequence against its KV cache (generation).

    ``qkv`` [B, (Hq + 2*Hk) * D]: fused projection of the new tokens, q / k already rotated;
    ``k_cache`` / ``v_cache`` [B, max_len, Hk * D] with the new token's k / v already stored at
    position ``lens[b] - 1``; ``lens`` [B] int32: live positions including the new token.
    ``window`` > 0 restricts every query to its last ``window`` positions.
    Returns [B, Hq * D]. Inference only (no autograd)."""
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    B = qkv.shape[0]
    if qkv.is_cuda:
        lib = _lib.cuda_lib()
        out = torch.empty((B, Hq * D), dtype=qkv.dtype, device=qkv.device)
        _lib.check_rc(lib.axb_decode_attn(qkv.data_ptr(), qkv.stride(0), 0, k_cache.data_ptr(), v_cache.data_ptr(),
                                          lens.data_ptr(), out.data_ptr(), out.stride(0), B, Hq, Hk, D,
                                          k_cache.shape[1], scale, int(window or 0), _lib.stream_ptr()), "decode_attn")
        return out
    q = qkv[:, : Hq * D].reshape(B, Hk, Hq // Hk, D).float()
    out = torch.empty(B, Hq * D, dtype=qkv.dtype)
    for b in range(B):
        n = int(lens[b])
        s0 = max(0, n - int(window)) if window else 0
        k = k_cache[b, s0:n].reshape(n - s0, Hk, D).float().transpose(0, 1)     # [Hk, n, D]
        v = v_cache[b, s0:n].reshape(n - s0, Hk, D).float().transpose(0, 1)
        p = torch.softmax((q[b] @ k.transpose(1, 2)) * scale, -1)        # [Hk, G, n]
        out[b] = (p @ v).reshape(-1).to(qkv.dtype)
    return out


# --------------------------------------------------------------------------------------- loss
class _LinearCE(torch.autograd.Function):
    """Chunked lm_head GEMM + cross entropy that never materialises [T, V] logits.

    For each chunk of rows: logits = h @ W^T (tcgen05 GEMM) -> in-place CE kernel that returns the
    per-row loss and overwrites the logits with their gradient -> dH chunk = dlogits @ W (and
    dW += dlogits^T @ h when the head is trainable). The backward pass only rescales.
    """

    @staticmethod
    def forward(ctx, h, w, labels, denom, chunk_rows, ignore_index, lora, softcap=0.0):
        from .gemm import gemm, pick_splits

        T, H = h.shape
        V = w.shape[0]
        need_dw = w.requires_grad
        dh = torch.empty_like(h)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device) if need_dw else None
        losses = torch.empty(T, dtype=torch.float32, device=h.device)
        lib = _lib.cuda_lib() if h.is_cuda else None
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            hc = h[r0:r1]
            logits = gemm(hc, w)
            if h.is_cuda and softcap:
                _lib.check_rc(
                    lib.axb_ce_fwd_bwd_softcap(logits.data_ptr(), labels[r0:r1].data_ptr(), losses[r0:r1].data_ptr(),
                                               None, r1 - r0, V, logits.stride(0), 1.0 / denom, ignore_index, 1,
                                               float(softcap), _lib.stream_ptr()), "ce_fwd_bwd_softcap")
                dlogits = logits
            elif h.is_cuda:
                _lib.check_rc(
                    lib.axb_ce_fwd_bwd(logits.data_ptr(), labels[r0:r1].data_ptr(),
                                       losses[r0:r1].data_ptr(), None, r1 - r0, V,
                                       logits.stride(0), 1.0 / denom, ignore_index, 1,
                                       _lib.stream_ptr()), "ce_fwd_bwd")
                dlogits = logits
            else:
                lf = logits.float()
                dcap = None
                if softcap:
                    t = torch.tanh(lf / softcap)
                    lf, dcap = t * softcap, 1.0 - t * t
                lab = labels[r0:r1]
                valid = lab != ignore_index
                lse = torch.logsumexp(lf, -1)
                tgt = lf.gather(1, lab.clamp(min=0)[:, None]).squeeze(1)
                losses[r0:r1] = torch.where(valid, lse - tgt, torch.zeros_like(lse))
                p = torch.softmax(lf, -1)
                p[torch.arange(r1 - r0), lab.clamp(min=0)] -= 1.0
                if dcap is not None:
                    p = p * dcap
                dlogits = (p * valid[:, None] / denom).to(logits.dtype)
            gemm(dlogits, w, trans_b=True, out=dh[r0:r1])
            if need_dw:
                sp = pick_splits(((V + 127) // 128) * ((H + 255) // 256), (r1 - r0 + 63) // 64)
                gemm(dlogits, hc, trans_a=True, trans_b=True, out=dw, accumulate=True, splits=sp)
        ctx.save_for_backward(dh, dw)
        ctx.w_dtype = w.dtype
        return losses.sum() / denom

    @staticmethod
    def backward(ctx, gout):
        dh, dw = ctx.saved_tensors
        return (dh * gout.to(dh.dtype), (dw * gout).to(ctx.w_dtype) if dw is not None else None,
                None, None, None, None, None, None)


def linear_cross_entropy(hidden, lm_head_weight, labels, num_items=None, chunk_rows=2048,
                         ignore_index=IGNORE_INDEX, softcap=0.0):
    """Mean (or ``sum / num_items``) token cross entropy of ``hidden @ W^T`` against ``labels``.

    ``labels`` must already be shifted (labels[t] is the target of position t). ``softcap``: the logits are
    soft-capped first, ``softcap * tanh(logits / softcap)`` (Gemma 2).
    """
    hidden = hidden.reshape(-1, hidden.shape[-1])
    labels = labels.reshape(-1).contiguous()
    if num_items is None:
        num_items = int((labels != ignore_index).sum().item())
    denom = float(max(num_items, 1))
    return _LinearCE.apply(hidden.contiguous(), lm_head_weight, labels, denom, chunk_rows,
                           ignore_index, None, float(softcap or 0.0))


class _LinearTokenLogps(torch.autograd.Function):
    """Per-token log-probability of ``labels`` under ``softmax(h @ W^T)`` without keeping [T, V].

    Forward: per chunk of rows, logits by the tcgen05 GEMM, then the cross-entropy kernel in
    loss-only mode. Backward: the chunk's logits are recomputed, the kernel overwrites them with
    ``softmax - onehot`` and ``dH = diag(-g) (dlogits @ W)``; the row scaling is applied to the
    [rows, H] product rather than to the [rows, V] logits. Ignored rows return 0 and get no
    gradient. Preference and policy-gradient objectives (which need a weight per token or per
    sequence, not one global mean) are built on this.
    """

    @staticmethod
    def forward(ctx, h, w, labels, chunk_rows, ignore_index, entropy_out=None):
        from .gemm import gemm

        T = h.shape[0]
        V = w.shape[0]
        nll = torch.zeros(T, dtype=torch.float32, device=h.device)
        if h.is_cuda:
            lib = _lib.cuda_lib()
            for r0 in range(0, T, chunk_rows):
                r1 = min(T, r0 + chunk_rows)
                logits = gemm(h[r0:r1], w)
                if entropy_out is not None:   # the logits chunk is still intact here
                    _lib.check_rc(lib.axb_entropy(logits.data_ptr(), entropy_out[r0:r1].data_ptr(), None, r1 - r0, V,
                                                  logits.stride(0), 1.0, _lib.stream_ptr()), "entropy")
                _lib.check_rc(lib.axb_ce_fwd_bwd(logits.data_ptr(), labels[r0:r1].data_ptr(), nll[r0:r1].data_ptr(),
                                                 None, r1 - r0, V, logits.stride(0), 1.0, ignore_index, 0,
                                                 _lib.stream_ptr()), "ce_fwd")
        else:
            for r0 in range(0, T, chunk_rows):
                r1 = min(T, r0 + chunk_rows)
                lf = (h[r0:r1] @ w.to(h.dtype).t()).float()
                lab = labels[r0:r1]
                valid = lab != ignore_index
                lsm = torch.log_softmax(lf, -1)
                if entropy_out is not None:
                    entropy_out[r0:r1] = -(lsm.exp() * lsm).sum(-1)
                lp = lsm.gather(1, lab.clamp(min=0)[:, None]).squeeze(1)
                nll[r0:r1] = torch.where(valid, -lp, torch.zeros_like(lp))
        ctx.save_for_backward(h, w, labels)
        ctx.chunk_rows, ctx.ignore_index = chunk_rows, ignore_index
        return -nll

    @staticmethod
    def backward(ctx, g):
        from .gemm import gemm, pick_splits

        h, w, labels = ctx.saved_tensors
        T, H = h.shape
        V = w.shape[0]
        need_dw = ctx.needs_input_grad[1]
        dh = torch.empty_like(h)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device) if need_dw else None
        s = (-g).float()
        for r0 in range(0, T, ctx.chunk_rows):
            r1 = min(T, r0 + ctx.chunk_rows)
            hc = h[r0:r1]
            if h.is_cuda:
                logits = gemm(hc, w)
                tmp = torch.empty(r1 - r0, dtype=torch.float32, device=h.device)
                _lib.check_rc(_lib.cuda_lib().axb_ce_fwd_bwd(
                    logits.data_ptr(), labels[r0:r1].data_ptr(), tmp.data_ptr(), None, r1 - r0, V,
                    logits.stride(0), 1.0, ctx.ignore_index, 1, _lib.stream_ptr()), "ce_bwd")
                dlogits = logits
            else:
                lf = (hc @ w.to(h.dtype).t()).float()
                lab = labels[r0:r1]
                valid = lab != ctx.ignore_index
                p = torch.softmax(lf, -1)
                p[torch.arange(r1 - r0), lab.clamp(min=0)] -= 1.0
                dlogits = (p * valid[:, None]).to(h.dtype)
            sc = s[r0:r1, None]
            dh[r0:r1] = (gemm(dlogits, w, trans_b=True).float() * sc).to(h.dtype)
            if need_dw:
                hs = (hc.float() * sc).to(h.dtype)
                sp = pick_splits(((V + 127) // 128) * ((H + 255) // 256), (r1 - r0 + 63) // 64) if h.is_cuda else 1
                gemm(dlogits, hs, trans_a=True, trans_b=True, out=dw, accumulate=True, splits=sp)
        return dh, (dw.to(w.dtype) if dw is not None else None), None, None, None, None


def linear_token_logps(hidden, lm_head_weight, labels, chunk_rows=2048, ignore_index=IGNORE_INDEX,
                       entropy_out=None):
    """log p(labels[t] | position t) for every row of ``hidden`` ([T] fp32; 0 where ignored).
    ``labels`` must already be shifted. ``entropy_out`` ([T] fp32, optional) receives the entropy of
    every row's distribution (a logged quantity: no gradient)."""
    hidden = hidden.reshape(-1, hidden.shape[-1]).contiguous()
    return _LinearTokenLogps.apply(hidden, lm_head_weight, labels.reshape(-1).contiguous(), chunk_rows, ignore_index,
                                   entropy_out)


class _XIELU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ap, an, beta, eps):
        ctx.save_for_backward(x, ap, an)
        ctx.consts = (float(beta), float(eps))
        y = torch.empty_like(x)
        _lib.check_rc(_lib.cuda_lib().axb_xielu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), float(ap), float(an), float(beta),
                                                    float(eps), _lib.stream_ptr()), "xielu_fwd")
        return y

    @staticmethod
    def backward(ctx, dy):
        x, ap, an = ctx.saved_tensors
        beta, eps = ctx.consts
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        sums = torch.zeros(2, dtype=torch.float32, device=x.device)
        _lib.check_rc(_lib.cuda_lib().axb_xielu_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), sums.data_ptr(), x.numel(),
                                                    float(ap), float(an), beta, eps, _lib.stream_ptr()), "xielu_bwd")
        return dx, sums[0].reshape(ap.shape).to(ap.dtype), sums[1].reshape(an.shape).to(an.dtype), None, None


def xielu(x, alpha_p, alpha_n, beta=0.5, eps=-1e-6):
    """xIELU activation: ``alpha_p x^2 + beta x`` for x > 0, ``alpha_n (expm1(min(x, eps)) - x) + beta x`` otherwise;
    ``alpha_p`` / ``alpha_n`` are the EFFECTIVE (already soft-plussed) one-element fp32 tensors, gradients flow to them."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _XIELU.apply(x.contiguous(), alpha_p.float().reshape(1), alpha_n.float().reshape(1), beta, eps)
    xf = x.float()
    neg = (torch.expm1(torch.clamp(xf, max=eps)) - xf) * alpha_n.float() + beta * xf
    return torch.where(xf > 0, alpha_p.float() * xf * xf + beta * xf, neg).to(x.dtype)


class _GatedPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kv, gate):
        M, W, D = kv.shape
        out = torch.empty((M, D), dtype=torch.float32, device=kv.device)
        _lib.check_rc(_lib.cuda_lib().axb_gated_pool_fwd(kv.data_ptr(), gate.data_ptr(), out.data_ptr(), M, W, D,
                                                         _lib.stream_ptr()), "gated_pool_fwd")
        ctx.save_for_backward(kv, gate, out)
        return out

    @staticmethod
    def backward(ctx, g):
        kv, gate, out = ctx.saved_tensors
        M, W, D = kv.shape
        g = g.contiguous().float()
        d_kv, d_gate = torch.empty_like(kv), torch.empty_like(gate)
        _lib.check_rc(_lib.cuda_lib().axb_gated_pool_bwd(kv.data_ptr(), gate.data_ptr(), out.data_ptr(), g.data_ptr(),
                                                         d_kv.data_ptr(), d_gate.data_ptr(), M, W, D, _lib.stream_ptr()),
                      "gated_pool_bwd")
        return d_kv, d_gate


def gated_softmax_pool(kv, gate):
    """``(kv * softmax(gate, dim=-2)).sum(-2)`` for [..., W, D] inputs in fp32 (the window pooling of DeepSeek-V4's
    compressors), one pass forward, probabilities recomputed in the backward pass."""
    if kv.is_cuda:
        lead = kv.shape[:-2]
        W, D = kv.shape[-2:]
        out = _GatedPool.apply(kv.float().reshape(-1, W, D).contiguous(), gate.float().reshape(-1, W, D).contiguous())
        return out.reshape(*lead, D)
    return (kv.float() * gate.float().softmax(dim=-2)).sum(-2)


class _AddLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, b, eps, w_offset):
        T, D = x.shape
        lib = _lib.cuda_lib()
        y = torch.empty_like(x)
        s = torch.empty_like(x) if residual is not None else x
        mean = torch.empty(T, dtype=torch.float32, device=x.device)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        _lib.check_rc(lib.axb_layernorm_fwd(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                            w.data_ptr() if w is not None else None, b.data_ptr() if b is not None else None,
                                            y.data_ptr(), s.data_ptr() if residual is not None else None, mean.data_ptr(),
                                            rstd.data_ptr(), T, D, float(eps), float(w_offset), _lib.stream_ptr()), "layernorm_fwd")
        ctx.save_for_backward(s, w, mean, rstd)
        ctx.has = (residual is not None, b is not None, float(w_offset))
        if residual is None:                 # no new stream: the second output is a placeholder
            dummy = x.new_empty(0)
            ctx.mark_non_differentiable(dummy)
            return y, dummy
        return y, s

    @staticmethod
    def backward(ctx, dy, ds):
        s, w, mean, rstd = ctx.saved_tensors
        has_res, has_b, w_offset = ctx.has
        T, D = s.shape
        dy = dy.contiguous()
        dres = ds.contiguous() if (has_res and ds is not None) else None
        dx = torch.empty_like(s)
        dw = torch.zeros(D, dtype=torch.float32, device=s.device) if w is not None else None
        db = torch.zeros(D, dtype=torch.float32, device=s.device) if has_b else None
        _lib.check_rc(_lib.cuda_lib().axb_layernorm_bwd(s.data_ptr(), dy.data_ptr(), dres.data_ptr() if dres is not None else None,
                                                        w.data_ptr() if w is not None else None, mean.data_ptr(), rstd.data_ptr(),
                                                        dx.data_ptr(), dw.data_ptr() if dw is not None else None,
                                                        db.data_ptr() if db is not None else None, T, D, w_offset,
                                                        _lib.stream_ptr()), "layernorm_bwd")
        return (dx, dx if has_res else None, dw.to(w.dtype) if w is not None else None,
                db.to(s.dtype) if has_b else None, None, None)


def add_layernorm(x, residual, w, b, eps, w_offset=0.0):
    """``s = x + residual`` (when given), ``y = LayerNorm(s) * (w + w_offset) + b``; returns (y, s). bf16 rows on the
    device take the fused kernel (the stream ``s`` is normalised as stored, in bf16), everything else the fp32 op."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] * 8 <= 200 * 1024:
        x = x.contiguous()
        y, s = _AddLayerNorm.apply(x, residual.contiguous() if residual is not None else None, w, b, eps, w_offset)
        return y, (s if residual is not None else x)
    s = x if residual is None else x + residual
    wf = None if w is None else (w.float() + w_offset if w_offset else w.float())
    y = torch.nn.functional.layer_norm(s.float(), (s.shape[-1],), wf, b.float() if b is not None else None, eps).to(s.dtype)
    return y, s


# ------------------------------------------------------------------------- hyper-connection mixer (DeepSeek-V4)
def sinkhorn_mix_ref(mixes, scale, base, hc=4, iters=20, eps=1e-6, post_mult=2.0):
    """Plain form of the hyper-connection mixer. mixes [M, hc (2 + hc)], scale [3], base [hc (2 + hc)] ->
    pre [M, hc] = sigmoid(.) + eps, post [M, hc] = post_mult sigmoid(.), comb [M, hc, hc]: row softmax + eps, then
    Sinkhorn-Knopp: column-normalise, then (iters - 1) x [row-normalise, column-normalise], each x / (sum + eps)."""
    m = mixes.float()
    pre = torch.sigmoid(m[:, :hc] * scale[0] + base[:hc]) + eps
    post = post_mult * torch.sigmoid(m[:, hc:2 * hc] * scale[1] + base[hc:2 * hc])
    c = torch.softmax((m[:, 2 * hc:] * scale[2] + base[2 * hc:]).view(-1, hc, hc), -1) + eps
    c = c / (c.sum(1, keepdim=True) + eps)
    for _ in range(iters - 1):
        c = c / (c.sum(2, keepdim=True) + eps)
        c = c / (c.sum(1, keepdim=True) + eps)
    return pre, post, c


class _SinkhornMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mixes, scale, base, iters, eps, post_mult):
        M = mixes.shape[0]
        pre = torch.empty((M, 4), dtype=torch.float32, device=mixes.device)
        post = torch.empty_like(pre)
        comb = torch.empty((M, 4, 4), dtype=torch.float32, device=mixes.device)
        _lib.check_rc(_lib.cuda_lib().axb_mhc_mix_fwd(mixes.data_ptr(), scale.data_ptr(), base.data_ptr(), pre.data_ptr(),
                                                      post.data_ptr(), comb.data_ptr(), M, 4, iters, eps, post_mult,
                                                      _lib.stream_ptr()), "mhc_mix_fwd")
        ctx.save_for_backward(mixes, scale, base)
        ctx.args = (iters, eps, post_mult)
        return pre, post, comb

    @staticmethod
    def backward(ctx, d_pre, d_post, d_comb):
        mixes, scale, base = ctx.saved_tensors
        iters, eps, post_mult = ctx.args
        M = mixes.shape[0]
        d_mixes = torch.empty_like(mixes)
        d_scale = torch.zeros(3, dtype=torch.float32, device=mixes.device)
        d_base = torch.zeros(24, dtype=torch.float32, device=mixes.device)
        z = lambda g, shape: (torch.zeros(shape, dtype=torch.float32, device=mixes.device) if g is None else g.contiguous().float())  # noqa: E731
        d_pre, d_post, d_comb = z(d_pre, (M, 4)), z(d_post, (M, 4)), z(d_comb, (M, 4, 4))
        _lib.check_rc(_lib.cuda_lib().axb_mhc_mix_bwd(mixes.data_ptr(), scale.data_ptr(), base.data_ptr(), d_pre.data_ptr(),
                                                      d_post.data_ptr(), d_comb.data_ptr(), d_mixes.data_ptr(),
                                                      d_scale.data_ptr(), d_base.data_ptr(), M, 4, iters, eps, post_mult,
                                                      _lib.stream_ptr()), "mhc_mix_bwd")
        return d_mixes, d_scale, d_base, None, None, None


def sinkhorn_mix(mixes, scale, base, hc=4, iters=20, eps=1e-6, post_mult=2.0):
    """(pre, post, comb) of the hyper-connection mixer; fp32. On a GPU with hc = 4 and iters <= 32 one kernel per
    direction holds a token's 4 x 4 matrix in registers for the whole Sinkhorn chain (the eager form is ~40 launches);
    the reference fuses the same chain in Triton (src/axolotl/integrations/kernels/libs/dsv4/mhc.py:260-350)."""
    if not (mixes.is_cuda and hc == 4 and 1 <= iters <= 32):
        return sinkhorn_mix_ref(mixes, scale, base, hc, iters, eps, post_mult)
    lead = mixes.shape[:-1]
    pre, post, comb = _SinkhornMix.apply(mixes.reshape(-1, 24).contiguous().float(), scale.float().contiguous(),
                                         base.float().contiguous(), int(iters), float(eps), float(post_mult))
    return pre.view(*lead, 4), post.view(*lead, 4), comb.view(*lead, 4, 4)


def hyperconnection_forward(streams, fn, base, scale, norm_eps=1e-6, hc=4, iters=20, eps=1e-6, post_mult=2.0):
    """One hyper-connection read: ``streams`` [..., hc, H] (the layer's residual streams) -> (post [..., hc],
    comb [..., hc, hc], collapsed [..., H]). The streams are RMS-normalised as one hc H-wide vector and projected by
    ``fn`` [hc (2 + hc), hc H] (the per-row RMS factor is applied after the product: one pass over the streams), mixed by
    ``sinkhorn_mix``, and collapsed into the layer input as sum_j pre[j] streams[j]. The layer's output y then goes back
    as streams'[i] = post[i] y + sum_j comb[i, j] streams[j]
    (src/axolotl/integrations/kernels/libs/dsv4/mhc.py:586-609)."""
    *lead, n, H = streams.shape
    flat = streams.reshape(-1, n * H)
    r = torch.rsqrt(flat.float().pow(2).mean(-1, keepdim=True) + norm_eps)
    mixes = (flat @ fn.to(flat.dtype).t()).float() * r
    pre, post, comb = sinkhorn_mix(mixes, scale, base, hc, iters, eps, post_mult)
    collapsed = torch.einsum("mj,mjh->mh", pre.to(streams.dtype), streams.reshape(-1, n, H))
    return post.view(*lead, n), comb.view(*lead, n, n), collapsed.view(*lead, H)
