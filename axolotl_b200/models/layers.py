"""Building blocks: fused multi-projection linear layers with LoRA adapters, RMSNorm.

A ``FusedLinear`` holds the row-concatenated weight of several projections that read the same
input (q|k|v, gate|up) so one tcgen05 GEMM serves them all. LoRA adapters attach per
sub-projection; their A matrices are stacked (``lora_A`` [R, in]) and their B matrices form the
diagonal blocks of ``lora_B`` [N, R], which the GEMM consumes as a K-extension. Per-projection
PEFT tensors (``<name>.lora_A.weight`` [r, in], ``<name>.lora_B.weight`` [out, r]) are views of
those buffers, so adapter checkpoints stay PEFT compatible
(reference adapter wiring: src/axolotl/loaders/adapter.py:140-202).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as Fn
from ..ops.lora import linear, lora_linear


_ADAPTERS_ON = True


def adapters_enabled() -> bool:
    return _ADAPTERS_ON


class disable_adapters:
    """Context manager: every adapter is skipped in the forward pass, so a LoRA model computes its
    frozen base model (the implicit reference policy of preference training; the reference gets the
    same effect from ``peft``'s ``disable_adapter`` inside trl)."""

    def __enter__(self):
        global _ADAPTERS_ON
        self._prev = _ADAPTERS_ON
        _ADAPTERS_ON = False

    def __exit__(self, *exc):
        global _ADAPTERS_ON
        _ADAPTERS_ON = self._prev


class RMSNorm(nn.Module):
    """``offset`` = 1 is the Gemma convention: the stored weight w starts at zero and the norm applies 1 + w."""

    def __init__(self, dim, eps=1e-6, dtype=torch.bfloat16, device=None, offset=0.0):
        super().__init__()
        self.offset = float(offset)
        self.weight = nn.Parameter(torch.full((dim,), 1.0 - self.offset, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x, residual=None):
        return Fn.add_rmsnorm(x, residual, self.weight, self.eps, w_offset=self.offset)

    def plain(self, x):
        """The norm alone (no residual stream)."""
        return Fn.rmsnorm(x, self.weight, self.eps, w_offset=self.offset)

    def effective_weight(self):
        return self.weight if not self.offset else (self.weight.float() + self.offset).to(self.weight.dtype)


class LayerNorm(nn.Module):
    """Mean-subtracting norm with the interface of ``RMSNorm`` (Cohere: weight only; StarCoder 2 / Nemotron: weight and
    bias; ``offset`` = 1 is Nemotron's stored-as-(w - 1) convention; OLMo: no parameters). bf16 rows on the device run
    the fused residual-add + LayerNorm kernel (``csrc/layernorm.cu``)."""

    def __init__(self, dim, eps=1e-5, dtype=torch.bfloat16, device=None, bias=True, offset=0.0, affine=True):
        super().__init__()
        self.offset = float(offset)
        self.weight = nn.Parameter(torch.full((dim,), 1.0 - self.offset, dtype=dtype, device=device)) if affine else None
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if (bias and affine) else None
        self.eps = eps

    def plain(self, x):
        shape = x.shape
        y, _ = Fn.add_layernorm(x.reshape(-1, shape[-1]), None, self.weight, self.bias, self.eps, self.offset)
        return y.reshape(shape)

    def forward(self, x, residual=None):
        return Fn.add_layernorm(x, residual, self.weight, self.bias, self.eps, self.offset)

    def effective_weight(self):
        return self.weight if not self.offset else (self.weight.float() + self.offset).to(self.weight.dtype)


def make_norm(cfg, dim, dtype, device, offset=0.0):
    """The architecture's hidden-state norm."""
    kind = cfg.norm_kind()
    if kind == "rms":
        return RMSNorm(dim, cfg.rms_norm_eps, dtype, device, offset=offset)
    return LayerNorm(dim, cfg.rms_norm_eps, dtype, device, bias=kind != "layernorm_nobias",
                     offset=1.0 if kind == "layernorm1p" else 0.0, affine=kind != "layernorm_fixed")


class FusedLinear(nn.Module):
    def __init__(self, in_features, out_features, names, bias=False, dtype=torch.bfloat16,
                 device=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = list(out_features)
        self.names = list(names)
        self.weight = nn.Parameter(torch.empty(sum(out_features), in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(sum(out_features), dtype=dtype, device=device)) if bias else None
        self.dora_magnitude = None
        self.qat = None   # {"weight_dtype": ..., "group_size": ...}: fake-quantised forward while training
        # LoRA state (absent until add_lora)
        self.lora_A = None
        self.lora_B = None
        self.lora_A16 = None
        self.lora_B16 = None
        self.lora_blocks = ()
        self.lora_names = []
        self.lora_r = 0
        self.scaling = 1.0
        self.lora_dropout = 0.0
        self.merged = False
        # MoRA state (absent until add_mora): one square matrix per adapted sub-projection
        self.mora_M = None
        self.mora_names = []
        self.mora_kind = 0

    # ------------------------------------------------------------------ sub-projection views
    def row_range(self, name):
        i = self.names.index(name)
        r0 = sum(self.out_features[:i])
        return r0, r0 + self.out_features[i]

    def sub_weight(self, name):
        r0, r1 = self.row_range(name)
        return self.weight[r0:r1]

    # ------------------------------------------------------------------ LoRA
    def add_lora(self, r, alpha, dropout=0.0, targets=None, use_rslora=False, dtype=torch.float32,
                 init_b_zero=True, use_dora=False):
        targets = [n for n in self.names if targets is None or n in targets]
        if not targets:
            return
        dev = self.weight.device
        if dev.type == "cuda" and r % 8:
            raise ValueError(f"lora_r={r}: the tensor-core path needs an adapter rank that is a multiple of 8 "
                             "(16-byte rows for the bulk tensor copies)")
        R = r * len(targets)
        N = self.weight.shape[0]
        A = torch.empty(R, self.in_features, dtype=dtype, device=dev)
        for i in range(len(targets)):  # PEFT default init: kaiming_uniform(a=sqrt(5)) on A, zeros on B
            nn.init.kaiming_uniform_(A[i * r:(i + 1) * r], a=math.sqrt(5))
        B = torch.zeros(N, R, dtype=dtype, device=dev)
        blocks = []
        for i, n in enumerate(targets):
            r0, r1 = self.row_range(n)
            blocks.append((r0, r1 - r0, i * r, r))
            if not init_b_zero:
                nn.init.normal_(B[r0:r1, i * r:(i + 1) * r], std=0.02)
        self.lora_A = nn.Parameter(A)
        self.lora_B = nn.Parameter(B)
        self.lora_blocks = tuple(blocks)
        self.lora_names = targets
        self.lora_r = r
        self.scaling = alpha / math.sqrt(r) if use_rslora else alpha / r
        self.lora_dropout = dropout
        self.refresh_shadows()
        if use_dora:
            self.add_dora_()

    # ------------------------------------------------------------------ MoRA
    def add_mora(self, r, kind, targets=None, dtype=torch.float32):
        """One zero-initialised square matrix of side ``sqrt((in + out) * r)`` per target."""
        from .mora import mora_rank

        targets = [n for n in self.names if targets is None or n in targets]
        if not targets:
            return
        dev = self.weight.device
        mult = 8 if dev.type == "cuda" else 2
        mats = []
        for n in targets:
            r0, r1 = self.row_range(n)
            rh = mora_rank(self.in_features, r1 - r0, r, mult)
            mats.append(nn.Parameter(torch.zeros(rh, rh, dtype=dtype, device=dev)))
        self.mora_M = nn.ParameterList(mats)
        self.mora_names, self.mora_kind = targets, int(kind)

    def _mora_update(self, x):
        """[.., N] update of all sub-projections (zero columns for the ones without an adapter)."""
        from .mora import mora_delta

        parts, have = [], dict(zip(self.mora_names, self.mora_M))
        for n, rows in zip(self.names, self.out_features):
            if n in have:
                parts.append(mora_delta(x, have[n], rows, self.mora_kind))
            else:
                parts.append(x.new_zeros(*x.shape[:-1], rows))
        return parts[0] if len(parts) == 1 else torch.cat(parts, -1)

    @torch.no_grad()
    def merge_mora_(self):
        from .mora import mora_dense_delta

        if self.mora_M is None:
            return
        self.dequantize_()
        for n, M in zip(self.mora_names, self.mora_M):
            r0, r1 = self.row_range(n)
            d = mora_dense_delta(M.detach(), self.in_features, r1 - r0, self.mora_kind)
            self.weight[r0:r1] = (self.weight[r0:r1].float() + d).to(self.weight.dtype)
            M.zero_()

    # ------------------------------------------------------------------ DoRA
    @torch.no_grad()
    def add_dora_(self):
        """Weight-decomposed LoRA: y_row = m_row / ||W + s B A||_row * (x W^T + s x A^T B^T)_row for
        the rows of adapted sub-projections. ``m`` starts at ||W||_row, so the layer is unchanged at
        initialisation; the norm is treated as a constant in the backward pass (as in PEFT)."""
        W = self._dense_weight().float()
        self.dora_w2 = (W * W).sum(1)                                   # ||W||^2 per row (frozen)
        mask = torch.zeros(W.shape[0], dtype=torch.bool, device=W.device)
        for (r0, rows, _, _) in self.lora_blocks:
            mask[r0:r0 + rows] = True
        self.dora_rows = mask
        self.dora_magnitude = nn.Parameter(self.dora_w2.sqrt().to(self.lora_A.dtype))

    def _dense_weight(self):
        st = getattr(self.weight, "_axb_quant", None)
        if st is not None:
            from ..ops.nf4 import dequantize_nf4

            return dequantize_nf4(self.weight.data, st, dtype=torch.bfloat16 if self.weight.is_cuda else torch.float32)
        return self.weight.detach()

    @torch.no_grad()
    def dora_weight_norm(self):
        """||W + s B A|| per output row without forming B A:
        ||W||^2 + 2 s <W, B A>_row + s^2 ||B A||^2_row, with <W, B A>_row = rowsum((W A^T) * B) and
        ||B A||^2_row = rowsum((B (A A^T)) * B)  (what the reference's fused DoRA-norm kernel computes,
        src/axolotl/kernels/dora.py:16-147)."""
        A, B = self.lora_A.detach().float(), self.lora_B.detach().float()
        W = self._dense_weight()
        if W.is_cuda:
            from ..ops import _lib
            from ..ops.gemm import gemm

            WA = gemm(W, self.lora_A16 if self.lora_A16 is not None else A.to(torch.bfloat16),
                      out_dtype=torch.float32)                          # [N, R] skinny tcgen05 GEMM
            A16 = self.lora_A16 if self.lora_A16 is not None else A.to(torch.bfloat16)
            G = gemm(A16, A16, out_dtype=torch.float32, bn=64)          # A A^T [R, R]
            norm = torch.empty(W.shape[0], dtype=torch.float32, device=W.device)
            Bc = B.contiguous()
            _lib.check_rc(_lib.cuda_lib().axb_dora_norm(WA.data_ptr(), Bc.data_ptr(), G.data_ptr(), self.dora_w2.data_ptr(),
                                                        norm.data_ptr(), W.shape[0], Bc.shape[1], float(self.scaling),
                                                        _lib.stream_ptr()), "dora_norm")
            return norm
        WA = W.float() @ A.t()
        cross = (WA * B).sum(1)
        quad = ((B @ (A @ A.t())) * B).sum(1)
        s = self.scaling
        return (self.dora_w2 + 2 * s * cross + s * s * quad).clamp(min=1e-12).sqrt()

    def dora_scale(self):
        """Per-row output scale (1 for rows without an adapter); carries the gradient of ``m``."""
        norm = self.dora_weight_norm()
        sc = self.dora_magnitude.float() / norm
        return torch.where(self.dora_rows, sc, torch.ones_like(sc))

    def refresh_shadows(self):
        """bf16 copies of the fp32 adapter masters for the GEMM kernels (CUDA only)."""
        if self.lora_A is None:
            return
        if self.lora_A.is_cuda:
            if self.lora_A16 is None or self.lora_A16.device != self.lora_A.device:
                self.lora_A16 = self.lora_A.detach().to(torch.bfloat16)
                self.lora_B16 = self.lora_B.detach().to(torch.bfloat16)
            else:
                self.lora_A16.copy_(self.lora_A.detach())
                self.lora_B16.copy_(self.lora_B.detach())
        else:
            self.lora_A16 = self.lora_B16 = None

    def peft_tensors(self):
        """{sub-projection name: (A [r, in], B [out, r])} views in PEFT layout."""
        out = {}
        for (r0, rows, c0, r), n in zip(self.lora_blocks, self.lora_names):
            out[n] = (self.lora_A[c0:c0 + r], self.lora_B[r0:r0 + rows, c0:c0 + r])
        return out

    def load_peft_tensors(self, name, A, B):
        i = self.lora_names.index(name)
        r0, rows, c0, r = self.lora_blocks[i]
        with torch.no_grad():
            self.lora_A[c0:c0 + r].copy_(A)
            self.lora_B[r0:r0 + rows, c0:c0 + r].copy_(B)

    @torch.no_grad()
    def quantize_nf4_(self, double_quant=True, blocksize=64):
        """Replaces the frozen bf16 weight by packed NF4 codes [N, K/2]; every GEMM that reads it
        expands it into a shared bf16 scratch first (QLoRA base weights)."""
        from ..ops.nf4 import quantize_nf4

        if getattr(self.weight, "_axb_quant", None) is not None:
            return
        N, K = self.weight.shape
        q, st = quantize_nf4(self.weight.detach(), blocksize, double_quant)
        w = nn.Parameter(q.view(N, K // 2), requires_grad=False)
        w._axb_quant = st
        self.weight = w

    @torch.no_grad()
    def dequantize_(self, dtype=torch.bfloat16):
        st = getattr(self.weight, "_axb_quant", None)
        if st is not None:
            from ..ops.nf4 import dequantize_nf4

            self.weight = nn.Parameter(dequantize_nf4(self.weight.data, st, dtype=dtype).clone(), requires_grad=False)

    @torch.no_grad()
    def merge_lora_(self):
        """W += s * B A (fp32 math, rounded once). Leaves the adapter zeroed out of the forward."""
        if self.lora_A is None or self.merged:
            return
        self.dequantize_()
        if self.dora_magnitude is not None:
            sc = self.dora_scale().detach()
            merged = (self.weight.float() + self.scaling * (self.lora_B.float() @ self.lora_A.float())) * sc[:, None]
            self.weight.copy_(merged.to(self.weight.dtype))
            self.dora_magnitude = None
            self.merged = True
            return
        delta = self.scaling * (self.lora_B.float() @ self.lora_A.float())
        self.weight.copy_((self.weight.float() + delta).to(self.weight.dtype))
        self.merged = True

    def _apply(self, fn, *a, **kw):
        st = getattr(self.weight, "_axb_quant", None)
        super()._apply(fn, *a, **kw)
        if st is not None:   # nn.Module._apply may rebuild the parameter object: carry the state along
            self.weight._axb_quant = st.to(self.weight.device)
        if self.lora_A is not None:
            self.lora_A16 = None
            self.refresh_shadows()
        return self

    def forward(self, x):
        if self.qat is not None and self.training and self.weight.requires_grad:
            from ..ops.fake_quant import fake_quantize_activation, ste_weight

            x = fake_quantize_activation(x, self.qat.get("activation_dtype"))
            return linear(x, ste_weight(self.weight, self.qat.get("weight_dtype"), self.qat.get("group_size")), self.bias)
        if self.mora_M is not None and _ADAPTERS_ON:
            return linear(x, self.weight, self.bias) + self._mora_update(x)
        if self.lora_A is None or self.merged or not _ADAPTERS_ON:
            return linear(x, self.weight, self.bias)
        if x.is_cuda and self.lora_A16 is None:
            self.refresh_shadows()
        if self.dora_magnitude is not None:
            y = lora_linear(x, self.weight, self.lora_A, self.lora_B, self.lora_A16, self.lora_B16,
                            self.scaling, self.lora_blocks, None, self.lora_dropout, self.training)
            y = y * self.dora_scale().to(y.dtype)
            return y if self.bias is None else y + self.bias.to(y.dtype)
        return lora_linear(x, self.weight, self.lora_A, self.lora_B, self.lora_A16, self.lora_B16,
                           self.scaling, self.lora_blocks, self.bias, self.lora_dropout,
                           self.training)

    def extra_repr(self):
        s = f"in={self.in_features}, out={dict(zip(self.names, self.out_features))}"
        if self.lora_A is not None:
            s += f", lora_r={self.lora_r} on {self.lora_names}, scaling={self.scaling:g}"
        return s
