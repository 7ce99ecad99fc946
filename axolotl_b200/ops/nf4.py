"""4-bit NormalFloat (NF4) weight storage for QLoRA, in the bitsandbytes layout: 64-element blocks,
two codes per byte (first element in the high nibble), fp32 absmax per block, optionally
"double quantised" (absmax minus its mean stored as 8-bit dynamic-map codes with one fp32 scale per
256 blocks). The reference dequantises this format through bitsandbytes' C entry points
(src/axolotl/kernels/quantize.py:27-106); here a CUDA kernel expands codes into a bf16 scratch
right before the tcgen05 GEMM that consumes them, in the forward and again in the backward pass.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

NF4_VALUES = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
              -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
              0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
              0.7229568362236023, 1.0)
_CODE = torch.tensor(NF4_VALUES, dtype=torch.float32)
_MID = (_CODE[:-1] + _CODE[1:]) / 2


def dynamic_map_8bit(signed=True, max_exponent_bits=7, total_bits=8):
    """The 256-entry non-uniform code used for the second-level (absmax) quantisation."""
    data = []
    non_sign_bits = total_bits - 1
    additional_items = 2 ** (non_sign_bits - max_exponent_bits) - 1
    i = 0
    for i in range(max_exponent_bits):
        n_frac = int(2 ** (i + non_sign_bits - max_exponent_bits) + 1) if signed else \
            int(2 ** (i + non_sign_bits - max_exponent_bits + 1) + 1)
        b = torch.linspace(0.1, 1, n_frac)
        means = (b[:-1] + b[1:]) / 2.0
        data += ((10 ** (-(max_exponent_bits - 1) + i)) * means).tolist()
        if signed:
            data += (-(10 ** (-(max_exponent_bits - 1) + i)) * means).tolist()
    if additional_items > 0:
        b = torch.linspace(0.1, 1, additional_items + 1)
        means = (b[:-1] + b[1:]) / 2.0
        data += ((10 ** (-(max_exponent_bits - 1) + i)) * means).tolist()
        if signed:
            data += (-(10 ** (-(max_exponent_bits - 1) + i)) * means).tolist()
    data += [0.0, 1.0]
    data += [0.0] * (2 ** total_bits - len(data))
    return torch.tensor(sorted(data), dtype=torch.float32)


_DYN = dynamic_map_8bit()


@dataclass
class NF4State:
    """Everything needed to expand ``qdata`` back to ``shape`` (besides the codes themselves)."""
    shape: tuple
    blocksize: int
    absmax: torch.Tensor | None = None        # fp32 per block (plain) ...
    absmax_q: torch.Tensor | None = None      # ... or uint8 codes into the dynamic map (double quant)
    absmax_scale: torch.Tensor | None = None  # fp32 per 256 blocks
    absmax_offset: torch.Tensor | None = None # fp32 scalar (mean of the block absmax values)

    def block_absmax(self):
        if self.absmax is not None:
            return self.absmax
        dyn = _DYN.to(self.absmax_q.device)
        v = dyn[self.absmax_q.long()].view(-1)
        n = v.numel()
        scale = self.absmax_scale.repeat_interleave(256)[:n]
        return v * scale + self.absmax_offset

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)
        return NF4State(self.shape, self.blocksize, mv(self.absmax), mv(self.absmax_q), mv(self.absmax_scale),
                        mv(self.absmax_offset))

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.absmax, self.absmax_q, self.absmax_scale) if t is not None)


def _nearest_code(x, code):
    mid = ((code[:-1] + code[1:]) / 2).to(x.device)
    return torch.bucketize(x, mid)


def quantize_nf4(w: torch.Tensor, blocksize=64, double_quant=True):
    """w [..]: returns (qdata uint8 [numel / 2], NF4State). numel must be a multiple of blocksize."""
    flat = w.detach().float().reshape(-1)
    if flat.numel() % blocksize:
        raise ValueError(f"NF4 needs numel divisible by the block size {blocksize}")
    blocks = flat.view(-1, blocksize)
    absmax = blocks.abs().amax(1)
    scaled = blocks / absmax.clamp(min=1e-30)[:, None]
    codes = _nearest_code(scaled, _CODE).to(torch.uint8).view(-1)
    qdata = (codes[0::2] << 4) | codes[1::2]
    st = NF4State(tuple(w.shape), blocksize)
    if double_quant:
        offset = absmax.mean()
        rem = absmax - offset
        pad = (-rem.numel()) % 256
        remp = torch.cat([rem, rem.new_zeros(pad)]).view(-1, 256)
        scale2 = remp.abs().amax(1).clamp(min=1e-30)
        q2 = _nearest_code(remp / scale2[:, None], _DYN).to(torch.uint8).view(-1)[: rem.numel()]
        st.absmax_q, st.absmax_scale, st.absmax_offset = q2.contiguous(), scale2.contiguous(), offset.reshape(())
    else:
        st.absmax = absmax.contiguous()
    return qdata.contiguous(), st


def dequantize_nf4(qdata: torch.Tensor, st: NF4State, out: torch.Tensor | None = None, dtype=torch.bfloat16):
    """Expands to ``st.shape``; on CUDA in bf16 this is one kernel launch into ``out``."""
    absmax = st.block_absmax().float().contiguous()
    n = qdata.numel() * 2
    if qdata.is_cuda and dtype == torch.bfloat16:
        if out is None:
            out = torch.empty(st.shape, dtype=torch.bfloat16, device=qdata.device)
        _lib.check_rc(_lib.cuda_lib().axb_nf4_dequant(qdata.data_ptr(), absmax.data_ptr(), out.data_ptr(), n,
                                                      st.blocksize, _lib.stream_ptr()), "nf4_dequant")
        return out.view(st.shape)
    code = _CODE.to(qdata.device)
    hi, lo = code[(qdata >> 4).long()], code[(qdata & 0xF).long()]
    vals = torch.stack([hi, lo], -1).reshape(-1, st.blocksize) * absmax[:, None]
    res = vals.reshape(st.shape).to(dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


_SCRATCH: dict = {}


def scratch_weight(shape, device):
    """One bf16 scratch per (device, numel): dequantised weights are consumed by the very next
    GEMM on the same stream, so all layers of equal size can share it."""
    n = 1
    for s in shape:
        n *= s
    key = (str(device), n)
    buf = _SCRATCH.get(key)
    if buf is None:
        buf = _SCRATCH[key] = torch.empty(n, dtype=torch.bfloat16, device=device)
    return buf.view(shape)


def dequantize_fp8_block(w_fp8: torch.Tensor, scale_inv: torch.Tensor, block=128, dtype=torch.bfloat16):
    """Blockwise-FP8 checkpoints (E4M3 weights, fp32 ``weight_scale_inv`` per 128x128 block) -> bf16
    (reference: src/axolotl/kernels/quantize.py:109-135)."""
    rows, cols = w_fp8.shape
    if w_fp8.is_cuda and dtype == torch.bfloat16 and cols % 8 == 0:
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=w_fp8.device)
        _lib.check_rc(_lib.cuda_lib().axb_fp8_block_dequant(
            w_fp8.contiguous().data_ptr(), scale_inv.float().contiguous().data_ptr(), out.data_ptr(), rows, cols,
            block, _lib.stream_ptr()), "fp8_block_dequant")
        return out
    s = scale_inv.float().repeat_interleave(block, 0)[:rows].repeat_interleave(block, 1)[:, :cols]
    return (w_fp8.float() * s).to(dtype)
