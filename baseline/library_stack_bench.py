"""Context number, NOT the reference arm: the same Llama-3-8B LoRA step built from stock library parts
that are installed on the box — Hugging Face ``transformers`` Llama (random init, bf16), flash-attn 2
varlen attention on packed rows (position ids restart per sample), cuBLAS GEMMs through
``torch.nn.functional.linear``, a minimal hand-written LoRA wrapper (r=16, alpha=32, all linear layers)
and ``torch.optim.AdamW(fused=True)``. It exists so that the headline tokens/s has one on-box
library-stack figure beside it while the reference itself cannot be installed offline. Its output says
``"impl": "library-stack (context only)"`` and must never be used as a reference ratio.

  python baseline/library_stack_bench.py --steps 5 --warmup 3
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import numpy as np
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
from ref_harness import LLAMA3_8B  # noqa: E402


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, r=16, alpha=32):
        super().__init__()
        self.base = base
        self.base.weight.requires_grad_(False)
        dev, dt = base.weight.device, base.weight.dtype
        self.A = nn.Parameter(torch.empty(r, base.in_features, device=dev, dtype=dt))
        self.B = nn.Parameter(torch.zeros(base.out_features, r, device=dev, dtype=dt))
        nn.init.kaiming_uniform_(self.A, a=math.sqrt(5))
        self.s = alpha / r

    def forward(self, x):
        return self.base(x) + self.s * nn.functional.linear(nn.functional.linear(x, self.A), self.B)


def wrap_lora(model):
    for mod in list(model.modules()):
        for name, child in list(mod.named_children()):
            if isinstance(child, nn.Linear) and name != "lm_head":
                setattr(mod, name, LoRALinear(child))


def packed_rows(n, seq_len, vocab, seed=0):
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(n):
        ids, pos, left = [], [], seq_len
        while left >= 256:
            l = int(min(rng.integers(256, 4097), left))
            ids.append(rng.integers(3, vocab, size=l))
            pos.append(np.arange(l))
            left -= l
        if left:
            ids.append(np.zeros(left, dtype=np.int64))
            pos.append(np.arange(left))
        rows.append((torch.from_numpy(np.concatenate(ids)).long()[None], torch.from_numpy(np.concatenate(pos)).long()[None]))
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None)
    args = ap.parse_args()
    from transformers import LlamaConfig, LlamaForCausalLM

    arch = dict(LLAMA3_8B)
    if args.layers:
        arch["num_hidden_layers"] = args.layers
    arch.pop("architectures"); arch.pop("torch_dtype")
    cfg = LlamaConfig(**arch)
    cfg._attn_implementation = "flash_attention_2"
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    for p in model.parameters():
        p.requires_grad_(False)
    wrap_lora(model)
    model.train()
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=2e-4, fused=True)
    W, K, S = max(args.warmup, 3), args.steps, 8192
    rows = [(a.pin_memory(), b.pin_memory()) for a, b in packed_rows(W + K, S, cfg.vocab_size)]

    def step(i):
        ids, pos = (t.to(dev, non_blocking=True) for t in rows[i])
        out = model(input_ids=ids, position_ids=pos, labels=ids)
        out.loss.backward()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return float(out.loss.item())

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        loss = step(W + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(json.dumps({"impl": "library-stack (context only)", "what": "HF transformers Llama + flash-attn 2 + cuBLAS + "
                      "hand-written LoRA wrapper + torch fused AdamW, packed 8192-token rows, host->device copy and loss "
                      "read every step", "value": S * K / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms / K, "steps": K,
                      "warmup": W, "n_gpus": 1, "last_loss": loss,
                      "peak_mem_gib": torch.cuda.max_memory_allocated() / 1024 ** 3,
                      "model": "llama-3-8b" + (f"[layers={args.layers}]" if args.layers else "")}))


if __name__ == "__main__":
    main()
