"""LoRA merge tools.

``merge_lora_sharded`` streams the base checkpoint shard by shard, adds ``scale * B @ A`` to every
targeted weight in fp32, rounds once to the base dtype and rewrites the shard plus a fresh
``model.safetensors.index.json`` -- peak memory is one shard, never the whole model (the
memory-efficient path of the reference, src/axolotl/cli/utils/lora_merge.py:1863-2278).
Handles: alpha/r and alpha/sqrt(r) (rsLoRA) scaling, rank/alpha patterns, per-expert adapters in
the PEFT ``target_parameters`` layout against fused (``experts.gate_up_proj``) or per-expert
checkpoints, NVFP4 expert weights (dequantise -> merge -> requantise with a fresh scale), and
copies every non-weight file. ``merge_sharded_fsdp_weights`` turns per-rank shard files into one
HF checkpoint.
"""
from __future__ import annotations

import json
import math
import os
import re
import shutil

import torch

from ..utils.logging import get_logger
from . import safetensors_io as st

LOG = get_logger(__name__)


def _adapter_scale(cfg: dict, module_path: str) -> float:
    r, alpha = _adapter_rank(cfg, module_path), cfg.get("lora_alpha", cfg.get("r", 8))
    for pat, av in (cfg.get("alpha_pattern") or {}).items():
        if _pattern_hits(pat, module_path):
            alpha = av
    return alpha / math.sqrt(r) if cfg.get("use_rslora") else alpha / r


def _pattern_hits(pat: str, module_path: str) -> bool:
    """PEFT's rule for ``rank_pattern`` / ``alpha_pattern`` keys: the key (a regular expression) has to
    match the module path as a whole or as a suffix that starts at a module boundary."""
    return re.match(rf"(.*\.)?({pat})$", module_path) is not None


def _adapter_rank(cfg, module_path: str) -> int:
    r = cfg.get("r", 8)
    for pat, rv in (cfg.get("rank_pattern") or {}).items():
        if _pattern_hits(pat, module_path):
            r = rv
    return r


def load_adapter_tensors(adapter_dir: str):
    with open(os.path.join(adapter_dir, "adapter_config.json")) as fh:
        cfg = json.load(fh)
    sd = st.load_file(os.path.join(adapter_dir, "adapter_model.safetensors"))
    pairs = {}
    for k, v in sd.items():
        m = re.match(r"base_model\.model\.(.+)\.lora_(A|B)(?:\.default)?\.weight$", k)
        if not m:
            mm = re.match(r"base_model\.model\.(.+)\.lora_magnitude_vector(?:\.default)?(?:\.weight)?$", k)
            if mm:   # DoRA magnitude
                pairs.setdefault(mm.group(1), {})["M"] = v.float().reshape(-1)
            continue
        pairs.setdefault(m.group(1), {})[m.group(2)] = v.float()
    return cfg, pairs


def _delta(pair, scale):
    return scale * (pair["B"] @ pair["A"])


def _expert_delta(pair, scale, e, num_experts):
    A, B = pair["A"], pair["B"]
    r = A.shape[0] // num_experts
    Ae = A[e * r:(e + 1) * r]
    Be = B.reshape(B.shape[0], r, num_experts)[:, :, e]
    return scale * (Be @ Ae)


def merge_tensor(name: str, w: torch.Tensor, cfg: dict, pairs: dict, shard: dict | None = None) -> torch.Tensor | None:
    """Merged replacement for checkpoint tensor ``name`` or None when no adapter targets it."""
    if name.endswith(".weight"):
        mod = name[: -len(".weight")]
        if mod not in pairs and mod.startswith("backbone."):      # Nemotron-H checkpoints of either prefix generation
            mod = "model." + mod[len("backbone."):]
        if mod in pairs and "A" in pairs[mod] and "B" in pairs[mod]:
            if cfg.get("fan_in_fan_out"):
                return (w.float() + _delta(pairs[mod], _adapter_scale(cfg, mod)).t()).to(w.dtype)
            merged = w.float() + _delta(pairs[mod], _adapter_scale(cfg, mod))
            if "M" in pairs[mod]:   # DoRA: rescale every output row to its learned magnitude
                merged = merged * (pairs[mod]["M"].to(merged.device) / merged.norm(dim=1).clamp(min=1e-12))[:, None]
            return merged.to(w.dtype)
        m = re.match(r"(.+\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)$", mod)
        if m:  # per-expert checkpoint, fused expert adapter
            base, e, sub = m.group(1), int(m.group(2)), m.group(3)
            key = f"{base}.{'down_proj' if sub == 'down_proj' else 'gate_up_proj'}"
            if key in pairs:
                E = pairs[key]["A"].shape[0] // _adapter_rank(cfg, key)
                d = _expert_delta(pairs[key], _adapter_scale(cfg, key), e, E)
                if sub != "down_proj":
                    half = d.shape[0] // 2
                    d = d[:half] if sub == "gate_proj" else d[half:]
                return (w.float() + d).to(w.dtype)
    m = re.match(r"(.+\.experts\.(?:gate_up_proj|down_proj))$", name)
    if m and name in pairs and w.dim() == 3:  # fused [E, out, in] expert tensor
        E = w.shape[0]
        out = w.float().clone()
        for e in range(E):
            out[e] += _expert_delta(pairs[name], _adapter_scale(cfg, name), e, E)
        return out.to(w.dtype)
    return None


def _merge_nvfp4_group(names, tensors, cfg, pairs):
    """names: {packed, scale, global} keys of one NVFP4 weight; returns replacement tensors."""
    from ..ops.nvfp4 import dequantize_nvfp4, quantize_nvfp4

    base = names["prefix"]
    if base not in pairs:
        return {}
    q, s = tensors[names["packed"]], tensors[names["scale"]]
    g = tensors[names["global"]].float()
    pts = g if names["global"].endswith("weight_scale_2") else 1.0 / g
    w = dequantize_nvfp4(q, s.to(torch.float8_e4m3fn) if s.dtype != torch.float8_e4m3fn else s, pts, dtype=torch.float32)
    if w.dim() == 3:
        for e in range(w.shape[0]):
            w[e] += _expert_delta(pairs[base], _adapter_scale(cfg, base), e, w.shape[0])
    else:
        w += _delta(pairs[base], _adapter_scale(cfg, base))
    q2, s2, p2 = quantize_nvfp4(w)  # fresh scales: the merged weight has a new dynamic range
    g2 = p2 if names["global"].endswith("weight_scale_2") else 1.0 / p2
    return {names["packed"]: q2, names["scale"]: s2, names["global"]: g2.reshape(tensors[names["global"]].shape)}


def _merge_quantised(k, w, tensors, cfg, pairs, device, nvfp4_scale_mode):
    """A weight stored as ``k`` + ``k_scale*`` companions (block-fp8 / MXFP8 / MXFP4 / NVFP4): expand, add the adapter
    delta, write back in the same format. Returns replacement tensors or {}."""
    from . import quant_formats as qf

    fmt, scales = qf.detect_format(k, w, tensors)
    if fmt is None:
        return {}
    full = qf.dequantize(fmt, w, scales, device)
    rep = merge_tensor(k, full, cfg, pairs)
    if rep is None:
        return {}
    q = qf.requantize(fmt, rep.float(), scales, device, nvfp4_scale_mode=nvfp4_scale_mode)
    return {k + suffix: t for suffix, t in q.items()}


def merge_lora_sharded(base_dir: str, adapter_dir: str, out_dir: str, device: str = "cpu", nvfp4_scale_mode: str = "reuse",
                       nf4_roundtrip: bool | None = None) -> dict:
    """Streams the base checkpoint shard by shard and writes the merged one. Quantised base weights keep their
    storage format (``nvfp4_scale_mode``: ``reuse`` the base block scales, or ``fresh`` ones from the merged weight).
    ``nf4_roundtrip``: merge into the NF4 quantise -> dequantise image of the base weights, i.e. what a QLoRA adapter
    trained against (default: when the adapter's config records ``load_in_4bit`` / a QLoRA run)."""
    cfg, pairs = load_adapter_tensors(adapter_dir)
    if nf4_roundtrip is None:
        nf4_roundtrip = bool(cfg.get("axolotl_load_in_4bit") or cfg.get("load_in_4bit") or cfg.get("qlora"))
    os.makedirs(out_dir, exist_ok=True)
    files = st.checkpoint_files(base_dir)
    if not files:
        raise FileNotFoundError(f"no safetensors checkpoint in {base_dir}")
    merged, wmap, total = set(), {}, 0
    for f in files:
        with st.SafeFile(f) as sf:
            tensors = {k: sf.get_tensor(k) for k in sf.keys()}
            meta = sf.metadata
        out = {}
        nv = {}
        for k in tensors:
            m = re.match(r"(.+)\.(weight_packed|weight_global_scale|weight_scale_2|weight_scale)$", k)
            if m and (tensors.get(m.group(1) + ".weight_packed") is not None or
                      (tensors.get(m.group(1) + ".weight") is not None and tensors[m.group(1) + ".weight"].dtype == torch.uint8)):
                d = nv.setdefault(m.group(1), {"prefix": m.group(1)})
                kind = m.group(2)
                d["packed" if kind == "weight_packed" else "scale" if kind == "weight_scale" else "global"] = k
        for pre, d in nv.items():
            if "packed" not in d and pre + ".weight" in tensors:
                d["packed"] = pre + ".weight"
            if {"packed", "scale", "global"} <= set(d):
                rep = _merge_nvfp4_group(d, tensors, cfg, pairs)
                if rep:
                    out.update(rep)
                    merged.add(pre)
        dev_pairs = {p: {a: t.to(device) for a, t in ab.items()} for p, ab in pairs.items()} if device != "cpu" else pairs
        for k, w in tensors.items():
            if k in out:
                continue
            if w.dtype in (torch.uint8, torch.float8_e4m3fn):
                rep = _merge_quantised(k, w, tensors, cfg, dev_pairs, device, nvfp4_scale_mode)
                if rep:
                    out.update(rep)
                    merged.add(k[: -len(".weight")] if k.endswith(".weight") else k)
                else:
                    out[k] = w
                continue
            base_w = w.to(device)
            if nf4_roundtrip and w.dim() == 2 and k.endswith(".weight") and k[: -len(".weight")] in pairs:
                from .quant_formats import simulate_nf4_roundtrip

                base_w = simulate_nf4_roundtrip(base_w)
            rep = merge_tensor(k, base_w, cfg, dev_pairs)
            if rep is not None:
                out[k] = rep.cpu()
                mm = re.match(r"(.+\.experts)\.\d+\.(gate_proj|up_proj|down_proj)\.weight$", k)
                merged.add(f"{mm.group(1)}.{'down_proj' if mm.group(2) == 'down_proj' else 'gate_up_proj'}" if mm and
                           k[: -len('.weight')] not in pairs else (k[: -len(".weight")] if k.endswith(".weight") else k))
            else:
                out[k] = w
        fn = os.path.basename(f)
        st.save_file(out, os.path.join(out_dir, fn), meta or {"format": "pt"})
        for k, t in out.items():
            wmap[k] = fn
            total += t.numel() * t.element_size()
    if len(files) > 1:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": {"total_size": total}, "weight_map": wmap}, fh, indent=2)
    for fn in os.listdir(base_dir):
        src = os.path.join(base_dir, fn)
        if os.path.isfile(src) and not fn.endswith(".safetensors") and fn != "model.safetensors.index.json":
            shutil.copy2(src, os.path.join(out_dir, fn))
    missing = set(pairs) - merged
    if missing:
        LOG.warning("%d adapter modules had no matching base tensor: %s", len(missing), sorted(missing)[:4])
    return {"merged": len(merged), "unmatched": sorted(missing), "files": len(files)}


def merge_sharded_fsdp_weights(shard_dir: str, out_dir: str, dtype=torch.bfloat16) -> list[str]:
    """Row-sharded per-rank files ``shard_rank{r}.safetensors`` (+ ``shard_index.json`` listing
    which tensors are split on dim 0) -> one HF checkpoint cast to ``dtype``."""
    with open(os.path.join(shard_dir, "shard_index.json")) as fh:
        index = json.load(fh)
    world = index["world_size"]
    parts = [st.load_file(os.path.join(shard_dir, f"shard_rank{r}.safetensors")) for r in range(world)]
    full = {}
    for k in parts[0]:
        if k in index["sharded"]:
            full[k] = torch.cat([p[k] for p in parts], 0)
        else:
            full[k] = parts[0][k]
        if full[k].is_floating_point() and full[k].dtype != torch.float8_e4m3fn:
            full[k] = full[k].to(dtype)
    os.makedirs(out_dir, exist_ok=True)
    for fn in ("config.json",):
        if os.path.exists(os.path.join(shard_dir, fn)):
            shutil.copy2(os.path.join(shard_dir, fn), os.path.join(out_dir, fn))
    return st.save_sharded(full, out_dir)
