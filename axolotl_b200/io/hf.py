"""Hugging Face checkpoint interchange for the model families in ``models.config``.

Our modules keep fused weights (qkv_proj, gate_up_proj, fused experts); checkpoints on disk use
the HF per-projection names, so loading concatenates and saving splits. NVFP4 expert checkpoints
(modelopt ``weight`` / ``weight_scale`` / ``weight_scale_2`` or compressed-tensors
``weight_packed`` / ``weight_scale`` / ``weight_global_scale``) are detected by "uint8 weight +
group scale" exactly like the reference loader
(src/axolotl/integrations/kernels/libs/scattermoe_lora/nvfp4_moe_loading.py:95-155, 189-243).
"""
from __future__ import annotations

import os
import re

import torch

from ..models.config import ModelConfig
from ..models.layers import FusedLinear
from ..models.moe import Experts
from ..models.transformer import CausalLM
from . import safetensors_io as st


def _split_name(hf_name: str):
    """'model.layers.3.self_attn.q_proj.weight' -> ('layers.3.self_attn', 'q_proj', 'weight')."""
    m = re.match(r"model\.(.*)\.(q_proj|k_proj|v_proj|qkv_proj|o_proj|gate_proj|up_proj|gate_up_proj|down_proj|"
                 r"q_a_proj|q_b_proj|kv_a_proj_with_mqa|kv_b_proj)\.(weight|bias)$", hf_name)
    return m.groups() if m else None


_FUSED_OF = {"q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj", "o_proj": "o_proj",
             "gate_proj": "gate_up_proj", "up_proj": "gate_up_proj", "down_proj": "down_proj",
             "qkv_proj": "qkv_proj", "gate_up_proj": "gate_up_proj",   # Phi-3 checkpoints are already fused
             "q_a_proj": "q_a_proj", "q_b_proj": "q_b_proj", "kv_a_proj_with_mqa": "kv_a_proj_with_mqa",
             "kv_b_proj": "kv_b_proj"}                                  # DeepSeek latent attention


@torch.no_grad()
def load_state_into(model: CausalLM, named_tensors, strict: bool = True):
    """Streams (hf_name, tensor) pairs into the model. Returns the set of missing parameter slots."""
    mods = dict(model.named_modules())
    filled = set()
    expert_parts = {}
    mxfp4_parts = {}
    llama4 = getattr(model.config, "model_type", "") == "llama4_text"
    bamba = getattr(model.config, "model_type", "") in ("bamba", "falcon_h1")       # the same names outside the mixers
    mamba_attr = ".mamba" if getattr(model.config, "model_type", "") == "falcon_h1" else ".self_attn"
    qwen3_next = getattr(model.config, "model_type", "") in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text")
    if getattr(model.config, "model_type", "") == "nemotron_h":
        return _nemotron_h_load(model, named_tensors, strict)
    glm = model.config.rope_pairs_interleaved() if hasattr(model.config, "rope_pairs_interleaved") else False
    hunyuan = getattr(model.config, "model_type", "") in ("hunyuan_v1_dense", "hunyuan_v1_moe")
    apertus = getattr(model.config, "model_type", "") == "apertus"
    lfm2 = getattr(model.config, "model_type", "") in ("lfm2", "lfm2_moe")
    afmoe = getattr(model.config, "model_type", "") == "afmoe"
    starcoder2 = getattr(model.config, "model_type", "") == "starcoder2"
    phi = getattr(model.config, "model_type", "") == "phi"
    falcon = getattr(model.config, "model_type", "") == "falcon"
    vision_params = None
    for name, t in named_tensors:
        if falcon:
            name = _falcon_in(name)
            if (m := re.match(r"model\.(layers\.\d+\.self_attn)\.query_key_value\.(weight|bias)$", name)):
                t = t.index_select(0, model.config.falcon_qkv_rows().to(t.device))     # rows into q | k | v order
                getattr(mods[m.group(1)].qkv_proj, m.group(2)).copy_(t)
                filled.add(name)
                continue
            elif (m := re.match(r"model\.(layers\.\d+)\.ln_mlp\.(weight|bias)$", name)):
                getattr(mods[m.group(1)].ln_mlp, m.group(2)).copy_(t)
                filled.add(name)
                continue
        if hunyuan:
            name = name.replace(".query_layernorm.", ".q_norm.").replace(".key_layernorm.", ".k_norm.") \
                .replace(".mlp.gate.wg.", ".mlp.gate.").replace(".mlp.shared_mlp.", ".mlp.shared_experts.")
        if afmoe:
            name = name.replace(".pre_mlp_layernorm.", ".pre_feedforward_layernorm.").replace(".post_mlp_layernorm.", ".post_feedforward_layernorm.") \
                .replace(".mlp.router.gate.", ".mlp.gate.").replace(".mlp.expert_bias", ".mlp.gate.e_score_correction_bias")
            if (m := re.match(r"model\.(layers\.\d+\.self_attn)\.gate_proj\.weight$", name)):
                mods[m.group(1)].out_gate.weight.copy_(t)
                filled.add(name)
                continue
        if lfm2:
            if (m := re.match(r"model\.(layers\.\d+)\.conv\.(.+)$", name)):
                mx, leaf = mods[m.group(1) + ".self_attn"], m.group(2)
                if leaf == "conv.weight":
                    mx.conv_weight.copy_(t.reshape(t.shape[0], t.shape[-1]))
                elif leaf == "conv.bias":
                    mx.conv_bias.copy_(t)
                else:
                    getattr(getattr(mx, leaf.split(".")[0]), leaf.split(".")[1]).copy_(t)
                filled.add(name)
                continue
            for theirs, ours in _LFM2_NAMES:
                if theirs in name:
                    name = name.replace(theirs, ours)
                    break
        if apertus:
            name = name.replace(".attention_layernorm.", ".input_layernorm.").replace(".feedforward_layernorm.", ".post_attention_layernorm.")
            if (m := re.match(r"model\.(layers\.\d+\.mlp)\.act_fn\.(alpha_p|alpha_n)$", name)):
                getattr(mods[m.group(1)], m.group(2)).copy_(t.reshape(-1))
                filled.add(name)
                continue
            if ".act_fn." in name:
                continue
        name = name.replace(".gate.moe_statics.e_score_correction_bias", ".gate.e_score_correction_bias")
        if starcoder2:
            name = name.replace(".mlp.c_fc.", ".mlp.up_proj.").replace(".mlp.c_proj.", ".mlp.down_proj.")
        if phi:
            name = name.replace(".mlp.fc1.", ".mlp.up_proj.").replace(".mlp.fc2.", ".mlp.down_proj.") \
                .replace(".self_attn.dense.", ".self_attn.o_proj.").replace("model.final_layernorm.", "model.norm.")
            if name == "lm_head.bias":
                model.lm_head_bias.copy_(t)
                filled.add(name)
                continue
        if glm:
            name, t = _glm_in(model, name, t)
        if llama4:
            name, t = _llama4_in(model, name, t)
        if qwen3_next:
            if (m := re.match(r"model\.(layers\.\d+)\.linear_attn\.(.+)$", name)):
                mx, leaf = mods[m.group(1) + ".self_attn"], m.group(2)
                if leaf == "conv1d.weight":
                    mx.conv_weight.copy_(t.reshape(t.shape[0], t.shape[-1]))
                elif leaf == "norm.weight":
                    mx.norm_weight.copy_(t)
                elif leaf in ("dt_bias", "A_log"):
                    getattr(mx, leaf).copy_(t)
                elif getattr(mx, "flat", False) and leaf.startswith("in_proj_"):
                    r0, r1 = mx.in_proj.row_range(leaf.split(".")[0])
                    mx.in_proj.weight[r0:r1].copy_(t)
                else:
                    getattr(getattr(mx, leaf.split(".")[0]), leaf.split(".")[1]).copy_(t)
                filled.add(name)
                continue
            if (m := re.match(r"model\.(layers\.\d+\.self_attn)\.q_proj\.(weight|bias)$", name)):
                at = mods[m.group(1)]           # rows per head: [query (D) | gate (D)]
                u = t.reshape(at.Hq, 2, at.D, *t.shape[1:])
                r0, r1 = at.qkv_proj.row_range("q_proj")
                (at.qkv_proj.weight if m.group(2) == "weight" else at.qkv_proj.bias)[r0:r1].copy_(u[:, 0].reshape(at.Hq * at.D, *t.shape[1:]))
                (at.out_gate.weight if m.group(2) == "weight" else at.out_gate.bias).copy_(u[:, 1].reshape(at.Hq * at.D, *t.shape[1:]))
                filled.add(name)
                continue
            if name.startswith("mtp."):
                continue                         # multi-token-prediction head: not part of the training graph
        if bamba:
            name = (name.replace(".pre_ff_layernorm.", ".post_attention_layernorm.").replace(".feed_forward.", ".mlp.")
                    .replace("model.final_layernorm.", "model.norm."))
        # multimodal wrappers (Gemma 3): the language model's tensors carry a prefix, the vision parts are not ours
        if name.startswith("language_model."):
            name = name[len("language_model."):]
        elif name.startswith("model.language_model."):
            name = "model." + name[len("model.language_model."):]
        if getattr(model, "vision", None) is not None and name.startswith(
                ("vision_tower.", "multi_modal_projector.", "model.vision_tower.", "model.multi_modal_projector.")):
            leaf = name[len("model."):] if name.startswith("model.") else name       # LLaVA: CLIP tower and projector
            if vision_params is None:
                vision_params = dict(model.vision.named_parameters())
            if leaf in vision_params:
                vision_params[leaf].copy_(t)
                filled.add(name)
            elif strict and not leaf.endswith("position_ids"):
                raise KeyError(f"unexpected checkpoint tensor '{name}'")
            continue
        if name.startswith(("vision_tower.", "multi_modal_projector.", "model.vision_tower.", "model.multi_modal_projector.",
                            "model.audio_tower.", "model.embed_vision.", "model.embed_audio.")):
            continue
        if name == "model.embed_tokens.weight":
            model.embed_tokens.copy_(t)
            filled.add("embed_tokens")
        elif name == "lm_head.weight":
            if model.lm_head is not None:
                model.lm_head.copy_(t)
            filled.add("lm_head")
        elif name == "model.norm.weight":
            model.norm.weight.copy_(t)
            filled.add("norm")
        elif (sp := _split_name(name)) is not None and ".experts." not in name:
            parent, sub, kind = sp
            fused = _FUSED_OF[sub]
            if fused == "qkv_proj" and f"{parent}.qkv_proj" not in mods:      # latent attention: a lone q_proj
                fused = sub
            if fused == "gate_up_proj" and f"{parent}.gate_up_proj" not in mods:   # ungated MLP: a lone up_proj
                fused = sub
            fl: FusedLinear = mods[f"{parent}.{fused}"]
            r0, r1 = fl.row_range(sub)
            (fl.weight if kind == "weight" else fl.bias)[r0:r1].copy_(t)
            filled.add(f"{parent}.{sub}.{kind}")
        elif (m := re.match(r"model\.(layers\.\d+)\.(input_layernorm|post_attention_layernorm|pre_feedforward_layernorm|post_feedforward_layernorm)\.(weight|bias)$", name)):
            getattr(mods[f"{m.group(1)}.{m.group(2)}"], m.group(3)).copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+)\.layer_scalar$", name)):
            mods[m.group(1)].layer_scalar.copy_(t.reshape(-1))
            filled.add(name)
        elif name in ("model.embed_tokens_per_layer.weight", "model.per_layer_model_projection.weight", "model.per_layer_projection_norm.weight"):
            leaf = name.split(".")[1]           # Gemma 4 per-layer input embeddings
            (model.embed_tokens_per_layer if leaf == "embed_tokens_per_layer" else getattr(model, leaf).weight).copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+)\.(per_layer_input_gate|per_layer_projection|post_per_layer_input_norm|"
                            r"post_feedforward_layernorm_1|post_feedforward_layernorm_2|pre_feedforward_layernorm_2)\.weight$", name)):
            getattr(mods[m.group(1)], m.group(2)).weight.copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+)\.router\.(proj\.weight|scale|per_expert_scale)$", name)):
            moe = mods[m.group(1)].g4_moe        # Gemma 4 expert block beside the dense MLP
            {"proj.weight": moe.gate, "scale": moe.router_scale, "per_expert_scale": moe.per_expert_scale}[m.group(2)].copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+)\.experts\.(gate_up_proj|down_proj)$", name)):
            getattr(mods[m.group(1)].g4_moe.experts, m.group(2)).copy_(t)
            filled.add(name)
        elif name == "model.norm.bias":
            model.norm.bias.copy_(t)
            filled.add("norm.bias")
        elif (m := re.match(r"model\.(layers\.\d+)\.mamba\.(.+)$", name)):
            # Granite 4.0-H state-space mixer (kept under `self_attn` in our layer)
            mx, leaf = mods[m.group(1) + mamba_attr], m.group(2)
            if leaf in ("in_proj.weight", "out_proj.weight", "in_proj.bias", "out_proj.bias"):
                getattr(getattr(mx, leaf.split(".")[0]), leaf.split(".")[1]).copy_(t)
            elif leaf == "conv1d.weight":
                mx.conv_weight.copy_(t.reshape(t.shape[0], t.shape[-1]))
            elif leaf == "conv1d.bias":
                mx.conv_bias.copy_(t)
            elif leaf == "norm.weight":
                mx.norm_weight.copy_(t)
            elif leaf in ("dt_bias", "A_log", "D"):
                getattr(mx, leaf).copy_(t)
            elif strict:
                raise KeyError(f"unexpected checkpoint tensor '{name}'")
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+)\.shared_mlp\.(input_linear|output_linear)\.weight$", name)):
            mlp = mods[m.group(1) + ".mlp"]
            mlp = mlp.shared_experts if getattr(mlp, "shared_experts", None) is not None else mlp
            (mlp.gate_up_proj if m.group(2) == "input_linear" else mlp.down_proj).weight.copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+)\.block_sparse_moe\.(input_linear|output_linear|router\.layer)\.weight$", name)):
            moe = mods[m.group(1) + ".mlp"]
            if m.group(2) == "router.layer":
                moe.gate.copy_(t)
            else:
                (moe.experts.gate_up_proj if m.group(2) == "input_linear" else moe.experts.down_proj).copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.self_attn)\.sinks$", name)):
            mods[m.group(1)].sinks.copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.mlp)\.router\.(weight|bias)$", name)):
            (mods[m.group(1)].gate if m.group(2) == "weight" else mods[m.group(1)].router_bias).copy_(t)
            filled.add(name)
        elif getattr(model.config, "model_type", "") == "gpt_oss" and (
                m := re.match(r"model\.(layers\.\d+\.mlp)\.experts\.(gate_up_proj|down_proj)_(blocks|scales)$", name)):
            # the released MXFP4 checkpoints: packed E2M1 blocks [E, out, in / 32, 16] + e8m0 scales [E, out, in / 32];
            # expanded to bf16 when both halves of a weight have arrived
            slot = mxfp4_parts.setdefault((m.group(1), m.group(2)), {})
            slot[m.group(3)] = t
            if len(slot) == 2:
                from .quant_formats import dequantize

                blocks = slot["blocks"]
                E, rows = blocks.shape[:2]
                w = dequantize("mxfp4", blocks.reshape(E, rows, -1), {"_scale": slot["scales"].reshape(E, rows, -1)})
                ex = mods[m.group(1)].experts
                if m.group(2) == "gate_up_proj":
                    ex.gate_up_proj.copy_(torch.cat([w[:, 0::2], w[:, 1::2]], 1))
                else:
                    ex.down_proj.copy_(w)
                del mxfp4_parts[(m.group(1), m.group(2))]
            filled.add(name)
        elif getattr(model.config, "model_type", "") == "gpt_oss" and (
                m := re.match(r"model\.(layers\.\d+\.mlp)\.experts\.(gate_up_proj|down_proj)(_bias)?$", name)):
            # gpt-oss stores [E, in, out] with gate / up interleaved along the output axis
            ex = mods[m.group(1)].experts
            if m.group(2) == "gate_up_proj":
                u = t if m.group(3) else t.transpose(1, 2)                  # [E, 2I(, H)] interleaved rows
                u = torch.cat([u[:, 0::2], u[:, 1::2]], 1)
                (ex.gate_up_bias if m.group(3) else ex.gate_up_proj).copy_(u)
            else:
                (ex.down_bias if m.group(3) else ex.down_proj).copy_(t if m.group(3) else t.transpose(1, 2))
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.self_attn\.indexer)\.(wq_b|wk|weights_proj)\.weight$", name)):
            getattr(mods[m.group(1)], m.group(2)).weight.copy_(t)        # sparse-attention indexer (GLM-5)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.self_attn\.indexer)\.k_norm\.(weight|bias)$", name)):
            getattr(mods[m.group(1)], "k_norm_" + m.group(2)).copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.mlp)\.(?:gate\.)?e_score_correction_bias$", name)):
            mods[m.group(1)].e_score_correction_bias.copy_(t.reshape(-1))
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.self_attn)\.(q_norm|k_norm|q_a_layernorm|kv_a_layernorm)\.weight$", name)):
            mods[f"{m.group(1)}.{m.group(2)}"].weight.copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.mlp)\.gate\.weight$", name)):
            mods[m.group(1)].gate.copy_(t)
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.mlp)\.shared_expert_gate\.weight$", name)):
            mods[m.group(1)].shared_expert_gate.copy_(t)      # Qwen2-MoE: sigmoid gate of the shared expert
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.mlp)\.experts\.(gate_up_proj|down_proj)$", name)):
            getattr(mods[m.group(1)].experts, m.group(2)).copy_(t)     # HF v5 fused expert tensors
            filled.add(name)
        elif (m := re.match(r"model\.(layers\.\d+\.mlp)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(\w+)$", name)):
            expert_parts.setdefault(m.group(1), {})[(int(m.group(2)), m.group(3), m.group(4))] = t
        elif name.endswith("rotary_emb.inv_freq"):
            continue
        elif strict:
            raise KeyError(f"unexpected checkpoint tensor '{name}'")
    for parent, parts in expert_parts.items():
        _fill_experts(mods[parent].experts, parts)
        filled.add(parent + ".experts")
    return filled


def _fill_experts(ex: Experts, parts: dict):
    from .nvfp4_loading import is_nvfp4_parts, fuse_nvfp4_experts

    if is_nvfp4_parts(parts):
        ex.nvfp4 = fuse_nvfp4_experts(parts, ex.E, device=ex.gate_up_proj.device)
        ex.gate_up_proj = None
        ex.down_proj = None
        return
    I = ex.I
    for (e, sub, kind), t in parts.items():
        if kind != "weight":
            continue
        if sub == "gate_proj":
            ex.gate_up_proj[e, :I].copy_(t)
        elif sub == "up_proj":
            ex.gate_up_proj[e, I:].copy_(t)
        else:
            ex.down_proj[e].copy_(t)


def load_pretrained(path: str, dtype=torch.bfloat16, device="cpu", config: ModelConfig | None = None,
                    strict: bool = True) -> CausalLM:
    cfg = config or ModelConfig.from_pretrained(path)
    model = CausalLM(cfg, dtype=dtype, device=device)
    load_state_into(model, st.iter_checkpoint(path), strict=strict)
    return model


def sharded_state_dict(model: CausalLM, rank: int) -> tuple[dict, list[str]]:
    """This rank's part of a SHARDED state dict under HF names, and the list of tensors that are split on
    dim 0. A row-sharded fused weight (q|k|v, gate|up) holds rows [rank * n, (rank + 1) * n) of the fused
    matrix; every sub-projection gets the overlap of that range with its own rows (possibly none: an empty
    [0, K] tensor keeps the per-rank files uniform). Tensors that are not sharded go into rank 0's file only.
    (The reference writes torch-DCP shards for ``fsdp_config.state_dict_type: SHARDED_STATE_DICT``,
    src/axolotl/monkeypatch/accelerate/fsdp2.py:348-433; this layout is what ``merge-sharded-fsdp-weights``
    reads back.)"""
    full = hf_state_dict(model) if rank == 0 else {}
    out, sharded = {}, []
    skip = set()
    for name, m in model.named_modules():
        if not isinstance(m, FusedLinear):
            continue
        info = getattr(m.weight, "_axb_shard", None)
        if info is None:
            continue
        parent = name.rsplit(".", 1)[0]
        rows = info.rows // info.world
        lo, hi = info.rank * rows, (info.rank + 1) * rows
        w = m.weight.detach()
        r0 = 0
        for sub, n in zip(m.names, m.out_features):
            r1 = r0 + n
            a, b = max(r0, lo), min(r1, hi)
            key = f"model.{parent}.{sub}.weight"
            out[key] = w[a - lo:b - lo] if b > a else w[:0]
            sharded.append(key)
            skip.add(key)
            r0 = r1
    for k, v in full.items():
        if k not in skip:
            out[k] = v
    return out, sharded


def save_sharded_state(model: CausalLM, out_dir: str, rank: int, world: int):
    """Every rank writes ``<out_dir>/pytorch_model_fsdp_0/shard_rank{rank}.safetensors``; rank 0 adds the
    index and the model config."""
    import json

    d = os.path.join(out_dir, "pytorch_model_fsdp_0")
    os.makedirs(d, exist_ok=True)
    sd, sharded = sharded_state_dict(model, rank)
    st.save_file({k: v.to("cpu").contiguous() for k, v in sd.items()}, os.path.join(d, f"shard_rank{rank}.safetensors"),
                 {"format": "pt"})
    if rank == 0:
        with open(os.path.join(d, "shard_index.json"), "w") as fh:
            json.dump({"world_size": world, "sharded": sharded}, fh, indent=1)
        model.config.save_pretrained(d)
    return d


def load_pretrained_from_rank0(path: str, dtype=torch.bfloat16, device="cpu", config: ModelConfig | None = None,
                               group=None, strict: bool = True) -> CausalLM:
    """``fsdp_config.cpu_ram_efficient_loading``: only rank 0 reads the checkpoint from disk; every other rank
    builds the empty model and receives the tensors by broadcast, so N ranks do not read (and hold in host
    memory) N copies of the files (src/axolotl/monkeypatch/accelerate/fsdp2.py:142-345 loads on rank 0 and
    scatters)."""
    import torch.distributed as dist

    cfg = config or ModelConfig.from_pretrained(path)
    model = CausalLM(cfg, dtype=dtype, device=device)
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if rank == 0:
        load_state_into(model, st.iter_checkpoint(path), strict=strict)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        src = dist.get_global_rank(group, 0) if group is not None else 0
        for _, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
            dist.broadcast(p.data, src=src, group=group)
        for _, b in sorted(model.named_buffers(), key=lambda kv: kv[0]):
            if b is not None and b.is_floating_point():
                dist.broadcast(b.data, src=src, group=group)
    return model


def _deinterleave_rows(w, heads, D, inverse=False):
    """Rotary pairs stored as (real, imaginary) neighbours <-> the half-split layout the rotary kernel works on:
    a permutation of the D output rows of every head (attention scores do not change when q and k share it)."""
    idx = torch.cat([torch.arange(0, D, 2), torch.arange(1, D, 2)])
    if inverse:
        idx = torch.argsort(idx)
    return w.reshape(heads, D, *w.shape[1:]).index_select(1, idx.to(w.device)).reshape(w.shape)


# LFM2 names (checkpoint, ours); the short-convolution operator sits where other families keep their attention module
_LFM2_NAMES = ((".feed_forward.expert_bias", ".mlp.gate.e_score_correction_bias"), (".feed_forward.gate.", ".mlp.gate."),
               (".feed_forward.experts.", ".mlp.experts."), (".operator_norm.", ".input_layernorm."), (".ffn_norm.", ".post_attention_layernorm."),
               (".feed_forward.w1.", ".mlp.gate_proj."), (".feed_forward.w3.", ".mlp.up_proj."), (".feed_forward.w2.", ".mlp.down_proj."),
               (".self_attn.out_proj.", ".self_attn.o_proj."), (".self_attn.q_layernorm.", ".self_attn.q_norm."),
               (".self_attn.k_layernorm.", ".self_attn.k_norm."), ("model.embedding_norm.", "model.norm."))


def _lfm2_state_dict(model, sd):
    out = {}
    for i, layer in enumerate(model.layers):
        mx = layer.self_attn
        if type(mx).__name__ == "ShortConv":
            pre = f"model.layers.{i}"
            for k in [k for k in sd if k.startswith(pre + ".self_attn.")]:
                sd.pop(k)
            out[f"{pre}.conv.in_proj.weight"] = mx.in_proj.weight.detach()
            out[f"{pre}.conv.out_proj.weight"] = mx.out_proj.weight.detach()
            out[f"{pre}.conv.conv.weight"] = mx.conv_weight.detach()[:, None, :]
            if mx.conv_bias is not None:
                out[f"{pre}.conv.in_proj.bias"] = mx.in_proj.bias.detach()
                out[f"{pre}.conv.out_proj.bias"] = mx.out_proj.bias.detach()
                out[f"{pre}.conv.conv.bias"] = mx.conv_bias.detach()
    for k, v in sd.items():
        for theirs, ours in _LFM2_NAMES:
            if ours in k:
                k = k.replace(ours, theirs)
                break
        out[k] = v
    return out


def _rotary_rows(w, heads, D, rot, inverse=False):
    """The first ``rot`` rows of every head: interleaved (real, imaginary) pairs <-> half-split layout."""
    idx = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, D)])
    if inverse:
        idx = torch.argsort(idx)
    return w.reshape(heads, D, *w.shape[1:]).index_select(1, idx.to(w.device)).reshape(w.shape)


_GLM4_NORMS = ((".post_self_attn_layernorm.", ".post_attention_layernorm."), (".post_attention_layernorm.", ".pre_feedforward_layernorm."),
               (".post_mlp_layernorm.", ".post_feedforward_layernorm."))


def _glm_in(model, name, t):
    """GLM checkpoints: rotary pairs of q / k stored as neighbours (rows are permuted); GLM-4 names its four norms
    `input`, `post_self_attn` (attention output), `post_attention` (MLP input), `post_mlp` (MLP output)."""
    cfg = model.config
    if cfg.model_type == "glm4":
        for src, dst in _GLM4_NORMS:
            if src in name:
                name = name.replace(src, dst)
                break
    m = re.search(r"\.self_attn\.(q|k)_proj\.(weight|bias)$", name)
    if m:
        heads = cfg.num_attention_heads if m.group(1) == "q" else cfg.num_key_value_heads
        t = _rotary_rows(t, heads, cfg.head_dim, cfg.rope_dim())
    return name, t


def _glm_out(model, sd):
    cfg, out = model.config, {}
    for name, t in sd.items():
        m = re.search(r"\.self_attn\.(q|k)_proj\.(weight|bias)$", name)
        if m:
            heads = cfg.num_attention_heads if m.group(1) == "q" else cfg.num_key_value_heads
            t = _rotary_rows(t, heads, cfg.head_dim, cfg.rope_dim(), inverse=True)
        if cfg.model_type == "glm4":
            for dst, src in reversed(_GLM4_NORMS):
                if src in name:
                    name = name.replace(src, dst)
                    break
        out[name] = t
    return out


def _llama4_in(model, name, t):
    """Llama 4 checkpoint names and layouts -> ours: `feed_forward` is `mlp`, `router` the gate, `shared_expert` the
    shared MLP; expert stacks are stored [E, in, out]; q / k rows use interleaved rotary pairs."""
    cfg = model.config
    name = name.replace("language_model.model.", "model.").replace("language_model.lm_head", "lm_head")
    name = name.replace(".feed_forward.", ".mlp.")
    if name.endswith(".mlp.router.weight"):
        return name.replace(".router.weight", ".gate.weight"), t
    name = name.replace(".mlp.shared_expert.", ".mlp.shared_experts.")
    if name.endswith(".mlp.experts.gate_up_proj") or name.endswith(".mlp.experts.down_proj"):
        return name, t.transpose(1, 2)
    if name.endswith(".self_attn.q_proj.weight"):
        return name, _deinterleave_rows(t, cfg.num_attention_heads, cfg.head_dim)
    if name.endswith(".self_attn.k_proj.weight"):
        return name, _deinterleave_rows(t, cfg.num_key_value_heads, cfg.head_dim)
    return name, t


def _llama4_out(model, sd):
    cfg, out = model.config, {}
    for name, t in sd.items():
        if name.endswith(".self_attn.q_proj.weight"):
            t = _deinterleave_rows(t, cfg.num_attention_heads, cfg.head_dim, inverse=True)
        elif name.endswith(".self_attn.k_proj.weight"):
            t = _deinterleave_rows(t, cfg.num_key_value_heads, cfg.head_dim, inverse=True)
        elif name.endswith(".mlp.experts.gate_up_proj") or name.endswith(".mlp.experts.down_proj"):
            t = t.transpose(1, 2).contiguous()
        name = name.replace(".mlp.gate.weight", ".mlp.router.weight").replace(".mlp.shared_experts.", ".mlp.shared_expert.")
        out[name.replace(".mlp.", ".feed_forward.")] = t
    return out


def _mamba_tensors(pre, mx, sd):
    sd[f"{pre}.mamba.in_proj.weight"] = mx.in_proj.weight.detach()
    sd[f"{pre}.mamba.out_proj.weight"] = mx.out_proj.weight.detach()
    if mx.in_proj.bias is not None:
        sd[f"{pre}.mamba.in_proj.bias"] = mx.in_proj.bias.detach()
    if mx.out_proj.bias is not None:
        sd[f"{pre}.mamba.out_proj.bias"] = mx.out_proj.bias.detach()
    sd[f"{pre}.mamba.conv1d.weight"] = mx.conv_weight.detach()[:, None, :]
    if mx.conv_bias is not None:
        sd[f"{pre}.mamba.conv1d.bias"] = mx.conv_bias.detach()
    if mx.norm_weight is not None:
        sd[f"{pre}.mamba.norm.weight"] = mx.norm_weight.detach()
    for leaf in ("dt_bias", "A_log", "D"):
        sd[f"{pre}.mamba.{leaf}"] = getattr(mx, leaf).detach()


def _nemotron_h_state_dict(model):
    """Nemotron-H names: `model.embeddings`, per layer `norm` + `mixer.*`, `model.norm_f`."""
    sd = {"model.embeddings.weight": model.embed_tokens.detach(), "model.norm_f.weight": model.norm.weight.detach()}
    if model.lm_head is not None:
        sd["lm_head.weight"] = model.lm_head.detach()
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}"
        sd[f"{pre}.norm.weight"] = layer.norm.weight.detach()
        mx = layer.mixer
        if layer.kind == "mamba":
            tmp = {}
            _mamba_tensors(pre, mx, tmp)
            sd.update({k.replace(".mamba.", ".mixer."): v for k, v in tmp.items()})
        else:
            for fl in ([mx.qkv_proj, mx.o_proj] if layer.kind == "attention" else [mx.up_proj, mx.down_proj]):
                for sub in fl.names:
                    r0, r1 = fl.row_range(sub)
                    sd[f"{pre}.mixer.{sub}.weight"] = fl.weight.detach()[r0:r1]
                    if fl.bias is not None:
                        sd[f"{pre}.mixer.{sub}.bias"] = fl.bias.detach()[r0:r1]
    return sd


@torch.no_grad()
def _nemotron_h_load(model, named_tensors, strict=True):
    filled = set()
    for name, t in named_tensors:
        name = name.replace("backbone.", "model.")
        if name == "model.embeddings.weight":
            model.embed_tokens.copy_(t)
        elif name == "model.norm_f.weight":
            model.norm.weight.copy_(t)
        elif name == "lm_head.weight":
            if model.lm_head is not None:
                model.lm_head.copy_(t)
        elif (m := re.match(r"model\.layers\.(\d+)\.norm\.weight$", name)):
            model.layers[int(m.group(1))].norm.weight.copy_(t)
        elif (m := re.match(r"model\.layers\.(\d+)\.mixer\.(.+)$", name)):
            layer, leaf = model.layers[int(m.group(1))], m.group(2)
            mx = layer.mixer
            if layer.kind == "mamba":
                if leaf == "conv1d.weight":
                    mx.conv_weight.copy_(t.reshape(t.shape[0], t.shape[-1]))
                elif leaf == "conv1d.bias":
                    mx.conv_bias.copy_(t)
                elif leaf == "norm.weight":
                    mx.norm_weight.copy_(t)
                elif leaf in ("dt_bias", "A_log", "D"):
                    getattr(mx, leaf).copy_(t)
                else:
                    getattr(getattr(mx, leaf.split(".")[0]), leaf.split(".")[1]).copy_(t)
            else:
                sub, kind = leaf.rsplit(".", 1)
                fl = {"q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj"}.get(sub, sub)
                fl = getattr(mx, fl)
                r0, r1 = fl.row_range(sub)
                (fl.weight if kind == "weight" else fl.bias)[r0:r1].copy_(t)
        elif name.endswith("rotary_emb.inv_freq"):
            continue
        elif strict:
            raise KeyError(f"unexpected checkpoint tensor '{name}'")
        filled.add(name)
    return filled


def _bamba_state_dict(model, sd):
    """Bamba / Falcon-H1 names: `mamba.*` mixers, `pre_ff_layernorm`, `feed_forward`, `final_layernorm`."""
    sd["model.final_layernorm.weight"] = sd.pop("model.norm.weight")
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}"
        sd[f"{pre}.input_layernorm.weight"] = layer.input_layernorm.weight.detach()
        sd[f"{pre}.pre_ff_layernorm.weight"] = layer.post_attention_layernorm.weight.detach()
        for mx in ([layer.mamba, layer.self_attn] if hasattr(layer, "mamba") else [layer.self_attn]):
            if type(mx).__name__ == "Mamba2Mixer":
                _mamba_tensors(pre, mx, sd)
            else:
                for fl in (mx.qkv_proj, mx.o_proj):
                    for sub in fl.names:
                        r0, r1 = fl.row_range(sub)
                        sd[f"{pre}.self_attn.{sub}.weight"] = fl.weight.detach()[r0:r1]
                        if fl.bias is not None:
                            sd[f"{pre}.self_attn.{sub}.bias"] = fl.bias.detach()[r0:r1]
        for fl in (layer.mlp.gate_up_proj, layer.mlp.down_proj):
            for sub in fl.names:
                r0, r1 = fl.row_range(sub)
                sd[f"{pre}.feed_forward.{sub}.weight"] = fl.weight.detach()[r0:r1]
    return sd


def _qwen3_next_out(model, sd):
    """Qwen3-Next names: `linear_attn.*` for the DeltaNet mixers; q_proj carries the output-gate rows head by head."""
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}"
        mx = layer.self_attn
        if type(mx).__name__ == "GatedDeltaNet":
            for k in [k for k in sd if k.startswith(pre + ".self_attn.")]:
                sd.pop(k)
            if mx.flat:
                for sub in mx.in_proj.names:
                    r0, r1 = mx.in_proj.row_range(sub)
                    sd[f"{pre}.linear_attn.{sub}.weight"] = mx.in_proj.weight.detach()[r0:r1]
            else:
                sd[f"{pre}.linear_attn.in_proj_qkvz.weight"] = mx.in_proj_qkvz.weight.detach()
                sd[f"{pre}.linear_attn.in_proj_ba.weight"] = mx.in_proj_ba.weight.detach()
            sd[f"{pre}.linear_attn.out_proj.weight"] = mx.out_proj.weight.detach()
            sd[f"{pre}.linear_attn.conv1d.weight"] = mx.conv_weight.detach()[:, None, :]
            sd[f"{pre}.linear_attn.norm.weight"] = mx.norm_weight.detach()
            sd[f"{pre}.linear_attn.dt_bias"] = mx.dt_bias.detach()
            sd[f"{pre}.linear_attn.A_log"] = mx.A_log.detach()
        else:
            q = sd.pop(f"{pre}.self_attn.q_proj.weight")
            gate = sd.pop(f"{pre}.self_attn.q_gate.weight")
            sd[f"{pre}.self_attn.q_proj.weight"] = torch.stack([q.reshape(mx.Hq, mx.D, -1), gate.reshape(mx.Hq, mx.D, -1)], 1) \
                .reshape(2 * mx.Hq * mx.D, -1)
    return sd


def _granite_hybrid_state_dict(model, sd):
    """Granite 4.0-H names: `mamba.*` mixers, `shared_mlp`, `block_sparse_moe`."""
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}"
        for nm in ("input_layernorm", "post_attention_layernorm"):
            sd[f"{pre}.{nm}.weight"] = getattr(layer, nm).weight.detach()
        mx = layer.self_attn
        if type(mx).__name__ == "Mamba2Mixer":
            sd[f"{pre}.mamba.in_proj.weight"] = mx.in_proj.weight.detach()
            sd[f"{pre}.mamba.out_proj.weight"] = mx.out_proj.weight.detach()
            if mx.in_proj.bias is not None:
                sd[f"{pre}.mamba.in_proj.bias"] = mx.in_proj.bias.detach()
                sd[f"{pre}.mamba.out_proj.bias"] = mx.out_proj.bias.detach()
            sd[f"{pre}.mamba.conv1d.weight"] = mx.conv_weight.detach()[:, None, :]
            if mx.conv_bias is not None:
                sd[f"{pre}.mamba.conv1d.bias"] = mx.conv_bias.detach()
            sd[f"{pre}.mamba.norm.weight"] = mx.norm_weight.detach()
            for leaf in ("dt_bias", "A_log", "D"):
                sd[f"{pre}.mamba.{leaf}"] = getattr(mx, leaf).detach()
        else:
            for fl in (mx.qkv_proj, mx.o_proj):
                for sub in fl.names:
                    r0, r1 = fl.row_range(sub)
                    sd[f"{pre}.self_attn.{sub}.weight"] = fl.weight.detach()[r0:r1]
        mlp = layer.mlp
        is_moe = isinstance(getattr(mlp, "experts", None), Experts)
        shared = getattr(mlp, "shared_experts", None) if is_moe else mlp
        if shared is not None:
            sd[f"{pre}.shared_mlp.input_linear.weight"] = shared.gate_up_proj.weight.detach()
            sd[f"{pre}.shared_mlp.output_linear.weight"] = shared.down_proj.weight.detach()
        if isinstance(getattr(mlp, "experts", None), Experts):
            sd[f"{pre}.block_sparse_moe.input_linear.weight"] = mlp.experts.gate_up_proj.detach()
            sd[f"{pre}.block_sparse_moe.output_linear.weight"] = mlp.experts.down_proj.detach()
            sd[f"{pre}.block_sparse_moe.router.layer.weight"] = mlp.gate.detach()
    return sd


_FALCON_NAMES = (("transformer.word_embeddings.", "model.embed_tokens."), ("transformer.ln_f.", "model.norm."),
                 ("transformer.h.", "model.layers."), (".self_attention.dense.", ".self_attn.o_proj."),
                 (".self_attention.", ".self_attn."), (".mlp.dense_h_to_4h.", ".mlp.up_proj."),
                 (".mlp.dense_4h_to_h.", ".mlp.down_proj."), (".ln_attn.", ".input_layernorm."))


def _falcon_in(name: str) -> str:
    for src, dst in _FALCON_NAMES:
        name = name.replace(src, dst)
    return name


def _falcon_out(model, sd: dict) -> dict:
    """This graph's names and q | k | v row order -> Falcon's (``transformer.h.N.self_attention.query_key_value`` ...)."""
    inv = torch.argsort(model.config.falcon_qkv_rows())
    two_norms = model.layers[0].ln_mlp is not None
    out = {}
    for k, v in sd.items():
        if ".self_attn.query_key_value." in k:
            v = v.index_select(0, inv.to(v.device))
        if two_norms:
            k = k.replace(".input_layernorm.", ".ln_attn.")
        k = k.replace(".self_attn.o_proj.", ".self_attention.dense.").replace(".self_attn.", ".self_attention.") \
            .replace(".mlp.up_proj.", ".mlp.dense_h_to_4h.").replace(".mlp.down_proj.", ".mlp.dense_4h_to_h.") \
            .replace("model.layers.", "transformer.h.").replace("model.embed_tokens.", "transformer.word_embeddings.") \
            .replace("model.norm.", "transformer.ln_f.")
        out[k] = v
    for i, layer in enumerate(model.layers):
        if layer.ln_mlp is not None:
            out[f"transformer.h.{i}.ln_mlp.weight"] = layer.ln_mlp.weight.detach()
            out[f"transformer.h.{i}.ln_mlp.bias"] = layer.ln_mlp.bias.detach()
    return out


def hf_state_dict(model: CausalLM, per_expert: bool = False) -> dict:
    """Model tensors under HF names (views where possible; the writer makes them contiguous)."""
    sd = {"model.embed_tokens.weight": model.embed_tokens.detach()}
    if model.norm.weight is not None:
        sd["model.norm.weight"] = model.norm.weight.detach()
    if getattr(model, "lm_head_bias", None) is not None:
        sd["lm_head.bias"] = model.lm_head_bias.detach()
    if model.lm_head is not None:
        sd["lm_head.weight"] = model.lm_head.detach()
    if getattr(model.norm, "bias", None) is not None:
        sd["model.norm.bias"] = model.norm.bias.detach()
    gpt_oss = getattr(model.config, "model_type", "") == "gpt_oss"
    if getattr(model.config, "model_type", "") in ("granitemoe", "granitemoeshared", "granitemoehybrid"):
        return _granite_hybrid_state_dict(model, sd)
    if getattr(model.config, "model_type", "") in ("bamba", "falcon_h1"):
        return _bamba_state_dict(model, sd)
    if getattr(model.config, "model_type", "") == "nemotron_h":
        return _nemotron_h_state_dict(model)
    for name, m in model.named_modules():
        if gpt_oss and isinstance(m, Experts):
            def interleave(u):            # [E, 2I, ...] gate rows then up rows -> alternating
                E, two_i = u.shape[:2]
                return torch.stack([u[:, : two_i // 2], u[:, two_i // 2:]], 2).reshape(u.shape)
            sd[f"model.{name}.gate_up_proj"] = interleave(m.gate_up_proj.detach()).transpose(1, 2).contiguous()
            sd[f"model.{name}.gate_up_proj_bias"] = interleave(m.gate_up_bias.detach())
            sd[f"model.{name}.down_proj"] = m.down_proj.detach().transpose(1, 2).contiguous()
            sd[f"model.{name}.down_proj_bias"] = m.down_bias.detach()
            continue
        if gpt_oss and getattr(m, "router_bias", None) is not None:
            sd[f"model.{name}.router.weight"] = m.gate.detach()
            sd[f"model.{name}.router.bias"] = m.router_bias.detach()
            continue
        if getattr(m, "sinks", None) is not None:
            sd[f"model.{name}.sinks"] = m.sinks.detach()
        if getattr(m, "layer_scalar", None) is not None:
            sd[f"model.{name}.layer_scalar"] = m.layer_scalar.detach()
        if type(m).__name__ == "LightningIndexer":
            sd[f"model.{name}.k_norm.weight"] = m.k_norm_weight.detach()
            sd[f"model.{name}.k_norm.bias"] = m.k_norm_bias.detach()
        if isinstance(m, FusedLinear):
            parent = name.rsplit(".", 1)[0]
            for sub in m.names:
                r0, r1 = m.row_range(sub)
                sd[f"model.{parent}.{sub}.weight"] = m.weight.detach()[r0:r1]
                if m.bias is not None:
                    sd[f"model.{parent}.{sub}.bias"] = m.bias.detach()[r0:r1]
        elif name.endswith(("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm",
                            "q_norm", "k_norm", "q_a_layernorm", "kv_a_layernorm")):
            if m.weight is not None:
                sd[f"model.{name}.weight"] = m.weight.detach()
            if getattr(m, "bias", None) is not None:
                sd[f"model.{name}.bias"] = m.bias.detach()
        elif isinstance(m, Experts):
            if m.nvfp4 is not None:
                for which in ("gate_up", "down"):
                    q = m.nvfp4[which]
                    sd[f"model.{name}.{which}_proj.weight_packed"] = q["qdata"]
                    sd[f"model.{name}.{which}_proj.weight_scale"] = q["scale"]
                    sd[f"model.{name}.{which}_proj.weight_global_scale"] = q["pts"]
            elif per_expert:
                I = m.I
                for e in range(m.E):
                    sd[f"model.{name}.{e}.gate_proj.weight"] = m.gate_up_proj.detach()[e, :I]
                    sd[f"model.{name}.{e}.up_proj.weight"] = m.gate_up_proj.detach()[e, I:]
                    sd[f"model.{name}.{e}.down_proj.weight"] = m.down_proj.detach()[e]
            else:
                sd[f"model.{name}.gate_up_proj"] = m.gate_up_proj.detach()
                sd[f"model.{name}.down_proj"] = m.down_proj.detach()
        elif hasattr(m, "gate") and isinstance(getattr(m, "gate"), torch.nn.Parameter):
            sd[f"model.{name}.gate.weight"] = m.gate.detach()
            if getattr(m, "shared_expert_gate", None) is not None:
                sd[f"model.{name}.shared_expert_gate.weight"] = m.shared_expert_gate.detach()
            if getattr(m, "e_score_correction_bias", None) is not None:
                where = "" if getattr(model.config, "model_type", "") == "minimax_m2" else "gate."    # MiniMax keeps it on the block
                sd[f"model.{name}.{where}e_score_correction_bias"] = m.e_score_correction_bias.detach()
    if getattr(model.config, "model_type", "") == "llama4_text":
        return _llama4_out(model, sd)
    if getattr(model.config, "model_type", "") in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text"):
        return _qwen3_next_out(model, sd)
    if model.config.rope_pairs_interleaved():
        sd = _glm_out(model, sd)
    mt_ = getattr(model.config, "model_type", "")
    if mt_ in ("hunyuan_v1_dense", "hunyuan_v1_moe"):
        return {k.replace(".q_norm.", ".query_layernorm.").replace(".k_norm.", ".key_layernorm.")
                .replace(".mlp.gate.weight", ".mlp.gate.wg.weight").replace(".mlp.shared_experts.", ".mlp.shared_mlp."): v
                for k, v in sd.items()}
    if mt_ == "ernie4_5_moe":
        return {k.replace(".gate.e_score_correction_bias", ".gate.moe_statics.e_score_correction_bias"):
                (v.reshape(1, -1) if k.endswith("e_score_correction_bias") else v) for k, v in sd.items()}
    if mt_ in ("lfm2", "lfm2_moe"):
        return _lfm2_state_dict(model, sd)
    if mt_ == "afmoe":
        return {k.replace(".pre_feedforward_layernorm.", ".pre_mlp_layernorm.").replace(".post_feedforward_layernorm.", ".post_mlp_layernorm.")
                .replace(".mlp.gate.e_score_correction_bias", ".mlp.expert_bias").replace(".mlp.gate.weight", ".mlp.router.gate.weight")
                .replace(".self_attn.out_gate.", ".self_attn.gate_proj."): v for k, v in sd.items()}
    if mt_ == "apertus":
        out = {k.replace(".input_layernorm.", ".attention_layernorm.").replace(".post_attention_layernorm.", ".feedforward_layernorm."): v
               for k, v in sd.items()}
        for i, layer in enumerate(model.layers):
            out[f"model.layers.{i}.mlp.act_fn.alpha_p"] = layer.mlp.alpha_p.detach()
            out[f"model.layers.{i}.mlp.act_fn.alpha_n"] = layer.mlp.alpha_n.detach()
            out[f"model.layers.{i}.mlp.act_fn.beta"] = torch.tensor(layer.mlp.xielu_beta, dtype=layer.mlp.alpha_p.dtype)
            out[f"model.layers.{i}.mlp.act_fn.eps"] = torch.tensor(layer.mlp.xielu_eps, dtype=layer.mlp.alpha_p.dtype)
        return out
    if mt_ == "phi":
        return {k.replace(".mlp.up_proj.", ".mlp.fc1.").replace(".mlp.down_proj.", ".mlp.fc2.")
                .replace(".self_attn.o_proj.", ".self_attn.dense.").replace("model.norm.", "model.final_layernorm."): v
                for k, v in sd.items()}
    if getattr(model.config, "model_type", "") == "starcoder2":
        return {k.replace(".mlp.up_proj.", ".mlp.c_fc.").replace(".mlp.down_proj.", ".mlp.c_proj."): v for k, v in sd.items()}
    if mt_ == "falcon":
        return _falcon_out(model, sd)
    if mt_ == "gemma4_text":
        out = {k.replace(".g4_moe.experts.", ".experts.").replace(".g4_moe.gate.weight", ".router.proj.weight")
               .replace("model.per_layer_model_projection.per_layer_model_projection.", "model.per_layer_model_projection."): v
               for k, v in sd.items()}
        if getattr(model, "ple_width", 0):
            out["model.embed_tokens_per_layer.weight"] = model.embed_tokens_per_layer.detach()
            out["model.per_layer_projection_norm.weight"] = model.per_layer_projection_norm.weight.detach()
        for i, layer in enumerate(model.layers):
            for nm in ("post_per_layer_input_norm", "post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                if hasattr(layer, nm):
                    out[f"model.layers.{i}.{nm}.weight"] = getattr(layer, nm).weight.detach()
            if layer.g4_moe is not None:
                out[f"model.layers.{i}.router.scale"] = layer.g4_moe.router_scale.detach()
                out[f"model.layers.{i}.router.per_expert_scale"] = layer.g4_moe.per_expert_scale.detach()
        return out
    return sd


def _with_vision(model, sd: dict) -> dict:
    """LLaVA layout: the language model's tensors under ``model.language_model.``, tower and projector beside it."""
    out = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v for k, v in sd.items()}
    if "lm_head.weight" not in out:          # the wrapper ties nothing by itself: write the head it would look for
        out["lm_head.weight"] = model.embed_tokens.detach()
    for k, v in model.vision.named_parameters():
        out["model." + k] = v.detach()
    return out


def save_pretrained(model: CausalLM, out_dir: str, max_shard_bytes: int = 5 * 1024 ** 3, per_expert=False):
    os.makedirs(out_dir, exist_ok=True)
    model.config.save_pretrained(out_dir)
    sd = hf_state_dict(model, per_expert=per_expert)
    if getattr(model, "vision", None) is not None:
        sd = _with_vision(model, sd)
    sd = {k: v.to("cpu") for k, v in sd.items()}
    return st.save_sharded(sd, out_dir, max_shard_bytes)
