"""LoRA adapter management: injection, PEFT-format state dicts, ``adapter_config.json``.

File format contract (what ``peft`` writes and what the reference's merge tool reads,
src/axolotl/cli/utils/lora_merge.py:1904-2000): keys
``base_model.model.<hf module path>.lora_A.weight`` [r, in] / ``.lora_B.weight`` [out, r];
expert adapters (PEFT ``target_parameters``) use ``<path>.lora_A.weight`` [E*r, in] and
``.lora_B.weight`` [out, r*E].
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import asdict, dataclass, field

import torch

from .layers import FusedLinear
from .moe import Experts

ALL_LINEAR = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj",
              "qkv_proj", "gate_up_proj")   # the last two: architectures whose checkpoints are fused (Phi-3)


@dataclass
class LoraSpec:
    r: int = 8
    lora_alpha: int = 16
    lora_dropout: float = 0.0
    target_modules: list | str | None = None       # names, or a regex string (PEFT semantics)
    target_parameters: list | None = None          # e.g. ["mlp.experts.gate_up_proj", "mlp.experts.down_proj"]
    use_rslora: bool = False
    use_dora: bool = False
    use_mora: bool = False
    mora_type: int = 6                              # 1 = sharing, 6 = rope (the MoRA fork's numbering)
    fan_in_fan_out: bool = False
    bias: str = "none"
    modules_to_save: list | None = None
    trainable_token_indices: list | dict | None = None
    rank_pattern: dict = field(default_factory=dict)
    alpha_pattern: dict = field(default_factory=dict)
    layers_to_transform: list | None = None
    base_model_name_or_path: str | None = None

    def to_peft_dict(self):
        tm = self.target_modules
        return {
            "peft_type": "LORA", "task_type": "CAUSAL_LM", "auto_mapping": None,
            "base_model_name_or_path": self.base_model_name_or_path, "bias": self.bias,
            "fan_in_fan_out": self.fan_in_fan_out, "inference_mode": True, "init_lora_weights": True,
            "layers_pattern": None, "layers_to_transform": self.layers_to_transform,
            "lora_alpha": self.lora_alpha, "lora_dropout": self.lora_dropout,
            "modules_to_save": self.modules_to_save, "r": self.r, "rank_pattern": self.rank_pattern,
            "alpha_pattern": self.alpha_pattern, "revision": None,
            "target_modules": sorted(tm) if isinstance(tm, (list, tuple, set)) else tm,
            "target_parameters": self.target_parameters, "use_dora": self.use_dora,
            "use_rslora": self.use_rslora, "trainable_token_indices": self.trainable_token_indices,
            **({"use_mora": True, "mora_type": self.mora_type} if self.use_mora else {}),
        }

    @classmethod
    def from_peft_dict(cls, d):
        keys = cls.__dataclass_fields__.keys()
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        return cls(**kw)

    def save(self, out_dir):
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "adapter_config.json"), "w") as fh:
            json.dump(self.to_peft_dict(), fh, indent=2)

    @classmethod
    def load(cls, adapter_dir):
        with open(os.path.join(adapter_dir, "adapter_config.json")) as fh:
            return cls.from_peft_dict(json.load(fh))


def _checkpoint_renames(model):
    """Where a family's checkpoint names its modules differently from this graph, (internal prefix, checkpoint
    prefix) pairs: adapters are saved under the CHECKPOINT's module names, so that PEFT and the merge tools find them."""
    cached = model.__dict__.get("_axb_hf_renames")
    if cached is not None:
        return cached
    mt = getattr(getattr(model, "config", None), "model_type", "")
    pairs = []
    for i, layer in enumerate(getattr(model, "layers", [])):
        pre = f"model.layers.{i}"
        mixer = type(getattr(layer, "self_attn", None)).__name__
        if mt in ("bamba", "granitemoehybrid") and mixer == "Mamba2Mixer":
            pairs.append((f"{pre}.self_attn.", f"{pre}.mamba."))
        if mt in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text") and mixer == "GatedDeltaNet":
            pairs.append((f"{pre}.self_attn.", f"{pre}.linear_attn."))
        if mt in ("bamba", "falcon_h1"):
            pairs.append((f"{pre}.mlp.", f"{pre}.feed_forward."))
        if mt in ("lfm2", "lfm2_moe"):
            if mixer == "ShortConv":
                pairs.append((f"{pre}.self_attn.", f"{pre}.conv."))
            pairs += [(f"{pre}.self_attn.o_proj", f"{pre}.self_attn.out_proj"), (f"{pre}.mlp.gate_proj", f"{pre}.feed_forward.w1"),
                      (f"{pre}.mlp.up_proj", f"{pre}.feed_forward.w3"), (f"{pre}.mlp.down_proj", f"{pre}.feed_forward.w2")]
        if mt == "hunyuan_v1_moe":
            pairs.append((f"{pre}.mlp.shared_experts.", f"{pre}.mlp.shared_mlp."))
        if mt == "afmoe":
            pairs.append((f"{pre}.self_attn.out_gate.gate_proj", f"{pre}.self_attn.gate_proj"))
        if mt == "phi":
            pairs += [(f"{pre}.mlp.up_proj", f"{pre}.mlp.fc1"), (f"{pre}.mlp.down_proj", f"{pre}.mlp.fc2"),
                      (f"{pre}.self_attn.o_proj", f"{pre}.self_attn.dense")]
        if mt == "falcon":
            fp = f"transformer.h.{i}"
            pairs += [(f"{pre}.self_attn.o_proj", f"{fp}.self_attention.dense"), (f"{pre}.self_attn.", f"{fp}.self_attention."),
                      (f"{pre}.mlp.up_proj", f"{fp}.mlp.dense_h_to_4h"), (f"{pre}.mlp.down_proj", f"{fp}.mlp.dense_4h_to_h")]
        if mt == "starcoder2":
            pairs.append((f"{pre}.mlp.up_proj", f"{pre}.mlp.c_fc"))
            pairs.append((f"{pre}.mlp.down_proj", f"{pre}.mlp.c_proj"))
        if mt == "llama4_text":
            pairs.append((f"{pre}.mlp.shared_experts.", f"{pre}.feed_forward.shared_expert."))
            pairs.append((f"{pre}.mlp.", f"{pre}.feed_forward."))
        if mt in ("granitemoeshared", "granitemoehybrid"):
            for inner in ("mlp.shared_experts", "mlp"):
                pairs.append((f"{pre}.{inner}.gate_up_proj", f"{pre}.shared_mlp.input_linear"))
                pairs.append((f"{pre}.{inner}.down_proj", f"{pre}.shared_mlp.output_linear"))
    if mt == "gemma4_text":          # a model-level projection: its module path is its own name
        pairs.append(("model.per_layer_model_projection.per_layer_model_projection", "model.per_layer_model_projection"))
    model.__dict__["_axb_hf_renames"] = pairs
    return pairs


def _hf_path(fused_name: str, sub: str, model=None) -> str:
    """'layers.3.self_attn.qkv_proj' + 'q_proj' -> 'model.layers.3.self_attn.q_proj' (in the checkpoint's own module
    names when ``model`` is given)."""
    parent = fused_name.rsplit(".", 1)[0]
    path = f"model.{parent}.{sub}"
    if model is not None:
        for src, dst in _checkpoint_renames(model):
            if path.startswith(src):
                path = dst + path[len(src):]
                break
        if getattr(model, "vision", None) is not None and path.startswith("model."):     # LLaVA keeps the language model one level down
            path = "model.language_model." + path[len("model."):]
    return path


def _B_rows_layout(model, name, sub, B, to_checkpoint: bool):
    """Output rows of an adapter's B in the CHECKPOINT's row order / count for the projections this graph stores
    differently: Llama 4 keeps rotary pairs interleaved in q / k (rows are permuted here), Qwen3-Next's q_proj carries
    the output-gate rows head by head (they get zero rows on the way out and are dropped on the way in)."""
    mt = getattr(getattr(model, "config", None), "model_type", "")
    if mt == "llama4_text" and sub in ("q_proj", "k_proj") and ".self_attn." in name:
        cfg = model.config
        heads = cfg.num_attention_heads if sub == "q_proj" else cfg.num_key_value_heads
        idx = torch.cat([torch.arange(0, cfg.head_dim, 2), torch.arange(1, cfg.head_dim, 2)])
        if to_checkpoint:
            idx = torch.argsort(idx)
        return B.reshape(heads, cfg.head_dim, -1).index_select(1, idx.to(B.device)).reshape(B.shape)
    if getattr(getattr(model, "config", None), "rope_pairs_interleaved", lambda: False)() and sub in ("q_proj", "k_proj") \
            and ".self_attn." in name:
        cfg = model.config
        heads, D, rot = (cfg.num_attention_heads if sub == "q_proj" else cfg.num_key_value_heads), cfg.head_dim, cfg.rope_dim()
        idx = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, D)])
        if to_checkpoint:
            idx = torch.argsort(idx)
        return B.reshape(heads, D, -1).index_select(1, idx.to(B.device)).reshape(B.shape)
    if mt == "falcon" and sub == "query_key_value":      # the checkpoint interleaves queries, keys and values by head / group
        idx = model.config.falcon_qkv_rows()
        if to_checkpoint:
            idx = torch.argsort(idx)
        return B.index_select(0, idx.to(B.device))
    if mt in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text") and sub == "q_proj" and ".self_attn." in name:
        cfg = model.config
        H, D = cfg.num_attention_heads, cfg.head_dim
        if to_checkpoint:
            if B.shape[0] != H * D:
                return B
            return torch.stack([B.reshape(H, D, -1), torch.zeros(H, D, B.shape[-1], dtype=B.dtype, device=B.device)], 1) \
                .reshape(2 * H * D, -1)
        if B.shape[0] == 2 * H * D:
            return B.reshape(H, 2, D, -1)[:, 0].reshape(H * D, -1)
    return B


# projections that `lora_target_linear` leaves alone: the sparse-attention indexer is not differentiated, and the
# attention output gate of Qwen3-Next lives inside q_proj in the checkpoint (no module of its own to attach to)
_NOT_AUTO_TARGETS = ("wq_b", "wk", "weights_proj", "q_gate")


def discover_linear_names(model) -> list[str]:
    """Leaf names of every projection in the decoder layers (what PEFT's ``all-linear`` finds on the HF graph)."""
    names = set()
    for _, m in model.fused_linears():
        names.update(n for n in m.names if n not in _NOT_AUTO_TARGETS)
    return sorted(names)


def _matches(spec: LoraSpec, hf_path: str, sub: str, layer_idx: int | None) -> bool:
    if spec.layers_to_transform is not None and layer_idx is not None and layer_idx not in spec.layers_to_transform:
        return False
    tm = spec.target_modules
    if tm is None:
        return False
    if isinstance(tm, str):
        if tm == "all-linear":
            return True
        return re.fullmatch(tm, hf_path) is not None
    return any(sub == t or hf_path.endswith("." + t) for t in tm)


def inject_lora(model, spec: LoraSpec, freeze_base: bool = True, adapter_dtype=torch.float32):
    """Adds adapters according to ``spec`` and freezes everything else. Returns the trainable
    parameter count."""
    if freeze_base:
        for p in model.parameters():
            p.requires_grad_(False)
    for name, m in model.fused_linears():
        mt = re.search(r"layers\.(\d+)\.", name)
        li = int(mt.group(1)) if mt else None
        targets = [s for s in m.names if _matches(spec, _hf_path(name, s, model), s, li)]
        if targets:
            r = spec.r
            for pat, rv in spec.rank_pattern.items():
                if any(re.search(pat, _hf_path(name, s, model)) for s in targets):
                    r = rv
            alpha = spec.lora_alpha
            for pat, av in spec.alpha_pattern.items():
                if any(re.search(pat, _hf_path(name, s, model)) for s in targets):
                    alpha = av
            if spec.use_mora:
                if not isinstance(m, FusedLinear) or getattr(m.weight, "_axb_quant", None) is not None:
                    raise NotImplementedError("MoRA needs full-precision, unsharded-by-TP base projections")
                m.add_mora(r, spec.mora_type, targets, adapter_dtype)
            elif spec.use_dora:
                if not isinstance(m, FusedLinear):
                    raise NotImplementedError("DoRA cannot be combined with tensor parallelism")
                m.add_lora(r, alpha, spec.lora_dropout, targets, spec.use_rslora, adapter_dtype, use_dora=True)
            else:
                m.add_lora(r, alpha, spec.lora_dropout, targets, spec.use_rslora, adapter_dtype)
    tm = spec.target_modules
    if isinstance(tm, (list, tuple, set)) and "embed_tokens" in tm:
        if model.lm_head is None:
            raise NotImplementedError("LoRA on embed_tokens with tied input/output embeddings is not supported")
        r = spec.r
        for pat, rv in spec.rank_pattern.items():
            if re.search(pat, "model.embed_tokens"):
                r = rv
        model.add_embedding_lora(r, spec.lora_alpha, spec.use_rslora, adapter_dtype)
    tti = spec.trainable_token_indices
    if tti:
        ids = tti.get("embed_tokens") if isinstance(tti, dict) else tti
        if ids:
            model.add_trainable_tokens(ids, adapter_dtype)
    if spec.target_parameters:
        for name, m in model.named_modules():
            if isinstance(m, Experts):
                wanted = [t for t in spec.target_parameters if t.endswith("gate_up_proj") or t.endswith("down_proj")]
                if wanted:
                    m.add_lora(spec.r, spec.lora_alpha, spec.use_rslora, adapter_dtype)
    if spec.modules_to_save:
        for n, p in model.named_parameters():
            if any(k in n for k in spec.modules_to_save):
                p.requires_grad_(True)
    return count_trainable_params(model)


@torch.no_grad()
def quantize_base_nf4_(model, double_quant=True):
    """QLoRA: every projection of the decoder layers is stored as NF4 (embeddings, norms, router
    and lm_head stay in bf16, as with bitsandbytes' ``load_in_4bit``). Returns bytes saved."""
    saved = 0
    for name, m in model.fused_linears():
        if not isinstance(m, FusedLinear) or not name.startswith("layers."):
            continue
        before = m.weight.numel() * m.weight.element_size()
        m.quantize_nf4_(double_quant)
        saved += before - m.weight.numel() - m.weight._axb_quant.nbytes()
    return saved


def count_trainable_params(model) -> int:
    """Trainable parameters as PEFT would count them (the zero off-diagonal blocks of a fused
    ``lora_B`` are storage, not parameters)."""
    n = 0
    fused_ids = set()
    for _, m in model.fused_linears():
        if m.lora_A is not None:
            fused_ids.update((id(m.lora_A), id(m.lora_B)))
            for A, B in m.peft_tensors().values():
                n += A.numel() + B.numel()
    n += sum(p.numel() for p in model.parameters() if p.requires_grad and id(p) not in fused_ids)
    return n


def get_peft_state_dict(model) -> dict:
    """Adapter tensors in PEFT naming (contiguous CPU-safe copies are made by the writer)."""
    sd = {}
    for name, m in model.fused_linears():
        if getattr(m, "mora_M", None) is not None:   # the MoRA fork keeps the square matrix under lora_A
            for sub, M in zip(m.mora_names, m.mora_M):
                sd[f"base_model.model.{_hf_path(name, sub, model)}.lora_A.weight"] = M.detach()
        if m.lora_A is None:
            continue
        tensors = m.gathered_peft_tensors() if hasattr(m, "gathered_peft_tensors") else m.peft_tensors()
        for sub, (A, B) in tensors.items():
            base = f"base_model.model.{_hf_path(name, sub, model)}"
            sd[f"{base}.lora_A.weight"] = A.detach()
            sd[f"{base}.lora_B.weight"] = _B_rows_layout(model, name, sub, B.detach(), True)
            if getattr(m, "dora_magnitude", None) is not None:
                r0, r1 = m.row_range(sub)
                sd[f"{base}.lora_magnitude_vector"] = m.dora_magnitude.detach()[r0:r1]
    if getattr(model, "token_rows", None) is not None:   # PEFT TrainableTokensLayer naming
        sd["base_model.model.model.embed_tokens.token_adapter.trainable_tokens_delta"] = model.token_rows.detach()
    if getattr(model, "embed_lora_At", None) is not None:
        sd["base_model.model.model.embed_tokens.lora_embedding_A"] = model.embed_lora_At.detach().t()
        sd["base_model.model.model.embed_tokens.lora_embedding_B"] = model.embed_lora_B.detach()
    ep_of = {id(m.experts): m.ep for m in model.modules() if getattr(m, "ep", None) is not None and hasattr(m, "experts")}
    for name, m in model.named_modules():
        if isinstance(m, Experts) and m.lora is not None:
            base = f"base_model.model.model.{name}"
            full = ep_of[id(m)].gather_expert_lora(m) if id(m) in ep_of else None
            for which in ("gate_up", "down"):
                sd[f"{base}.{which}_proj.lora_A.weight"] = (full or m.lora)[which + "_A"].detach()
                sd[f"{base}.{which}_proj.lora_B.weight"] = (full or m.lora)[which + "_B"].detach()
    return sd


def set_peft_state_dict(model, sd: dict, strict: bool = True):
    """Loads PEFT-named adapter tensors (any ``.default`` adapter-name infix is tolerated)."""
    norm = {k.replace(".lora_A.default.", ".lora_A.").replace(".lora_B.default.", ".lora_B.")
            .replace(".lora_magnitude_vector.default", ".lora_magnitude_vector"): v for k, v in sd.items()}
    used = set()
    for name, m in model.fused_linears():
        if getattr(m, "mora_M", None) is not None:
            for sub, M in zip(m.mora_names, m.mora_M):
                k = f"base_model.model.{_hf_path(name, sub, model)}.lora_A.weight"
                if k in norm:
                    with torch.no_grad():
                        M.copy_(norm[k])
                    used.add(k)
                    used.add(k.replace("lora_A", "lora_B")) if k.replace("lora_A", "lora_B") in norm else None
                elif strict:
                    raise KeyError(f"adapter tensor {k} is missing")
        if m.lora_A is None:
            continue
        for sub in m.lora_names:
            base = f"base_model.model.{_hf_path(name, sub, model)}"
            ka, kb = f"{base}.lora_A.weight", f"{base}.lora_B.weight"
            if ka in norm and kb in norm:
                m.load_peft_tensors(sub, norm[ka].to(m.lora_A.device),
                                    _B_rows_layout(model, name, sub, norm[kb], False).to(m.lora_B.device))
                used.update((ka, kb))
                for km in (f"{base}.lora_magnitude_vector", f"{base}.lora_magnitude_vector.weight"):
                    if km in norm and getattr(m, "dora_magnitude", None) is not None:
                        r0, r1 = m.row_range(sub)
                        with torch.no_grad():
                            m.dora_magnitude[r0:r1].copy_(norm[km].reshape(-1))
                        used.add(km)
            elif strict:
                raise KeyError(f"adapter tensors for {base} are missing")
        m.refresh_shadows()
    if getattr(model, "token_rows", None) is not None:
        kt = "base_model.model.model.embed_tokens.token_adapter.trainable_tokens_delta"
        src = {k.replace(".default", ""): v for k, v in sd.items() if "trainable_tokens_delta" in k}
        if kt in src:
            with torch.no_grad():
                model.token_rows.copy_(src[kt])
            norm[kt] = src[kt]
            used.add(kt)
        elif strict:
            raise KeyError("adapter tensor for the trainable token rows is missing")
    if getattr(model, "embed_lora_At", None) is not None:
        ka = "base_model.model.model.embed_tokens.lora_embedding_A"
        kb = "base_model.model.model.embed_tokens.lora_embedding_B"
        norm.update({k.replace(".default", ""): v for k, v in sd.items() if "lora_embedding_" in k})
        if ka in norm and kb in norm:
            with torch.no_grad():
                model.embed_lora_At.copy_(norm[ka].t())
                model.embed_lora_B.copy_(norm[kb])
            used.update((ka, kb))
        elif strict:
            raise KeyError("adapter tensors for embed_tokens are missing")
    for name, m in model.named_modules():
        if isinstance(m, Experts) and m.lora is not None:
            base = f"base_model.model.model.{name}"
            for which in ("gate_up", "down"):
                for ab in ("A", "B"):
                    k = f"{base}.{which}_proj.lora_{ab}.weight"
                    if k in norm:
                        with torch.no_grad():
                            m.lora[f"{which}_{ab}"].copy_(norm[k])
                        used.add(k)
                    elif strict:
                        raise KeyError(f"adapter tensor {k} is missing")
    from ..ops.grouped import bump_param_epoch

    bump_param_epoch()   # cached operand copies of expert adapters are stale
    unused = set(norm) - used
    if strict and unused:
        raise KeyError(f"unexpected adapter tensors: {sorted(unused)[:5]} ...")
    return unused


def save_adapter(model, spec: LoraSpec, out_dir: str):
    from ..io.safetensors_io import save_file

    os.makedirs(out_dir, exist_ok=True)
    sd = {k: v.to("cpu").contiguous() for k, v in get_peft_state_dict(model).items()}
    save_file(sd, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    spec.save(out_dir)


def load_adapter(model, adapter_dir: str, strict: bool = True) -> LoraSpec:
    from ..io.safetensors_io import load_file

    spec = LoraSpec.load(adapter_dir)
    sd = load_file(os.path.join(adapter_dir, "adapter_model.safetensors"))
    set_peft_state_dict(model, sd, strict=strict)
    return spec


@torch.no_grad()
def merge_and_unload(model):
    """Folds every adapter into its base weight (W += s * B A) and removes the adapters."""
    if getattr(model, "embed_lora_At", None) is not None:
        model.merge_embedding_lora_()
    if getattr(model, "token_rows", None) is not None:
        model.merge_trainable_tokens_()
    for _, m in model.fused_linears():
        if getattr(m, "mora_M", None) is not None:
            m.merge_mora_()
            m.mora_M, m.mora_names = None, []
        if m.lora_A is not None:
            m.merge_lora_()
            m.lora_A = m.lora_B = m.lora_A16 = m.lora_B16 = None
            m.lora_blocks, m.lora_names, m.merged = (), [], False
    for m in model.modules():
        if isinstance(m, Experts) and m.lora is not None:
            if m.nvfp4 is not None:
                raise NotImplementedError("merge into NVFP4 experts goes through io.merge (requantising writer)")
            r = m.lora_r
            for e in range(m.E):
                for which, W in (("gate_up", m.gate_up_proj), ("down", m.down_proj)):
                    A, B = m.expert_lora(which, e)
                    W[e].copy_((W[e].float() + m.scaling * (B.float() @ A.float())).to(W.dtype))
            m.lora = None
    return model
