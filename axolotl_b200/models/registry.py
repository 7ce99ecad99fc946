"""Per-architecture capability declarations and checks.

One table says what each supported ``model_type`` can be combined with; ``validate_cfg`` turns a
mismatch into a clear configuration error before any weight is loaded. Reference counterpart: the
``model_support`` registry (per-arch Supported / Unsupported / Experimental declarations and the
``validate_cfg`` hook, src/axolotl/model_support/).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class ArchSupport:
    packing: bool = True              # multipack + varlen attention
    lora: bool = True
    qlora: bool = True
    tensor_parallel: bool = True
    context_parallel: bool = True
    expert_parallel: bool = False     # MoE families only
    nvfp4_experts: bool = False
    head_dims: tuple = (64, 128)      # what the attention kernels are built for
    notes: tuple = field(default_factory=tuple)


ARCHS = {
    "llama": ArchSupport(),
    "mistral": ArchSupport(notes=("sliding_window is applied by the attention kernels (not with context parallelism)",)),
    "phi3": ArchSupport(tensor_parallel=False, notes=("longrope: the long factors apply when a document exceeds the original context",)),
    "qwen2": ArchSupport(),
    "granite": ArchSupport(notes=("embedding / attention / residual / logits multipliers are applied as scalar ops",)),
    "smollm3": ArchSupport(notes=("layers listed in no_rope_layers run without rotary embedding",)),
    "qwen3": ArchSupport(),
    "qwen3_moe": ArchSupport(tensor_parallel=False, expert_parallel=True, nvfp4_experts=True),
    "mixtral": ArchSupport(tensor_parallel=False, expert_parallel=True, nvfp4_experts=True),
    "olmoe": ArchSupport(tensor_parallel=False, expert_parallel=True, nvfp4_experts=True,
                         notes=("q / k RMSNorm over all heads runs as separate norm launches before RoPE",)),
    "qwen2_moe": ArchSupport(tensor_parallel=False, expert_parallel=True, nvfp4_experts=True,
                             notes=("the shared expert is a dense MLP replicated on every expert-parallel rank",)),
}

# architectures the reference lists that have no model graph here (named so that the error can say so)
KNOWN_UNSUPPORTED = ("gemma", "gemma2", "gemma3", "gemma4", "deepseek_v2", "deepseek_v3", "deepseek_v4", "falcon",
                     "falcon_h1", "phi", "gpt_neox", "mamba", "jamba", "glm", "glm4", "glm_moe_dsa", "llama4", "mllama",
                     "qwen2_vl", "qwen3_vl", "qwen3_5", "qwen3_next", "nemotron_h", "granitemoehybrid", "kimi_linear",
                     "olmo", "olmo2", "cohere", "starcoder2", "bamba", "lfm2")


def support_for(model_type: str) -> ArchSupport:
    if model_type not in ARCHS:
        hint = " (the reference supports it; this framework has no model graph for it)" if model_type in KNOWN_UNSUPPORTED else ""
        raise ValueError(f"model_type '{model_type}' is not supported{hint}; supported: {sorted(ARCHS)}")
    return ARCHS[model_type]


def validate_cfg(cfg, model_cfg) -> list[str]:
    """Raises on combinations the architecture cannot run; returns informational notes."""
    sup = support_for(model_cfg.model_type)
    g = cfg.get
    if (g("tensor_parallel_size") or 1) > 1 and not sup.tensor_parallel:
        raise ValueError(f"tensor parallelism is not available for model_type '{model_cfg.model_type}'")
    if (g("context_parallel_size") or 1) > 1 and not sup.context_parallel:
        raise ValueError(f"context parallelism is not available for model_type '{model_cfg.model_type}'")
    if (g("expert_parallel_size") or 1) > 1 and not sup.expert_parallel:
        raise ValueError(f"expert parallelism needs a mixture-of-experts architecture, not '{model_cfg.model_type}'")
    if g("expert_weights_nvfp4") and not sup.nvfp4_experts:
        raise ValueError(f"NVFP4 expert weights need a mixture-of-experts architecture, not '{model_cfg.model_type}'")
    if g("sample_packing") and not sup.packing:
        raise ValueError(f"sample packing is not available for model_type '{model_cfg.model_type}'")
    if model_cfg.head_dim not in sup.head_dims:
        raise ValueError(f"head_dim {model_cfg.head_dim} is not supported by the attention kernels {sup.head_dims}")
    ep = g("expert_parallel_size") or 1
    if ep > 1 and model_cfg.num_experts % ep:
        raise ValueError(f"{model_cfg.num_experts} experts cannot be split over expert_parallel_size={ep}")
    return list(sup.notes)
