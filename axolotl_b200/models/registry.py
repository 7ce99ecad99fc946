"""Per-architecture support descriptors.

One descriptor per ``model_type`` declares what the architecture can be combined with. A capability is
``Supported`` (verified), ``Unsupported(reason)`` (enabling it is a configuration error that cites the reason) or
``Experimental(note)`` (runs, warns once). ``validate_cfg`` checks a run's configuration against the descriptor
before any weight is loaded, so that a combination the graph cannot run fails with one clear message instead of a
``NotImplementedError`` from inside the first step. Out-of-tree architectures register their own descriptor with
``register_model_support`` (from a plugin or any imported module).

Reference counterpart: the ``model_support`` registry (Supported / Unsupported / Experimental declarations,
``check_capability`` and the ``validate_cfg`` hook: src/axolotl/model_support/base.py:18-130,
src/axolotl/model_support/registry.py:22-80).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Union

from ..utils.logging import get_logger

LOG = get_logger(__name__)


@dataclass(frozen=True)
class Supported:
    note: str = ""


@dataclass(frozen=True)
class Unsupported:
    reason: str = ""


@dataclass(frozen=True)
class Experimental:
    note: str = ""


Capability = Union[Supported, Unsupported, Experimental]
_WARNED = set()

# capability names
PACKING, LORA, QLORA = "sample_packing", "lora", "qlora"
TP, CP, EP = "tensor_parallel", "context_parallel", "expert_parallel"
NVFP4, KV_CACHE = "nvfp4_experts", "kv_cache_generation"


class ModelSupport:
    """Everything the framework needs to know about one architecture, in one place. Subclass, set the class
    attributes, register. A missing capability key means "no special knowledge": the generic path applies."""

    model_types: ClassVar[tuple] = ()
    is_multimodal: ClassVar[bool] = False
    capabilities: ClassVar[dict] = {}
    head_dims: ClassVar[tuple | None] = None      # widths with a tensor-core kernel (others take the blocked library path)
    notes: ClassVar[tuple] = ()

    def validate_cfg(self, cfg, model_cfg) -> None:
        """Model-specific checks; raise ValueError on a bad combination."""

    def pre_model_load(self, cfg) -> None: ...

    def post_model_load(self, cfg, model) -> None: ...


_REGISTRY: dict[str, ModelSupport] = {}


def register_model_support(cls):
    """Class decorator: registers the descriptor under each of its ``model_types`` (a later registration of the same
    type overrides the earlier one)."""
    if not cls.model_types:
        raise ValueError(f"{cls.__name__} must define `model_types`")
    inst = cls()
    for mt in cls.model_types:
        if mt in _REGISTRY:
            LOG.warning("overriding model support for %s with %s", mt, cls.__name__)
        _REGISTRY[mt] = inst
    return cls


def get_model_support(model_type: str | None) -> ModelSupport | None:
    return _REGISTRY.get(model_type) if model_type else None


def check_capability(support: ModelSupport | None, name: str, model_type: str | None, *, feature: str | None = None,
                     hint: str = "") -> None:
    """Raise on ``Unsupported``, warn once on ``Experimental``; anything else passes."""
    cap = support.capabilities.get(name) if support is not None else None
    feature = feature or name
    if isinstance(cap, Unsupported):
        raise ValueError(f"{feature} is not supported for model_type={model_type}."
                         + (f" {cap.reason}" if cap.reason else "") + (f" {hint}" if hint else ""))
    if isinstance(cap, Experimental) and (feature, model_type) not in _WARNED:
        _WARNED.add((feature, model_type))
        LOG.warning("%s is experimental for model_type=%s.%s", feature, model_type, f" {cap.note}" if cap.note else "")


# ------------------------------------------------------------------------------------------- built-in descriptors
_NO_EP = Unsupported("Expert parallelism needs a mixture-of-experts architecture.")
_NO_NVFP4 = Unsupported("NVFP4 expert weights need a mixture-of-experts architecture.")
_DENSE = {EP: _NO_EP, NVFP4: _NO_NVFP4}
_MOE_NO_TP = Unsupported("The expert stacks are not sharded over a tensor-parallel group; use expert parallelism.")
_WIDE_NO_CP = Unsupported("The context-parallel attention kernels take head widths 64 and 128 only.")
_WIDE_NO_KV = Unsupported("The decode attention kernel takes head widths 64 and 128; generation recomputes the sequence.")
_MIXER_NO_TP = Unsupported("State-space / linear-attention mixers are not sharded over a tensor-parallel group.")
_MIXER_NO_KV = Unsupported("Recurrent-state decoding is not built; generation recomputes the sequence.")


def _register(name, types, caps, head_dims=(64, 128), notes=(), validate=None):
    body = {"model_types": tuple(types), "capabilities": dict(caps), "head_dims": head_dims, "notes": tuple(notes)}
    if validate is not None:
        body["validate_cfg"] = lambda self, cfg, mc: validate(cfg, mc)
    return register_model_support(type(name, (ModelSupport,), body))


_register("LlamaLike", ("llama", "qwen2", "qwen3", "seed_oss", "ernie4_5", "hunyuan_v1_dense"), _DENSE)
_register("Glm4Moe", ("glm4_moe", "minimax_m2", "hunyuan_v1_moe", "ernie4_5_moe"), {TP: _MOE_NO_TP})
_register("Afmoe", ("afmoe",), {TP: _MOE_NO_TP, KV_CACHE: Unsupported("The gated attention output is not part of the cached decode path; generation recomputes the sequence.")})
_register("GraniteMoe", ("granitemoe", "granitemoeshared"), {TP: _MOE_NO_TP})
_register("Glm", ("glm", "glm4"), {**_DENSE, TP: Unsupported("The checkpoint's fused gate|up projection is kept fused.")},
          notes=("rotary pairs stored as neighbours are permuted to the half-split layout at load and back at save",))
_register("Olmo2", ("olmo2", "olmo3"), {**_DENSE, TP: Unsupported("q / k norms span all heads of the unsharded projection.")},
          notes=("norms sit on the branch outputs; q / k RMSNorm over all heads runs as separate launches before RoPE",))
_register("LayerNormFamilies", ("nemotron", "starcoder2", "cohere", "cohere2", "olmo", "phi", "falcon"),
          {**_DENSE, TP: Unsupported("These graphs have no sharding rule here.")},
          notes=("mean-subtracting norms run the fused residual-add + LayerNorm kernel",))
_register("Arcee", ("arcee", "apertus"), {**_DENSE, TP: Unsupported("The ungated MLP has no sharding rule here.")})
_register("Mistral", ("mistral", "ministral", "ministral3"), _DENSE,
          notes=("sliding_window is applied by the attention kernels (not with context parallelism)",))
_register("Phi3", ("phi3",), {**_DENSE, TP: Unsupported("The checkpoint's fused projections are kept fused.")},
          notes=("longrope: the long factors apply when a document exceeds the original context",))
_register("Granite", ("granite",), _DENSE,
          notes=("embedding / attention / residual / logits multipliers are applied as scalar ops",))
_register("SmolLM3", ("smollm3",), _DENSE, notes=("layers listed in no_rope_layers run without rotary embedding",))
_MOE = {TP: _MOE_NO_TP}
_register("SparseMoE", ("qwen3_moe", "mixtral"), _MOE)
_register("OLMoE", ("olmoe",), _MOE, notes=("q / k RMSNorm over all heads runs as separate norm launches before RoPE",))
_register("Qwen2MoE", ("qwen2_moe",), _MOE,
          notes=("the shared expert is a dense MLP replicated on every expert-parallel rank",))
_register("Gemma", ("gemma", "gemma2", "gemma3_text"),
          {**_DENSE, CP: _WIDE_NO_CP, KV_CACHE: _WIDE_NO_KV, TP: Experimental("Checked on the Llama-style graphs only.")},
          head_dims=None,
          notes=("head width 256 and the tanh soft caps run through the wide-head attention kernels",))
_register("Gemma4", ("gemma4_text",),
          {**_DENSE, CP: _WIDE_NO_CP, KV_CACHE: _WIDE_NO_KV, TP: Unsupported("Layers differ in head width and key / value head count.")},
          head_dims=None,
          notes=("sliding layers (256-wide heads) run the wide-head attention kernels; global layers (512-wide heads) run the "
                 "blocked library path",
                 "per-layer input embeddings, the expert block beside the dense MLP (grouped tcgen05 GEMMs) and the layers "
                 "that attend an earlier layer's keys / values are built; the bidirectional (vision) attention mode is not"))
_register("GptOss", ("gpt_oss",),
          {TP: _MOE_NO_TP, CP: Unsupported("Attention sinks are not carried through the context-parallel kernels."),
           KV_CACHE: Unsupported("Attention sinks are not part of the decode kernel; generation recomputes the sequence."),
           NVFP4: Experimental("MXFP4 checkpoints are dequantised at load; NVFP4 re-quantisation of biased experts is unverified.")},
          notes=("attention sinks are applied as a rescale of the kernel's output and log-sum-exp",))
_LATENT = {TP: _MOE_NO_TP, CP: _WIDE_NO_CP, KV_CACHE: Unsupported("A latent-attention KV cache is not built; generation recomputes the sequence.")}
_register("Mistral4", ("mistral4",), {TP: _MOE_NO_TP, CP: Experimental("128-wide latent-attention heads take the context-parallel kernels; not exercised on ranks."),
                                     KV_CACHE: Unsupported("A latent-attention KV cache is not built; generation recomputes the sequence.")},
          notes=("latent attention with 128-wide q/k and v runs the standard varlen attention kernels",))
_register("DeepSeek", ("deepseek_v2", "deepseek_v3"), _LATENT, head_dims=None,
          notes=("latent attention expands k / v per head and runs the 192/128 wide-head kernels",))
_register("GlmMoeDsa", ("glm_moe_dsa",), _LATENT, head_dims=None,
          notes=("documents longer than index_topk take the dense-mask form of the selected-key attention",))
_register("Llama4Text", ("llama4_text",),
          {TP: _MOE_NO_TP, CP: Unsupported("Chunked attention layers are not available with context parallelism."),
           KV_CACHE: Unsupported("Chunked attention is not part of the decode kernel; generation recomputes the sequence.")})
_HYBRID = {TP: _MIXER_NO_TP, KV_CACHE: _MIXER_NO_KV,
           CP: Experimental("Mamba-2 layers hand their state and convolution halo across chunks; checked against the "
                            "single-rank scan on CPU ranks.")}
_register("GraniteHybrid", ("granitemoehybrid",), _HYBRID)
_register("Bamba", ("bamba",), {**_HYBRID, **_DENSE})
_register("NemotronH", ("nemotron_h",), {**_HYBRID, **_DENSE},
          notes=("blocks of type `moe` (latent, non-gated experts) are rejected when the config is read",))
_register("FalconH1", ("falcon_h1",), {**_HYBRID, **_DENSE})
_register("Lfm2Moe", ("lfm2_moe",), {TP: _MIXER_NO_TP, KV_CACHE: _MIXER_NO_KV})
_register("Lfm2", ("lfm2",), {**_DENSE, TP: _MIXER_NO_TP, KV_CACHE: _MIXER_NO_KV,
                             CP: Experimental("The convolution halo crosses chunk borders like the Mamba-2 one; not exercised on ranks.")})
_register("Qwen3Next", ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text"),
          {TP: _MIXER_NO_TP, KV_CACHE: _MIXER_NO_KV,
           CP: Unsupported("A Gated DeltaNet chunk's transition is a full matrix per head; its hand-over is not built.")},
          head_dims=None)

# architectures the reference lists that have no model graph here (named so that the error can say so)
KNOWN_UNSUPPORTED = ("deepseek_v4", "gpt_neox", "mamba", "jamba", "mllama", "qwen2_vl", "qwen3_vl", "kimi_linear", "gemmoe")


def support_for(model_type: str) -> ModelSupport:
    sup = get_model_support(model_type)
    if sup is None:
        hint = " (the reference supports it; this framework has no model graph for it)" if model_type in KNOWN_UNSUPPORTED else ""
        raise ValueError(f"model_type '{model_type}' is not supported{hint}; supported: {sorted(_REGISTRY)}")
    return sup


def validate_cfg(cfg, model_cfg) -> list[str]:
    """Raises on combinations the architecture cannot run; returns informational notes."""
    mt = model_cfg.model_type
    sup = support_for(mt)
    g = cfg.get
    moe = bool(getattr(model_cfg, "num_experts", 0))
    if (g("tensor_parallel_size") or 1) > 1:
        check_capability(sup, TP, mt, feature="tensor parallelism")
    if (g("context_parallel_size") or 1) > 1:
        check_capability(sup, CP, mt, feature="context parallelism")
    ep = g("expert_parallel_size") or 1
    if ep > 1:
        if not moe:
            raise ValueError(f"expert parallelism needs a mixture-of-experts model, not this '{mt}' configuration")
        check_capability(sup, EP, mt, feature="expert parallelism")
        if model_cfg.num_experts % ep:
            raise ValueError(f"{model_cfg.num_experts} experts cannot be split over expert_parallel_size={ep}")
    if g("expert_weights_nvfp4"):
        if not moe:
            raise ValueError(f"NVFP4 expert weights need a mixture-of-experts model, not this '{mt}' configuration")
        check_capability(sup, NVFP4, mt, feature="NVFP4 expert weights")
    if g("sample_packing"):
        check_capability(sup, PACKING, mt, feature="sample packing")
    if g("adapter") in ("lora", "qlora"):
        check_capability(sup, QLORA if g("adapter") == "qlora" else LORA, mt, feature=g("adapter"))
    if (g("context_parallel_size") or 1) > 1 and model_cfg.head_dim not in (64, 128):
        raise ValueError(f"head_dim {model_cfg.head_dim}: the context-parallel attention kernels take head widths 64 and 128")
    sup.validate_cfg(cfg, model_cfg)
    return list(sup.notes)
