"""Model configuration: a single dataclass covering the decoder-only families we own
(Llama / Mistral / Qwen2 / Qwen3 dense, Qwen3-MoE / Mixtral-style sparse), filled from a Hugging
Face ``config.json`` so checkpoints stay interchangeable with ``transformers``.

The reference resolves architectures through ``transformers.AutoConfig``
(src/axolotl/utils/config/__init__.py:259-372); we read the same file ourselves.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Any

SUPPORTED_MODEL_TYPES = ("llama", "mistral", "phi3", "qwen2", "qwen3", "qwen3_moe", "mixtral", "granite", "smollm3", "qwen2_moe", "olmoe",
                         "gemma", "gemma2", "gemma3_text", "deepseek_v2", "deepseek_v3", "gpt_oss", "granitemoehybrid", "llama4_text", "bamba", "nemotron_h", "qwen3_next", "falcon_h1", "glm_moe_dsa",
                         "glm", "glm4", "olmo2", "olmo3", "seed_oss", "arcee", "glm4_moe", "ernie4_5", "hunyuan_v1_dense",
                         "granitemoe", "granitemoeshared", "nemotron", "starcoder2", "cohere", "cohere2", "ministral", "ministral3", "qwen3_5_text", "qwen3_5_moe_text", "minimax_m2",
                         "hunyuan_v1_moe", "ernie4_5_moe", "apertus", "lfm2", "lfm2_moe", "mistral4", "olmo", "phi", "afmoe", "gemma4_text", "falcon")
GEMMA_TYPES = ("gemma", "gemma2", "gemma3_text")
MLA_TYPES = ("deepseek_v2", "deepseek_v3", "glm_moe_dsa", "mistral4")      # multi-head latent attention
GRANITE_MOE_TYPES = ("granitemoe", "granitemoeshared", "granitemoehybrid")
QWEN3_NEXT_TYPES = ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text")   # Gated DeltaNet hybrids
ZERO_CENTERED_NORM_TYPES = GEMMA_TYPES + QWEN3_NEXT_TYPES     # RMSNorm weights stored as w, applied as 1 + w


@dataclass
class ModelConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int | None = None
    head_dim: int | None = None
    hidden_act: str = "silu"
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    attention_bias: bool = False
    mlp_bias: bool = False
    tie_word_embeddings: bool = False
    initializer_range: float = 0.02
    qk_norm: bool = False  # Qwen3: per-head RMSNorm on q and k before RoPE
    # sparse MoE (qwen3_moe / mixtral)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    decoder_sparse_step: int = 1
    mlp_only_layers: list = field(default_factory=list)
    bos_token_id: int | None = None
    eos_token_id: Any = None
    pad_token_id: int | None = None
    torch_dtype: str = "bfloat16"
    architectures: list = field(default_factory=list)
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.model_type in ("qwen3", "qwen3_moe"):
            self.qk_norm = True
        if self.model_type in ("qwen2", "qwen2_moe"):
            self.attention_bias = True
        if self.model_type in ("gemma3_text", "gemma4_text", "olmo2", "olmo3", "minimax_m2") + QWEN3_NEXT_TYPES:
            self.qk_norm = True

    # ------------------------------------------------------------------ HF interchange
    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        d = dict(d)
        mt = d.get("model_type", "llama")
        if mt == "llava" and isinstance(d.get("text_config"), dict):    # image front end + one of the causal graphs
            wrapper = {k: d[k] for k in ("vision_config", "vision_feature_layer", "vision_feature_select_strategy",
                                         "projector_hidden_act", "multimodal_projector_bias", "image_seq_length") if k in d}
            wrapper["image_token_id"] = d.get("image_token_id", d.get("image_token_index", 32000))
            wrapper["model_type"] = "llava"
            d = dict(d["text_config"], vision_wrapper=wrapper)
            d.setdefault("model_type", "llama")
            mt = d["model_type"]
        if mt == "gemma3" and isinstance(d.get("text_config"), dict):   # the multimodal wrapper: its language model
            wrapper = None
            if isinstance(d.get("vision_config"), dict) and d["vision_config"].get("hidden_size"):   # + SigLIP tower and projector
                wrapper = {k: d[k] for k in ("vision_config", "mm_tokens_per_image", "boi_token_index", "eoi_token_index") if k in d}
                wrapper["image_token_id"] = d.get("image_token_index", d.get("image_token_id", 262144))
                wrapper["model_type"] = "gemma3"
            d = dict(d["text_config"], model_type="gemma3_text")
            if wrapper:
                d["vision_wrapper"] = wrapper
            mt = "gemma3_text"
        if mt == "gemma4" and isinstance(d.get("text_config"), dict):      # the multimodal wrapper: its language model
            d = dict(d["text_config"], model_type="gemma4_text")
            mt = "gemma4_text"
        if mt == "gemma4_text":
            # sliding layers: 256-wide heads, plain rope; global layers: `global_head_dim`-wide heads, a quarter of the
            # angle pairs rotate; weights of the norms are plain scales; scores are not scaled; values are RMS-normalised
            L = d.get("num_hidden_layers", 0)
            d.setdefault("tie_word_embeddings", True)
            d["hidden_act"] = d.get("hidden_activation") or "gelu_pytorch_tanh"
            d.setdefault("rms_norm_eps", 1e-6)
            d.setdefault("head_dim", 256)
            d.setdefault("global_head_dim", 512)
            d.setdefault("sliding_window", 512)
            if not d.get("layer_types"):
                d["layer_types"] = ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(L)]
            d["layer_types"] = list(d["layer_types"][:-1]) + ["full_attention"] if L else []
            if not isinstance(d.get("rope_parameters"), dict) or "full_attention" not in d["rope_parameters"]:
                d["rope_parameters"] = {"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                        "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1000000.0}}
            d["rope_theta"] = d["rope_parameters"]["sliding_attention"].get("rope_theta", 10000.0)
            if d.get("hidden_size_per_layer_input") is None:
                d["hidden_size_per_layer_input"] = 256
            d.setdefault("vocab_size_per_layer_input", d.get("vocab_size"))
            if d.get("enable_moe_block"):     # the expert block runs BESIDE the dense MLP of every layer: kept out of the generic MoE switches
                d["g4_experts"] = {"num_experts": int(d["num_experts"]), "top_k": int(d["top_k_experts"]),
                                   "intermediate": int(d["moe_intermediate_size"])}
            d["num_experts"] = 0
            if d.get("use_bidirectional_attention"):
                raise ValueError("gemma4_text: use_bidirectional_attention is not supported")
        if mt in GEMMA_TYPES:
            d.setdefault("tie_word_embeddings", True)
            d["hidden_act"] = d.get("hidden_activation") or "gelu_pytorch_tanh"   # HF forces the tanh form
            d.setdefault("rms_norm_eps", 1e-6)
            if mt == "gemma3_text":
                # checkpoints write only what differs from the architecture's defaults (the 4B config gives four keys)
                for key, val in (("vocab_size", 262208), ("hidden_size", 2304), ("intermediate_size", 9216), ("num_hidden_layers", 26),
                                 ("num_attention_heads", 8), ("num_key_value_heads", 4), ("max_position_embeddings", 131072),
                                 ("rope_theta", 1000000.0), ("rope_local_base_freq", 10000.0)):
                    d.setdefault(key, val)
                d.setdefault("head_dim", 256)
                d.setdefault("query_pre_attn_scalar", 256)
                d.setdefault("sliding_window", 4096)
                rp = d.get("rope_parameters")
                if isinstance(rp, dict) and "full_attention" in rp:        # transformers v5: one rope set per layer type
                    loc = rp.get("sliding_attention") or {}
                    d.setdefault("rope_local_base_freq", loc.get("rope_theta", 10000.0))
                    d["rope_parameters"] = rp["full_attention"]
            if mt == "gemma2":
                d.setdefault("head_dim", 256)
                d.setdefault("query_pre_attn_scalar", 256)
                d.setdefault("sliding_window", 4096)
                d.setdefault("attn_logit_softcapping", 50.0)
                d.setdefault("final_logit_softcapping", 30.0)
        if mt == "llama4" and isinstance(d.get("text_config"), dict):      # the multimodal wrapper: its language model
            d = dict(d["text_config"], model_type="llama4_text")
            mt = "llama4_text"
        if mt == "llama4_text":
            L = d.get("num_hidden_layers", 0)
            d["num_experts"] = d.get("num_local_experts") or 0
            d["moe_intermediate_size"] = d.get("intermediate_size") or 0          # routed and shared experts
            step = d.get("interleave_moe_layer_step") or 1
            moe_layers = d.get("moe_layers")
            if moe_layers is None:
                moe_layers = list(range(step - 1, L, step))
            d["mlp_only_layers"] = [i for i in range(L) if i not in set(moe_layers)]
            d["dense_intermediate_size"] = d.get("intermediate_size_mlp") or d.get("intermediate_size")
            if d.get("no_rope_layers") in (None, []):
                every = d.get("no_rope_layer_interval") or 4
                d["no_rope_layers"] = [int((i + 1) % every != 0) for i in range(L)]
            d.setdefault("rms_norm_eps", 1e-5)
        if mt in ("qwen3_5", "qwen3_5_moe") and isinstance(d.get("text_config"), dict):    # the multimodal wrapper: its language model
            d = dict(d["text_config"], model_type=mt + "_text")
            mt = d["model_type"]
        if mt in QWEN3_NEXT_TYPES:
            L = d.get("num_hidden_layers", 0)
            if not d.get("layer_types"):
                every = d.get("full_attention_interval") or 4
                d["layer_types"] = ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(L)]
            d.setdefault("partial_rotary_factor", 0.25)
            d.setdefault("norm_topk_prob", True)
        if mt == "nemotron_h":
            types = d.get("layers_block_type")
            if not types and d.get("hybrid_override_pattern"):          # "M" mamba, "*" attention, "-" MLP
                types = [{"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}[c] for c in d["hybrid_override_pattern"]]
            if not types:
                raise ValueError("nemotron_h: the config lists neither layers_block_type nor hybrid_override_pattern")
            if "moe" in types:
                raise ValueError("nemotron_h: blocks of type `moe` (latent, non-gated experts) are not supported")
            d["block_types"] = list(types)
            d["num_hidden_layers"] = len(types)
            d["rms_norm_eps"] = d.get("layer_norm_epsilon", 1e-5)
            d["hidden_act"] = d.get("mlp_hidden_act", "relu2")
        if mt == "bamba":
            if d.get("mamba_d_head") in (None, "auto"):
                d["mamba_d_head"] = int((d.get("mamba_expand") or 2) * d["hidden_size"]) // int(d.get("mamba_n_heads") or 128)
            rp = d.get("rope_parameters") or {}
            d.setdefault("partial_rotary_factor", rp.get("partial_rotary_factor", 0.5))
        if mt == "afmoe":              # Arcee Trinity: four norms, q / k norms, gated attention output, rope on sliding layers only
            L = d.get("num_hidden_layers", 0)
            d["qk_norm"] = True
            d.setdefault("head_dim", 128)
            d.setdefault("norm_topk_prob", True)
            d["mlp_only_layers"] = list(range(int(d.get("num_dense_layers") or 0)))
            if not d.get("layer_types"):
                every = d.get("global_attn_every_n_layers") or 4
                d["layer_types"] = ["full_attention" if (i + 1) % every == 0 else "sliding_attention" for i in range(L)]
            d["routed_scaling_factor"] = d.get("route_scale", 1.0)
            d["n_shared_experts"] = d.get("num_shared_experts") or 0
        if mt == "minimax_m2":         # q / k norms over all heads, sigmoid routing with a selection bias, no shared expert
            d["num_experts"] = d.get("num_local_experts") or 0
            d["moe_intermediate_size"] = d.get("intermediate_size") or 0
            d["norm_topk_prob"] = True
        if mt == "glm4_moe":           # Llama-style attention (optional per-head q/k norms, half of a head rotates) + DeepSeek-V3 routing
            d["num_experts"] = d.get("n_routed_experts") or 0
            d.setdefault("norm_topk_prob", True)
            d.setdefault("partial_rotary_factor", 0.5)
            d["qk_norm"] = bool(d.get("use_qk_norm", False))
            k1 = d.get("first_k_dense_replace") or 0
            d["mlp_only_layers"] = [i for i in range(d.get("num_hidden_layers", 0)) if i < k1]
        if mt == "ernie4_5":
            d["attention_bias"] = d["mlp_bias"] = bool(d.get("use_bias", False))
        if mt in ("hunyuan_v1_dense", "hunyuan_v1_moe"):
            d["qk_norm"] = True        # per head, AFTER the rotary embedding
        if mt == "hunyuan_v1_moe":     # softmax top-k routing renormalised, one always-on shared MLP of the same width
            if not isinstance(d.get("num_experts"), int) or not isinstance(d.get("moe_topk", 1), int):
                raise ValueError("hunyuan_v1_moe: per-layer expert counts / top-k lists are not supported")
            d["num_experts_per_tok"] = d.get("moe_topk") or 1
            d["moe_intermediate_size"] = d.get("intermediate_size") or 0
            d["norm_topk_prob"] = True
        if mt == "ernie4_5_moe":       # ERNIE attention; softmax scores, selection with a bias, ungated shared experts
            L = d.get("num_hidden_layers", 0)
            d["attention_bias"] = d["mlp_bias"] = bool(d.get("use_bias", False))
            d["num_experts"] = d.get("moe_num_experts") or 0
            d["num_experts_per_tok"] = d.get("moe_k") or 1
            d["norm_topk_prob"] = True
            start, every = d.get("moe_layer_start_index") or 0, d.get("moe_layer_interval") or 1
            end = d.get("moe_layer_end_index")
            end = L - 1 if end in (None, -1) else end
            d["mlp_only_layers"] = [i for i in range(L) if not ((i + 1) % every == 0 and start <= i <= end)]
        if mt == "lfm2_moe":           # LFM2 with routed experts after the first dense layers (sigmoid scores, selection bias)
            d["block_auto_adjust_ff_dim"] = False
            d["mlp_only_layers"] = list(range(int(d.get("num_dense_layers") or 0)))
            d.setdefault("norm_topk_prob", True)
        if mt in ("lfm2", "lfm2_moe"):   # gated short convolutions beside a few attention layers (q / k norms per head)
            L = d.get("num_hidden_layers", 0)
            d["rms_norm_eps"] = d.get("norm_eps", 1e-5)
            d["qk_norm"] = True
            d.setdefault("tie_word_embeddings", True)
            if not d.get("layer_types"):
                full = set(d.get("full_attn_idxs") or range(L))
                d["layer_types"] = ["full_attention" if i in full else "conv" for i in range(L)]
            inter = d.get("intermediate_size") or d.get("block_ff_dim") or 0
            if d.get("block_auto_adjust_ff_dim", True):
                inter = int(2 * inter / 3)
                mult = d.get("block_ffn_dim_multiplier", 1.0)
                if mult is not None:
                    mo = int(d.get("block_multiple_of") or 256)
                    inter = mo * ((int(mult * inter) + mo - 1) // mo)
            d["mlp_width"] = inter
        if mt == "apertus":            # q / k norms per head, ungated MLP with the learnable xIELU activation
            d["qk_norm"] = True
            d.setdefault("hidden_act", "xielu")
        if mt in GRANITE_MOE_TYPES:
            d["num_experts"] = d.get("num_local_experts") or 0
            d["moe_intermediate_size"] = d.get("intermediate_size") or 0     # width of a routed expert
            d.setdefault("norm_topk_prob", True)
            if not d.get("layer_types") and d.get("layers_block_type"):
                d["layer_types"] = d["layers_block_type"]
        if mt == "gpt_oss":
            d["num_experts"] = d.get("num_local_experts") or 0
            d["moe_intermediate_size"] = d.get("intermediate_size") or 0
            d["hidden_act"] = "gpt_oss_swiglu"        # g * sigmoid(1.702 g) * (up + 1), both branches clamped
            d.setdefault("swiglu_limit", 7.0)
            d.setdefault("attention_bias", True)
            d.setdefault("sliding_window", 128)
            if not d.get("rope_scaling") and not d.get("rope_parameters"):     # the family's default: YaRN x32 over 4096
                d["rope_scaling"] = {"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                     "truncate": False, "original_max_position_embeddings": 4096}
        if mt in ("glm", "glm4"):      # half of every head rotates, pairs stored as neighbours; fused gate|up; q/k/v biases
            d.setdefault("partial_rotary_factor", 0.5)
            d.setdefault("attention_bias", True)
            d.setdefault("rms_norm_eps", 1.5625e-07)
        if mt in ("olmo2", "olmo3"):   # norms on the branch OUTPUTS only, q/k norms over all heads
            d["qk_norm"] = True
            d.setdefault("rms_norm_eps", 1e-5)
            if mt == "olmo3" and not d.get("layer_types"):
                L = d.get("num_hidden_layers", 0)
                d["layer_types"] = ["sliding_attention" if (i + 1) % 4 else "full_attention" for i in range(L)]
        if mt == "seed_oss":
            d.setdefault("attention_bias", True)
            d.setdefault("attention_out_bias", False)
        if mt == "arcee":
            d.setdefault("hidden_act", "relu2")
        if mt == "olmo":               # LayerNorm without parameters, optional clamp of q / k / v
            d["rms_norm_eps"] = 1e-5
        if mt == "phi":                # one LayerNorm per layer, attention and MLP side by side, biases everywhere incl. the head
            d["rms_norm_eps"] = d.get("layer_norm_eps", 1e-5)
            d["attention_bias"] = d["mlp_bias"] = True
            d.setdefault("hidden_act", "gelu_new")
            d.setdefault("partial_rotary_factor", (d.get("rope_parameters") or {}).get("partial_rotary_factor", 0.5))
            if d.get("qk_layernorm"):
                raise ValueError("phi: qk_layernorm (per-head LayerNorm of q / k) is not supported")
        if mt == "falcon":             # LayerNorm, ungated GELU MLP, one fused query_key_value projection in three row layouts
            if d.get("alibi"):
                raise ValueError("falcon: ALiBi position biases (alibi: true) are not supported; the rotary checkpoints are")
            d.setdefault("num_attention_heads", d.get("n_head", 71))
            d.setdefault("num_hidden_layers", d.get("n_layer", 32))
            new = bool(d.get("new_decoder_architecture", False))
            d["new_decoder_architecture"] = new
            d.setdefault("multi_query", True)
            d.setdefault("parallel_attn", True)
            d["num_key_value_heads"] = (d.get("num_kv_heads") or d["num_attention_heads"]) if new \
                else (1 if d["multi_query"] else d["num_attention_heads"])
            if d.get("num_ln_in_parallel_attn") is None:
                d["num_ln_in_parallel_attn"] = 2 if new else 1
            d["intermediate_size"] = d.get("ffn_hidden_size") or 4 * d.get("hidden_size", 4544)
            d["rms_norm_eps"] = d.get("layer_norm_epsilon", 1e-5)
            d["attention_bias"] = d["mlp_bias"] = bool(d.get("bias", False))
            d["hidden_act"] = d.get("activation", "gelu")
            d.setdefault("tie_word_embeddings", True)
            d.setdefault("max_position_embeddings", 2048)
        if mt == "nemotron":           # LayerNorm with (1 + w) and bias, half of a head rotates, ungated squared-ReLU MLP
            d["rms_norm_eps"] = d.get("norm_eps", 1e-5)
            d.setdefault("partial_rotary_factor", 0.5)
            d.setdefault("hidden_act", "relu2")
        if mt == "starcoder2":         # LayerNorm with bias, ungated GELU MLP (c_fc / c_proj), biases everywhere
            d["rms_norm_eps"] = d.get("norm_epsilon", 1e-5)
            d["attention_bias"] = d["mlp_bias"] = bool(d.get("use_bias", True))
            d.setdefault("hidden_act", "gelu_pytorch_tanh")
            d.setdefault("tie_word_embeddings", True)
        if mt in ("cohere", "cohere2"):   # one mean-subtracting norm per layer, attention and MLP side by side, scaled logits
            d["rms_norm_eps"] = d.get("layer_norm_eps", 1e-5)
            d.setdefault("tie_word_embeddings", True)
            d.setdefault("logit_scale", 0.0625)
            if d.get("use_qk_norm"):
                raise ValueError(f"{mt}: use_qk_norm (per-head LayerNorm of q / k) is not supported")
            if mt == "cohere2" and not d.get("layer_types"):
                pat = d.get("sliding_window_pattern") or 4
                d["layer_types"] = ["sliding_attention" if (i + 1) % pat else "full_attention"
                                    for i in range(d.get("num_hidden_layers", 0))]
        if mt == "ministral3" and not d.get("rope_parameters") and not d.get("rope_scaling"):
            d["rope_parameters"] = {"rope_type": "yarn", "rope_theta": 1000000.0, "factor": 16.0, "original_max_position_embeddings": 16384,
                                    "beta_fast": 32.0, "beta_slow": 1.0, "mscale_all_dim": 1.0, "mscale": 1.0,
                                    "llama_4_scaling_beta": 0.1}
        if mt == "glm_moe_dsa":        # GLM-5: DeepSeek-V3 style latent attention + routing, plus the sparse-attention indexer
            L = d.get("num_hidden_layers", 0)
            for key, default in (("qk_nope_head_dim", 192), ("qk_rope_head_dim", 64), ("v_head_dim", 256), ("kv_lora_rank", 512),
                                 ("q_lora_rank", 2048), ("n_shared_experts", 1), ("routed_scaling_factor", 2.5), ("n_group", 1),
                                 ("topk_group", 1), ("index_topk", 2048), ("index_head_dim", 128), ("index_n_heads", 32)):
                d.setdefault(key, default)
            d["num_experts"] = d.get("n_routed_experts") or 0
            d.setdefault("norm_topk_prob", True)
            d["head_dim"] = d["qk_nope_head_dim"] + d["qk_rope_head_dim"]
            types = d.get("mlp_layer_types") or (["dense"] * min(3, L) + ["sparse"] * max(L - 3, 0))
            d["mlp_layer_types"] = list(types)
            d["mlp_only_layers"] = [i for i, t in enumerate(types) if t != "sparse"]
            d["rope_interleave"] = False                        # split-half rotation
        if mt == "mistral4":           # latent attention (128-wide q/k and v), position-scaled queries, softmax group routing
            for key, default in (("qk_nope_head_dim", 64), ("qk_rope_head_dim", 64), ("v_head_dim", 128), ("kv_lora_rank", 256),
                                 ("q_lora_rank", 1024), ("n_shared_experts", 1), ("routed_scaling_factor", 1.0), ("n_group", 1),
                                 ("topk_group", 1), ("rope_interleave", True)):
                d.setdefault(key, default)
            d.setdefault("num_experts_per_tok", 4)
            d.setdefault("norm_topk_prob", True)
            if not d.get("rope_parameters") and not d.get("rope_scaling"):
                d["rope_parameters"] = {"rope_type": "yarn", "rope_theta": 10000.0, "factor": 128.0,
                                        "original_max_position_embeddings": 8192, "beta_fast": 32.0, "beta_slow": 1.0,
                                        "mscale_all_dim": 1.0, "mscale": 1.0, "llama_4_scaling_beta": 0.1}
        if mt in ("deepseek_v2", "deepseek_v3", "mistral4"):
            d["num_experts"] = d.get("n_routed_experts") or 0
            d.setdefault("norm_topk_prob", mt == "deepseek_v3")
            d["head_dim"] = (d.get("qk_nope_head_dim") or 128) + (d.get("qk_rope_head_dim") or 64)
            k1 = d.get("first_k_dense_replace") or 0
            step = d.get("moe_layer_freq") or 1
            d["mlp_only_layers"] = [i for i in range(d.get("num_hidden_layers", 0)) if i < k1 or i % step]
            d["router_aux_loss_coef"] = d.get("aux_loss_alpha") or 0.0
        if mt not in SUPPORTED_MODEL_TYPES:
            raise ValueError(
                f"model_type '{mt}' is not supported by axolotl_b200 (supported: {SUPPORTED_MODEL_TYPES})")
        known = {f for f in cls.__dataclass_fields__ if f != "extra"}
        kw = {k: v for k, v in d.items() if k in known}
        if "rope_parameters" in d and isinstance(d["rope_parameters"], dict):  # transformers v5 layout
            rp = d["rope_parameters"]
            kw.setdefault("rope_theta", rp.get("rope_theta", 10000.0))
            if rp.get("rope_type", "default") != "default":
                kw["rope_scaling"] = rp
        if mt in ("qwen2_moe", "olmoe"):
            kw.setdefault("norm_topk_prob", False)      # the HF default of these families
        if mt == "olmoe":
            kw.setdefault("moe_intermediate_size", d.get("intermediate_size", 0))
        if mt == "mixtral":
            kw["num_experts"] = d.get("num_local_experts", 0)
            kw["moe_intermediate_size"] = d.get("intermediate_size", 0)
        if "torch_dtype" not in kw and "dtype" in d:
            kw["torch_dtype"] = d["dtype"]
        extra = {k: v for k, v in d.items() if k not in known}
        cfg = cls(**kw)
        cfg.extra = extra
        return cfg

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        f = os.path.join(path, "config.json") if os.path.isdir(path) else path
        with open(f) as fh:
            return cls.from_hf_dict(json.load(fh))

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        extra = d.pop("extra")
        d.pop("qk_norm")
        if self.model_type == "mixtral":
            d["num_local_experts"] = d.pop("num_experts")
        if self.model_type == "gpt_oss":
            d["num_local_experts"] = d.pop("num_experts")
            d["intermediate_size"] = d.pop("moe_intermediate_size")
            d["hidden_act"] = "silu"
        if self.model_type == "nemotron_h":
            d["layers_block_type"] = list(extra.get("block_types") or [])
            d["layer_norm_epsilon"] = d.get("rms_norm_eps", 1e-5)
            d["mlp_hidden_act"] = d.pop("hidden_act", "relu2")
        if self.model_type == "llama4_text":
            d["num_local_experts"] = d.pop("num_experts")
            d["intermediate_size"] = d.pop("moe_intermediate_size") or d.get("intermediate_size")
            d["intermediate_size_mlp"] = extra.get("dense_intermediate_size") or d["intermediate_size"]
            d["moe_layers"] = [i for i in range(self.num_hidden_layers) if i not in set(self.mlp_only_layers)]
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
        if self.model_type == "gemma4_text":      # rope settings live per layer type in rope_parameters only
            d.pop("rope_theta", None)
            d.pop("rope_scaling", None)
            d["hidden_activation"] = d.pop("hidden_act", "gelu_pytorch_tanh")
        if self.model_type == "falcon":
            d["layer_norm_epsilon"] = d.pop("rms_norm_eps", 1e-5)
            d["bias"] = bool(d.pop("attention_bias", False))
            d["activation"] = d.pop("hidden_act", "gelu")
            d["ffn_hidden_size"] = d.pop("intermediate_size")
            d["num_kv_heads"] = d.pop("num_key_value_heads")
            for k in ("mlp_bias", "head_dim", "rope_scaling"):
                d.pop(k, None)
            rt = d.pop("rope_theta", None)
            if rt and not extra.get("rope_parameters"):
                d["rope_parameters"] = {"rope_type": "default", "rope_theta": rt}
        if self.model_type == "afmoe":
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
            d.pop("norm_topk_prob", None)
            extra.pop("routed_scaling_factor", None)
            extra.pop("n_shared_experts", None)
        if self.model_type == "lfm2_moe":
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
        if self.model_type == "hunyuan_v1_moe":
            d["moe_topk"] = d.pop("num_experts_per_tok")
            d.pop("moe_intermediate_size", None)
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
        if self.model_type == "ernie4_5_moe":
            d["moe_num_experts"] = d.pop("num_experts")
            d["moe_k"] = d.pop("num_experts_per_tok")
            d["use_bias"] = bool(self.attention_bias)
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
        if self.model_type == "minimax_m2":
            d["num_local_experts"] = d.pop("num_experts")
            d["intermediate_size"] = d.pop("moe_intermediate_size") or d.get("intermediate_size")
        if self.model_type == "glm4_moe":
            d["n_routed_experts"] = d.pop("num_experts")
            d["use_qk_norm"] = bool(self.qk_norm)
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
        if self.model_type == "ernie4_5":
            d["use_bias"] = bool(self.attention_bias)
        if self.model_type in GRANITE_MOE_TYPES:
            d["num_local_experts"] = d.pop("num_experts")
            d["intermediate_size"] = d.pop("moe_intermediate_size") or extra.get("intermediate_size") or d.get("intermediate_size")
        if self.model_type == "glm_moe_dsa":
            extra.pop("rope_interleave", None)
        if self.model_type in MLA_TYPES:
            d["n_routed_experts"] = d.pop("num_experts")
            d.pop("head_dim", None)
            d.pop("mlp_only_layers", None)
            d.pop("decoder_sparse_step", None)
        if not self.num_experts:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                      "router_aux_loss_coef", "decoder_sparse_step", "mlp_only_layers"):
                d.pop(k, None)
        if self.model_type == "gemma4_text" and (g4 := extra.pop("g4_experts", None)):
            d.update(num_experts=g4["num_experts"], top_k_experts=g4["top_k"], moe_intermediate_size=g4["intermediate"], enable_moe_block=True)
        if not d.get("architectures"):
            d["architectures"] = [_ARCH_NAME[self.model_type]]
        out = dict(extra)
        out.update(d)
        if (vw := out.pop("vision_wrapper", None)):
            vw = dict(vw)
            if vw["model_type"] == "gemma3":
                vw["image_token_index"] = vw.pop("image_token_id")
                return {"model_type": vw.pop("model_type"), "architectures": ["Gemma3ForConditionalGeneration"],
                        "text_config": {k: v for k, v in out.items() if k != "architectures"},
                        "torch_dtype": out.get("torch_dtype", "bfloat16"), **vw}
            return {"model_type": vw.pop("model_type"), "architectures": ["LlavaForConditionalGeneration"],
                    "text_config": {k: v for k, v in out.items() if k != "architectures"},
                    "tie_word_embeddings": out.get("tie_word_embeddings", False), "torch_dtype": out.get("torch_dtype", "bfloat16"), **vw}
        return out

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as fh:
            json.dump(self.to_hf_dict(), fh, indent=2)

    # ------------------------------------------------------------------ derived
    def multiplier(self, name: str) -> float:
        """Granite's scalar multipliers (embedding / attention / residual / logits_scaling); 1 elsewhere
        (``attention_multiplier`` falls back to 1/sqrt(head_dim))."""
        if self.model_type == "gemma4_text":
            if name == "embedding_multiplier":
                import torch

                return float(torch.tensor(self.hidden_size ** 0.5, dtype=torch.bfloat16))
            return 1.0                                # (scores are not scaled: q / k are RMS-normalised)
        if self.model_type in GEMMA_TYPES:
            if name == "embedding_multiplier":      # sqrt(hidden) rounded to the activation dtype, as HF does
                import torch

                return float(torch.tensor(self.hidden_size ** 0.5, dtype=torch.bfloat16))
            if name == "attention_multiplier":
                qpas = (self.extra or {}).get("query_pre_attn_scalar")
                return float(qpas) ** -0.5 if qpas and self.model_type != "gemma" else 1.0 / math.sqrt(self.head_dim)
            return 1.0
        if self.model_type == "afmoe":
            if name == "embedding_multiplier" and (self.extra or {}).get("mup_enabled"):
                return float(self.hidden_size) ** 0.5
            return 1.0 / math.sqrt(self.head_dim) if name == "attention_multiplier" else 1.0
        if self.model_type in ("cohere", "cohere2"):
            if name == "logits_scaling":
                return 1.0 / float((self.extra or {}).get("logit_scale") or 1.0)
            return 1.0 / math.sqrt(self.head_dim) if name == "attention_multiplier" else 1.0
        if self.model_type == "falcon_h1":
            # maximal-update scalars: on the embeddings, on the keys (folded into the score scale: the rotary
            # embedding is linear), on the logits (a division elsewhere, hence the reciprocal)
            ex = self.extra or {}
            if name == "embedding_multiplier":
                return float(ex.get("embedding_multiplier") or 1.0)
            if name == "attention_multiplier":
                return float(ex.get("key_multiplier") or 1.0) / math.sqrt(self.head_dim)
            if name == "logits_scaling":
                return 1.0 / float(ex.get("lm_head_multiplier") or 1.0)
            return 1.0
        if self.model_type not in ("granite",) + GRANITE_MOE_TYPES:
            return 1.0 / math.sqrt(self.head_dim) if name == "attention_multiplier" else 1.0
        default = 1.0 / math.sqrt(self.head_dim) if name == "attention_multiplier" else 1.0
        v = (self.extra or {}).get(name)
        return float(v) if v is not None else default

    def norm_offset(self) -> float:
        """Gemma stores RMSNorm weights as ``w`` and applies ``1 + w``."""
        return 1.0 if self.model_type in ZERO_CENTERED_NORM_TYPES else 0.0

    def sandwich_norms(self) -> bool:
        """Gemma 2 / 3 and GLM-4 normalise the output of the attention and MLP branches too (four norms per layer)."""
        return self.model_type in ("gemma2", "gemma3_text", "gemma4_text", "glm4", "afmoe")

    def norm_kind(self) -> str:
        """"rms", or a mean-subtracting LayerNorm: with bias (StarCoder 2), stored as w - 1 with bias (Nemotron),
        weight only (Cohere)."""
        return {"starcoder2": "layernorm", "nemotron": "layernorm1p", "cohere": "layernorm_nobias", "phi": "layernorm", "falcon": "layernorm",
                "cohere2": "layernorm_nobias", "olmo": "layernorm_fixed"}.get(self.model_type, "rms")

    def parallel_block(self) -> bool:
        """Cohere: attention and MLP read the same normalised input and are added to the stream together."""
        if self.model_type == "falcon":
            ex = self.extra or {}
            return bool(ex.get("new_decoder_architecture") or ex.get("parallel_attn", True))
        return self.model_type in ("cohere", "cohere2", "phi")

    def falcon_qkv_rows(self):
        """Falcon stores one ``query_key_value`` projection. Row i of this graph's q | k | v block is row ``idx[i]`` of the
        checkpoint's: per key / value group [its queries, key, value] (new decoder architecture), [all queries, key, value]
        (multi-query), or per head [query, key, value]."""
        import torch

        Hq, Hk, D = self.num_attention_heads, self.num_key_value_heads, self.head_dim
        ex = self.extra or {}
        if ex.get("new_decoder_architecture"):
            G = Hq // Hk
            blk = torch.arange(Hk * (G + 2) * D).view(Hk, G + 2, D)
            return torch.cat([blk[:, :G].reshape(-1), blk[:, G].reshape(-1), blk[:, G + 1].reshape(-1)])
        if ex.get("multi_query", True):
            return torch.arange((Hq + 2) * D)
        blk = torch.arange(Hq * 3 * D).view(Hq, 3, D)
        return torch.cat([blk[:, 0].reshape(-1), blk[:, 1].reshape(-1), blk[:, 2].reshape(-1)])

    def post_norm_only(self) -> bool:
        """OLMo 2 / 3: no norm on a branch's input, one on its output."""
        return self.model_type in ("olmo2", "olmo3")

    def rope_pairs_interleaved(self) -> bool:
        """GLM checkpoints store the rotated part of every head with (real, imaginary) neighbours; the rows of q / k are
        permuted to the half-split layout at load (scores do not change when q and k share the permutation)."""
        return self.model_type in ("glm", "glm4", "ernie4_5", "ernie4_5_moe", "cohere", "cohere2")

    def attn_softcap(self) -> float:
        v = (self.extra or {}).get("attn_logit_softcapping") if self.model_type == "gemma2" else None
        return float(v) if v else 0.0

    def final_softcap(self) -> float:
        v = (self.extra or {}).get("final_logit_softcapping") if self.model_type in ("gemma2", "gemma3_text", "gemma4_text") else None
        return float(v) if v else 0.0

    def layer_head_dim(self, idx: int) -> int:
        """Gemma 4: full-attention layers have wider heads than sliding ones."""
        if self.model_type == "gemma4_text" and (self.extra or {})["layer_types"][idx] == "full_attention":
            return int((self.extra or {}).get("global_head_dim") or self.head_dim)
        return self.head_dim

    def layer_kv_heads(self, idx: int) -> int:
        ex = self.extra or {}
        if self.model_type == "gemma4_text" and ex.get("attention_k_eq_v") and ex["layer_types"][idx] == "full_attention":
            return int(ex.get("num_global_key_value_heads") or self.num_key_value_heads)
        return self.num_key_value_heads

    def layer_inv_freq(self, idx: int):
        """Gemma 4: (inverse frequencies of layer ``idx`` over ALL angle pairs of its head, or None). Global layers rotate
        only the first ``partial_rotary_factor`` of the pairs (i, i + D/2); the others get frequency 0."""
        if self.model_type != "gemma4_text":
            return None
        import torch

        ex = self.extra or {}
        kind = ex["layer_types"][idx]
        rp = (ex.get("rope_parameters") or {}).get(kind) or {}
        D = self.layer_head_dim(idx)
        theta, factor = float(rp.get("rope_theta", 10000.0)), float(rp.get("factor", 1.0))
        if rp.get("rope_type", "default") == "proportional":
            n = int(float(rp.get("partial_rotary_factor", 1.0)) * D // 2)
            inv = torch.zeros(D // 2, dtype=torch.float32)
            inv[:n] = 1.0 / (theta ** (torch.arange(0, 2 * n, 2, dtype=torch.float32) / D))
            return inv / factor
        return 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D)) / factor

    def local_rope_theta(self, idx: int) -> float | None:
        """Gemma 3: sliding-window layers rotate with their own base frequency and no scaling."""
        if self.model_type != "gemma3_text" or not self.sliding_window(idx):
            return None
        return float((self.extra or {}).get("rope_local_base_freq", 10000.0))

    def sliding_window(self, idx: int | None = None) -> int:
        """Causal sliding window in tokens of layer ``idx`` (0 = full attention). Mistral / Phi-3 /
        Mixtral checkpoints carry ``sliding_window`` for every layer; Qwen2 / Qwen3 / SmolLM3-style
        configs apply theirs only with ``use_sliding_window`` and only to the layers whose
        ``layer_types`` entry is ``sliding_attention`` (by default the layers from ``max_window_layers``
        upwards)."""
        ex = self.extra or {}
        w = ex.get("sliding_window")
        if not w:
            return 0
        if self.model_type in ("mistral", "phi3", "mixtral", "ministral3"):
            return int(w)
        if self.model_type == "gpt_oss":
            if idx is None:
                return int(w)
            types = ex.get("layer_types")
            return int(w) if (types[idx] == "sliding_attention" if types else idx % 2 == 0) else 0
        if self.model_type in ("gemma2", "gemma3_text"):
            if idx is None:
                return int(w)
            types = ex.get("layer_types")
            if types:
                return int(w) if types[idx] == "sliding_attention" else 0
            if self.model_type == "gemma2":
                return int(w) if idx % 2 == 0 else 0          # even layers slide
            pat = ex.get("sliding_window_pattern") or 6
            return int(w) if (idx + 1) % pat else 0           # every pat-th layer is global
        if self.model_type == "starcoder2":
            return int(w)
        if self.model_type in ("olmo3", "cohere2", "ministral", "afmoe", "gemma4_text"):
            types = ex.get("layer_types")
            if idx is None or not types:
                return int(w)
            return int(w) if types[idx] == "sliding_attention" else 0
        if self.model_type in ("qwen2", "qwen2_moe", "qwen3", "qwen3_moe", "smollm3"):
            if not ex.get("use_sliding_window"):
                return 0
            types = ex.get("layer_types")
            if idx is None:
                return int(w)
            if types:
                return int(w) if types[idx] == "sliding_attention" else 0
            return int(w) if idx >= (ex.get("max_window_layers") or 0) else 0
        return 0

    def layer_kind(self, idx: int) -> str:
        """"attention" or "mamba" (hybrid families list their layers in ``layer_types``)."""
        if self.model_type in ("lfm2", "lfm2_moe"):
            return "attention" if (self.extra or {})["layer_types"][idx] == "full_attention" else "shortconv"
        if self.model_type not in ("granitemoehybrid", "bamba", "nemotron_h") + QWEN3_NEXT_TYPES:
            return "attention"
        if self.model_type in QWEN3_NEXT_TYPES:
            return "deltanet" if (self.extra or {})["layer_types"][idx] == "linear_attention" else "attention"
        if self.model_type == "nemotron_h":
            return (self.extra or {})["block_types"][idx]          # "mamba" | "attention" | "mlp": one block per layer
        if self.model_type == "bamba":
            return "attention" if idx in set((self.extra or {}).get("attn_layer_indices") or []) else "mamba"
        types = (self.extra or {}).get("layer_types") or (self.extra or {}).get("layers_block_type")
        return "mamba" if types and types[idx] == "mamba" else "attention"

    def uses_rope(self, idx: int) -> bool:
        """SmolLM3 drops the rotary embedding in every layer whose ``no_rope_layers`` entry is 0; Granite 4.0-H
        attention layers carry no position signal unless ``position_embedding_type`` is ``rope``."""
        if self.model_type == "granitemoehybrid":
            return (self.extra or {}).get("position_embedding_type") == "rope"
        if self.model_type in ("granitemoe", "granitemoeshared"):
            return True
        if self.model_type in ("cohere2", "afmoe"):
            return (self.extra or {})["layer_types"][idx] == "sliding_attention"     # global layers carry no position signal
        if self.model_type == "nemotron_h":
            return False                                           # its attention blocks carry no position signal
        if self.model_type == "llama4_text":
            return bool((self.extra or {})["no_rope_layers"][idx])           # 1 = this layer rotates
        if self.model_type != "smollm3":
            return True
        ex = self.extra or {}
        flags = ex.get("no_rope_layers")
        if flags is None:
            every = ex.get("no_rope_layer_interval", 4)
            return (idx + 1) % every != 0
        return bool(flags[idx])

    def is_moe_layer(self, idx: int) -> bool:
        return (self.num_experts > 0 and idx not in self.mlp_only_layers
                and (idx + 1) % max(self.decoder_sparse_step, 1) == 0)

    def rope_dim(self) -> int:
        """Width of the rotated part of a head (DeepSeek latent attention rotates only its shared 64-wide part)."""
        if self.model_type in MLA_TYPES:
            return int((self.extra or {}).get("qk_rope_head_dim") or 64)
        ex = self.extra or {}
        f = ex.get("partial_rotary_factor") or (ex.get("rope_parameters") or {}).get("partial_rotary_factor") \
            or (self.rope_scaling or {}).get("partial_rotary_factor")
        if f and float(f) < 1.0:
            return int(self.head_dim * float(f))
        return self.head_dim

    def rope_inv_freq(self):
        """(inv_freq tensor [rope_dim/2] fp32, attention scaling factor) incl. the llama3, linear
        and yarn variants of ``rope_scaling``."""
        import torch

        D = self.rope_dim()
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        scale = 1.0
        rs = self.rope_scaling
        if rs:
            kind = rs.get("rope_type", rs.get("type", "default"))
            if kind == "linear":
                inv = inv / float(rs["factor"])
            elif kind == "llama3":
                factor, lo, hi = rs["factor"], rs.get("low_freq_factor", 1.0), rs.get("high_freq_factor", 4.0)
                old = rs.get("original_max_position_embeddings", 8192)
                wavelen = 2 * math.pi / inv
                smooth = (old / wavelen - lo) / (hi - lo)
                scaled = torch.where(wavelen > old / lo, inv / factor, inv)
                mid = (wavelen <= old / lo) & (wavelen >= old / hi)
                inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
            elif kind == "yarn":
                # NTK-by-parts (YaRN): high-frequency dimensions keep their wavelength, low-frequency ones
                # are interpolated by `factor`, with a linear ramp between the two correction dimensions;
                # cos / sin are scaled by the attention factor 0.1 ln(factor) + 1
                factor = float(rs["factor"])
                old = rs.get("original_max_position_embeddings") or self.max_position_embeddings
                beta_fast, beta_slow = rs.get("beta_fast") or 32.0, rs.get("beta_slow") or 1.0
                mscale, mscale_all = rs.get("mscale"), rs.get("mscale_all_dim")

                def get_mscale(f, m=1.0):
                    return 1.0 if f <= 1 else 0.1 * m * math.log(f) + 1.0

                if rs.get("attention_factor") is not None:
                    scale = float(rs["attention_factor"])
                elif mscale and mscale_all:
                    scale = get_mscale(factor, mscale) / get_mscale(factor, mscale_all)
                else:
                    scale = get_mscale(factor)

                def corr_dim(n_rot):
                    return (D * math.log(old / (n_rot * 2 * math.pi))) / (2 * math.log(self.rope_theta))

                low, high = corr_dim(beta_fast), corr_dim(beta_slow)
                if rs.get("truncate", True):
                    low, high = math.floor(low), math.ceil(high)
                low, high = max(low, 0), min(high, D - 1)
                if low == high:
                    high += 0.001
                ramp = ((torch.arange(D // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
                extrap = 1 - ramp
                inv = (inv / factor) * (1 - extrap) + inv * extrap
            elif kind == "longrope":
                # Phi-3 long context: per-dimension rescale factors, one set for sequences within the
                # original context (returned here) and one beyond it (``rope_inv_freq_long``)
                inv = inv / torch.tensor(rs["short_factor"], dtype=torch.float32)
                scale = self._longrope_attention_factor()
            elif kind in ("default", None):
                pass
            else:
                raise ValueError(f"rope_scaling type '{kind}' is not supported")
        return inv, scale

    def _longrope_orig(self) -> int:
        rs = self.rope_scaling or {}
        return int(rs.get("original_max_position_embeddings") or (self.extra or {}).get("original_max_position_embeddings")
                   or self.max_position_embeddings)

    def _longrope_attention_factor(self) -> float:
        rs = self.rope_scaling or {}
        if rs.get("attention_factor") is not None:
            return float(rs["attention_factor"])
        orig = self._longrope_orig()
        factor = rs.get("factor") or self.max_position_embeddings / orig
        return 1.0 if factor <= 1.0 else math.sqrt(1 + math.log(factor) / math.log(orig))

    def rope_inv_freq_long(self):
        """(inv_freq for documents longer than the original context, that context length) for the
        ``longrope`` scaling of Phi-3; None for every other configuration."""
        import torch

        rs = self.rope_scaling
        if not rs or rs.get("rope_type", rs.get("type")) != "longrope":
            return None
        D = self.head_dim
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        return inv / torch.tensor(rs["long_factor"], dtype=torch.float32), self._longrope_orig()

    def num_params(self, include_embeddings: bool = True) -> int:
        H, L, V = self.hidden_size, self.num_hidden_layers, self.vocab_size
        D, Hq, Hk = self.head_dim, self.num_attention_heads, self.num_key_value_heads
        attn = H * (Hq + 2 * Hk) * D + Hq * D * H
        n = 0
        for i in range(L):
            if self.is_moe_layer(i):
                mlp = self.num_experts * 3 * H * self.moe_intermediate_size + H * self.num_experts
            else:
                mlp = 3 * H * self.intermediate_size
            n += attn + mlp + 2 * H
        n += H
        if include_embeddings:
            n += V * H * (1 if self.tie_word_embeddings else 2)
        return n


_ARCH_NAME = {
    "llama": "LlamaForCausalLM",
    "mistral": "MistralForCausalLM",
    "phi3": "Phi3ForCausalLM",
    "qwen2": "Qwen2ForCausalLM",
    "qwen3": "Qwen3ForCausalLM",
    "qwen3_moe": "Qwen3MoeForCausalLM",
    "mixtral": "MixtralForCausalLM",
    "granite": "GraniteForCausalLM",
    "qwen2_moe": "Qwen2MoeForCausalLM",
    "olmoe": "OlmoeForCausalLM",
    "smollm3": "SmolLM3ForCausalLM",
    "gemma": "GemmaForCausalLM",
    "gemma2": "Gemma2ForCausalLM",
    "gemma3_text": "Gemma3ForCausalLM",
    "gemma4_text": "Gemma4ForCausalLM",
    "deepseek_v2": "DeepseekV2ForCausalLM",
    "deepseek_v3": "DeepseekV3ForCausalLM",
    "gpt_oss": "GptOssForCausalLM",
    "granitemoehybrid": "GraniteMoeHybridForCausalLM",
    "llama4_text": "Llama4ForCausalLM",
    "bamba": "BambaForCausalLM",
    "nemotron_h": "NemotronHForCausalLM",
    "falcon_h1": "FalconH1ForCausalLM",
    "glm_moe_dsa": "GlmMoeDsaForCausalLM",
    "glm": "GlmForCausalLM",
    "glm4": "Glm4ForCausalLM",
    "olmo2": "Olmo2ForCausalLM",
    "olmo3": "Olmo3ForCausalLM",
    "seed_oss": "SeedOssForCausalLM",
    "arcee": "ArceeForCausalLM",
    "glm4_moe": "Glm4MoeForCausalLM",
    "ernie4_5": "Ernie4_5ForCausalLM",
    "hunyuan_v1_dense": "HunYuanDenseV1ForCausalLM",
    "granitemoe": "GraniteMoeForCausalLM",
    "granitemoeshared": "GraniteMoeSharedForCausalLM",
    "nemotron": "NemotronForCausalLM",
    "starcoder2": "Starcoder2ForCausalLM",
    "cohere": "CohereForCausalLM",
    "cohere2": "Cohere2ForCausalLM",
    "minimax_m2": "MiniMaxM2ForCausalLM",
    "hunyuan_v1_moe": "HunYuanMoEV1ForCausalLM",
    "ernie4_5_moe": "Ernie4_5_MoeForCausalLM",
    "apertus": "ApertusForCausalLM",
    "lfm2": "Lfm2ForCausalLM",
    "mistral4": "Mistral4ForCausalLM",
    "olmo": "OlmoForCausalLM",
    "phi": "PhiForCausalLM",
    "falcon": "FalconForCausalLM",
    "afmoe": "AfmoeForCausalLM",
    "lfm2_moe": "Lfm2MoeForCausalLM",
    "ministral": "MinistralForCausalLM",
    "ministral3": "Ministral3ForCausalLM",
    "qwen3_next": "Qwen3NextForCausalLM",
    "qwen3_5_text": "Qwen3_5ForCausalLM",
    "qwen3_5_moe_text": "Qwen3_5MoeForCausalLM",
}


# Named architectures used by the benchmark configs (random-init, no download needed).
PRESETS = {
    "tiny-llama": dict(model_type="llama", vocab_size=32000, hidden_size=256, intermediate_size=688,
                       num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=2048),
    "llama-3-8b": dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                       rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=8192),
    "llama-3-70b": dict(model_type="llama", vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                        num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                        rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=8192),
    "qwen3-8b": dict(model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                     num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960),
    "qwen3-moe-30b-a3b": dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048,
                              intermediate_size=6144, moe_intermediate_size=768, num_hidden_layers=48,
                              num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                              num_experts=128, num_experts_per_tok=8, norm_topk_prob=True,
                              router_aux_loss_coef=0.001, rope_theta=1000000.0, rms_norm_eps=1e-6,
                              max_position_embeddings=40960),
    "tiny-gemma2": dict(model_type="gemma2", vocab_size=4096, hidden_size=256, intermediate_size=512,
                        num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
                        hidden_act="gelu_pytorch_tanh", rms_norm_eps=1e-6, tie_word_embeddings=True,
                        extra=dict(query_pre_attn_scalar=256, sliding_window=64, attn_logit_softcapping=50.0,
                                   final_logit_softcapping=30.0)),
    "tiny-gemma3": dict(model_type="gemma3_text", vocab_size=4096, hidden_size=256, intermediate_size=512,
                        num_hidden_layers=6, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
                        hidden_act="gelu_pytorch_tanh", rms_norm_eps=1e-6, tie_word_embeddings=True,
                        rope_theta=1000000.0,
                        extra=dict(query_pre_attn_scalar=256, sliding_window=64, rope_local_base_freq=10000.0,
                                   sliding_window_pattern=6)),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", vocab_size=4096, hidden_size=256, intermediate_size=512,
                           moe_intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=64, num_experts=8, num_experts_per_tok=2,
                           router_aux_loss_coef=0.001, rms_norm_eps=1e-6),
}


def preset(name: str, **overrides) -> ModelConfig:
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return ModelConfig(**kw)
