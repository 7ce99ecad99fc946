"""Cross-field validation rules (the semantics of the reference's validator mixins,
src/axolotl/utils/schemas/validation.py:26-1916 and config.py:1760-2211, restated for this
framework). Each rule raises ``ValueError`` with an actionable message or rewrites deprecated
spellings in place; warnings are returned as strings."""
from __future__ import annotations

import os


def validate(cfg: dict, capabilities: dict | None = None) -> list[str]:
    from .rules import run_rules

    w: list[str] = run_rules(cfg)
    cap = capabilities or {}
    g = cfg.get

    # ---- deprecated / remapped spellings
    if g("evaluation_strategy") and not g("eval_strategy"):
        cfg["eval_strategy"] = cfg.pop("evaluation_strategy")
        w.append("`evaluation_strategy` is deprecated, use `eval_strategy`")
    if g("sequence_parallel_degree") and not g("context_parallel_size"):
        cfg["context_parallel_size"] = cfg.pop("sequence_parallel_degree")
        w.append("`sequence_parallel_degree` is deprecated, use `context_parallel_size`")
    if g("include_tokens_per_second") is not None and g("include_tkps") is None:
        cfg["include_tkps"] = cfg["include_tokens_per_second"]
    if g("dataset_processes") and not g("dataset_num_proc"):
        cfg["dataset_num_proc"] = cfg.pop("dataset_processes")
    if g("noisy_embedding_alpha") and not g("neftune_noise_alpha"):
        cfg["neftune_noise_alpha"] = cfg.pop("noisy_embedding_alpha")
    if g("max_packed_sequence_len"):
        raise ValueError("`max_packed_sequence_len` was removed; use `sample_packing: true` with `sequence_len`")
    if g("rl_beta") is not None and g("dpo_beta") is None:
        cfg["dpo_beta"] = cfg["rl_beta"]
    for legacy, impl in (("flash_attention", "flash_attention_2"), ("sdp_attention", "sdpa"),
                         ("eager_attention", "eager"), ("flex_attention", "flex_attention")):
        if g(legacy):
            if g("attn_implementation") and g("attn_implementation") != impl:
                raise ValueError(f"`{legacy}: true` conflicts with `attn_implementation: {g('attn_implementation')}`")
            cfg["attn_implementation"] = impl
    if g("fsdp") and not g("fsdp_config"):
        w.append("`fsdp` list without `fsdp_config`: defaults are used")
    if g("fsdp_config") and not g("fsdp_version") and (g("fsdp_config") or {}).get("fsdp_version"):
        cfg["fsdp_version"] = cfg["fsdp_config"]["fsdp_version"]

    # ---- model source
    if not g("base_model") and not g("model_preset"):
        raise ValueError("`base_model` (an HF model directory) or `model_preset` is required")

    # ---- batch arithmetic
    if g("gradient_accumulation_steps") and g("batch_size"):
        raise ValueError("set only one of `gradient_accumulation_steps` and `batch_size`")
    if g("batch_size"):
        w.append("`batch_size` is not recommended; set `gradient_accumulation_steps` (and `micro_batch_size`)")
    if g("micro_batch_size") is not None and g("micro_batch_size") < 1:
        raise ValueError("`micro_batch_size` must be >= 1")
    if g("eval_batch_size") and g("eval_sample_packing") is False and g("sample_packing") \
            and g("eval_batch_size") != g("micro_batch_size"):
        w.append("eval_batch_size != micro_batch_size with packing on train only: eval batches are unpacked")

    # ---- precision
    if g("bf16") and g("fp16"):
        raise ValueError("`bf16` and `fp16` are mutually exclusive")
    if g("fp16") or g("float16"):
        raise ValueError("fp16 training is not supported: the tensor-core kernels are bf16 (set `bf16: true`)")
    if g("bf16") is True and cap.get("bf16") is False:
        raise ValueError("`bf16: true` but this device has no bf16 support")
    if g("tf32") is True and cap.get("tf32") is False:
        raise ValueError("`tf32: true` but this device has no tf32 support")

    # ---- adapters
    ad = g("adapter")
    if ad == "mora":
        if g("load_in_4bit") or g("load_in_8bit") or g("gptq"):
            raise ValueError("adapter: mora currently requires a full-precision base model. "
                             "Use adapter: lora or qlora for quantized training.")
        if (g("tensor_parallel_size") or 1) > 1:
            raise ValueError("adapter: mora cannot be combined with tensor parallelism")
    if ad in ("lora", "qlora", "mora"):
        if not g("lora_r"):
            raise ValueError("`lora_r` is required with `adapter: lora`")
        if g("lora_alpha") is None and ad != "mora":
            raise ValueError("`lora_alpha` is required with `adapter: lora`")
        if not (g("lora_target_modules") or g("lora_target_linear") or g("lora_target_parameters")):
            raise ValueError("no LoRA targets: set `lora_target_linear: true`, `lora_target_modules` or `lora_target_parameters`")
    if ad == "qlora":
        if not g("load_in_4bit") and not g("expert_weights_nvfp4"):
            raise ValueError("`adapter: qlora` requires `load_in_4bit: true`")
        if g("merge_lora"):
            raise ValueError("cannot merge a LoRA into a 4-bit base in place; run `merge-lora` on the bf16 checkpoint")
    if g("load_in_4bit") and ad != "qlora":
        raise ValueError("`load_in_4bit` without `adapter: qlora` is not supported")
    if g("load_in_4bit") and (g("tensor_parallel_size") or 1) > 1:
        raise ValueError("NF4 base weights cannot be combined with tensor parallelism")
    if ad == "llama-adapter":
        raise ValueError("`adapter: llama-adapter` is not supported")
    if g("lora_dropout") and (g("lora_mlp_kernel") or g("lora_qkv_kernel") or g("lora_o_kernel")):
        w.append("lora_dropout > 0: the fused LoRA K-extension path is replaced by the two-GEMM path during training")
    if g("unfrozen_parameters") and ad:
        w.append("`unfrozen_parameters` together with an adapter: listed base parameters are trained in bf16 with fp32 masters")
    if g("loraplus_lr_ratio") is not None and not ad:
        raise ValueError("`loraplus_lr_ratio` needs a LoRA adapter")

    # ---- data / packing
    if not g("datasets") and not g("pretraining_dataset") and not g("is_preprocess") and not g("test_datasets") \
            and not g("rl"):
        raise ValueError("no `datasets` (or `pretraining_dataset`) configured")
    if g("sample_packing") and g("group_by_length"):
        raise ValueError("`group_by_length` cannot be combined with `sample_packing`")
    if g("sample_packing") and g("attn_implementation") in ("eager",):
        raise ValueError("sample packing needs a varlen attention path; `eager` attention cannot isolate packed documents")
    if g("sample_packing") and g("pad_to_sequence_len") is None:
        cfg["pad_to_sequence_len"] = True
    if g("eval_sample_packing") is None and g("sample_packing"):
        cfg["eval_sample_packing"] = True if (g("val_set_size") or g("test_datasets")) else None
    if g("val_set_size") and g("test_datasets"):
        raise ValueError("`val_set_size` and `test_datasets` are mutually exclusive")
    if g("pretraining_dataset") and not g("max_steps"):
        raise ValueError("`max_steps` is required with a streaming `pretraining_dataset`")
    if g("streaming") and g("sample_packing") and not g("pretrain_multipack_attn", True):
        w.append("streaming packing without pretrain_multipack_attn lets documents attend across boundaries")
    if g("use_pose") and not g("sample_packing"):
        w.append("PoSE is usually combined with sample packing")
    if g("curriculum_sampling") and g("shuffle_merged_datasets", True):
        w.append("curriculum_sampling keeps dataset order only if `shuffle_merged_datasets: false`")
    if g("sequence_len") and g("sequence_len") % 8:
        w.append("sequence_len is not a multiple of 8; rows are padded to a multiple of 64 anyway")

    # ---- schedule
    if g("warmup_steps") is not None and g("warmup_ratio") is not None:
        raise ValueError("set only one of `warmup_steps` and `warmup_ratio`")
    if g("save_steps") and g("saves_per_epoch"):
        raise ValueError("set only one of `save_steps` and `saves_per_epoch`")
    if g("eval_steps") and g("evals_per_epoch"):
        raise ValueError("set only one of `eval_steps` and `evals_per_epoch`")
    if g("save_strategy") == "epoch" and g("save_steps"):
        raise ValueError("`save_strategy: epoch` conflicts with `save_steps`")
    if g("eval_strategy") == "no" and g("eval_steps"):
        raise ValueError("`eval_strategy: no` conflicts with `eval_steps`")
    if g("load_best_model_at_end") and g("save_strategy") and g("eval_strategy") \
            and g("save_strategy") != g("eval_strategy"):
        raise ValueError("`load_best_model_at_end` needs matching save and eval strategies")
    if g("early_stopping_patience") and not (g("eval_steps") or g("evals_per_epoch")):
        raise ValueError("`early_stopping_patience` needs periodic evaluation (`eval_steps`/`evals_per_epoch`)")
    if g("lr_scheduler") == "one_cycle" and g("warmup_steps"):
        w.append("one_cycle ignores warmup_steps")

    # ---- optimizer
    opt = (g("optimizer") or "adamw_torch_fused").lower()
    if opt in ("adamw_bnb_8bit", "adamw_8bit", "paged_adamw_8bit", "paged_adamw_32bit", "lion_8bit", "ao_adamw_8bit",
               "ao_adamw_4bit", "ao_adamw_fp8"):
        raise ValueError(f"optimizer '{opt}' needs bitsandbytes/torchao, which are not available; use `adamw_torch_fused`")
    if opt in ("dion", "galore_adamw", "q_galore_adamw8bit", "optimi_adamw", "flash_adamw"):
        raise ValueError(f"optimizer '{opt}' is not implemented on axolotl_b200")

    # ---- parallelism
    tp, cp = g("tensor_parallel_size") or 1, g("context_parallel_size") or 1
    ep = g("expert_parallel_size") or 1
    world = int(g("world_size") or os.environ.get("WORLD_SIZE", 1))
    if cp > 1:
        if not g("sample_packing") and (g("micro_batch_size") or 1) != 1:
            w.append("context parallelism without packing: micro batches are flattened into one packed row")
        if g("sample_packing") and (g("micro_batch_size") or 1) != 1:
            raise ValueError("context parallelism with sample packing requires `micro_batch_size: 1`")
        if g("ring_attn_func") not in (None, "varlen_llama3", "batch_ring", "zigzag"):
            raise ValueError(f"unknown ring_attn_func '{g('ring_attn_func')}'")
    if tp > 1 and ep > 1:
        raise ValueError("expert parallelism cannot be combined with tensor parallelism")
    if world % (tp * cp * ep * (g("dp_replicate_size") or 1)) and world > 1:
        raise ValueError(f"world size {world} is not divisible by tp*cp*ep*dp_replicate")
    if g("fsdp_config") and (g("fsdp_version") or 2) == 1:
        w.append("FSDP1 semantics are served by the native sharding runtime (same as fsdp_version: 2)")
    if g("fsdp_config") and g("fsdp_config").get("offload_params"):
        raise ValueError("fsdp offload_params is not supported (180 GB HBM per GPU makes it unnecessary)")

    # ---- RL
    rl = g("rl")
    if rl and rl not in ("dpo", "ipo", "orpo", "kto", "simpo", "grpo", "gdpo", "ebft"):
        raise ValueError(f"unknown rl method '{rl}'")
    if rl == "ebft":
        eb = g("ebft")
        if not eb:
            raise ValueError("`ebft` config section is required when `rl: ebft` is set. "
                             "Add an `ebft:` section with at least `mode: structured`.")
        if (eb.get("mode") or "structured") not in ("structured", "strided"):
            raise ValueError(f"unknown ebft.mode '{eb.get('mode')}' (structured or strided)")
        if eb.get("embed_method") not in (None, "last_token", "mean_pooling", "completion_mean", "concat"):
            raise ValueError(f"unknown ebft.embed_method '{eb.get('embed_method')}'")
    if rl in ("grpo", "gdpo") and not (g("trl") or {}).get("reward_funcs"):
        raise ValueError(f"rl: {rl} needs trl.reward_funcs (dotted paths of reward functions)")
    if rl and g("sample_packing"):
        raise ValueError("sample packing is not supported for preference training")

    # ---- memory features
    if g("tiled_mlp"):
        w.append("tiled_mlp is implemented as sequence-chunked MLP evaluation inside each layer")
    return w
