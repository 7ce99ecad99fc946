"""Table of cross-field config rules, one small function per rule.

Every entry restates one validator of the reference (src/axolotl/utils/schemas/validation.py:26-1916,
src/axolotl/utils/schemas/config.py:1760-2211); its name is the reference's so that the two can be read
side by side. A rule receives the raw config dict and either returns ``None``, returns a warning string,
rewrites the dict in place (deprecated spellings, derived defaults), or raises ``ValueError``. Rules
whose subject does not exist in this framework (DeepSpeed JSON rewriting, NPU, BetterTransformer) reject
the key itself in ``schema.UNSUPPORTED_KEYS`` and are not repeated here.
"""
from __future__ import annotations

from math import gcd

SUPPORTED_METRICS = {"sacrebleu", "comet", "ter", "chrf", "perplexity"}
RULES = []


def rule(fn):
    RULES.append(fn)
    return fn


def _adapter(c):
    return c.get("adapter") in ("lora", "qlora")


# ------------------------------------------------------------------------------- datasets
@rule
def check_deprecated_unsloth_fields(c):
    found = [f for f in ("unsloth_cross_entropy_loss", "unsloth_lora_mlp", "unsloth_lora_qkv", "unsloth_lora_o",
                         "unsloth_rms_norm", "unsloth_rope") if c.get(f)]
    if found:
        raise ValueError(f"`{'`, `'.join(found)}` {'has' if len(found) == 1 else 'have'} been removed. "
                         "Please use `lora_mlp_kernel`, `lora_qkv_kernel`, `lora_o_kernel` instead.")


@rule
def deprecate_sharegpt_datasets(c):
    for ds in c.get("datasets") or []:
        t = ds.get("type") if isinstance(ds, dict) else None
        if isinstance(t, str) and t.startswith("sharegpt"):
            raise ValueError("`type: sharegpt.*` is deprecated. Please use `type: chat_template` instead.")


@rule
def check_pretraining_streaming_deprecation(c):
    if c.get("pretraining_dataset") and not c.get("streaming"):
        return ("Setting `pretraining_dataset` without `streaming: true` is deprecated; streaming is enabled "
                "automatically for now")


@rule
def check_push_ds_auth(c):
    if c.get("push_dataset_to_hub") and c.get("hf_use_auth_token") is not True:
        raise ValueError("Require cfg.hf_use_auth_token to be True for push_dataset_to_hub")


@rule
def check_test_datasets_bench(c):
    if c.get("do_bench_eval") and not c.get("test_datasets") and not c.get("val_set_size"):
        raise ValueError("`do_bench_eval` needs a test dataset (`test_datasets` or `val_set_size`): there is no hub "
                         "access to fetch an empty placeholder dataset")


@rule
def check_eval_packing(c):
    if c.get("sample_packing") and c.get("eval_table_size") and c.get("eval_sample_packing") is not False:
        raise ValueError("eval_table_size and eval_sample_packing are not supported together with sample_packing. "
                         "Please set 'eval_sample_packing' to false.")
    if c.get("sample_packing") and c.get("eval_sample_packing") is False and c.get("remove_unused_columns") is None:
        c["remove_unused_columns"] = False


@rule
def check_mm_prepare(c):
    if c.get("skip_prepare_dataset") and c.get("remove_unused_columns") is None:
        c["remove_unused_columns"] = False


# ------------------------------------------------------------------------------- attention
@rule
def check_scaling_softmax_requires_flex(c):
    if c.get("scaling_softmax"):
        raise ValueError("scaling_softmax requires flex attention, which this framework does not provide "
                         "(attention always runs the varlen flash kernel)")


@rule
def check_attention_backend(c):
    impl = c.get("attn_implementation")
    if impl in ("xformers", "sage", "fp8", "flash_attention_3", "flash_attention_4"):
        return (f"attn_implementation: {impl} is served by the native varlen flash kernel "
                "(packed documents stay isolated)")
    if impl == "eager" and not c.get("sample_packing"):
        return "attn_implementation: eager is served by the native varlen flash kernel"


# ------------------------------------------------------------------------------- training
@rule
def check_batch_size_fields(c):
    fields = ("micro_batch_size", "gradient_accumulation_steps", "batch_size")
    if c.get("strict_batch_fields") and sum(1 for f in fields if c.get(f)) < 2:
        raise ValueError(f"At least two of {', '.join(fields)} must be set")


@rule
def hint_sample_packing_padding(c):
    if c.get("sample_packing") and c.get("pad_to_sequence_len") is False:
        return "`pad_to_sequence_len: true` is recommended when using sample_packing"


@rule
def hint_reward_model_pad(c):
    if c.get("reward_model") and not c.get("pad_to_sequence_len"):
        if c.get("pad_to_sequence_len") is None:
            c["pad_to_sequence_len"] = True
        return "`pad_to_sequence_len: true` is recommended when using reward_model"


@rule
def set_reward_model_defaults(c):
    if c.get("reward_model"):
        if c.get("num_labels") is None:
            c["num_labels"] = 1
        if not (c.get("type_of_model") or c.get("model_type")):
            c["model_type"] = "AutoModelForSequenceClassification"
    if c.get("process_reward_model"):
        if c.get("num_labels") is None:
            c["num_labels"] = 2
        if not (c.get("type_of_model") or c.get("model_type")):
            c["model_type"] = "AutoModelForTokenClassification"


@rule
def hint_eval_train_mbsz(c):
    if c.get("eval_batch_size") and c.get("micro_batch_size") and c.get("eval_batch_size") != c.get("micro_batch_size"):
        return "eval_batch_size != micro_batch_size. This can lead to VRAM instability."


@rule
def check_saves(c):
    if c.get("save_strategy") and c.get("save_steps") and c.get("save_strategy") != "steps":
        raise ValueError("save_strategy and save_steps mismatch. Please set save_strategy to 'steps' or remove save_steps.")


@rule
def check_push_save(c):
    if c.get("hub_model_id") and c.get("save_strategy") not in ("steps", "epoch", None):
        return "hub_model_id is set without any models being saved. To save a model, set save_strategy."


@rule
def check_evals(c):
    if c.get("eval_strategy") and c.get("eval_steps") and c.get("eval_strategy") != "steps":
        raise ValueError("eval_strategy and eval_steps mismatch. Please set eval_strategy to 'steps' or remove eval_steps.")
    if (c.get("val_set_size") == 0 and (c.get("eval_steps") or c.get("eval_strategy")) and not c.get("test_datasets")
            and c.get("eval_strategy") != "no"):
        raise ValueError("eval_steps and eval_strategy are not supported with val_set_size == 0")
    if c.get("evals_per_epoch") and c.get("eval_strategy") and c.get("eval_strategy") != "steps":
        raise ValueError("eval_strategy must be empty or set to `steps` when used with evals_per_epoch.")
    if c.get("do_bench_eval") and not (c.get("evals_per_epoch") or c.get("eval_steps")):
        raise ValueError("do_bench_eval requires evals_per_epoch or eval_steps to be set.")


@rule
def check_neftune(c):
    if c.get("noisy_embedding_alpha") and c.get("neftune_noise_alpha"):
        raise ValueError("noisy_embedding_alpha is deprecated, use neftune_noise_alpha; both are set, please remove the "
                         "deprecated noisy_embedding_alpha setting")
    if c.get("neftune_noise_alpha") is not None and c["neftune_noise_alpha"] <= 0.0:
        raise ValueError("neftune_noise_alpha must be > 0.0")


@rule
def check_multipack_buffer_size(c):
    if c.get("pretrain_multipack_buffer_size") and c.get("streaming_multipack_buffer_size"):
        raise ValueError("pretrain_multipack_buffer_size is deprecated, use streaming_multipack_buffer_size; both are set, "
                         "please remove the deprecated pretrain_multipack_buffer_size setting")
    if c.get("pretrain_multipack_buffer_size"):
        c["streaming_multipack_buffer_size"] = c.pop("pretrain_multipack_buffer_size")
        return "`pretrain_multipack_buffer_size` is deprecated. Use `streaming_multipack_buffer_size` instead."


@rule
def check_use_reentrant_mismatch(c):
    if c.get("unfrozen_parameters") and (c.get("gradient_checkpointing_kwargs") or {}).get("use_reentrant") is True:
        raise ValueError("`use_reentrant` must be false when used with partially frozen model.")


@rule
def check_causal_lm_evals(c):
    if c.get("do_causal_lm_eval") and c.get("eval_sample_packing"):
        raise ValueError("do_causal_lm_eval is enabled, eval_sample_packing must be set to False")
    m = c.get("eval_causal_lm_metrics")
    if m:
        if not isinstance(m, list):
            raise ValueError("eval_causal_lm_metrics must be a list")
        if set(m) - SUPPORTED_METRICS:
            raise ValueError(f"eval_causal_lm_metrics must be one of {sorted(SUPPORTED_METRICS)}")


@rule
def check_mistral_common_incompatible_options(c):
    if not c.get("tokenizer_use_mistral_common"):
        return
    raise ValueError("tokenizer_use_mistral_common needs the mistral-common package, which is not available here; "
                     "use the model's Hugging Face tokenizer files")


@rule
def pretrain_with_tps(c):
    if c.get("pretraining_dataset") and c.get("include_tokens_per_second"):
        raise ValueError("pretraining_dataset and include_tokens_per_second cannot be used together.")


# ------------------------------------------------------------------------------- adapters
@rule
def check_lr_groups(c):
    if c.get("lr_groups") and c.get("loraplus_lr_ratio"):
        raise ValueError("lr_groups and loraplus_lr_ratio cannot be used together.")


@rule
def check_frozen(c):
    if c.get("adapter") and c.get("peft_layers_to_transform") and c.get("unfrozen_parameters"):
        raise ValueError("`unfrozen_parameters` used with `peft_layers_to_transform` can have unexpected behavior.")


@rule
def check_peft_layers_pattern(c):
    if c.get("peft_layers_pattern") and not c.get("peft_layers_to_transform"):
        raise ValueError("peft_layers_pattern requires peft_layers_to_transform to be set")


@rule
def check_fused_lora(c):
    if _adapter(c) and c.get("flash_attn_fuse_mlp"):
        raise ValueError("Fused modules are not supported with LoRA/QLoRA")


@rule
def check_lora_kernels_trust_remote_code(c):
    if (c.get("lora_mlp_kernel") or c.get("lora_qkv_kernel") or c.get("lora_o_kernel")) and c.get("trust_remote_code"):
        raise ValueError("lora_mlp_kernel, lora_qkv_kernel, and lora_o_kernel are not compatible with trust_remote_code. "
                         "Please disable trust_remote_code or explicitly set lora_*_kernel to false.")


@rule
def check_trust_remote_code(c):
    if c.get("trust_remote_code"):
        return ("trust_remote_code has no effect: models are built from this framework's own block graph, "
                "no code is loaded from the checkpoint directory")


@rule
def check_lora_config_values(c):
    if not c.get("adapter"):
        return
    r = c.get("lora_r")
    if r is not None and r <= 0:
        raise ValueError("lora_r must be a positive integer")
    d = c.get("lora_dropout")
    if d is not None and not 0.0 <= d < 1.0:
        raise ValueError("lora_dropout must be in [0, 1)")
    if c.get("peft_use_dora") and c.get("adapter") == "mora":
        raise ValueError("peft_use_dora cannot be combined with adapter: mora")
    if c.get("peft_use_dora") and c.get("lora_target_parameters"):
        raise ValueError("DoRA is defined for linear-layer targets; remove lora_target_parameters or peft_use_dora")
    if c.get("lora_modules_to_save") and (c.get("tensor_parallel_size") or 1) > 1:
        raise ValueError("lora_modules_to_save (full copies of embeddings / lm_head) cannot be combined with tensor parallelism")


@rule
def check_loftq(c):
    if c.get("loftq_config") or (c.get("peft") or {}).get("loftq_config"):
        raise ValueError("LoftQ initialisation is not implemented; remove `loftq_config` (PEFT default init is used)")


@rule
def check_layer_replication(c):
    if c.get("peft_layer_replication"):
        raise ValueError("peft_layer_replication (layer duplication by index ranges) is not implemented")


# ------------------------------------------------------------------------------- preference / RL
@rule
def check_kto_config(c):
    if c.get("rl") == "kto":
        if c.get("sample_packing") or c.get("eval_sample_packing"):
            raise ValueError("sample_packing is not supported with kto")


@rule
def check_grpo_liger_sequence_parallel(c):
    if c.get("rl") == "grpo" and (c.get("trl") or {}).get("use_liger_loss") and (c.get("context_parallel_size") or 1) > 1:
        raise ValueError("GRPO + SP + Liger not currently supported")


@rule
def check_rl_config_gradient_checkpointing(c):
    if (c.get("rl") and c.get("gradient_checkpointing") and (c.get("gradient_checkpointing_kwargs") or {}).get("use_reentrant")
            and c.get("load_in_4bit") and c.get("adapter") == "qlora" and (c.get("world_size") or 1) > 1):
        raise ValueError("The `use_reentrant: True` implementation of gradient checkpointing is not supported for "
                         "distributed RL training with QLoRA. Please set `use_reentrant: False` in "
                         "`gradient_checkpointing_kwargs`.")


@rule
def check_gdpo(c):
    if c.get("rl") == "gdpo" and (c.get("trl") or {}).get("multi_objective_aggregation") == "sum_then_normalize":
        raise ValueError("`multi_objective_aggregation` value set as `sum_then_normalize` => GRPO, but GDPO was selected")


@rule
def check_dpo(c):
    lt, lw, rl = c.get("dpo_loss_type"), c.get("dpo_loss_weights"), c.get("rl")
    warn = None
    if rl == "ipo":
        warn = "rl: ipo will soon be deprecated. Use `rl: dpo` with `dpo_loss_type: ['ipo']` instead."
    if rl == "dpo":
        if lw is not None and lt is None:
            raise ValueError("`dpo_loss_weights` requires `dpo_loss_type` to be set")
        if lt is not None and lw is not None and len(lt) != len(lw):
            raise ValueError(f"`dpo_loss_type` and `dpo_loss_weights` must be the same length, but got {len(lt)} losses "
                             f"and {len(lw)} weights")
    elif lt is not None or lw is not None:
        raise ValueError(f"`dpo_loss_type` and `dpo_loss_weights` are for DPO only, but got rl={rl!r}")
    return warn


@rule
def check_grpo_batch_size_divisibility(c):
    if c.get("rl") != "grpo":
        return
    trl = c.get("trl") or {}
    n = trl.get("num_generations")
    if n is None:
        return
    if n < 2:
        raise ValueError(f"GRPO requires `trl.num_generations >= 2` (got {n}). With num_generations=1, every group has "
                         "zero advantage and the policy never updates.")
    if trl.get("generation_batch_size") is not None:
        gbs, src, explicit = int(trl["generation_batch_size"]), "trl.generation_batch_size", True
    else:
        mb, ga = c.get("micro_batch_size") or 1, c.get("gradient_accumulation_steps") or 1
        gbs, src, explicit = int(mb) * int(ga), f"micro_batch_size ({mb}) * gradient_accumulation_steps ({ga})", False
    if gbs % n:
        hint = ""
        if not explicit:
            mb = int(c.get("micro_batch_size") or 1)
            ga = (n * mb // gcd(n, mb)) // mb
            hint = (f" Smallest fix: set `gradient_accumulation_steps: {ga}` (so micro_batch_size * GA = {mb * ga} is a "
                    f"multiple of {n}).")
        raise ValueError(f"GRPO: generation batch size must be divisible by `trl.num_generations`. Got "
                         f"effective_gbs={gbs} (from {src}) and num_generations={n}.{hint}")
    world = c.get("world_size") or 1
    if world > 1 and gbs < n * world:
        raise ValueError(f"GRPO with world_size={world} requires effective_gbs >= num_generations * world_size = "
                         f"{n * world}, got {gbs}. Increase gradient_accumulation_steps or micro_batch_size.")


@rule
def check_simpo_warmup(c):
    if c.get("rl") == "simpo" and c.get("warmup_ratio"):
        raise ValueError("warmup_ratio is not supported with the simpo trainer. Please use `warmup_steps` instead")


@rule
def check_rl_beta(c):
    if c.get("rl_beta") is not None and c.get("dpo_beta") is not None and c["rl_beta"] != c["dpo_beta"]:
        raise ValueError("`rl_beta` and `dpo_beta` are both set to different values; keep one")


@rule
def check_vllm_mode_set(c):
    trl = c.get("trl") or {}
    if trl.get("use_vllm") and not trl.get("vllm_mode"):
        trl["vllm_mode"] = "server"
        c["trl"] = trl
    if trl.get("vllm_mode") == "colocate":
        raise ValueError("trl.vllm_mode: colocate is not available; rollouts come from the training model itself "
                         "(use_vllm: false) or from `axolotl vllm-serve` (vllm_mode: server)")


@rule
def check_ebft(c):
    if c.get("rl") != "ebft":
        return
    eb = c.get("ebft") or {}
    if c.get("torch_compile"):
        raise ValueError("ebft cannot be combined with torch_compile")
    if (c.get("gradient_checkpointing_kwargs") or {}).get("use_reentrant"):
        raise ValueError("ebft needs non-reentrant gradient checkpointing (use_reentrant: false)")
    if c.get("activation_offloading"):
        raise ValueError("ebft is not compatible with activation_offloading")
    if eb.get("mode") == "strided":
        stride, ctx, gen = eb.get("stride"), eb.get("context_length"), eb.get("generate_max_len")
        if stride is not None and stride <= 0:
            raise ValueError("ebft.stride must be positive")
        if c.get("sequence_len") and ctx and gen and ctx + gen > c["sequence_len"]:
            raise ValueError("ebft strided mode: context_length + generate_max_len exceeds sequence_len")
        for ds in c.get("datasets") or []:
            if isinstance(ds, dict) and ds.get("split") and "test" in str(ds["split"]):
                return "ebft strided mode trains on anchors cut from the dataset; a test split is unusual here"


# ------------------------------------------------------------------------------- optimizer
@rule
def check_adamw_optimizer_params(c):
    if any(c.get(k) for k in ("adam_beta1", "adam_beta2", "adam_epsilon")) and \
            (c.get("optimizer") and "adamw" not in str(c["optimizer"]).lower()):
        return "adamw hyperparameters found, but no adamw optimizer set"


@rule
def check_muon_deepspeed_fsdp(c):
    if c.get("optimizer") == "muon" and (c.get("fsdp") or c.get("fsdp_config")):
        v = c.get("fsdp_version") or (c.get("fsdp_config") or {}).get("fsdp_version") or 1
        if str(v) != "2":
            raise ValueError("Muon optimizer is only compatible with FSDP2. Set fsdp_version: 2 to use Muon with FSDP.")


@rule
def check_qgalore(c):
    if c.get("optimizer") == "q_galore_adamw8bit" and c.get("adapter"):
        raise ValueError(f"q_galore_adamw8bit operates on full-precision parameters and is incompatible with "
                         f"adapter='{c['adapter']}'. Remove the adapter setting or pick a different optimizer.")


@rule
def check_batch_flattening_fa(c):
    bf = c.get("batch_flattening")
    if not bf:
        return
    if bf != "auto" and c.get("sample_packing"):
        raise ValueError("batch_flattening not compatible with sample_packing")
    if bf != "auto" and (c.get("micro_batch_size") or 1) == 1:
        return "batch_flattening has no effect with micro_batch_size == 1"
    c["batch_flattening"] = bool(not c.get("sample_packing") and (c.get("micro_batch_size") or 1) > 1)


@rule
def check_cross_entropy_conflicts(c):
    on = [k for k in ("cut_cross_entropy", "chunked_cross_entropy", "liger_cross_entropy", "liger_fused_linear_cross_entropy")
          if c.get(k)]
    if len(on) > 1:
        raise ValueError(f"Only one cross entropy optimization can be enabled at a time. Found {len(on)} enabled: "
                         f"{', '.join(on)}. Please disable all but one.")


@rule
def check_tensor_parallel_optimizer(c):
    if (c.get("tensor_parallel_size") or 1) > 1 and str(c.get("optimizer") or "").lower() in ("muon", "sinkgd", "came_pytorch"):
        raise ValueError(f"optimizer {c['optimizer']} works on whole matrices and cannot be combined with tensor parallelism")


@rule
def check_lr_and_decay_ranges(c):
    if c.get("learning_rate") is not None and float(c["learning_rate"]) < 0:
        raise ValueError("learning_rate must be >= 0")
    if c.get("weight_decay") is not None and float(c["weight_decay"]) < 0:
        raise ValueError("weight_decay must be >= 0")
    if c.get("max_grad_norm") is not None and float(c["max_grad_norm"]) < 0:
        raise ValueError("max_grad_norm must be >= 0")
    if c.get("warmup_ratio") is not None and not 0.0 <= float(c["warmup_ratio"]) <= 1.0:
        raise ValueError("warmup_ratio must be in [0, 1]")
    if c.get("cosine_min_lr_ratio") is not None and not 0.0 <= float(c["cosine_min_lr_ratio"]) <= 1.0:
        raise ValueError("cosine_min_lr_ratio must be in [0, 1]")


# ------------------------------------------------------------------------------- sharding
@rule
def check_fsdp_config_kwargs_prefix(c):
    fc = c.get("fsdp_config")
    if not fc:
        return
    if any(k.startswith("fsdp_") and k != "fsdp_version" for k in fc):
        c["fsdp_config"] = {(k[len("fsdp_"):] if k.startswith("fsdp_") and k != "fsdp_version" else k): v for k, v in fc.items()}
        return ("Configuring FSDP fields with the `fsdp_` prefix is deprecated. Please omit the `fsdp_` prefix from any "
                "fields in `fsdp_config`.")


@rule
def check_fsdp_version_in_fsdp_config(c):
    fc = c.get("fsdp_config") or {}
    if not c.get("fsdp_version") and fc.get("version"):
        c["fsdp_version"] = fc.pop("version")
    elif not c.get("fsdp_version") and fc.get("fsdp_version"):
        c["fsdp_version"] = fc["fsdp_version"]
    if fc and not c.get("fsdp_version"):
        c["fsdp_version"] = 1
    if fc and c.get("fsdp_version"):
        fc["fsdp_version"] = c["fsdp_version"]


@rule
def check_fsdp2_cpu_offload_pin_memory(c):
    fc = c.get("fsdp_config") or {}
    if fc.get("cpu_offload_pin_memory") is False:
        if str(c.get("fsdp_version")) != "2":
            raise ValueError("FSDP1 does not support disabling cpu_offload_pin_memory, please set `fsdp_version` to 2")
        if not fc.get("offload_params"):
            raise ValueError("disabling cpu_offload_pin_memory requires enabling offload_params")


@rule
def check_fsdp2_base_model_quant_rl(c):
    if str(c.get("fsdp_version")) == "2" and c.get("rl") in ("dpo", "kto", "orpo", "ipo") \
            and (c.get("load_in_8bit") or c.get("load_in_4bit")):
        raise ValueError(f"FSDP2 does not support load_in_8bit or load_in_4bit with {c.get('rl')}.")


@rule
def check_fsdp_state_dict_type(c):
    t = (c.get("fsdp_config") or {}).get("state_dict_type")
    if t and str(t).upper() not in ("FULL_STATE_DICT", "SHARDED_STATE_DICT", "LOCAL_STATE_DICT"):
        raise ValueError(f"unknown fsdp_config.state_dict_type '{t}' (FULL_STATE_DICT or SHARDED_STATE_DICT)")
    if t and str(t).upper() == "LOCAL_STATE_DICT":
        raise ValueError("fsdp_config.state_dict_type LOCAL_STATE_DICT is not supported; use SHARDED_STATE_DICT")


@rule
def check_mem_mismatch(c):
    if c.get("max_memory") is not None and c.get("gpu_memory_limit") is not None:
        raise ValueError("max_memory and gpu_memory_limit are mutually exclusive and cannot be used together.")


@rule
def check_model_quantization_config_vs_bnb(c):
    if c.get("model_quantization_config") and (c.get("load_in_8bit") or c.get("load_in_4bit")):
        raise ValueError("model_quantization_config and load_in_8bit or load_in_4bit cannot be used together.")


@rule
def check_gpt_oss_fsdp_loading(c):
    if c.get("model_quantization_config") == "Mxfp4Config" and (c.get("fsdp_config") or {}).get("cpu_ram_efficient_loading"):
        raise ValueError("FSDP cpu_ram_efficient_loading is not supported for Mxfp4Config model quantization.")


@rule
def check_hsdp(c):
    if c.get("dp_replicate_size") is not None and c["dp_replicate_size"] < 1:
        raise ValueError("dp_replicate_size must be >= 1")
    rep, sh = c.get("dp_replicate_size") or 1, c.get("dp_shard_size")
    if rep > 1 and sh == 1:
        return "dp_replicate_size > 1 with dp_shard_size: 1 is plain replicated data parallelism"
    if sh is not None and sh < 1:
        raise ValueError("dp_shard_size must be >= 1")
    if rep < 1:
        raise ValueError("dp_replicate_size must be >= 1")


@rule
def check_expert_parallel(c):
    if c.get("expert_parallel_size") is not None and c["expert_parallel_size"] < 1:
        raise ValueError("expert_parallel_size must be >= 1")
    ep = c.get("expert_parallel_size") or 1
    if ep > 1 and (c.get("context_parallel_size") or 1) > 1 and not c.get("sample_packing"):
        return "expert parallelism with context parallelism: every cp rank routes its own slice of the row"
    if ep < 1:
        raise ValueError("expert_parallel_size must be >= 1")


# ------------------------------------------------------------------------------- templates / streaming
@rule
def check_chat_template_config(c):
    if c.get("chat_template") == "jinja" and not c.get("chat_template_jinja"):
        raise ValueError("chat_template_jinja is required when chat_template is set to 'jinja'. Please provide the Jinja "
                         "template string in chat_template_jinja field.")
    if c.get("chat_template_jinja") and not c.get("chat_template"):
        c["chat_template"] = "jinja"


@rule
def check_pretraining_w_group_by_length(c):
    if c.get("pretraining_dataset") and c.get("group_by_length"):
        return "You probably want to disable group_by_length as it will force a streamed dataset to download completely."


@rule
def check_pretraining_w_val_set_size(c):
    if c.get("pretraining_dataset") and c.get("val_set_size"):
        raise ValueError("val_set_size is not supported with pretraining_dataset. Use test_datasets to specify evaluation "
                         "datasets for pretraining.")


@rule
def check_streaming_w_val_set_size(c):
    if c.get("streaming") and c.get("val_set_size"):
        raise ValueError("val_set_size is not supported with streaming datasets. Use test_datasets to specify evaluation "
                         "datasets when streaming is enabled.")


@rule
def check_streaming_w_max_steps(c):
    if c.get("streaming") and not c.get("max_steps"):
        raise ValueError("max_steps must be set when using streaming datasets. Trainer cannot infer dataset length for "
                         "iterable datasets.")


@rule
def check_streaming_w_multiple_datasets(c):
    if c.get("streaming") and c.get("sample_packing") and c.get("datasets") and len(c["datasets"]) > 1:
        raise ValueError("Sample packing with multiple streaming datasets is not yet supported")


# ------------------------------------------------------------------------------- model-specific
@rule
def check_falcon_fsdp(c):
    if c.get("base_model") and "falcon" in str(c["base_model"]).lower() and c.get("fsdp"):
        raise ValueError("FSDP is not supported for falcon models")


@rule
def check_mpt_checkpointing(c):
    if c.get("base_model") and "mpt" in str(c["base_model"]).lower() and c.get("gradient_checkpointing"):
        raise ValueError("gradient_checkpointing is not supported for MPT models")


@rule
def check_gptq_w_revision(c):
    if c.get("gptq") and c.get("revision_of_model"):
        raise ValueError("revision_of_model is not supported for GPTQ models.")


# ------------------------------------------------------------------------------- activation memory
@rule
def check_gradient_checkpointing_w_offload(c):
    gc = c.get("gradient_checkpointing")
    if gc == "offload":
        c["gradient_checkpointing"] = True
        if c.get("activation_offloading") is None:
            c["activation_offloading"] = True
        return "`offload` is deprecated for gradient_checkpointing, use `activation_offloading: true`"
    if gc == "offload_disk":
        c["gradient_checkpointing"] = True
        c["activation_offloading"] = "disk"
        return "`offload_disk` is deprecated for gradient_checkpointing, use `activation_offloading: disk`"
    if gc == "unsloth":
        c["gradient_checkpointing"] = True
        if c.get("activation_offloading") is None:
            c["activation_offloading"] = True
        return "`gradient_checkpointing: unsloth` is served by `activation_offloading: true`"


@rule
def check_activation_offloading_wo_gc(c):
    ao = c.get("activation_offloading")
    if ao and ao not in (True, "legacy", "disk", "hidden_states"):
        raise ValueError(f"unknown activation_offloading mode '{ao}' (true, legacy, disk or hidden_states)")
    if ao and not c.get("gradient_checkpointing"):
        raise ValueError("activation_offloading requires gradient_checkpointing")


@rule
def check_selective_checkpointing(c):
    sc = c.get("selective_checkpointing")
    if not sc:
        return
    if not c.get("gradient_checkpointing"):
        raise ValueError("selective_checkpointing requires gradient_checkpointing")
    if (c.get("gradient_checkpointing_kwargs") or {}).get("use_reentrant"):
        raise ValueError("selective_checkpointing requires non-reentrant checkpointing (use_reentrant: false)")
    if c.get("activation_offloading") and c.get("activation_offloading") != "hidden_states":
        raise ValueError("selective_checkpointing is only compatible with activation_offloading: hidden_states (or false)")
    save = (sc.get("save") if isinstance(sc, dict) else None) or ["attention"]
    allowed = {"attention", "mlp", "norm"}
    bad = [s for s in save if s not in allowed]
    if bad:
        raise ValueError(f"selective_checkpointing.save entries {bad} are not known; choose from {sorted(allowed)}")
    if _adapter(c) and "mlp" in save:
        return "selective_checkpointing: keeping MLP outputs with a LoRA adapter saves little recompute for much memory"


@rule
def check_hidden_states_offloading(c):
    if c.get("activation_offloading") != "hidden_states":
        return
    kw = c.setdefault("gradient_checkpointing_kwargs", {}) if c.get("gradient_checkpointing_kwargs") is None else c["gradient_checkpointing_kwargs"]
    if kw.get("use_reentrant") and c.get("unfrozen_parameters"):
        raise ValueError("activation_offloading: hidden_states with reentrant checkpointing is incompatible with "
                         "`unfrozen_parameters` (partially frozen model).")
    if _adapter(c):
        return ("activation_offloading: hidden_states uses gradient checkpointing; with LoRA/QLoRA, "
                "activation_offloading: true can be faster because it avoids recompute")


@rule
def check_layer_offloading(c):
    if c.get("layer_offloading") and (c.get("fsdp_config") or (c.get("tensor_parallel_size") or 1) > 1):
        raise ValueError("layer_offloading keeps whole frozen layers in host memory and cannot be combined with "
                         "parameter sharding or tensor parallelism")


# ------------------------------------------------------------------------------- ReLoRA / early stopping
@rule
def check_relora(c):
    if not c.get("relora"):
        return
    if not c.get("jagged_restart_steps"):
        raise ValueError("jagged_restart_steps must be set to use ReLoRA")
    if c.get("adapter") not in ("lora", "qlora"):
        raise ValueError("cfg.adapter must support ReLoRA to use ReLoRA restart semantics")
    if c.get("lr_scheduler") == "one_cycle":
        raise ValueError("ReLoRA is not compatible with the one_cycle scheduler")
    if c.get("flash_attn_fuse_mlp"):
        raise ValueError("Fused modules are not supported with ReLoRA")


@rule
def check_early_stopping(c):
    if c.get("early_stopping_patience"):
        if c.get("save_steps") and c.get("eval_steps") and isinstance(c["save_steps"], int) and isinstance(c["eval_steps"], int) \
                and c["save_steps"] % c["eval_steps"]:
            raise ValueError("`early_stopping_patience` requires that eval_steps should evenly divide save_steps.")


# ------------------------------------------------------------------------------- parallelism
@rule
def check_context_parallel_size(c):
    cp = c.get("context_parallel_size") or 1
    if cp > 1:
        if c.get("attn_implementation") in ("sdpa", "eager"):
            raise ValueError("context_parallel_size > 1 requires the flash attention path (remove attn_implementation "
                             f"'{c['attn_implementation']}')")
        if c.get("heads_k_stride") is not None and c["heads_k_stride"] < 1:
            raise ValueError("heads_k_stride must be >= 1")
        mt = c.get("model_config_type") or ""
        if mt in ("nemotron_h", "falcon_h1", "granitemoehybrid", "qwen3_next"):
            raise ValueError(f"context parallelism for hybrid SSM model type {mt} is not implemented")
        return (f"Sequence parallelism (SP) is enabled with context_parallel_size={cp}. Each rank logs the loss of its own "
                "slice; the logged mean is over ranks.")


@rule
def check_tensor_parallel_size(c):
    if c.get("tensor_parallel_size") is not None and c["tensor_parallel_size"] < 1:
        raise ValueError("tensor_parallel_size must be >= 1")
    tp = c.get("tensor_parallel_size") or 1
    if tp > 1 and c.get("tp_plan") not in (None, "auto"):
        raise ValueError("only the automatic tensor-parallel plan (column/row split of every projection) is available")


# ------------------------------------------------------------------------------- quantisation / QAT
@rule
def check_qat(c):
    q = c.get("qat")
    if not q:
        return
    if _adapter(c):
        raise ValueError("QAT fake-quantises trainable dense weights and cannot be combined with a LoRA adapter")
    wd = (q.get("weight_dtype") or "int8").lower()
    if wd not in ("int4", "int8", "fp8", "float8_e4m3fn", "nvfp4", "mxfp4"):
        raise ValueError(f"unknown qat.weight_dtype '{wd}'")
    ad = q.get("activation_dtype")
    if ad and str(ad).lower() not in ("int8", "fp8", "float8_e4m3fn"):
        raise ValueError(f"unknown qat.activation_dtype '{ad}'")
    gs = q.get("group_size")
    if gs is not None and (gs <= 0 or gs & (gs - 1)):
        raise ValueError("qat.group_size must be a positive power of two")
    if q.get("fake_quant_after_n_steps") is not None and q["fake_quant_after_n_steps"] < 0:
        raise ValueError("qat.fake_quant_after_n_steps must be >= 0")


@rule
def check_sequence_len(c):
    s = c.get("sequence_len")
    if s is not None and s <= 0:
        raise ValueError("sequence_len must be positive")
    if c.get("min_sample_len") and s and c["min_sample_len"] > s:
        raise ValueError("min_sample_len exceeds sequence_len: every sample would be dropped")
    if c.get("excess_length_strategy") not in (None, "drop", "truncate", "raise"):
        raise ValueError("excess_length_strategy must be one of drop, truncate, raise")


@rule
def check_sample_packing_bin_options(c):
    if c.get("sample_packing_bin_size") is not None and c["sample_packing_bin_size"] < 1:
        raise ValueError("sample_packing_bin_size must be >= 1")
    if c.get("sample_packing_group_size") is not None and c["sample_packing_group_size"] < 1:
        raise ValueError("sample_packing_group_size must be >= 1")
    if c.get("sample_packing_sequentially") and c.get("curriculum_sampling") is False and c.get("shuffle_merged_datasets"):
        return "sample_packing_sequentially keeps the dataset order inside bins; the merged datasets are still shuffled first"


@rule
def check_dataset_entries(c):
    for key in ("datasets", "test_datasets"):
        for i, ds in enumerate(c.get(key) or []):
            if not isinstance(ds, dict):
                raise ValueError(f"{key}[{i}] must be a mapping with at least `path`")
            if not ds.get("path"):
                if str(ds.get("type") or "").startswith("_synthetic"):
                    continue   # generated in memory
                raise ValueError(f"{key}[{i}] has no `path`")
            if ds.get("shards") is not None and ds["shards"] < 1:
                raise ValueError(f"{key}[{i}].shards must be >= 1")
            if ds.get("shards_idx") is not None and ds.get("shards") and not 0 <= ds["shards_idx"] < ds["shards"]:
                raise ValueError(f"{key}[{i}].shards_idx must be in [0, shards)")
            for cloud in ("s3://", "gs://", "gcs://", "abfs://", "az://", "adl://", "oci://"):
                if str(ds["path"]).startswith(cloud):
                    raise ValueError(f"{key}[{i}].path '{ds['path']}': cloud object stores are not reachable from this "
                                     "framework (no fsspec back ends); copy the data to a local directory")


@rule
def check_special_tokens(c):
    st = c.get("special_tokens")
    if st is not None and not isinstance(st, dict):
        raise ValueError("special_tokens must be a mapping (e.g. {pad_token: '<pad>'})")
    if c.get("tokens") is not None and not isinstance(c["tokens"], list):
        raise ValueError("tokens must be a list of strings")
    if c.get("added_tokens_overrides") is not None and not isinstance(c["added_tokens_overrides"], dict):
        raise ValueError("added_tokens_overrides must map token ids to new token strings")


@rule
def check_loss_watchdog(c):
    if c.get("loss_watchdog_patience") and not c.get("loss_watchdog_threshold"):
        raise ValueError("loss_watchdog_patience needs loss_watchdog_threshold")


@rule
def check_kd(c):
    if c.get("kd_trainer"):
        if c.get("kd_ce_alpha") is not None and not 0.0 <= c["kd_ce_alpha"] <= 1.0:
            raise ValueError("kd_ce_alpha must be in [0, 1]")
        if c.get("kd_temperature") is not None and c["kd_temperature"] <= 0:
            raise ValueError("kd_temperature must be positive")
        if c.get("sample_packing") and c.get("kd_online_server_base_url"):
            raise ValueError("online knowledge distillation does not support sample packing")


@rule
def check_behaviour_bearing_inert_keys(c):
    """Keys that change numerics in the reference and have no implementation here are refused
    instead of being ignored."""
    if c.get("fp32_norms") or c.get("fp32_norm_classes"):
        return "fp32_norms: normalisation layers already accumulate in fp32 inside the kernels; weights stay bf16"
    if c.get("activation_dtype") and str(c["activation_dtype"]).lower() not in ("bf16", "bfloat16"):
        raise ValueError("activation_dtype other than bf16 is not supported: the tensor-core kernels are bf16")
    if c.get("dpo_norm_loss"):
        raise ValueError("dpo_norm_loss (length-normalised DPO) is not implemented; use rl: ipo or simpo for length "
                         "normalisation")
    if c.get("streaming_partial_batch") is False and c.get("streaming"):
        return "streaming_partial_batch: false — the last partial batch of the stream is dropped"


def run_rules(cfg: dict) -> list[str]:
    """Applies every rule in order; returns the collected warnings."""
    warnings = []
    for fn in RULES:
        msg = fn(cfg)
        if msg:
            warnings.append(msg)
    return warnings
