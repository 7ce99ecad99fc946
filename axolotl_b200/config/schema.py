"""Configuration schema: the axolotl YAML surface as a pydantic model.

Every key of the reference schema (src/axolotl/utils/schemas/config.py:189-209 and its mixins) is
*recognised*. Keys this framework implements are typed fields below; keys that configure machinery
we deliberately do not have (DeepSpeed, bitsandbytes 8-bit, xformers, torch.compile, ...) are listed
in ``UNSUPPORTED_KEYS`` and rejected with a clear message when set to a truthy value; the remaining
reference keys are accepted and carried through untouched (``INERT_KEYS``). Unknown keys are an
error with a did-you-mean hint.
"""
from __future__ import annotations

import difflib
from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field, field_validator, model_validator


class _Base(BaseModel):
    model_config = ConfigDict(extra="allow", protected_namespaces=(), populate_by_name=True)


# ------------------------------------------------------------------------------------ datasets
class SFTDataset(_Base):
    path: str | None = None
    split: str | None = None
    type: str | dict | None = None
    input_transform: str | None = None
    shards: int | None = None
    shards_idx: int | None = None
    preprocess_shards: int | None = None
    conversation: str | None = None
    chat_template: str | None = None
    chat_template_jinja: str | None = None
    data_files: str | list[str] | None = None
    input_format: str | None = None
    name: str | None = None
    ds_type: str | None = None
    field: str | None = None
    field_human: str | None = None
    field_model: str | None = None
    field_messages: str | None = None
    field_tools: str | None = None
    field_thinking: str | None = None
    template_thinking_key: str | None = None
    message_field_role: str | None = None
    message_field_content: str | None = None
    message_property_mappings: dict[str, str] | None = None
    message_field_training: str | None = None
    message_field_training_detail: str | None = None
    split_thinking: bool | None = None
    logprobs_field: str | None = None
    temperature: float | None = None
    roles_to_train: list[str] | None = None
    train_on_eos: Literal["all", "turn", "last"] | None = None
    train_on_eot: Literal["all", "turn", "last"] | None = None
    roles: dict[str, list[str]] | None = None
    drop_system_message: bool | None = None
    trust_remote_code: bool | None = False
    revision: str | None = None
    text_column: str | None = None
    # _synthetic
    length: int | None = None
    sequence_length: int | None = None
    min_input_id: int | None = None
    max_input_id: int | None = None
    seed: int | None = None
    # variable-length synthetic (extension used by the benchmark configs)
    min_length: int | None = None
    max_length: int | None = None
    mask_prefix_fraction: float | None = None


class UserDefinedPrompterType(_Base):
    system_prompt: str | None = None
    system_format: str | None = None
    field_system: str | None = None
    field_instruction: str | None = None
    field_input: str | None = None
    field_output: str | None = None
    format: str | None = None
    no_input_format: str | None = None


class PretrainingDataset(_Base):
    name: str | None = None
    path: str | None = None
    split: str | None = "train"
    text_column: str | None = "text"
    type: str | None = "pretrain"
    trust_remote_code: bool | None = False
    data_files: str | list[str] | None = None
    skip: int | None = None


class FSDPConfig(_Base):
    fsdp_version: int | None = None
    activation_checkpointing: bool | None = None
    offload_params: bool | None = None
    sync_module_states: bool | None = None
    cpu_ram_efficient_loading: bool | None = None
    cpu_offload_pin_memory: bool | None = None
    use_orig_params: bool | None = None
    state_dict_type: Literal["FULL_STATE_DICT", "LOCAL_STATE_DICT", "SHARDED_STATE_DICT"] | None = None
    final_state_dict_type: Literal["FULL_STATE_DICT", "LOCAL_STATE_DICT", "SHARDED_STATE_DICT"] | None = None
    auto_wrap_policy: str | None = None
    transformer_layer_cls_to_wrap: str | None = None
    reshard_after_forward: bool | None = None
    mixed_precision_policy: str | None = None

    @model_validator(mode="before")
    @classmethod
    def strip_prefix(cls, data):
        # the reference accepts both `fsdp_xxx` and `xxx` spellings inside fsdp_config
        if isinstance(data, dict):
            out = {}
            for k, v in data.items():
                nk = k[5:] if k.startswith("fsdp_") and k != "fsdp_version" else k
                out[nk] = v
            return out
        return data


class SpecialTokens(_Base):
    bos_token: str | None = None
    eos_token: str | None = None
    pad_token: str | None = None
    unk_token: str | None = None
    additional_special_tokens: list[str] | None = None


class LrGroup(_Base):
    name: str
    modules: list[str]
    lr: float


class TRLConfig(_Base):
    beta: float | None = None
    max_completion_length: int | None = None
    num_generations: int | None = None
    use_vllm: bool | None = False
    vllm_server_host: str | None = None
    vllm_server_port: int | None = None
    reward_funcs: list[str] | None = None
    reward_weights: list[float] | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    loss_type: str | None = None
    epsilon: float | None = None
    epsilon_high: float | None = None
    scale_rewards: bool | str | None = None
    num_iterations: int | None = None
    log_completions: bool | None = None
    sync_ref_model: bool | None = None
    ref_model_mixup_alpha: float | None = None
    ref_model_sync_steps: int | None = None
    importance_sampling_level: str | None = None
    mask_truncated_completions: bool | None = None
    async_prefetch: int | None = None
    replay_buffer_size: int | None = None


QuantDType = Literal["int4", "int8", "fp8", "float8_e4m3fn", "nvfp4", "mxfp4", "mxfp8"]


class QATConfig(_Base):
    """Quantisation-aware training: which fake-quantiser wraps the trainable dense weights
    (src/axolotl/utils/schemas/quantization.py:31-58)."""
    activation_dtype: QuantDType | None = None
    weight_dtype: QuantDType = "int8"
    quantize_embedding: bool | None = False
    group_size: int | None = 32
    fake_quant_after_n_steps: int | None = None


class PTQConfig(_Base):
    """Post-training quantisation applied by ``axolotl quantize`` (quantization.py:61-80)."""
    weight_dtype: QuantDType = "nvfp4"
    activation_dtype: QuantDType | None = None
    quantize_embedding: bool | None = None
    group_size: int | None = 16


class VllmConfig(_Base):
    """Arguments of ``axolotl vllm-serve`` (src/axolotl/utils/schemas/vllm.py)."""
    device: str | None = "auto"
    tensor_parallel_size: int | None = None
    data_parallel_size: int | None = None
    gpu_memory_utilization: float | None = 0.9
    dtype: str | None = "auto"
    max_model_len: int | None = None
    enable_prefix_caching: bool | None = None
    host: str | None = "0.0.0.0"  # nosec B104
    port: int | None = 8000
    enable_reasoning: bool | None = None
    reasoning_parser: str | None = None
    enforce_eager: bool | None = None
    serve_module: str | None = None
    worker_extension_cls: str | None = None


class EBFTConfig(_Base):
    """Energy-based fine-tuning block (src/axolotl/utils/schemas/config.py:76-190)."""
    feature_layers: list[float] = [0.25, 0.5, 0.75]
    embed_method: Literal["last_token", "mean_pooling", "completion_mean", "concat"] = "last_token"
    use_whitening: bool = False
    alignment_coef: float = 1.0
    diversity_coef: float = 1.0
    ce_coef: float = 0.0
    adaptive_max_tokens: bool = True
    gt_length_multiplier: float = 1.5
    mode: Literal["structured", "strided"] = "structured"
    stride: int = 8
    context_length: int = 8
    generate_max_len: int = 8
    n_samples_per_prompt: int = 4
    temperature: float = 0.6
    top_p: float = 1.0
    rl_coef: float = 1.0
    advantage_estimator: Literal["rloo", "group_norm", "reinforce"] = "rloo"
    min_completion_prefix: int = 0


class SelectiveCheckpointing(_Base):
    save: list[str] = ["attention"]


class DynamicCheckpointConfig(_Base):
    enabled: bool = False
    check_interval: int = 10
    trigger_file_path: str = ""


# ------------------------------------------------------------------------------------ top level
class AxolotlConfig(_Base):
    # ---- model
    base_model: str | None = None
    base_model_config: str | None = None
    model_preset: str | None = None  # extension: a named architecture from models.config.PRESETS
    tokenizer_config: str | None = None
    tokenizer_type: str | None = None
    tokenizer_use_fast: bool | None = None
    tokenizer_legacy: bool | None = None
    trust_remote_code: bool | None = None
    type_of_model: str | None = None
    model_type: str | None = None
    revision_of_model: str | None = None
    overrides_of_model_config: dict | None = None
    reinit_weights: bool | None = None
    resize_token_embeddings_to_32x: bool | None = None
    shrink_embeddings: bool | None = None
    mean_resizing_embeddings: bool | None = False
    rope_scaling: dict | None = None
    # ---- outputs
    output_dir: str = "./model-out"
    hub_model_id: str | None = None
    hub_strategy: str | None = None
    save_safetensors: bool | None = True
    # ---- precision
    bf16: bool | Literal["auto", "full"] | None = None
    fp16: bool | None = None
    tf32: bool | Literal["auto"] | None = None
    float32: bool | None = None
    bfloat16: bool | None = None
    float16: bool | None = None
    fp8: bool | None = None
    # ---- adapters
    adapter: Literal["lora", "qlora", "llama-adapter"] | str | None = None
    lora_model_dir: str | None = None
    lora_r: int | None = None
    lora_alpha: int | None = None
    lora_dropout: float | None = 0.0
    lora_target_modules: list[str] | str | None = None
    lora_target_parameters: list[str] | str | None = None
    lora_target_linear: bool | None = None
    lora_modules_to_save: list[str] | None = None
    lora_fan_in_fan_out: bool | None = None
    lora_rank_pattern: dict | None = None
    lora_alpha_pattern: dict | None = None
    peft_use_dora: bool | None = None
    peft_use_rslora: bool | None = None
    peft_layers_to_transform: list[int] | None = None
    peft_layers_pattern: list[str] | None = None
    peft_init_lora_weights: bool | str | None = None
    peft_autocast_adapter_dtype: bool | None = None
    peft_trainable_token_indices: Any = None
    loraplus_lr_ratio: float | None = None
    loraplus_lr_embedding: float | None = 1e-6
    merge_lora: bool | None = None
    merge_method: Literal["legacy", "memory_efficient"] | None = "memory_efficient"
    lora_mlp_kernel: bool | None = None
    lora_qkv_kernel: bool | None = None
    lora_o_kernel: bool | None = None
    lora_embedding_kernel: bool | None = None
    load_in_4bit: bool | None = False
    load_in_8bit: bool | None = False
    quantize_moe_experts: bool | None = None
    unfrozen_parameters: list[str] | None = None
    # ---- data
    datasets: list[SFTDataset] | None = None
    test_datasets: list[SFTDataset] | None = None
    pretraining_dataset: list[PretrainingDataset] | None = None
    dataset_prepared_path: str | None = None
    dataset_processes: int | None = None
    dataset_num_proc: int | None = None
    dataset_exact_deduplication: bool | None = None
    dataset_keep_in_memory: bool | None = None
    dataset_shard_num: int | None = None
    dataset_shard_idx: int | None = None
    skip_prepare_dataset: bool | None = False
    shuffle_merged_datasets: bool | None = True
    shuffle_before_merging_datasets: bool | None = False
    push_dataset_to_hub: str | None = None
    hf_use_auth_token: bool | None = None
    val_set_size: float | None = 0.0
    sequence_len: int = 512
    eval_sequence_len: int | None = None
    min_sample_len: int | None = None
    excess_length_strategy: Literal["drop", "truncate", "raise"] | None = None
    sample_packing: bool | None = None
    eval_sample_packing: bool | None = None
    sample_packing_group_size: int | None = 100_000
    sample_packing_bin_size: int | None = 200
    sample_packing_sequentially: bool | None = None
    sample_packing_eff_est: float | None = None
    sample_packing_mp_start_method: str | None = None
    multipack_real_batches: bool | None = None
    pad_to_sequence_len: bool | None = None
    pad_to_multiple_of: int | None = None
    curriculum_sampling: bool | None = None
    group_by_length: bool | None = None
    train_on_inputs: bool | None = False
    chat_template: str | None = None
    chat_template_jinja: str | None = None
    chat_template_kwargs: dict | None = None
    # multimodal (LLaVA-style checkpoints: CLIP tower + projector in front of the language model)
    processor_type: str | None = None
    processor_config: str | None = None
    is_multimodal: bool | None = None
    image_size: int | list[int] | None = None
    image_resize_algorithm: str | None = None
    role_boundaries: list[dict] | None = None
    freeze_mm_modules: bool | None = None        # False: the vision tower trains too (the projector follows the adapter / freezing rules)
    eot_tokens: list[str] | None = None
    default_system_message: str | None = None
    special_tokens: SpecialTokens | None = None
    tokens: list[str] | None = None
    added_tokens_overrides: dict[int, str] | None = None
    streaming: bool | None = None
    streaming_multipack_buffer_size: int | None = 10_000
    pretrain_multipack_buffer_size: int | None = None
    pretrain_multipack_attn: bool | None = True
    pretraining_sample_concatenation: bool | None = None
    use_pose: bool | None = None
    pose_split_on_token_ids: list[int] | None = None
    pose_max_context_len: int | None = None
    pose_num_chunks: int | None = None
    dataloader_num_workers: int | None = None
    dataloader_pin_memory: bool | None = None
    dataloader_prefetch_factor: int | None = None
    dataloader_drop_last: bool | None = None
    remove_unused_columns: bool | None = None
    # ---- batch / schedule
    micro_batch_size: int | None = 1
    gradient_accumulation_steps: int | None = None
    batch_size: int | None = None
    eval_batch_size: int | None = None
    num_epochs: float = 1.0
    max_steps: int | None = None
    learning_rate: float | str = 5e-5
    weight_decay: float | None = 0.0
    optimizer: str | None = "adamw_torch_fused"
    optim_args: str | dict | None = None
    optim_target_modules: list[str] | str | None = None
    adam_beta1: float | None = None
    adam_beta2: float | None = None
    adam_beta3: float | None = None
    adam_epsilon: float | None = None
    adam_epsilon2: float | None = None
    max_grad_norm: float | None = None
    lr_scheduler: str | None = "cosine"
    lr_scheduler_kwargs: dict | None = None
    lr_quadratic_warmup: bool | None = None
    cosine_min_lr_ratio: float | None = None
    cosine_constant_lr_ratio: float | None = None
    lr_div_factor: float | None = None
    lr_groups: list[LrGroup] | None = None
    embedding_lr: float | None = None
    embedding_lr_scale: float | None = None
    warmup_steps: int | None = None
    warmup_ratio: float | None = None
    jagged_restart_steps: int | None = None
    jagged_restart_warmup_steps: int | None = None
    jagged_restart_anneal_steps: int | None = None
    neftune_noise_alpha: float | None = None
    seed: int | None = None
    # ---- logging / saving / eval
    logging_steps: int | None = None
    save_steps: int | float | None = None
    saves_per_epoch: int | None = None
    save_strategy: Literal["steps", "epoch", "no", "best"] | None = None
    save_total_limit: int | None = None
    save_only_model: bool | None = False
    save_first_step: bool | None = None
    eval_steps: int | float | None = None
    evals_per_epoch: int | None = None
    eval_strategy: str | None = None
    early_stopping_patience: int | None = None
    load_best_model_at_end: bool | None = False
    metric_for_best_model: str | None = None
    greater_is_better: bool | None = None
    include_tokens_per_second: bool | None = None
    include_tkps: bool | None = True
    loss_watchdog_threshold: float | None = None
    loss_watchdog_patience: int | None = None
    resume_from_checkpoint: str | None = None
    auto_resume_from_checkpoints: bool | None = None
    dynamic_checkpoint: DynamicCheckpointConfig | None = None
    profiler_steps: int | None = None
    profiler_steps_start: int | None = 0
    gc_steps: int | None = None
    torch_empty_cache_steps: int | None = None
    do_causal_lm_eval: bool | None = None
    eval_causal_lm_metrics: list[str] | None = None
    eval_max_new_tokens: int | None = None
    eval_table_size: int | None = None
    do_bench_eval: bool | None = None
    bench_dataset: str | None = None
    generate_samples: bool | None = None
    num_generation_samples: int | None = 3
    generation_max_new_tokens: int | None = 50
    generation_temperature: float | None = 0.7
    generation_top_p: float | None = None
    generation_top_k: int | None = None
    generation_prompt_ratio: float | None = 0.5
    generation_do_sample: bool | None = True
    # ---- reporting
    use_wandb: bool | None = None
    # Ray Train launcher (cli/launchers.py)
    use_ray: bool | None = None
    ray_num_workers: int | None = None
    ray_run_name: str | None = None
    resources_per_worker: dict | None = None
    wandb_project: str | None = None
    wandb_entity: str | None = None
    wandb_name: str | None = None
    wandb_run_id: str | None = None
    wandb_mode: str | None = None
    wandb_watch: str | None = None
    wandb_log_model: str | None = None
    use_mlflow: bool | None = None
    mlflow_tracking_uri: str | None = None
    mlflow_experiment_name: str | None = None
    mlflow_run_name: str | None = None
    hf_mlflow_log_artifacts: bool | None = None
    use_comet: bool | None = None
    comet_project_name: str | None = None
    use_tensorboard: bool | None = None
    use_trackio: bool | None = None
    use_otel_metrics: bool | None = None
    otel_metrics_host: str | None = "localhost"
    otel_metrics_port: int | None = 8000
    # ---- memory
    gradient_checkpointing: bool | Literal["offload", "offload_disk", "unsloth"] | None = False
    gradient_checkpointing_kwargs: dict | None = None
    activation_offloading: bool | str | None = False
    layer_offloading: bool | None = None
    selective_checkpointing: bool | SelectiveCheckpointing | None = None
    tiled_mlp: bool | None = None
    tiled_mlp_num_shards: int | None = None
    chunked_cross_entropy: bool | None = None
    chunked_cross_entropy_num_chunks: int | None = None
    # ---- attention
    attn_implementation: str | None = None
    flash_attention: bool | None = None
    sdp_attention: bool | None = None
    eager_attention: bool | None = None
    flex_attention: bool | None = None
    sdpa_varlen: bool | None = None
    # ---- parallelism
    fsdp: list[str] | None = None
    fsdp_config: FSDPConfig | None = None
    fsdp_version: int | None = None
    fsdp_final_state_dict_type: str | None = None
    dp_shard_size: int | None = None
    dp_replicate_size: int | None = None
    tensor_parallel_size: int | None = None
    context_parallel_size: int | None = None
    sequence_parallel_degree: int | None = None
    expert_parallel_size: int | None = None
    heads_k_stride: int | None = None
    ring_attn_func: str | None = None
    ddp: bool | None = None
    ddp_timeout: int | None = None
    ddp_bucket_cap_mb: int | None = None
    ddp_broadcast_buffers: bool | None = None
    ddp_find_unused_parameters: bool | None = None
    world_size: int | None = None
    local_rank: int | None = None
    device: Any = None
    device_map: Any = None
    # ---- RL / preference
    rl: str | None = None
    trl: TRLConfig | None = None
    ebft: EBFTConfig | None = None
    rl_beta: float | None = None
    dpo_beta: float | None = None
    dpo_label_smoothing: float | None = None
    dpo_loss_type: str | list[str] | None = None
    dpo_use_weighting: bool | None = None
    orpo_alpha: float | None = None
    rpo_alpha: float | None = None
    simpo_gamma: float | None = None
    cpo_alpha: float | None = None
    kto_desirable_weight: float | None = None
    kto_undesirable_weight: float | None = None
    reward_model: bool | None = None
    process_reward_model: bool | None = None
    lisa_n_layers: int | None = None
    lisa_step_interval: int | None = None
    peer_heartbeat_timeout: float | None = None   # extension: seconds before a silent peer is declared failed (0 = off)
    center_rewards_coefficient: float | None = None
    cpo_loss_type: str | None = None
    max_prompt_len: int | None = None
    precompute_ref_log_probs: bool | None = None
    vllm: VllmConfig | None = None
    use_comet: bool | None = None
    comet_api_key: str | None = None
    comet_workspace: str | None = None
    comet_project_name: str | None = None
    comet_experiment_key: str | None = None
    comet_mode: str | None = None
    comet_online: bool | None = None
    comet_experiment_config: dict | None = None
    use_trackio: bool | None = None
    trackio_project_name: str | None = None
    trackio_run_name: str | None = None
    trackio_space_id: str | None = None
    # ---- MoE
    experts_implementation: str | None = None
    router_aux_loss_coef: float | None = None
    expert_weights_nvfp4: bool | None = None  # extension: quantise frozen expert weights to NVFP4 at load
    # ---- misc
    plugins: list[str] | None = None
    strict: bool | None = False
    debug: bool | None = None
    is_preprocess: bool | None = None
    use_ray: bool | None = False
    capabilities: dict | None = None
    env_capabilities: dict | None = None
    axolotl_config_path: str | None = None
    relora: bool | None = None
    relora_prune_ratio: float | None = None
    relora_cpu_offload: bool | None = None
    qat: QATConfig | None = None
    quantization: PTQConfig | None = None
    fix_untrained_tokens: int | list[int] | None = None
    # derived (filled by normalisation)
    is_llama_derived_model: bool | None = None
    is_mistral_derived_model: bool | None = None
    is_qwen_derived_model: bool | None = None
    model_config_type: str | None = None
    total_num_tokens: int | None = None
    total_supervised_tokens: int | None = None

    @field_validator("learning_rate", mode="before")
    @classmethod
    def _lr_to_float(cls, v):
        return float(v) if isinstance(v, str) else v

    @field_validator("datasets", "test_datasets", mode="before")
    @classmethod
    def _ds_list(cls, v):
        if v is not None and not isinstance(v, list):
            raise ValueError("datasets must be a list")
        return v


KNOWN_KEYS = set(AxolotlConfig.model_fields)

# Reference keys that configure machinery this framework does not contain. Setting them to a truthy
# value is an error (the message names the native replacement where there is one).
UNSUPPORTED_KEYS = {
    "deepspeed": "DeepSpeed is not used; sharding is native (fsdp_config / dp_shard_size)",
    "deepcompile": "DeepSpeed is not used",
    "load_in_8bit": "bitsandbytes int8 is not available; use bf16 or NVFP4 expert weights",
    "gptq": "GPTQ checkpoints are not supported",
    "xformers_attention": "attention always runs the native varlen flash kernel",
    "sage_attention": "attention always runs the native varlen flash kernel",
    "s2_attention": "shifted-sparse attention is not implemented",
    "torch_compile": "no tracing compiler is used; kernels are hand-written",
    "unsloth_cross_entropy_loss": "the native chunked linear+CE kernel is always used",
    "llama4_linearized_experts": "checkpoints with per-expert linear modules are not loaded directly; convert them with `axolotl delinearize-llama4` first",
    "use_onebitllms": "1-bit LLM training is not supported",
    "flash_optimum": "BetterTransformer is not used",
    "fp8": "fp8 mixed precision is not implemented; bf16 tensor-core kernels are used",
    "large_head_attention": "head widths 64, 128, 256 (and 192/128 latent attention) have native kernels; 512 does not",
}

# Reference keys that are accepted and carried through without effect on this framework (their
# purpose is served natively or is irrelevant here).
INERT_KEYS = {
    "accelerator_config", "activation_checkpointing", "async_prefetch", "auto_find_batch_size",
    "bnb_config_kwargs", "cls_model_config", "dion_lr", "dion_momentum",
    "dion_rank_fraction", "dion_rank_multiple_of", "dpo_generate_during_eval", "dpo_padding_free",
    "dpo_use_liger_kernel", "dpo_use_logits_to_keep", "dpo_loss_weights", "embeddings_skip_upcast",
    "experimental_skip_move_to_device", "flash_attn_cross_entropy", "flash_attn_d512", "flash_attn_rms_norm", "flex_attn_compile_kwargs", "fp8_enable_fsdp_float8_all_gather", "fused_attn_kernel", "gc_collect_steps",
    "gemma4_hybrid_attn_impl", "gradio_max_new_tokens", "gradio_server_name",
    "gradio_server_port", "gradio_share", "gradio_temperature", "gradio_title", "hub_revision",
    "is_falcon_derived_model",
    "lisa_layers_attribute", "lora_on_cpu", "low_cpu_mem_usage",
    "model_quantization_config_kwargs", "num_dataset_shards_to_save",
    "overrides_of_model_kwargs", "peft", "peft_ensure_weight_tying", "preprocess_iterable", "processor_kwargs", "qgalore_cos_threshold", "qgalore_gamma_proj",
    "qgalore_proj_bits", "qgalore_proj_group_size", "qgalore_proj_quant", "qgalore_proj_type", "qgalore_queue_size",
    "qgalore_rank", "qgalore_scale", "qgalore_update_proj_gap", "qlora_sharded_model_loading", "quantize_embedding",
    "recompute_layer_types", "relora_prune_method",
    "save_sliding_window", "scaling_softmax_bias", "scaling_softmax_factor", "streaming_min_groups",
    "tokenizer_save_jinja_files", "tokenizer_use_mistral_common", "torch_compile_backend",
    "torch_compile_mode", "torch_compile_options", "torchdistx_path", "trainer_cls", "use_eaft", "eaft_alpha", "eaft_k", "use_kernels", "use_liger_loss",
    "liger_rope", "liger_rms_norm", "liger_glu_activation", "liger_layer_norm", "kd_online_server_base_url", "tiled_mlp_use_original_mlp", "min_num_params",
}


# Reference keys without a schema field whose effect is decided by a validation rule (config/rules.py):
# rewritten to their current spelling, honoured, or refused with a message.
RULED_KEYS = {
    "activation_dtype", "dpo_norm_loss", "fp32_norm_classes", "fp32_norms", "loftq_config",
    "peft_layer_replication", "streaming_partial_batch", "max_packed_sequence_len", "noisy_embedding_alpha", "evaluation_strategy",
    "batch_flattening", "cut_cross_entropy", "liger_cross_entropy", "liger_fused_linear_cross_entropy", "flash_attn_fuse_mlp",
    "max_memory", "gpu_memory_limit", "model_quantization_config", "scaling_softmax",
}


def check_keys(raw: dict) -> list[str]:
    """Raises on unknown or unsupported keys; returns the list of inert keys that were set."""
    inert = []
    for k, v in raw.items():
        if k in UNSUPPORTED_KEYS:
            if v:
                raise ValueError(f"config key '{k}' is unsupported on axolotl_b200: {UNSUPPORTED_KEYS[k]}")
            continue
        if k in KNOWN_KEYS or k in RULED_KEYS:
            continue
        if k in INERT_KEYS:
            inert.append(k)
            continue
        hint = difflib.get_close_matches(k, sorted(KNOWN_KEYS | INERT_KEYS | RULED_KEYS), n=1)
        raise ValueError(f"unknown config key '{k}'" + (f" (did you mean '{hint[0]}'?)" if hint else ""))
    return inert
