"""``train(cfg, dataset_meta)``: config -> tokenizer -> data -> model (+adapter) -> parallel runtime
-> optimizer/schedule -> Trainer -> saved artefacts. The call graph of the reference
(src/axolotl/train.py:54-668) collapsed into one module because there is no HF Trainer,
accelerate or PEFT layer underneath.

Artefacts (reference contract, src/axolotl/train.py:254-488): ``adapter_config.json`` +
``config.json`` (+ tokenizer) are written up front; periodic ``checkpoint-N/`` directories carry
the adapter (or full model), optimizer, RNG, ``trainer_state.json`` and ``tokens_state.json``; the
end of training writes ``adapter_model.safetensors`` (LoRA) or ``model*.safetensors`` (full).
"""
from __future__ import annotations

import os
import signal

import numpy as np
import torch

from ..data.collator import PackedCollator
from ..data.loading import TrainDatasetMeta, load_datasets
from ..data.packing import MultipackBatchSampler
from ..io import hf as hf_io
from ..models.config import ModelConfig, preset
from ..models.lora import ALL_LINEAR, LoraSpec, inject_lora, load_adapter, save_adapter
from ..models.transformer import CausalLM
from ..plugins.base import PluginManager
from ..utils.logging import get_logger, start_debug_log, stop_debug_log
from .callbacks import build_callbacks
from .optimizer import (FlatAdamW, TorchOptimizerAdapter, build_param_groups, default_warmup_steps, make_lr_lambda)
from .trainer import Callback, TrainArgs, Trainer, find_last_checkpoint

LOG = get_logger(__name__)


def model_config_from_cfg(cfg) -> ModelConfig:
    if cfg.get("model_preset"):
        mc = preset(cfg["model_preset"], **(cfg.get("overrides_of_model_config") or {}))
    else:
        mc = ModelConfig.from_pretrained(cfg.get("base_model_config") or cfg["base_model"])
        for k, v in (cfg.get("overrides_of_model_config") or {}).items():
            setattr(mc, k, v)
    if cfg.get("rope_scaling"):
        mc.rope_scaling = dict(cfg["rope_scaling"])
    if cfg.get("router_aux_loss_coef") is not None:
        mc.router_aux_loss_coef = cfg["router_aux_loss_coef"]
    return mc


def build_model(cfg, device) -> CausalLM:
    dtype = torch.bfloat16 if cfg.get("torch_dtype") == "bfloat16" else torch.float32
    mc = model_config_from_cfg(cfg)
    from ..models.registry import validate_cfg as validate_arch

    for note in validate_arch(cfg, mc):
        LOG.info("%s: %s", mc.model_type, note)
    pm = PluginManager.get_instance()
    pm.call("pre_model_load", cfg)
    src = cfg.get("base_model")
    have_weights = bool(src) and os.path.isdir(src) and bool(hf_io.st.checkpoint_files(src)) and not cfg.get("reinit_weights")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if have_weights and world > 1 and (cfg.get("fsdp_config") or {}).get("cpu_ram_efficient_loading") \
            and torch.distributed.is_initialized():
        model = hf_io.load_pretrained_from_rank0(src, dtype=dtype, device=device, config=mc)
        LOG.info("cpu_ram_efficient_loading: rank 0 read the checkpoint, the other ranks received it by broadcast")
    elif have_weights:
        model = hf_io.load_pretrained(src, dtype=dtype, device=device, config=mc)
    else:
        if not cfg.get("reinit_weights") and not cfg.get("model_preset"):
            LOG.warning("no weights found under %r: initialising randomly", src)
        model = CausalLM(mc, dtype=dtype, device=device).init_weights(cfg.get("seed") or 0)
    if cfg.get("expert_weights_nvfp4"):
        from ..ops.grouped import quantize_experts_nvfp4_

        quantize_experts_nvfp4_(model)
    fix = cfg.get("fix_untrained_tokens")
    if fix:
        n = model.fix_untrained_tokens(None if fix is True or isinstance(fix, bool) else ([fix] if isinstance(fix, int) else fix))
        LOG.info("fix_untrained_tokens: %d embedding rows set to the mean of the trained rows", n)
    pm.call("post_model_build", cfg, model)
    return model


def _mora_type(v):
    from ..models.mora import mora_type_id

    return mora_type_id(v)


def lora_spec_from_cfg(cfg) -> LoraSpec | None:
    if cfg.get("adapter") not in ("lora", "qlora", "mora"):
        return None
    mora = cfg.get("mora") or {}
    use_mora = cfg.get("adapter") == "mora"
    if use_mora and mora.get("use_mora") is False:
        raise ValueError("mora.use_mora must be true when adapter: mora is set")
    tm = cfg.get("lora_target_modules")
    if cfg.get("lora_target_linear"):
        tm = sorted(set(ALL_LINEAR) | set(tm or [])) if not isinstance(tm, str) else tm
    tp = cfg.get("lora_target_parameters")
    if isinstance(tp, str):
        tp = [tp]
    return LoraSpec(r=cfg["lora_r"], lora_alpha=cfg.get("lora_alpha") or cfg["lora_r"], lora_dropout=cfg.get("lora_dropout") or 0.0,
                    target_modules=tm, target_parameters=tp, use_rslora=bool(cfg.get("peft_use_rslora")),
                    use_dora=bool(cfg.get("peft_use_dora")), use_mora=use_mora,
                    trainable_token_indices=cfg.get("peft_trainable_token_indices"),
                    mora_type=_mora_type(mora.get("mora_type", "rope")) if use_mora else 6, modules_to_save=cfg.get("lora_modules_to_save"),
                    rank_pattern=cfg.get("lora_rank_pattern") or {}, alpha_pattern=cfg.get("lora_alpha_pattern") or {},
                    layers_to_transform=cfg.get("peft_layers_to_transform"),
                    base_model_name_or_path=cfg.get("base_model"))


def setup_adapter(cfg, model):
    pm = PluginManager.get_instance()
    spec = lora_spec_from_cfg(cfg)
    if spec is None:
        _apply_freezing(cfg, model)
        return None
    pm.call("pre_lora_load", cfg, model)
    if cfg.get("adapter") == "qlora" and cfg.get("load_in_4bit"):
        from ..models.lora import quantize_base_nf4_

        qcfg = cfg.get("bnb_config_kwargs") or {}
        saved = quantize_base_nf4_(model, double_quant=qcfg.get("bnb_4bit_use_double_quant", True) is not False)
        LOG.info("base projections stored as NF4: %.2f GiB saved", saved / 1024 ** 3)
    adapter_dtype = torch.float32 if cfg.get("peft_autocast_adapter_dtype", True) is not False else model.dtype
    if cfg.get("lora_target_linear") and isinstance(spec.target_modules, (list, tuple)):
        from ..models.lora import discover_linear_names

        # every projection of THIS architecture (latent-attention bottlenecks, state-space in/out projections ...)
        spec.target_modules = sorted(set(spec.target_modules) | set(discover_linear_names(model)))
    n = inject_lora(model, spec, adapter_dtype=adapter_dtype)
    if cfg.get("lora_model_dir"):
        load_adapter(model, cfg["lora_model_dir"])
        LOG.info("loaded adapter from %s", cfg["lora_model_dir"])
    _apply_freezing(cfg, model, keep_frozen=True)
    total = sum(p.numel() for p in model.parameters())
    LOG.info("trainable params: %s || all params: %s || trainable%%: %.4f", f"{n:,}", f"{total:,}", 100 * n / max(total, 1))
    pm.call("post_lora_load", cfg, model)
    return spec


def _apply_freezing(cfg, model, keep_frozen=False):
    """``unfrozen_parameters``: regex list; everything else is frozen (src/axolotl/utils/freeze.py:52-211)."""
    import re

    pats = cfg.get("unfrozen_parameters")
    if not pats:
        return
    regs = [re.compile(p) for p in pats]
    for n, p in model.named_parameters():
        hit = any(r.search(n) for r in regs)
        if hit:
            p.requires_grad_(True)
        elif not keep_frozen:
            p.requires_grad_(False)


def build_optimizer(cfg, model, parallel=None):
    pm = PluginManager.get_instance()
    custom = pm.first("create_optimizer", cfg, model)
    if custom is not None:
        return TorchOptimizerAdapter(custom, [p for p in model.parameters() if p.requires_grad],
                                     cfg.get("max_grad_norm") or 0.0, model)
    name = (cfg.get("optimizer") or "adamw_torch_fused").lower()
    groups = build_param_groups(model.named_parameters(), weight_decay=cfg.get("weight_decay") or 0.0,
                                embedding_lr=cfg.get("embedding_lr"), embedding_lr_scale=cfg.get("embedding_lr_scale"),
                                loraplus_lr_ratio=cfg.get("loraplus_lr_ratio"),
                                lr_groups=[dict(g) for g in (cfg.get("lr_groups") or [])] or None,
                                lr=float(cfg["learning_rate"]), per_layer=bool(cfg.get("lisa_n_layers")))
    betas = (cfg.get("adam_beta1") or 0.9, cfg.get("adam_beta2") or 0.999)
    eps = cfg.get("adam_epsilon") or 1e-8
    if name in ("adamw_torch", "adamw_torch_fused", "adamw_hf", "adamw", "adamw_anyprecision", "adamw_apex_fused"):
        world = parallel.dp_size if parallel is not None else 1
        opt = FlatAdamW(groups, lr=float(cfg["learning_rate"]), betas=betas, eps=eps,
                        max_grad_norm=cfg.get("max_grad_norm") or 0.0,
                        alloc=parallel.optimizer_alloc() if parallel is not None else None, pad_multiple=8 * max(world, 1),
                    moment_shard=parallel.moment_shard() if parallel is not None else None)
        opt.bind_model_shadows(model)
        return opt
    from .optimizers_extra import build_torch_optimizer

    params = [{"params": [p for _, p in g["params"]], "lr": float(cfg["learning_rate"]) * g["lr_scale"],
               "weight_decay": g["weight_decay"]} for g in groups]
    topt = build_torch_optimizer(name, params, lr=float(cfg["learning_rate"]), betas=betas, eps=eps, cfg=cfg)
    if hasattr(topt, "mark_adamw"):   # Muon: embeddings, the output head and adapter-side matrices keep AdamW
        topt.mark_adamw([p for g in groups for n, p in g["params"]
                         if any(k in n for k in ("embed_tokens", "lm_head", "embed_lora", "token_rows"))])
    return TorchOptimizerAdapter(topt, [p for g in groups for _, p in g["params"]], cfg.get("max_grad_norm") or 0.0, model)


def make_batches_fn(cfg, ds, rank, dp_size, parallel=None, is_eval=False):
    """callable(epoch) -> iterator of collated micro-batches for this data-parallel rank."""
    tok_pad = cfg.get("pad_token_id") or 0
    packing = bool(cfg.get("eval_sample_packing") if is_eval else cfg.get("sample_packing"))
    mbs = (cfg.get("eval_batch_size") if is_eval else cfg.get("micro_batch_size")) or 1
    seq = (cfg.get("eval_sequence_len") if is_eval else None) or cfg["sequence_len"]
    pad_to_seq = bool(cfg.get("pad_to_sequence_len"))
    coll = PackedCollator(tok_pad, cfg.get("pad_to_multiple_of") or 64, seq, pad_to_seq)
    custom = PluginManager.get_instance().first("get_collator_cls_and_kwargs", cfg, is_eval)
    if custom is not None:   # a plugin supplies the collator (e.g. knowledge distillation targets)
        coll = custom[0](**custom[1])
    agree = (lambda n: int(parallel.min_scalar(n))) if (parallel is not None and dp_size > 1) else None

    if packing:
        samp = MultipackBatchSampler(ds.lengths, seq, mbs, real_batches=bool(cfg.get("multipack_real_batches")),
                                     bin_size=cfg.get("sample_packing_bin_size") or 200,
                                     group_size=cfg.get("sample_packing_group_size") or 100_000,
                                     sequential=bool(cfg.get("sample_packing_sequentially")),
                                     shuffle=not (is_eval or cfg.get("curriculum_sampling")), seed=cfg.get("seed") or 42,
                                     rank=rank, world_size=dp_size, len_agree_fn=agree)

        def packed(epoch=0):
            samp.set_epoch(epoch)
            for bins in samp:
                yield coll([[ds[i] for i in b] for b in bins])

        return packed, samp

    def plain(epoch=0):
        n = len(ds)
        order = np.arange(n) if (is_eval or cfg.get("curriculum_sampling")) else np.random.default_rng((cfg.get("seed") or 42) + epoch).permutation(n)
        if cfg.get("group_by_length") and not is_eval:
            chunks = [order[i:i + mbs * 50] for i in range(0, n, mbs * 50)]
            order = np.concatenate([c[np.argsort(-ds.lengths[c], kind="stable")] for c in chunks]) if chunks else order
        per_rank = (n // (mbs * dp_size)) * mbs if not is_eval else None
        mine = order[rank::dp_size]
        if per_rank is not None:
            mine = mine[:per_rank]
        for i in range(0, len(mine), mbs):
            idx = mine[i:i + mbs]
            if len(idx) < mbs and not is_eval:
                break
            yield coll([[ds[j]] for j in idx])

    return plain, None


class RowDataset:
    """Pre-tokenised rows kept as dicts (extra per-token fields survive, unlike TokenizedDataset)."""

    def __init__(self, rows):
        self.rows = rows
        self.lengths = np.array([len(r["input_ids"]) for r in rows], dtype=np.int32)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[int(i)]


def load_row_datasets(cfg) -> TrainDatasetMeta:
    from ..data.loading import _shard, calculate_total_num_steps, read_raw

    rows = []
    for d in cfg.get("datasets") or []:
        for r in _shard(read_raw(dict(d)), dict(d)):
            if len(r["input_ids"]) <= cfg["sequence_len"]:
                r.setdefault("labels", r["input_ids"])
                rows.append(r)
    ds = RowDataset(rows)
    meta = TrainDatasetMeta(ds, None, None)
    meta.total_num_steps = calculate_total_num_steps(cfg, ds)
    return meta


def build_objective_run(cfg, model, tokenizer, device, parallel, dp_rank, dp_size, spec):
    """Batches + ``compute_loss`` object for ``rl:`` / ``reward_model`` runs. Returns
    (train_batches(epoch) callable, objective, micro-batches per epoch)."""
    import copy

    rl = cfg.get("rl")
    pad = cfg.get("pad_token_id") or 0
    seed = cfg.get("seed") or 42
    mbs = cfg["micro_batch_size"]
    if rl in ("grpo", "gdpo", "ebft"):
        from ..rl import grpo as G

        st = G.GRPOSettings(cfg)
        eos = tokenizer.eos_token_id if tokenizer is not None else cfg.get("eos_token_id")
        if st.use_vllm:
            sync_dir = os.path.join(cfg["output_dir"], "rollout_adapter")
            engine = G.VLLMServerRollout(st.host, st.port, adapter_sync_dir=sync_dir if spec is not None else None,
                                         save_adapter_fn=(lambda d: save_adapter(model, spec, d)) if spec is not None else None)
        else:
            engine = G.LocalRollout(model, eos, pad, seed + dp_rank)
        if eos is not None and cfg.get("eos_token_id") is None:
            cfg["eos_token_id"] = eos
        engine = PluginManager.get_instance().first("wrap_rollout_engine", cfg, engine) or engine
        eb = dict(cfg.get("ebft") or {}) if rl == "ebft" else {}
        if eb.get("mode") == "strided":
            from ..rl.ebft import load_strided_records

            # short anchored rollouts: sample count, length and sampling temperature come from the ebft block
            st.num_generations = int(eb.get("n_samples_per_prompt") or 4)
            st.max_completion_length = int(eb.get("generate_max_len") or 8)
            st.temperature = float(eb.get("temperature") if eb.get("temperature") is not None else 0.6)
            st.top_p = float(eb.get("top_p") if eb.get("top_p") is not None else 1.0)
            st.scale_rewards = "rloo" if (eb.get("advantage_estimator") or "rloo") == "rloo" else st.scale_rewards
            records = load_strided_records(cfg, tokenizer)
        else:
            records = G.load_prompt_records(cfg, tokenizer)
        extra = (cfg.get("trl") or {}).get("reward_funcs") or []
        reward_funcs = G.load_reward_funcs(extra) if (extra or rl != "ebft") else []
        if rl == "ebft":   # feature-matching reward from the frozen policy (adapters off, or a frozen copy)
            from ..rl.ebft import FeatureMatchingReward

            frozen = copy.deepcopy(model).requires_grad_(False) if spec is None else None
            reward_funcs = [FeatureMatchingReward(model, tokenizer, cfg.get("ebft"), st.num_generations, frozen)] + reward_funcs
        producer = G.RolloutProducer(model, engine, reward_funcs,
                                     st, records, mbs, tokenizer, pad, eos, dp_rank, dp_size, seed)
        return producer, G.GRPOObjective(st, producer), len(producer) * st.num_iterations
    from ..rl.data import PreferenceBatches, load_preference_dataset
    from ..rl.objectives import build_objective, precompute_reference_logps

    ref_model = None
    if spec is None and rl in ("dpo", "ipo", "kto"):
        ref_model = copy.deepcopy(model).requires_grad_(False)   # full fine-tune: frozen copy as reference
    dp_group = parallel.dp_group if parallel is not None else None
    obj = build_objective(cfg, ref_model, pad, dp_group)
    if cfg.get("process_reward_model"):
        meta = load_datasets(cfg)
        fn, _ = make_batches_fn(cfg, meta.train, dp_rank, dp_size, parallel)
        coll = obj.collator()

        def prm_batches(epoch):
            for b in fn(epoch):
                b["labels_preshifted"] = True
                b["n_trainable"] = int((b["labels"] != -100).sum())
                yield b

        return prm_batches, obj, max(len(meta.train) // (mbs * dp_size), 1)
    records = load_preference_dataset(cfg, tokenizer)
    coll = obj.collator()
    if cfg.get("precompute_ref_log_probs") and rl in ("dpo", "ipo"):
        precompute_reference_logps(model, records, coll, device, mbs, ref_model, average=getattr(obj, "average", False))
    batches = PreferenceBatches(records, coll, mbs, dp_rank, dp_size, seed)
    return batches, obj, len(batches)


def save_model_artifacts(model, cfg, spec, out_dir, parallel=None, rank=0):
    """Adapter (LoRA) or full HF checkpoint into ``out_dir`` (rank 0 writes)."""
    if spec is not None:
        if rank == 0:
            save_adapter(model, spec, out_dir)
        return
    sd_type = str((cfg.get("fsdp_config") or {}).get("state_dict_type") or "FULL_STATE_DICT").upper()
    if parallel is not None and parallel.fsdp is not None and sd_type == "SHARDED_STATE_DICT":
        # every rank writes its own rows; `axolotl merge-sharded-fsdp-weights` assembles the HF checkpoint
        hf_io.save_sharded_state(model, out_dir, parallel.fsdp.rank, parallel.fsdp.world)
        return
    if parallel is not None and parallel.fsdp is not None:
        parallel.materialize_full_weights(model)  # gathers sharded weights for saving
    if rank == 0:
        hf_io.save_pretrained(model, out_dir)


def setup_signal_handler(trainer, model, cfg, spec):
    def handler(signum, frame):  # SIGINT: save what we have and stop
        LOG.warning("signal %s received: saving and stopping", signum)
        trainer.should_stop = True
        trainer.should_save = True

    if trainer.rank == 0:
        try:
            signal.signal(signal.SIGINT, handler)
        except ValueError:
            pass  # not the main thread


def train(cfg, dataset_meta: TrainDatasetMeta | None = None):
    try:
        return _train(cfg, dataset_meta)
    finally:
        stop_debug_log()


def _train(cfg, dataset_meta: TrainDatasetMeta | None = None):
    torch.manual_seed(cfg.get("seed") or 42)
    np.random.seed(cfg.get("seed") or 42)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    use_cuda = torch.cuda.is_available() and cfg.get("device") != "cpu"
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1:
        from ..parallel.runtime import init_distributed

        init_distributed(timeout_s=cfg.get("ddp_timeout"))
    start_debug_log(cfg["output_dir"], append=bool(cfg.get("resume_from_checkpoint")))
    pm = PluginManager.get_instance()

    tokenizer = None
    if cfg.get("base_model") and os.path.isdir(cfg["base_model"]) and any(
            os.path.exists(os.path.join(cfg["base_model"], f)) for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        from ..data.tokenizer import load_tokenizer

        tokenizer = load_tokenizer(cfg)
        cfg["pad_token_id"] = tokenizer.pad_token_id
    objective_mode = bool(cfg.get("rl") or cfg.get("reward_model"))   # preference / online-RL objectives
    streaming = bool(cfg.get("pretraining_dataset") or cfg.get("streaming")) and not objective_mode
    multimodal = bool(cfg.get("processor_type") or cfg.get("is_multimodal")) and not objective_mode
    if dataset_meta is None and multimodal:
        from ..data.loading import _shard, read_raw
        from ..data.multimodal import RawConversationDataset

        rows = [r for d in (cfg.get("datasets") or []) for r in _shard(read_raw(dict(d)), dict(d))]
        n_val = int(len(rows) * cfg["val_set_size"]) if cfg.get("val_set_size") and cfg["val_set_size"] < 1 else int(cfg.get("val_set_size") or 0)
        dataset_meta = TrainDatasetMeta(RawConversationDataset(rows[n_val:]), RawConversationDataset(rows[:n_val]) if n_val else None)
        per_step = cfg["micro_batch_size"] * cfg["gradient_accumulation_steps"] * int(os.environ.get("WORLD_SIZE", "1"))
        dataset_meta.total_num_steps = max(int(len(rows[n_val:]) // per_step * (cfg.get("num_epochs") or 1)), 1)
    if dataset_meta is None and cfg.get("kd_trainer"):
        dataset_meta = load_row_datasets(cfg)
    if dataset_meta is None and not objective_mode and not streaming:
        dataset_meta = load_datasets(cfg)

    remote = pm.first("run_training", cfg, dataset_meta, tokenizer)
    if remote is not None:            # a plugin trained elsewhere (remote service): no local model, nothing to save
        return remote

    model = build_model(cfg, device)
    if tokenizer is not None:
        want = len(tokenizer)
        if want > model.config.vocab_size or (cfg.get("shrink_embeddings") and want < model.config.vocab_size):
            new = model.resize_token_embeddings(want, 32 if cfg.get("resize_token_embeddings_to_32x") else None,
                                                bool(cfg.get("mean_resizing_embeddings")))
            LOG.info("token embeddings resized to %d rows (tokenizer has %d tokens)", new, want)
    parallel = None
    if world > 1:
        from ..parallel.runtime import create_runtime

        parallel = create_runtime(device=device, dp_shard=cfg.get("dp_shard_size"),
                                  dp_replicate=cfg.get("dp_replicate_size") or 1, tp=cfg.get("tensor_parallel_size") or 1,
                                  cp=cfg.get("context_parallel_size") or 1, ep=cfg.get("expert_parallel_size") or 1)
        parallel.tp_max_tokens = cfg["micro_batch_size"] * cfg["sequence_len"]
        raf = (cfg.get("fsdp_config") or {}).get("reshard_after_forward")
        parallel.reshard_after_forward = True if raf is None else bool(raf)
        parallel.apply_tp(model)          # shards projections before adapters are created
    spec = setup_adapter(cfg, model)
    if getattr(model, "vision", None) is not None and cfg.get("freeze_mm_modules") is False:
        for p_ in model.vision.parameters():       # the image tower and projector train with the language model
            p_.requires_grad_(True)
    pm.call("post_model_load", cfg, model)
    if cfg.get("gradient_checkpointing") or (cfg.get("fsdp_config") or {}).get("activation_checkpointing"):
        ao = cfg.get("activation_offloading") or None
        model.enable_gradient_checkpointing(True, offload=ao, selective=bool(cfg.get("selective_checkpointing")),
                                            offload_dir=os.path.join(cfg["output_dir"], "activation_offload") if ao == "disk" else None)
        if ao in (True, "legacy", "disk"):
            model.offload_saved_store = model.ckpt_store   # also park what autograd saves outside the layers
        if ao:
            LOG.info("activation offloading: checkpointed layer inputs go to %s", "disk" if ao == "disk" else "pinned host memory")
    if cfg.get("layer_offloading"):
        from .activation_memory import LayerOffloader

        model.layer_offloader = LayerOffloader(model, device)
        LOG.info("layer offloading: %.2f GiB of frozen layer weights kept in pinned host memory",
                 sum(model.layer_offloader.bytes_per_layer) / 1024 ** 3)

    dp_size, dp_rank = 1, 0
    if parallel is not None:
        parallel.shard_model(model)       # FSDP row-sharding of the frozen weights
        dp_size, dp_rank = parallel.dp_size, parallel.dp_rank

    if cfg.get("reward_model") or cfg.get("process_reward_model"):
        from ..rl.objectives import add_score_head

        add_score_head(model, 2 if cfg.get("process_reward_model") else 1, cfg.get("seed") or 42)
    opt = build_optimizer(cfg, model, parallel)
    if parallel is not None:
        parallel.attach_optimizer(opt)

    objective = None
    eval_fn = None
    if objective_mode:
        train_fn, objective, n_batches = build_objective_run(cfg, model, tokenizer, device, parallel, dp_rank, dp_size, spec)
        dataset_meta = TrainDatasetMeta(train=None, eval=None, total_num_steps=max(
            int(n_batches * (cfg.get("num_epochs") or 1)) // cfg["gradient_accumulation_steps"], 1))
    elif streaming:
        from ..data.streaming import StreamingPackedBatches

        if tokenizer is None:
            from ..data.tokenizer import load_tokenizer

            tokenizer = load_tokenizer(cfg)
            cfg["pad_token_id"] = tokenizer.pad_token_id
        train_fn = StreamingPackedBatches(cfg, cfg.get("pretraining_dataset") or cfg.get("datasets"), tokenizer,
                                          dp_rank, dp_size)
        dataset_meta = TrainDatasetMeta(train=None, eval=None, total_num_steps=cfg["max_steps"])
        if cfg.get("test_datasets"):
            ev = load_datasets(dict(cfg, datasets=cfg["test_datasets"], test_datasets=None, val_set_size=None), tokenizer)
            eval_fn, _ = make_batches_fn(cfg, ev.train, dp_rank, dp_size, parallel, is_eval=True)
    elif multimodal:
        from ..data import multimodal as mm

        if getattr(model, "vision", None) is None:
            raise ValueError(f"multimodal training needs a checkpoint with an image front end this package builds (LLaVA: CLIP "
                             f"tower + projector; Gemma 3: SigLIP tower + pooling projector); '{model.config.model_type}' was loaded as a language model only")
        if cfg.get("sample_packing"):
            raise ValueError("sample_packing is not available for multimodal datasets (batches are already padding-free)")
        processor = mm.load_processor(cfg, tokenizer)
        d0 = dict((cfg.get("datasets") or [{}])[0])
        strategy = mm.get_processing_strategy(
            processor, cfg.get("chat_template_jinja"), cfg.get("chat_template"), image_size=cfg.get("image_size"),
            image_resize_algorithm=cfg.get("image_resize_algorithm"), train_on_inputs=bool(cfg.get("train_on_inputs")),
            roles_to_train=d0.get("roles_to_train"), train_on_eos=d0.get("train_on_eos"),
            role_boundaries=d0.get("role_boundaries") or cfg.get("role_boundaries"), field_messages=d0.get("field_messages"))
        collator = mm.MultiModalChatCollator(getattr(processor, "tokenizer", tokenizer), strategy)
        train_fn, sampler = mm.make_multimodal_batches_fn(cfg, dataset_meta.train, collator, dp_rank, dp_size), None
        if dataset_meta.eval is not None and len(dataset_meta.eval):
            eval_fn = mm.make_multimodal_batches_fn(cfg, dataset_meta.eval, collator, dp_rank, dp_size, is_eval=True)
    else:
        train_fn, sampler = make_batches_fn(cfg, dataset_meta.train, dp_rank, dp_size, parallel)
        if dataset_meta.eval is not None and len(dataset_meta.eval):
            eval_fn, _ = make_batches_fn(cfg, dataset_meta.eval, dp_rank, dp_size, parallel, is_eval=True)
    total = dataset_meta.total_num_steps or cfg.get("max_steps") or 0
    if cfg.get("max_steps"):
        total = min(total, cfg["max_steps"]) if total else cfg["max_steps"]
    warm = default_warmup_steps(total, cfg.get("warmup_steps"), cfg.get("warmup_ratio"))
    sched = pm.first("create_lr_scheduler", cfg, opt, total)
    lr_lambda = sched or make_lr_lambda(
        "cosine_with_quadratic_warmup" if cfg.get("lr_quadratic_warmup") else
        ("cosine_with_min_lr" if cfg.get("cosine_min_lr_ratio") and (cfg.get("lr_scheduler") or "cosine") == "cosine" else cfg.get("lr_scheduler")),
        total, warm, min_lr_ratio=cfg.get("cosine_min_lr_ratio") or 0.0,
        constant_lr_ratio=cfg.get("cosine_constant_lr_ratio"), **(cfg.get("lr_scheduler_kwargs") or {}))
    if cfg.get("jagged_restart_steps") and sched is None:
        from .optimizer import jagged_restarts

        lr_lambda = jagged_restarts(lr_lambda, cfg["jagged_restart_steps"], cfg.get("jagged_restart_warmup_steps") or 10,
                                    cfg.get("jagged_restart_anneal_steps") or 1)
    logging_steps = cfg.get("logging_steps") or max(min(int(0.005 * total), 10), 1)
    args = TrainArgs(output_dir=cfg["output_dir"], max_steps=total, num_epochs=cfg.get("num_epochs") or 1,
                     micro_batch_size=cfg["micro_batch_size"], gradient_accumulation_steps=cfg["gradient_accumulation_steps"],
                     learning_rate=float(cfg["learning_rate"]), weight_decay=cfg.get("weight_decay") or 0.0,
                     max_grad_norm=cfg.get("max_grad_norm") or 0.0, logging_steps=logging_steps,
                     save_steps=cfg.get("save_steps"), save_strategy=cfg.get("save_strategy") or ("steps" if cfg.get("save_steps") else "no"),
                     save_total_limit=cfg.get("save_total_limit"), save_only_model=bool(cfg.get("save_only_model")),
                     save_first_step=bool(cfg.get("save_first_step")), eval_steps=cfg.get("eval_steps"),
                     eval_strategy=cfg.get("eval_strategy") or "no", seed=cfg.get("seed") or 42,
                     include_tkps=cfg.get("include_tkps", True) is not False,
                     gradient_checkpointing=bool(cfg.get("gradient_checkpointing")))
    resume = cfg.get("resume_from_checkpoint")
    if not resume and cfg.get("auto_resume_from_checkpoints"):
        resume = find_last_checkpoint(cfg["output_dir"])
    args.resume_from_checkpoint = resume

    def save_fn(trainer, ckpt_dir):
        save_model_artifacts(model, cfg, spec, ckpt_dir, parallel, trainer.rank)

    callbacks = build_callbacks(cfg) + pm.collect_callbacks("add_callbacks_pre_trainer", cfg, model)
    trainer_cls = pm.first("get_trainer_cls", cfg) or Trainer
    trainer = trainer_cls(model, opt, lr_lambda, args, train_fn, eval_batches=eval_fn, parallel=parallel,
                          callbacks=callbacks, save_fn=save_fn, device=device, total_steps=total,
                          compute_loss=objective or pm.first("compute_loss", cfg))
    if world > 1 and cfg.get("peer_heartbeat_timeout") != 0:
        from ..parallel.health import HeartbeatCallback, HeartbeatMonitor

        trainer.callbacks.append(HeartbeatCallback(HeartbeatMonitor(timeout_s=cfg.get("peer_heartbeat_timeout") or 600)))
    trainer.callbacks += pm.collect_callbacks("add_callbacks_post_trainer", cfg, trainer)
    pm.call("post_trainer_create", cfg, trainer)

    # up-front artefacts
    if rank == 0:
        os.makedirs(cfg["output_dir"], exist_ok=True)
        model.config.save_pretrained(cfg["output_dir"])
        if spec is not None:
            spec.save(cfg["output_dir"])
        if tokenizer is not None:
            tokenizer.save_pretrained(cfg["output_dir"])
    if resume and spec is not None and os.path.exists(os.path.join(resume, "adapter_model.safetensors")):
        load_adapter(model, resume)
    setup_signal_handler(trainer, model, cfg, spec)
    if cfg.get("generate_samples") and dataset_meta is not None and (dataset_meta.eval or dataset_meta.train) is not None:
        from .callbacks import SampleGenerationCallback

        src = dataset_meta.eval if dataset_meta.eval is not None and len(dataset_meta.eval) else dataset_meta.train
        n = min(cfg.get("num_generation_samples") or 3, len(src))
        trainer.callbacks.append(SampleGenerationCallback(cfg, [src[i] for i in range(n)], tokenizer))
    if cfg.get("tiled_mlp"):
        import math as _math

        shards = cfg.get("tiled_mlp_num_shards") or max(1, _math.ceil(cfg["sequence_len"] * cfg["micro_batch_size"] / 8192))
        rows = max(256, _math.ceil(cfg["sequence_len"] * cfg["micro_batch_size"] / shards / 128) * 128)
        n = 0
        for layer in model.layers:
            if hasattr(layer.mlp, "tile_rows"):
                layer.mlp.tile_rows = rows
                n += 1
        LOG.info("tiled MLP: %d layers, %d rows per tile", n, rows)
    if cfg.get("qat"):
        q = dict(cfg["qat"])
        start = q.get("fake_quant_after_n_steps") or 0
        mods = [m for n, m in model.fused_linears() if n.startswith("layers.") and hasattr(m, "qat")]

        class _QATStart(Callback):
            def on_step_end(self, trainer, logs):
                if trainer.global_step == start:
                    for m in mods:
                        m.qat = q

        if start <= 0:
            for m in mods:
                m.qat = q
        else:
            trainer.callbacks.append(_QATStart())
        if q.get("quantize_embedding"):
            # the embedding table is rounded to the weight grid in place at every optimizer step end
            from ..ops.fake_quant import fake_quantize

            class _QATEmbedding(Callback):
                def on_step_end(self, trainer, logs):
                    if trainer.global_step >= start and model.embed_tokens.requires_grad:
                        with torch.no_grad():
                            model.embed_tokens.copy_(fake_quantize(model.embed_tokens, q.get("weight_dtype"), q.get("group_size")))

            trainer.callbacks.append(_QATEmbedding())
        LOG.info("QAT: %d projections fake-quantised to %s (group %s, activations %s)", len(mods), q.get("weight_dtype"),
                 q.get("group_size"), q.get("activation_dtype"))
    if cfg.get("neftune_noise_alpha"):
        model.neftune_noise_alpha = float(cfg["neftune_noise_alpha"])

    trainer.train()

    if cfg.get("merge_lora") and spec is not None:
        from ..models.lora import merge_and_unload

        merge_and_unload(model)
        spec = None
    save_model_artifacts(model, cfg, spec, cfg["output_dir"], parallel, rank)
    if rank == 0:
        _write_model_card(cfg, trainer)
    pm.call("post_train", cfg, model)
    if parallel is not None:
        parallel.barrier()
    return model, tokenizer, trainer


def _write_model_card(cfg, trainer):
    last = next((l for l in reversed(trainer.log_history) if "loss" in l), {})
    with open(os.path.join(cfg["output_dir"], "README.md"), "w") as fh:
        fh.write(f"# {os.path.basename(os.path.normpath(cfg['output_dir']))}\n\n"
                 f"Fine-tuned from `{cfg.get('base_model') or cfg.get('model_preset')}` with axolotl_b200.\n\n"
                 f"- steps: {trainer.global_step}\n- final loss: {last.get('loss')}\n"
                 f"- adapter: {cfg.get('adapter')}\n- sequence_len: {cfg.get('sequence_len')}\n"
                 f"- learning_rate: {cfg.get('learning_rate')}\n")
