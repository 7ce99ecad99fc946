"""Drives the unmodified reference (installed under ``baseline/_ref``) on the headline config.

``run_reference(n_gpus, steps, warmup)`` writes, into a scratch directory,
  * a model directory with only ``config.json`` (Llama-3-8B architecture) and a minimal word-level
    tokenizer — the weights are random (``reinit_weights: true``, src/axolotl/loaders/model.py:942-943),
  * a PRE-TOKENISED json dataset with sample lengths uniform in [256, 4096] (``input_ids``,
    ``attention_mask``, ``labels``: the reference takes such rows as they are,
    src/axolotl/utils/data/wrappers.py:134-141),
  * the YAML of the run: LoRA r=16 / alpha=32 on all linear layers, ``sample_packing`` into
    8192-token rows, micro-batch 1, no accumulation, bf16, fused AdamW, FSDP2 when more than one rank,
then calls the reference's own entry point ``axolotl.cli.train.do_cli`` in THIS process (under
torchrun every rank does so, exactly like ``axolotl train``), with ``ref_timing_plugin.TimingPlugin``
registered through the reference's plugin list to time steps W+1..W+K. Returns the bench line as a
dict, or ``{"impl": "reference", "unavailable": reason}``. Nothing of ``axolotl_b200`` is imported.
"""
from __future__ import annotations

import importlib
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REQUIRED = ("peft", "accelerate", "trl", "colorama", "datasets")
SEQ_LEN = 8192

LLAMA3_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096, "intermediate_size": 14336,
    "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "vocab_size": 128256,
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "hidden_act": "silu",
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
    "attention_bias": False, "mlp_bias": False,
}


def missing_modules(required=REQUIRED):
    out = []
    for mod in required:
        try:
            importlib.import_module(mod)
        except Exception:
            out.append(mod)
    return out


def write_model_dir(path, arch=None):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(arch or LLAMA3_8B, fh, indent=1)
    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2, "<unk>": 3}
    vocab.update({f"t{i}": i for i in range(4, 64)})
    tok = {"version": "1.0", "truncation": None, "padding": None,
           "added_tokens": [{"id": i, "content": c, "single_word": False, "lstrip": False, "rstrip": False,
                             "normalized": False, "special": True} for c, i in list(vocab.items())[:4]],
           "normalizer": None, "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
           "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "<unk>"}}
    with open(os.path.join(path, "tokenizer.json"), "w") as fh:
        json.dump(tok, fh)
    with open(os.path.join(path, "tokenizer_config.json"), "w") as fh:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "bos_token": "<s>", "eos_token": "</s>",
                   "pad_token": "<pad>", "unk_token": "<unk>", "model_max_length": SEQ_LEN}, fh)
    with open(os.path.join(path, "special_tokens_map.json"), "w") as fh:
        json.dump({"bos_token": "<s>", "eos_token": "</s>", "pad_token": "<pad>", "unk_token": "<unk>"}, fh)


def write_dataset(path, n_samples, vocab_size, seed=0, min_len=256, max_len=4096):
    """One json line per sample, already tokenised; labels equal the inputs."""
    import numpy as np

    rng = np.random.default_rng(seed)
    with open(path, "w") as fh:
        for _ in range(n_samples):
            n = int(rng.integers(min_len, max_len + 1))
            ids = rng.integers(3, vocab_size, size=n).tolist()
            fh.write(json.dumps({"input_ids": ids, "attention_mask": [1] * n, "labels": ids}) + "\n")


def write_config(path, *, model_dir, data_file, out_dir, n_gpus, steps, warmup, seq_len=SEQ_LEN):
    import yaml

    cfg = {
        "base_model": model_dir, "reinit_weights": True, "tokenizer_type": "AutoTokenizer",
        "load_in_8bit": False, "load_in_4bit": False,
        "adapter": "lora", "lora_r": 16, "lora_alpha": 32, "lora_dropout": 0.0, "lora_target_linear": True,
        "datasets": [{"path": data_file, "ds_type": "json", "type": None}],
        "dataset_prepared_path": os.path.join(out_dir, "prepared"), "val_set_size": 0,
        "sequence_len": seq_len, "sample_packing": True, "pad_to_sequence_len": True,
        "micro_batch_size": 1, "gradient_accumulation_steps": 1, "max_steps": steps + warmup, "num_epochs": 1,
        "optimizer": "adamw_torch_fused", "lr_scheduler": "constant", "learning_rate": 2e-4, "warmup_steps": 0,
        "bf16": True, "tf32": True, "flash_attention": True, "gradient_checkpointing": False,
        "logging_steps": 1, "save_strategy": "no", "output_dir": os.path.join(out_dir, "out"),
        "plugins": ["ref_timing_plugin.TimingPlugin"], "seed": 0, "strict": False,
    }
    if n_gpus > 1:
        cfg["fsdp_version"] = 2
        cfg["fsdp_config"] = {"offload_params": False, "state_dict_type": "FULL_STATE_DICT",
                              "auto_wrap_policy": "TRANSFORMER_BASED_WRAP",
                              "transformer_layer_cls_to_wrap": "LlamaDecoderLayer", "reshard_after_forward": True}
    with open(path, "w") as fh:
        yaml.safe_dump(cfg, fh, sort_keys=False)
    return cfg


def run_reference(n_gpus, steps, warmup, *, ref_path=None, required=REQUIRED, arch=None, seq_len=SEQ_LEN,
                  work_dir=None):
    ref_path = ref_path or os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_path, "axolotl")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-index --no-deps "
                                                    "--target baseline/_ref <reference checkout>)"}
    miss = missing_modules(required)
    if miss:
        return {"impl": "reference",
                "unavailable": "reference installed with --no-deps but its runtime dependencies are not in the image or "
                               f"the offline wheelhouse: {', '.join(miss)} (axolotl.train imports them at module load)"}
    for p in (ref_path, HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    arch = arch or LLAMA3_8B
    # every rank must see the same files: the directory name is derived from the rendezvous, rank 0 writes
    tag = os.environ.get("MASTER_PORT", "0") + "_" + os.environ.get("TORCHELASTIC_RUN_ID", "solo")
    work = work_dir or os.path.join(tempfile.gettempdir(), f"axb_ref_{tag}_{steps}_{warmup}")
    model_dir, data_file, cfg_path = os.path.join(work, "model"), os.path.join(work, "data.jsonl"), os.path.join(work, "cfg.yml")
    timing = os.path.join(work, "timing.json")
    done_flag = os.path.join(work, "inputs_ready")
    if rank == 0:
        os.makedirs(work, exist_ok=True)
        if os.path.exists(timing):
            os.remove(timing)
        write_model_dir(model_dir, arch)
        per_step = max(8, 2 * seq_len // 2176 + 2)      # mean sample length 2176: ~4 samples per row, with slack
        write_dataset(data_file, (steps + warmup + 2) * per_step * max(world, 1), arch["vocab_size"])
        write_config(cfg_path, model_dir=model_dir, data_file=data_file, out_dir=work, n_gpus=world, steps=steps,
                     warmup=warmup, seq_len=seq_len)
        open(done_flag, "w").close()
    else:
        import time

        t0 = time.time()
        while not os.path.exists(done_flag):
            if time.time() - t0 > 600:
                return {"impl": "reference", "unavailable": "rank 0 never wrote the benchmark inputs"}
            time.sleep(0.2)
    os.environ["AXB_REF_WARMUP"], os.environ["AXB_REF_STEPS"] = str(warmup), str(steps)
    os.environ["AXB_REF_TIMING_OUT"] = timing
    try:
        train_cli = importlib.import_module("axolotl.cli.train")
    except Exception as exc:
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"}
    argv = sys.argv
    sys.argv = ["axolotl.cli.train", cfg_path]
    try:
        train_cli.do_cli(config=cfg_path)
    except SystemExit:
        pass
    except Exception as exc:
        return {"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}"}
    finally:
        sys.argv = argv
    if rank != 0:
        return None
    if not os.path.exists(timing):
        return {"impl": "reference", "unavailable": "the reference run ended without reaching the timed steps"}
    with open(timing) as fh:
        t = json.load(fh)
    tokens = seq_len * world * t["steps"]
    value = tokens / (t["device_ms"] / 1e3)
    e2e = tokens / (t["host_ms"] / 1e3)
    return {
        "metric": "train tokens/s/box (max over ranks), Llama-3-8B LoRA FSDP2", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": t["steps"], "warmup": t["warmup"], "ms_per_step": t["device_ms"] / t["steps"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, lengths U[256,4096], pre-tokenised, packed to 8192 by the reference's "
                "multipack sampler; random-init weights (reinit_weights)",
        "impl": "reference",
        "config": {"model": "llama-3-8b" if arch is LLAMA3_8B else arch.get("model_type", "?"), "global_batch": world,
                   "seq_len": seq_len, "parallelism": f"fsdp{world}" if world > 1 else "single", "lora_r": 16,
                   "lora_alpha": 32, "optimizer": "adamw_torch_fused", "grad_accum": 1, "micro_batch": 1},
        # the reference's loop copies every batch from the host and logs the loss every step: its
        # device-timed and end-to-end figures cover the same work
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": t["host_ms"] / t["steps"],
                "h2d_bytes_per_step": 3 * seq_len * 8, "d2h_bytes_per_step": 4, "last_loss": t["last_loss"]},
        "peak_mem_gib": t["peak_mem_gib"],
    }
