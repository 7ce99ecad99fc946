"""Headline benchmark: train tokens/s per box, Llama-3-8B LoRA (r=16, alpha=32, all linear layers,
frozen bf16 base), FSDP-style sharding over N GPUs of one node, synthetic packed data.

  python bench.py --gpus 1 --steps 5 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
         --master-port P bench.py --gpus N --steps K --warmup W

Prints ONE JSON line (rank 0). ``value`` is the device-timed aggregate over all GPUs with the
step's inputs already resident on the device; ``e2e`` repeats the measurement through the public
``Trainer.training_step`` API with a host->device copy of every step's pinned inputs and a
device->host read of every step's loss. ``--impl reference`` runs the unmodified reference package
from ``baseline/_ref`` on the same config through its own CLI entry (baseline/ref_harness.py); it
reports ``unavailable`` with the reason when that package or its dependencies cannot be imported.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEQ_LEN = 8192
MODEL = "llama-3-8b"


def _env_int(k, d):
    return int(os.environ.get(k, d))


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        # median over samples taken under load (upper half of the distribution)
        load = sm[len(sm) // 2:] if sm else []
        med = load[len(load) // 2] if load else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """Runs the unmodified reference from baseline/_ref through its own ``axolotl.cli.train`` entry
    (see baseline/ref_harness.py), or explains in one line why it cannot run here. Nothing of
    axolotl_b200 is imported on this path."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import ref_harness

    if args.config != "lora8b":
        res = {"impl": "reference", "unavailable": "the reference arm is wired for the headline config only"}
    else:
        res = ref_harness.run_reference(args.gpus, args.steps, max(args.warmup, 3))
    if _env_int("RANK", 0) == 0 and res is not None:
        print(json.dumps(res))
    return 0


def build_batches(n_batches, vocab, seed, rank, seq_len=SEQ_LEN, rows=1, min_len=256, max_len=4096):
    """Synthetic packed batches: sample lengths uniform in [256, 4096], packed first-fit into
    ``seq_len``-token rows (``rows`` rows per micro-batch), labels == inputs, position ids restart
    per sample."""
    from axolotl_b200.data.collator import PackedCollator
    from axolotl_b200.data.packing import MultipackBatchSampler
    from axolotl_b200.data.synthetic import synthetic_varlen

    ds = synthetic_varlen(max(64, n_batches * 6 * rows * max(1, seq_len // 8192)), min_len, min(max_len, seq_len), 3, vocab,
                          0.0, seed=seed + 1000 * rank)
    samp = MultipackBatchSampler(ds.lengths, seq_len, rows, real_batches=True, seed=seed)
    coll = PackedCollator(pad_token_id=0, sequence_len=seq_len, pad_to_sequence_len=True)
    out = []
    for b in samp:
        out.append(coll([[ds[i] for i in bin_] for bin_ in b]))
        if len(out) == n_batches:
            break
    while len(out) < n_batches:
        out.append(out[len(out) % max(1, len(out))])
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is then not the headline config)")
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--config", default="lora8b", choices=["lora8b", "moe", "tp70b", "cp64k"],
                    help="lora8b: the headline Llama-3-8B LoRA FSDP run; moe: Qwen3-MoE-30B-A3B with NVFP4 experts, "
                         "expert + attention LoRA, expert parallelism over all ranks (4096-token rows, micro-batch 2); "
                         "tp70b: Llama-3-70B LoRA, TP=2 x FSDP=N/2, activation checkpointing; "
                         "cp64k: Llama-3-8B full fine-tune, context parallel over all ranks, one 65536-token row")
    ap.add_argument("--reshard-after-forward", default="true", choices=["true", "false"],
                    help="fsdp_config.reshard_after_forward of the headline run (false keeps gathered weights from the "
                         "forward to the backward pass of a step)")
    args = ap.parse_args()
    if args.model == MODEL:
        args.model = {"moe": "qwen3-moe-30b-a3b", "tp70b": "llama-3-70b"}.get(args.config, MODEL)
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from axolotl_b200.models.config import preset
    from axolotl_b200.models.lora import ALL_LINEAR, LoraSpec, inject_lora
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.ops import _lib
    from axolotl_b200.train.optimizer import FlatAdamW, build_param_groups, make_lr_lambda
    from axolotl_b200.train.trainer import TrainArgs, Trainer, h2d_bytes, to_device_batch

    world = _env_int("WORLD_SIZE", 1)
    rank = _env_int("RANK", 0)
    local_rank = _env_int("LOCAL_RANK", 0)
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    parallel = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    W, K = max(args.warmup, 3), args.steps

    overrides = {} if args.layers is None else {"num_hidden_layers": args.layers}
    cfg = preset(args.model, **overrides)
    torch.manual_seed(0)
    model = CausalLM(cfg, dtype=torch.bfloat16, device=dev).init_weights(0)
    if args.config == "moe":
        # random-init routers are far less balanced than trained ones: start the expert-parallel row capacity at
        # 3 x the mean load (an overflow would skip the step and grow it; skipped steps are reported below)
        os.environ.setdefault("AXB_EP_CAPACITY", "3.0")
        from axolotl_b200.ops.grouped import quantize_experts_nvfp4_

        quantize_experts_nvfp4_(model)
        inject_lora(model, LoraSpec(r=16, lora_alpha=32, target_modules=["q_proj", "k_proj", "v_proj", "o_proj"],
                                    target_parameters=["mlp.experts.gate_up_proj", "mlp.experts.down_proj"]))
        if world > 1:
            from axolotl_b200.parallel import build_parallel

            parallel = build_parallel(model, ep=world, device=dev)
    elif args.config == "tp70b":
        from axolotl_b200.parallel.runtime import create_runtime

        if world > 1:
            parallel = create_runtime(device=dev, tp=2, dp_shard=world // 2)
            parallel.tp_max_tokens = SEQ_LEN
            parallel.apply_tp(model)            # before the adapters exist
        inject_lora(model, LoraSpec(r=16, lora_alpha=32, target_modules=list(ALL_LINEAR)))
        if parallel is not None:
            parallel.shard_model(model)
        model.enable_gradient_checkpointing(True)
    elif args.config == "cp64k":
        if world > 1:
            from axolotl_b200.parallel import build_parallel

            parallel = build_parallel(model, cp=world, device=dev)
        model.enable_gradient_checkpointing(True)
    else:
        inject_lora(model, LoraSpec(r=16, lora_alpha=32, target_modules=list(ALL_LINEAR)))
        if world > 1:
            from axolotl_b200.parallel import build_parallel

            parallel = build_parallel(model, dp_shard=world, device=dev,
                                      reshard_after_forward=args.reshard_after_forward == "true")
    opt = FlatAdamW(build_param_groups(model.named_parameters(), weight_decay=0.0), lr=2e-4, max_grad_norm=1.0,
                    alloc=parallel.optimizer_alloc() if parallel is not None else None, pad_multiple=8 * max(world, 1),
                    moment_shard=parallel.moment_shard() if parallel is not None else None)
    opt.bind_model_shadows(model)
    if parallel is not None:
        parallel.attach_optimizer(opt)
    targs = TrainArgs(max_steps=10 ** 9, micro_batch_size=1, gradient_accumulation_steps=1, learning_rate=2e-4,
                      logging_steps=10 ** 9, include_tkps=False)
    trainer = Trainer(model, opt, make_lr_lambda("constant", 10 ** 6, 0), targs, lambda e: [], parallel=parallel, device=dev)
    model.train()

    seq_len = {"moe": 4096, "cp64k": 65536}.get(args.config, SEQ_LEN)
    # ranks of one context- or tensor-parallel group must see the same batch
    data_rank = 0 if args.config == "cp64k" else (rank // 2 if args.config == "tp70b" else rank)
    cpu_batches = build_batches(W + K, cfg.vocab_size, seed=0, rank=data_rank, seq_len=seq_len,
                                rows=2 if args.config == "moe" else 1, max_len=8192 if args.config == "cp64k" else 4096,
                                min_len=1024 if args.config == "cp64k" else 256)
    for b in cpu_batches:
        for k in ("input_ids", "labels", "position_ids"):
            b[k] = b[k].pin_memory()
    tokens_per_step = int(cpu_batches[0]["input_ids"].numel())
    # real (non-pad) and trainable tokens of the timed steps, next to the padded slot count
    real_tokens = sum(int((b["labels"] != -100).sum()) + int(((b["labels"] == -100) & (b["input_ids"] != 0)).sum())
                      for b in cpu_batches[W:W + K])
    trainable_tokens = sum(int((b["labels"][:, 1:] != -100).sum()) for b in cpu_batches[W:W + K])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-timed arm
    def stage(b):
        cp = getattr(parallel, "cp", None) if parallel is not None else None
        if cp is None:
            return to_device_batch(b, dev)
        sb = cp.slice_batch(b)               # this rank's chunk of the row, labels shifted globally
        d = to_device_batch(sb, dev)
        d["attn_meta"] = cp.make_meta(*sb["cp_meta_args"])
        return d

    staged = [stage(b) for b in cpu_batches]
    torch.cuda.synchronize()
    for i in range(W):
        trainer.training_step([staged[i]])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(K):
        trainer.training_step([staged[W + i]])
    ev1.record()
    barrier()
    launches = _lib.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = ev0.elapsed_time(ev1)
    _lib.check_status()

    # ---------------------------------------------------------------- end-to-end arm (public API)
    barrier()
    t0 = time.perf_counter()
    last_loss = 0.0
    for i in range(K):
        loss = trainer.training_step([cpu_batches[W + i]])  # pinned host batch -> H2D inside
        last_loss = float(loss.item())                       # D2H read of the step's result
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    mem_gib = torch.cuda.max_memory_allocated(dev) / 1024 ** 3
    # symmetric (peer-mapped) arenas are allocated outside torch's caching allocator: sharded weights, flat
    # fp32 masters / gradients / bf16 shadows, staging and exchange buffers
    symm_bytes = 0
    if parallel is not None:
        from axolotl_b200.parallel.symm import allocated_bytes

        symm_bytes = allocated_bytes()
    free_b, total_b = torch.cuda.mem_get_info(dev)
    counts = torch.tensor([real_tokens, trainable_tokens], dtype=torch.float64, device=dev)
    if world > 1 and args.config not in ("cp64k",):
        dist.all_reduce(counts)
        if args.config == "tp70b":
            counts /= 2          # both ranks of a tensor-parallel pair count the same batch
    real_tokens, trainable_tokens = float(counts[0]), float(counts[1])
    if rank == 0:
        groups = {"cp64k": 1, "tp70b": max(world // 2, 1)}.get(args.config, world)   # data-parallel replicas
        total_tokens = tokens_per_step * groups * K
        value = total_tokens / (ms / 1e3)
        e2e_value = total_tokens / (e2e_ms / 1e3)
        print(json.dumps({
            "metric": {"lora8b": "train tokens/s/box (max over ranks), Llama-3-8B LoRA FSDP2",
                       "moe": "train tokens/s/box (max over ranks), Qwen3-MoE-30B-A3B NVFP4 expert-LoRA EP",
                       "tp70b": "train tokens/s/box (max over ranks), Llama-3-70B LoRA TP2 x FSDP",
                       "cp64k": "train tokens/s/box (max over ranks), Llama-3-8B full fine-tune CP @ 64k"}[args.config],
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16",
            "data": {"moe": "synthetic uniform token ids, sample lengths U[256,4096] packed to 4096-token rows, 2 rows per step; "
                            "random-init weights, experts quantised to NVFP4",
                     "cp64k": "synthetic uniform token ids, sample lengths U[1024,8192] packed to one 65536-token row; "
                              "random-init weights"}.get(args.config, "synthetic uniform token ids, lengths U[256,4096] "
                                                                      "packed to 8192; random-init weights"),
            "impl": "ours",
            "config": {"model": args.model + ("" if args.layers is None else f"[layers={args.layers}]"),
                       "global_batch": {"moe": 2 * world, "cp64k": 1, "tp70b": max(world // 2, 1)}.get(args.config, world),
                       "seq_len": seq_len,
                       "parallelism": ({"moe": f"ep{world}", "tp70b": f"tp2 x fsdp{world // 2}", "cp64k": f"cp{world}"}
                                       .get(args.config, f"fsdp{world}")) if world > 1 else "single",
                       "lora_r": 16, "lora_alpha": 32, "reshard_after_forward": args.reshard_after_forward == "true",
                       "optimizer": "adamw (fused, fp32 states)", "grad_accum": 1, "micro_batch": 2 if args.config == "moe" else 1,
                       "l2": "per-step working set (16 GB of weights + activations) far exceeds the 126 MB L2",
                       **({"ep_capacity_factor": getattr(getattr(parallel, "ep", None), "capacity_factor", None),
                           "ep_skipped_steps": int(getattr(getattr(parallel, "ep", None), "skipped_steps", 0))}
                          if args.config == "moe" and world > 1 else {})},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": h2d_bytes(cpu_batches[W]) + 16 * (getattr(staged[W]["attn_meta"], "n_tiles", 0) * 2),
                    "d2h_bytes_per_step": 4, "last_loss": last_loss},
            "gpu_launches": launches,
            "tokens": {"slots_per_s": value, "non_pad_per_s": real_tokens / (ms / 1e3),
                       "trainable_per_s": trainable_tokens / (ms / 1e3),
                       "note": "`value` counts every slot of the packed rows (the reference's tokens/s does too); "
                               "non_pad leaves out the padding at the end of each row, trainable counts label positions"},
            "peak_mem_gib": mem_gib,
            "memory": {"torch_peak_allocated_gib": mem_gib, "symmetric_arenas_gib": symm_bytes / 1024 ** 3,
                       "device_in_use_gib": (total_b - free_b) / 1024 ** 3},
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
