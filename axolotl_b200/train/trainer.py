"""The training loop we own end to end (the reference delegates it to ``transformers.Trainer``;
its own additions live in src/axolotl/core/trainers/base.py:141-994).

One optimizer step = ``gradient_accumulation_steps`` micro-batches (each a packed [B, S] batch
with position-id document boundaries) -> loss normalised by the trainable tokens of the whole
step -> gradient sync through the parallel runtime -> fused clip + AdamW -> LR schedule ->
callbacks. Logs carry loss, ppl, grad_norm, learning_rate, memory/* and the reference's
``tokens/train_per_sec_per_gpu`` (trainable tokens, host clock) next to device-timed totals.
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from ..models.transformer import IGNORE_INDEX
from ..ops import functional as Fn
from ..utils.logging import get_logger

LOG = get_logger(__name__)
TOKENS_STATE_FILE = "tokens_state.json"


@dataclass
class TrainArgs:
    output_dir: str = "./outputs"
    max_steps: int = -1
    num_epochs: float = 1.0
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    learning_rate: float = 2e-4
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    logging_steps: int = 1
    save_steps: int | float | None = None
    save_strategy: str = "steps"
    save_total_limit: int | None = 4
    save_only_model: bool = False
    save_first_step: bool = False
    eval_steps: int | float | None = None
    eval_strategy: str = "no"
    seed: int = 42
    include_tkps: bool = True
    gradient_checkpointing: bool = False
    loss_watchdog_threshold: float | None = None
    loss_watchdog_patience: int = 3
    resume_from_checkpoint: str | None = None
    bf16: bool = True
    extra: dict = field(default_factory=dict)


def count_trainable(labels: torch.Tensor) -> int:
    """Targets that survive the shift-by-one inside each row."""
    lab = labels if labels.dim() == 2 else labels[None]
    return int((lab[:, 1:] != IGNORE_INDEX).sum().item())


def to_device_batch(batch: dict, device, pin=True):
    """Async H2D copy of a collated batch (pinned staging) + varlen metadata for the kernels.
    A batch that was staged before (has ``attn_meta``) is passed through."""
    if "attn_meta" in batch:
        return batch
    out = {"n_trainable": batch["n_trainable"] if "n_trainable" in batch else count_trainable(batch["labels"]),
           "n_tokens": batch["n_tokens"] if "n_tokens" in batch else int(batch["input_ids"].numel())}
    if batch.get("labels_preshifted"):
        out["labels_preshifted"] = True
    for k in ("input_ids", "labels", "position_ids"):
        t = batch[k]
        if device.type == "cuda":
            if pin and not t.is_pinned():
                t = t.pin_memory()
            t = t.to(device, non_blocking=True)
        out[k] = t
    for k, t in (batch.get("aux_tensors") or {}).items():   # objective-specific tensors (seq ids, rewards, ...)
        if device.type == "cuda":
            if pin and not t.is_pinned():
                t = t.pin_memory()
            t = t.to(device, non_blocking=True)
        out[k] = t
    out.update(batch.get("meta") or {})
    cu = batch.get("cu_seqlens")
    if "cp_meta_args" in batch:
        out["attn_meta"] = None   # built by the context-parallel runtime
        return out
    causal = not batch.get("bidirectional", False)
    if cu is None:
        from ..models.transformer import build_attn_meta

        out["attn_meta"] = build_attn_meta(batch["position_ids"], device, causal)
    else:
        out["attn_meta"] = Fn.AttnMeta(cu, device, causal)
    return out


def h2d_bytes(batch: dict) -> int:
    return sum(batch[k].numel() * batch[k].element_size() for k in ("input_ids", "labels", "position_ids")
               if isinstance(batch.get(k), torch.Tensor))


class Callback:
    def on_train_begin(self, trainer): ...
    def on_pre_step(self, trainer): ...
    def on_pre_optimizer_step(self, trainer): ...
    def on_step_end(self, trainer, logs): ...
    def on_log(self, trainer, logs): ...
    def on_save(self, trainer, ckpt_dir): ...
    def on_evaluate(self, trainer, metrics): ...
    def on_train_end(self, trainer): ...


class Trainer:
    def __init__(self, model, optimizer, lr_lambda, args: TrainArgs, train_batches, *, eval_batches=None,
                 parallel=None, callbacks=None, save_fn=None, device=None, total_steps=None,
                 compute_loss=None):
        """train_batches: callable(epoch) -> iterable of collated micro-batches for THIS rank."""
        self.model, self.opt, self.lr_lambda, self.args = model, optimizer, lr_lambda, args
        self.train_batches, self.eval_batches = train_batches, eval_batches
        self.parallel = parallel
        self.callbacks = list(callbacks or [])
        self.save_fn = save_fn
        self.device = device or next(model.parameters()).device
        self.total_steps = total_steps
        self.compute_loss = compute_loss
        self.global_step = 0
        self.epoch = 0
        self.tokens = {"total": 0, "trainable": 0}
        self.log_history = []
        self.should_stop = False
        self.should_save = False
        self.batches_in_epoch = 0      # micro-batches consumed in the current epoch (resume skips exactly these)
        self._last_log_time = None
        self._last_log_trainable = 0
        self._loss_acc = None
        self._loss_acc_n = 0
        self.rank = parallel.rank if parallel is not None else 0
        self.world_size = parallel.world_size if parallel is not None else 1

    # ------------------------------------------------------------------ one optimizer step
    def training_step(self, micro_batches):
        """micro_batches: list of collated CPU batches. Returns the (device) loss of the step."""
        model, opt = self.model, self.opt
        n_items = sum(b["n_trainable"] if "n_trainable" in b else count_trainable(b["labels"])
                      for b in micro_batches)
        n_items = max(n_items, 1)
        loss_total = None
        par = self.parallel
        cp = getattr(par, "cp", None) if par is not None else None
        for i, cpu_batch in enumerate(micro_batches):
            if cp is not None and "attn_meta" not in cpu_batch:
                cpu_batch = cp.slice_batch(cpu_batch)   # this rank's chunk, labels shifted globally
            b = to_device_batch(cpu_batch, self.device)
            if cp is not None and "cp_meta_args" in cpu_batch and not getattr(b["attn_meta"], "cp", False):
                b["attn_meta"] = cp.make_meta(*cpu_batch["cp_meta_args"])
            last = i == len(micro_batches) - 1
            if par is not None:
                par.before_micro_batch(last)
            with self._saved_tensor_scope():
                if self.compute_loss is not None:
                    b["ga_steps"] = len(micro_batches)
                    loss = self.compute_loss(model, b, n_items)
                else:
                    media = {"pixel_values": b["pixel_values"]} if "pixel_values" in b else {}
                    out = model(b["input_ids"], b["position_ids"], b["labels"], attn_meta=b["attn_meta"],
                                num_items=n_items, shift_labels=not b.get("labels_preshifted", False),
                                aux_scale=1.0 / len(micro_batches), **media)
                    loss = out.loss
            loss.backward()
            loss_total = loss.detach() if loss_total is None else loss_total + loss.detach()
            self.tokens["total"] += b["n_tokens"]
        self.tokens["trainable"] += n_items
        lr = self.args.learning_rate * self.lr_lambda(self.global_step)
        for cb in self.callbacks:
            cb.on_pre_optimizer_step(self)
        if par is not None:
            gnorm_sq = par.optimizer_step(opt, lr)
        else:
            gnorm_sq = opt.step(lr=lr)
        opt.zero_grad()
        from ..ops.grouped import bump_param_epoch

        bump_param_epoch()   # cached bf16 operand copies of adapters are stale now
        if par is not None:
            par.after_optimizer_step()
        self.global_step += 1
        self._last_lr = lr
        self._last_gnorm_sq = gnorm_sq
        return loss_total

    def _saved_tensor_scope(self):
        """``activation_offloading: true | legacy | disk``: large tensors that autograd saves outside the
        checkpointed layers (embedding output, final norm, loss chunks) go to the same store as the layers'
        inputs while the forward pass runs."""
        store = getattr(self.model, "offload_saved_store", None)
        if store is None:
            import contextlib

            return contextlib.nullcontext()
        from .activation_memory import OffloadSavedTensors

        return OffloadSavedTensors(store)

    # ------------------------------------------------------------------ loop
    def train(self):
        args = self.args
        if args.resume_from_checkpoint:
            self.load_checkpoint(args.resume_from_checkpoint)
        if args.gradient_checkpointing and hasattr(self.model, "enable_gradient_checkpointing") \
                and not getattr(self.model, "gradient_checkpointing", False):
            self.model.enable_gradient_checkpointing(True)
        self.model.train()
        for cb in self.callbacks:
            cb.on_train_begin(self)
        ga = args.gradient_accumulation_steps
        max_steps = args.max_steps if args.max_steps and args.max_steps > 0 else (self.total_steps or 0)
        start_epoch = self.epoch
        n_epochs = max(1, math.ceil(args.num_epochs or 1))
        self._last_log_time = time.time()
        skip = getattr(self, "_resume_skip_batches", 0)
        done = False
        # an explicit max_steps wins over num_epochs: the data is cycled until the steps are done
        explicit_steps = bool(args.max_steps and args.max_steps > 0)
        epoch = start_epoch
        while (explicit_steps or epoch < n_epochs) and not done:
            self.epoch = epoch
            self.batches_in_epoch = 0
            pending = []
            seen = 0
            for bi, batch in enumerate(self.train_batches(epoch)):
                seen += 1
                self.batches_in_epoch += 1
                if skip > 0:
                    skip -= 1
                    continue
                pending.append(batch)
                if len(pending) < ga:
                    continue
                try:
                    for cb in self.callbacks:   # nothing of this rank is in flight here (health checks)
                        cb.on_pre_step(self)
                except Exception as exc:
                    from ..parallel.health import PeerFailure

                    if isinstance(exc, PeerFailure):
                        # a peer is gone: no collective may be entered any more. Keep what this rank
                        # alone can write (optimizer state, RNG, counters), then leave.
                        LOG.error("peer failure before step %d: %s", self.global_step + 1, exc)
                        self.should_stop = True
                        try:
                            self.save_local_state()
                        except Exception as save_exc:   # pragma: no cover
                            LOG.warning("emergency state could not be written: %s", save_exc)
                    raise
                loss = self.training_step(pending)
                pending = []
                self._after_step(loss)
                if (max_steps > 0 and self.global_step >= max_steps) or self.should_stop:
                    done = True
                    break
            if seen == 0:
                break   # an empty epoch: nothing to cycle over
            skip = 0    # a resume skips inside its own epoch only
            if not done:
                self._after_epoch()
            epoch += 1
        if args.save_strategy == "epoch" and getattr(self, "_last_saved_step", -1) != self.global_step \
                and not self.should_stop:
            self._after_epoch()   # the run ended on max_steps inside (or exactly at the end of) an epoch
        for cb in self.callbacks:
            cb.on_train_end(self)
        return self.log_history

    def _after_epoch(self):
        """``save_strategy: epoch`` / ``eval_strategy: epoch``: act at every epoch boundary."""
        args = self.args
        if args.save_strategy == "epoch":
            self.save_checkpoint()
        if args.eval_strategy == "epoch" and self.eval_batches is not None:
            self.evaluate()

    def _after_step(self, loss):
        args = self.args
        self._loss_acc = loss if self._loss_acc is None else self._loss_acc + loss
        self._loss_acc_n += 1
        logs = None
        if self.global_step % max(1, args.logging_steps) == 0 or self.global_step == 1:
            logs = self._make_logs()
        for cb in self.callbacks:
            cb.on_step_end(self, logs)
        if logs is not None:
            self.log_history.append(logs)
            for cb in self.callbacks:
                cb.on_log(self, logs)
            if self.rank == 0:
                LOG.info(json.dumps({k: (round(v, 6) if isinstance(v, float) else v) for k, v in logs.items()}))
        save_every = self._resolve_interval(args.save_steps)
        if (self.should_save or (args.save_strategy == "steps" and save_every and self.global_step % save_every == 0)
                or (args.save_first_step and self.global_step == 1)):
            self.save_checkpoint()
            self.should_save = False
        eval_every = self._resolve_interval(args.eval_steps)
        if self.eval_batches is not None and eval_every and self.global_step % eval_every == 0:
            self.evaluate()

    def _resolve_interval(self, v):
        if not v:
            return None
        if isinstance(v, float) and v < 1:
            return max(1, int(v * (self.total_steps or 1)))
        return int(v)

    def _make_logs(self):
        loss = float((self._loss_acc / max(1, self._loss_acc_n)).item())
        self._loss_acc, self._loss_acc_n = None, 0
        if self.parallel is not None and self.world_size > 1:
            loss = self.parallel.mean_scalar(loss)
        now = time.time()
        logs = {"step": self.global_step, "epoch": self.epoch, "loss": loss,
                "learning_rate": self._last_lr}
        try:
            logs["ppl"] = math.exp(loss)
        except OverflowError:
            logs["ppl"] = float("inf")
        for k, v in (getattr(self.compute_loss, "last_metrics", None) or {}).items():
            logs[k] = v   # objective-specific metrics (rewards/*, kl, clip_ratio, ...)
        if self._last_gnorm_sq is not None:
            logs["grad_norm"] = float(torch.as_tensor(self._last_gnorm_sq).sqrt().item())
        if self.args.include_tkps:
            trainable_all = self.tokens["trainable"]
            if self.parallel is not None and self.world_size > 1:
                trainable_all = self.parallel.sum_scalar(trainable_all)
            dt = max(now - self._last_log_time, 1e-9)
            logs["tokens/train_per_sec_per_gpu"] = (trainable_all - self._last_log_trainable) / self.world_size / dt
            logs["tokens/trainable"] = trainable_all
            logs["tokens/total"] = self.tokens["total"]
            self._last_log_trainable = trainable_all
        self._last_log_time = now
        if self.device.type == "cuda":
            gib = 1024 ** 3
            logs["memory/max_active (GiB)"] = torch.cuda.max_memory_allocated(self.device) / gib
            logs["memory/max_allocated (GiB)"] = torch.cuda.max_memory_allocated(self.device) / gib
            logs["memory/device_reserved (GiB)"] = torch.cuda.memory_reserved(self.device) / gib
            if self.parallel is not None:   # peer-mapped arenas live outside torch's allocator
                from ..parallel.symm import allocated_bytes

                logs["memory/symmetric_arenas (GiB)"] = allocated_bytes() / gib
        return logs

    # ------------------------------------------------------------------ eval
    @torch.no_grad()
    def evaluate(self):
        was = self.model.training
        self.model.eval()
        tot_loss, tot_items = 0.0, 0
        for cpu_batch in self.eval_batches():
            b = to_device_batch(cpu_batch, self.device)
            n = max(count_trainable(cpu_batch["labels"]), 1)
            with torch.enable_grad():  # the fused loss computes its gradient in the forward pass
                media = {"pixel_values": b["pixel_values"]} if "pixel_values" in b else {}
                out = self.model(b["input_ids"], b["position_ids"], b["labels"], attn_meta=b["attn_meta"], num_items=n, **media)
            tot_loss += float(out.loss.item()) * n
            tot_items += n
        if self.parallel is not None and self.world_size > 1:
            tot_loss = self.parallel.sum_scalar(tot_loss)
            tot_items = self.parallel.sum_scalar(tot_items)
        ev = tot_loss / max(tot_items, 1)
        metrics = {"step": self.global_step, "eval_loss": ev, "eval_ppl": math.exp(min(ev, 50))}
        self.log_history.append(metrics)
        for cb in self.callbacks:
            cb.on_evaluate(self, metrics)
        if self.rank == 0:
            LOG.info(json.dumps(metrics))
        self.model.train(was)
        return metrics

    # ------------------------------------------------------------------ checkpoints
    def checkpoint_dir(self, step=None):
        return os.path.join(self.args.output_dir, f"checkpoint-{self.global_step if step is None else step}")

    def save_checkpoint(self):
        if self.device.type == "cuda":
            from ..ops import _lib

            _lib.check_status(self.device)   # never persist weights of a step whose device wait ran out
        d = self.checkpoint_dir()
        if self.rank == 0:
            os.makedirs(d, exist_ok=True)
        if self.parallel is not None:
            self.parallel.barrier()
        if self.save_fn is not None:
            self.save_fn(self, d)
        if not self.args.save_only_model:
            try:
                torch.save(self.opt.state_dict(), os.path.join(d, f"optimizer_rank{self.rank}.pt" if self.world_size > 1 else "optimizer.pt"))
            except Exception as exc:  # the reference tolerates optimizer-save failures as well
                LOG.warning("could not save optimizer state: %s", exc)
            rng = {"torch": torch.get_rng_state(), "numpy": np.random.get_state()}
            if self.device.type == "cuda":
                rng["cuda"] = torch.cuda.get_rng_state(self.device)
            torch.save(rng, os.path.join(d, f"rng_state_{self.rank}.pth" if self.world_size > 1 else "rng_state.pth"))
        if self.rank == 0:
            state = {"global_step": self.global_step, "epoch": self.epoch, "log_history": self.log_history,
                     "max_steps": self.args.max_steps, "total_steps": self.total_steps,
                     "batches_in_epoch": self.batches_in_epoch}
            with open(os.path.join(d, "trainer_state.json"), "w") as fh:
                json.dump(state, fh, indent=1)
            with open(os.path.join(d, TOKENS_STATE_FILE), "w") as fh:
                json.dump(self.tokens, fh)
            self._rotate_checkpoints()
        self._last_saved_step = self.global_step
        for cb in self.callbacks:
            cb.on_save(self, d)
        return d

    def save_local_state(self):
        """Collective-free emergency dump of this rank's optimizer state, RNG and counters into
        ``<output_dir>/emergency-<step>/`` (used when a peer failed: barriers and weight gathers are
        off limits then). Replicated trainable weights are part of the optimizer's fp32 masters."""
        d = os.path.join(self.args.output_dir, f"emergency-{self.global_step}")
        os.makedirs(d, exist_ok=True)
        torch.save(self.opt.state_dict(), os.path.join(d, f"optimizer_rank{self.rank}.pt"))
        state = {"global_step": self.global_step, "epoch": self.epoch, "batches_in_epoch": self.batches_in_epoch,
                 "tokens": self.tokens, "rank": self.rank, "world_size": self.world_size}
        with open(os.path.join(d, f"trainer_state_rank{self.rank}.json"), "w") as fh:
            json.dump(state, fh, indent=1)
        return d

    def _rotate_checkpoints(self):
        limit = self.args.save_total_limit
        if not limit or limit <= 0:
            return
        out = self.args.output_dir
        cks = sorted((int(n.split("-")[1]), n) for n in os.listdir(out)
                     if n.startswith("checkpoint-") and n.split("-")[1].isdigit())
        import shutil

        for _, n in cks[:-limit]:
            shutil.rmtree(os.path.join(out, n), ignore_errors=True)

    def load_checkpoint(self, d):
        with open(os.path.join(d, "trainer_state.json")) as fh:
            st = json.load(fh)
        self.global_step, self.epoch = st["global_step"], st.get("epoch", 0)
        self.log_history = st.get("log_history", [])
        tok = os.path.join(d, TOKENS_STATE_FILE)
        if os.path.exists(tok):
            with open(tok) as fh:
                self.tokens = json.load(fh)
            self._last_log_trainable = self.tokens["trainable"]
        for cand in (f"optimizer_rank{self.rank}.pt", "optimizer.pt"):
            p = os.path.join(d, cand)
            if os.path.exists(p):
                self.opt.load_state_dict(torch.load(p, map_location="cpu", weights_only=False))
                break
        for cand in (f"rng_state_{self.rank}.pth", "rng_state.pth"):
            p = os.path.join(d, cand)
            if os.path.exists(p):
                rng = torch.load(p, map_location="cpu", weights_only=False)
                torch.set_rng_state(rng["torch"])
                np.random.set_state(rng["numpy"])
                if "cuda" in rng and self.device.type == "cuda":
                    torch.cuda.set_rng_state(rng["cuda"], self.device)
                break
        self._resume_skip_batches = st.get("batches_in_epoch", 0)
        LOG.info("resumed from %s at step %d", d, self.global_step)


def find_last_checkpoint(output_dir):
    """Newest ``checkpoint-N`` directory (``auto_resume_from_checkpoints``,
    src/axolotl/utils/train.py:11-47)."""
    if not os.path.isdir(output_dir):
        return None
    cks = [(int(n.split("-")[1]), n) for n in os.listdir(output_dir)
           if n.startswith("checkpoint-") and n.split("-")[1].isdigit()
           and os.path.exists(os.path.join(output_dir, n, "trainer_state.json"))]
    return os.path.join(output_dir, max(cks)[1]) if cks else None
