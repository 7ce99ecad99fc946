"""Trainer callbacks: loss watchdog, on-demand checkpoints, profiler, GC, early stopping, metric
reporters (tensorboard / wandb / mlflow when importable, Prometheus exporter)
(reference: src/axolotl/utils/callbacks/__init__.py:57-880, profiler.py, dynamic_checkpoint.py,
opentelemetry.py)."""
from __future__ import annotations

import gc
import json
import os
import time

import torch

from ..utils.logging import get_logger
from .trainer import Callback

LOG = get_logger(__name__)


class LossWatchdogCallback(Callback):
    """Stops training when the loss stays above a threshold for ``patience`` consecutive logs."""

    def __init__(self, threshold, patience=3):
        self.threshold, self.patience, self.bad = threshold, patience, 0

    def on_log(self, trainer, logs):
        loss = logs.get("loss")
        if loss is None:
            return
        if loss != loss or loss > self.threshold:
            self.bad += 1
            if self.bad >= self.patience:
                LOG.warning("loss watchdog: loss %.4f above %.4f for %d logs, stopping", loss, self.threshold, self.bad)
                trainer.should_stop = True
        else:
            self.bad = 0


class DynamicCheckpointCallback(Callback):
    """`touch <output_dir>/axolotl_checkpoint.save` triggers a checkpoint at the next check; rank 0
    looks, the decision is broadcast so every rank saves at the same step."""

    TRIGGER = "axolotl_checkpoint.save"

    def __init__(self, check_interval=10, trigger_file_path=None):
        self.interval, self.trigger = max(1, check_interval), trigger_file_path

    def on_step_end(self, trainer, logs):
        if trainer.global_step % self.interval:
            return
        path = self.trigger or os.path.join(trainer.args.output_dir, self.TRIGGER)
        flag = 0
        if trainer.rank == 0 and os.path.exists(path):
            flag = 1
            try:
                os.remove(path)
            except OSError:
                pass
        if trainer.parallel is not None and trainer.world_size > 1:
            flag = int(trainer.parallel.sum_scalar(flag) > 0)
        if flag:
            LOG.info("dynamic checkpoint requested at step %d", trainer.global_step)
            trainer.should_save = True


class SaveFirstStepCallback(Callback):
    def on_step_end(self, trainer, logs):
        if trainer.global_step == 1:
            trainer.should_save = True


class GCCallback(Callback):
    def __init__(self, gc_steps=None, empty_cache_steps=None):
        self.gc_steps, self.empty_cache_steps = gc_steps, empty_cache_steps

    def on_step_end(self, trainer, logs):
        if self.gc_steps and trainer.global_step % self.gc_steps == 0:
            gc.collect()
        if self.empty_cache_steps and trainer.global_step % self.empty_cache_steps == 0 and torch.cuda.is_available():
            torch.cuda.empty_cache()


class EarlyStoppingCallback(Callback):
    def __init__(self, patience, metric="eval_loss", greater_is_better=False):
        self.patience, self.metric, self.gib = patience, metric, greater_is_better
        self.best, self.bad = None, 0

    def on_evaluate(self, trainer, metrics):
        v = metrics.get(self.metric)
        if v is None:
            return
        better = self.best is None or (v > self.best if self.gib else v < self.best)
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                LOG.info("early stopping: %s did not improve for %d evaluations", self.metric, self.bad)
                trainer.should_stop = True


class ProfilerCallback(Callback):
    """torch.profiler trace (`profiler_trace.json`) and CUDA memory snapshot (`snapshot.pickle`) of
    ``steps`` optimizer steps starting at ``start``."""

    def __init__(self, steps, start=0):
        self.steps, self.start, self.prof = steps, start, None

    def on_step_end(self, trainer, logs):
        s = trainer.global_step
        if s == self.start and self.prof is None:
            if torch.cuda.is_available():
                torch.cuda.memory._record_memory_history(max_entries=100_000)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.prof = torch.profiler.profile(activities=acts, record_shapes=True, with_stack=False)
            self.prof.__enter__()
        elif self.prof is not None and s >= self.start + self.steps:
            self.prof.__exit__(None, None, None)
            out = trainer.args.output_dir
            os.makedirs(out, exist_ok=True)
            self.prof.export_chrome_trace(os.path.join(out, "profiler_trace.json"))
            if torch.cuda.is_available():
                torch.cuda.memory._dump_snapshot(os.path.join(out, "snapshot.pickle"))
                torch.cuda.memory._record_memory_history(enabled=None)
            self.prof = None
            self.steps = 0


class JsonlReporter(Callback):
    """Always-on reporter: one JSON line per log into ``<output_dir>/train_log.jsonl``."""

    def on_log(self, trainer, logs):
        if trainer.rank != 0:
            return
        os.makedirs(trainer.args.output_dir, exist_ok=True)
        with open(os.path.join(trainer.args.output_dir, "train_log.jsonl"), "a") as fh:
            fh.write(json.dumps(logs) + "\n")

    on_evaluate = on_log


class TensorboardReporter(Callback):
    def __init__(self, log_dir):
        from torch.utils.tensorboard import SummaryWriter  # noqa: WPS433 (optional dependency)

        self.w = SummaryWriter(log_dir)

    def on_log(self, trainer, logs):
        if trainer.rank == 0:
            for k, v in logs.items():
                if isinstance(v, (int, float)) and k != "step":
                    self.w.add_scalar(k if "/" in k else f"train/{k}", v, logs.get("step", trainer.global_step))

    on_evaluate = on_log


class WandbReporter(Callback):
    def __init__(self, cfg):
        import wandb  # optional dependency

        self.wandb = wandb
        self.run = wandb.init(project=cfg.get("wandb_project"), entity=cfg.get("wandb_entity"), name=cfg.get("wandb_name"),
                              id=cfg.get("wandb_run_id"), mode=cfg.get("wandb_mode"), config=dict(cfg), resume="allow")

    def on_log(self, trainer, logs):
        if trainer.rank == 0:
            self.wandb.log(logs, step=logs.get("step"))

    on_evaluate = on_log


class MLflowReporter(Callback):
    def __init__(self, cfg):
        import mlflow  # optional dependency

        self.mlflow = mlflow
        if cfg.get("mlflow_tracking_uri"):
            mlflow.set_tracking_uri(cfg["mlflow_tracking_uri"])
        if cfg.get("mlflow_experiment_name"):
            mlflow.set_experiment(cfg["mlflow_experiment_name"])
        mlflow.start_run(run_name=cfg.get("mlflow_run_name"))

    def on_log(self, trainer, logs):
        if trainer.rank == 0:
            self.mlflow.log_metrics({k.replace("/", "_").replace(" ", "_").replace("(", "").replace(")", ""): v
                                     for k, v in logs.items() if isinstance(v, (int, float))}, step=logs.get("step"))


class CometReporter(Callback):
    """``use_comet``: metrics to a Comet experiment (src/axolotl/core/builders/base.py:526-548,
    src/axolotl/utils/callbacks/comet_.py)."""

    def __init__(self, cfg):
        import comet_ml  # optional dependency

        kw = {k: cfg.get(f"comet_{k}") for k in ("api_key", "workspace", "project_name", "experiment_key", "mode", "online")
              if cfg.get(f"comet_{k}") is not None}
        kw.update(cfg.get("comet_experiment_config") or {})
        self.exp = comet_ml.start(**{k: v for k, v in kw.items() if k in ("api_key", "workspace", "project_name",
                                                                          "experiment_key", "mode", "online")})
        self.exp.log_parameters({k: v for k, v in dict(cfg).items() if isinstance(v, (str, int, float, bool))})

    def on_log(self, trainer, logs):
        if trainer.rank == 0:
            self.exp.log_metrics({k: v for k, v in logs.items() if isinstance(v, (int, float))}, step=logs.get("step"))

    on_evaluate = on_log

    def on_train_end(self, trainer):
        if trainer.rank == 0:
            self.exp.end()


class TrackioReporter(Callback):
    """``use_trackio``: metrics to a Trackio project (local dashboard or a Space)."""

    def __init__(self, cfg):
        import trackio  # optional dependency

        self.trackio = trackio
        trackio.init(project=cfg.get("trackio_project_name") or "axolotl", name=cfg.get("trackio_run_name"),
                     space_id=cfg.get("trackio_space_id"), config={k: v for k, v in dict(cfg).items()
                                                                   if isinstance(v, (str, int, float, bool))})

    def on_log(self, trainer, logs):
        if trainer.rank == 0:
            self.trackio.log({k: v for k, v in logs.items() if isinstance(v, (int, float))})

    on_evaluate = on_log

    def on_train_end(self, trainer):
        if trainer.rank == 0:
            self.trackio.finish()


class PrometheusExporter(Callback):
    """`use_otel_metrics`: exposes the latest training metrics as Prometheus gauges on
    ``otel_metrics_host:otel_metrics_port``."""

    def __init__(self, host="localhost", port=8000):
        from prometheus_client import Gauge, start_http_server

        self.Gauge, self.g = Gauge, {}
        try:
            start_http_server(port, addr=host)
        except OSError as exc:
            LOG.warning("metrics exporter could not bind %s:%s (%s)", host, port, exc)

    def on_log(self, trainer, logs):
        if trainer.rank != 0:
            return
        for k, v in logs.items():
            if not isinstance(v, (int, float)):
                continue
            name = "axolotl_" + "".join(c if c.isalnum() else "_" for c in k).strip("_").lower()
            if name not in self.g:
                self.g[name] = self.Gauge(name, k)
            self.g[name].set(v)


class StatusCheckCallback(Callback):
    """Reads the kernels' status word at every log (and the trainer reads it again before it writes a
    checkpoint): a bounded device wait that ran out becomes a Python exception instead of a silent
    wrong result or a persisted half-reduced step."""

    def on_log(self, trainer, logs):
        if trainer.device.type == "cuda":
            from ..ops import _lib

            _lib.check_status(trainer.device)


class SampleGenerationCallback(Callback):
    """Monitoring: at every evaluation / save interval, continues a few evaluation (or training)
    samples from a prefix with the current weights and logs prompt, reference continuation and
    generation (``generate_samples`` and the ``generation_*`` keys of the reference,
    src/axolotl/utils/schemas/config.py:1429-1468). Written to ``<output_dir>/generations.jsonl``."""

    def __init__(self, cfg, samples, tokenizer=None, every=None):
        self.n = cfg.get("num_generation_samples") or 3
        self.max_new = cfg.get("generation_max_new_tokens") or 50
        do_sample = cfg.get("generation_do_sample", True) is not False
        self.temperature = (cfg.get("generation_temperature") if cfg.get("generation_temperature") is not None else 0.7) \
            if do_sample else 0.0
        self.top_p = cfg.get("generation_top_p") or 1.0
        self.ratio = cfg.get("generation_prompt_ratio") if cfg.get("generation_prompt_ratio") is not None else 0.5
        self.samples, self.tok = samples, tokenizer
        self.every = every or cfg.get("eval_steps") or cfg.get("save_steps") or 100
        self.out = os.path.join(cfg["output_dir"], "generations.jsonl")

    def on_step_end(self, trainer, logs):
        every = self.every if self.every >= 1 else max(int(self.every * max(trainer.total_steps or 1, 1)), 1)
        if trainer.global_step % every or trainer.rank != 0:
            return
        model = trainer.model
        dev = model.embed_tokens.device
        rows = []
        for i in range(min(self.n, len(self.samples))):
            ids = [int(t) for t in self.samples[i]["input_ids"]]
            cut = max(1, int(len(ids) * self.ratio))
            out = model.generate(torch.tensor([ids[:cut]], device=dev), max_new_tokens=self.max_new,
                                 temperature=self.temperature, top_p=self.top_p,
                                 eos_token_id=getattr(self.tok, "eos_token_id", None))
            gen = out[0].tolist()[cut:]
            dec = (lambda t: self.tok.decode(t, skip_special_tokens=True)) if self.tok is not None else (lambda t: t)
            rows.append({"step": trainer.global_step, "prompt": dec(ids[:cut]), "reference": dec(ids[cut:cut + self.max_new]),
                         "generation": dec(gen)})
        os.makedirs(os.path.dirname(self.out) or ".", exist_ok=True)
        with open(self.out, "a") as fh:
            for r in rows:
                fh.write(json.dumps(r) + "\n")
        model.train()
        LOG.info("generated %d monitoring samples at step %d", len(rows), trainer.global_step)


class LISACallback(Callback):
    """Layerwise importance sampling for full fine-tuning: every ``interval`` steps a new random set
    of ``n_layers`` decoder layers is trainable, all others are frozen (no gradient is computed for
    them and the optimizer leaves their weights and moments alone); embeddings, final norm and head
    always train. Reference: src/axolotl/utils/callbacks/lisa.py:23 (``lisa_n_layers``,
    ``lisa_step_interval``)."""

    def __init__(self, n_layers, interval, seed=0):
        import random

        self.n, self.interval, self.rng = int(n_layers), max(int(interval), 1), random.Random(seed)
        self.active = None

    def _switch(self, trainer):
        layers = trainer.model.layers
        self.active = sorted(self.rng.sample(range(len(layers)), min(self.n, len(layers))))
        for i, layer in enumerate(layers):
            on = i in self.active
            for p in layer.parameters():
                if getattr(p, "_axb_grad", None) is not None or p.requires_grad:   # parameters the optimizer owns
                    p.requires_grad_(on)
        if hasattr(trainer.opt, "set_active_layers"):
            trainer.opt.set_active_layers(self.active)
        LOG.info("LISA: training layers %s", self.active)

    def on_train_begin(self, trainer):
        self._switch(trainer)

    def on_step_end(self, trainer, logs):
        if trainer.global_step % self.interval == 0:
            self._switch(trainer)


class ReLoRACallback(Callback):
    """ReLoRA: every ``restart_steps`` optimizer steps the adapters are folded into the base
    weights (W += s B A), A is re-initialised, B zeroed and the adapters' AdamW moments pruned, so
    successive low-rank updates add up to a high-rank one. Pair with the jagged-restart schedule
    (reference: src/axolotl/monkeypatch/relora.py and ReLoRAConfig)."""

    def __init__(self, restart_steps, prune_ratio=0.9):
        self.every, self.prune = int(restart_steps), float(prune_ratio if prune_ratio is not None else 0.9)

    def on_step_end(self, trainer, logs):
        import math

        import torch

        if self.every <= 0 or trainer.global_step == 0 or trainer.global_step % self.every:
            return
        model = trainer.model
        touched = []
        with torch.no_grad():
            for _, m in model.fused_linears():
                if getattr(m, "mora_M", None) is not None:   # ReMoRA: fold the square matrices in, restart at zero
                    m.merge_mora_()
                    touched += list(m.mora_M)
                if getattr(m, "lora_A", None) is None or getattr(m.weight, "_axb_quant", None) is not None:
                    continue
                if getattr(m.weight, "_axb_shard", None) is not None or getattr(m, "tp", None) is not None:
                    continue   # sharded base weights are merged at export time instead
                delta = m.scaling * (m.lora_B.float() @ m.lora_A.float())
                m.weight.add_(delta.to(m.weight.dtype))
                r = m.lora_r
                for i in range(len(m.lora_names)):
                    torch.nn.init.kaiming_uniform_(m.lora_A[i * r:(i + 1) * r], a=math.sqrt(5))
                m.lora_B.zero_()
                touched += [m.lora_A, m.lora_B]
        if hasattr(trainer.opt, "reset_state"):
            trainer.opt.reset_state(touched, self.prune)
        model.refresh_lora_shadows()
        LOG.info("ReLoRA restart at step %d: merged and reset %d adapter tensors", trainer.global_step, len(touched))


def build_callbacks(cfg):
    from ..utils.telemetry import TelemetryCallback

    cbs = [JsonlReporter(), StatusCheckCallback(), TelemetryCallback(cfg)]
    if cfg.get("lisa_n_layers") and cfg.get("lisa_step_interval"):
        cbs.append(LISACallback(cfg["lisa_n_layers"], cfg["lisa_step_interval"], cfg.get("seed") or 0))
    if cfg.get("relora") and cfg.get("jagged_restart_steps"):
        cbs.append(ReLoRACallback(cfg["jagged_restart_steps"], cfg.get("relora_prune_ratio")))
    if cfg.get("loss_watchdog_threshold") is not None:
        cbs.append(LossWatchdogCallback(cfg["loss_watchdog_threshold"], cfg.get("loss_watchdog_patience") or 3))
    dc = cfg.get("dynamic_checkpoint")
    if dc and dc.get("enabled"):
        cbs.append(DynamicCheckpointCallback(dc.get("check_interval") or 10, dc.get("trigger_file_path") or None))
    if cfg.get("gc_steps") or cfg.get("torch_empty_cache_steps"):
        cbs.append(GCCallback(cfg.get("gc_steps"), cfg.get("torch_empty_cache_steps")))
    if cfg.get("early_stopping_patience"):
        cbs.append(EarlyStoppingCallback(cfg["early_stopping_patience"], cfg.get("metric_for_best_model") or "eval_loss",
                                         bool(cfg.get("greater_is_better"))))
    if cfg.get("profiler_steps"):
        cbs.append(ProfilerCallback(cfg["profiler_steps"], cfg.get("profiler_steps_start") or 0))
    for flag, factory in (("use_tensorboard", lambda: TensorboardReporter(os.path.join(cfg["output_dir"], "runs"))),
                          ("use_wandb", lambda: WandbReporter(cfg)), ("use_mlflow", lambda: MLflowReporter(cfg)),
                          ("use_comet", lambda: CometReporter(cfg)), ("use_trackio", lambda: TrackioReporter(cfg)),
                          ("use_otel_metrics", lambda: PrometheusExporter(cfg.get("otel_metrics_host") or "localhost",
                                                                          cfg.get("otel_metrics_port") or 8000))):
        if cfg.get(flag) or (flag == "use_wandb" and cfg.get("wandb_project")) \
                or (flag == "use_comet" and cfg.get("comet_project_name")) \
                or (flag == "use_trackio" and cfg.get("trackio_project_name")):
            try:
                cbs.append(factory())
            except Exception as exc:
                LOG.warning("%s requested but unavailable: %s", flag, exc)
    return cbs
