"""Timing plugin for the reference arm of ``bench.py``.

Loaded by the UNMODIFIED reference through its own plugin mechanism (``plugins:`` in the YAML,
``BasePlugin.add_callbacks_post_trainer``; src/axolotl/integrations/base.py:260-273): it adds one
``transformers.TrainerCallback`` that brackets optimizer steps W+1 .. W+K with a barrier and a device
synchronisation on both sides, times them with CUDA events and with the host clock, writes the result
to the file named by ``AXB_REF_TIMING_OUT`` and then stops the run. Nothing of ``axolotl_b200`` is
imported here.
"""
from __future__ import annotations

import json
import os
import time

import torch
from transformers import TrainerCallback

try:   # the real reference; the test suite substitutes a stand-in package of the same name
    from axolotl.integrations.base import BasePlugin
except Exception:   # pragma: no cover
    class BasePlugin:   # type: ignore
        pass


def _barrier():
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


class StepTimer(TrainerCallback):
    def __init__(self):
        self.warmup = int(os.environ.get("AXB_REF_WARMUP", "3"))
        self.steps = int(os.environ.get("AXB_REF_STEPS", "5"))
        self.out = os.environ.get("AXB_REF_TIMING_OUT")
        self.t0 = None
        self.ev0 = self.ev1 = None
        self.last_loss = None

    def on_log(self, args, state, control, logs=None, **kw):
        if logs and "loss" in logs:
            self.last_loss = float(logs["loss"])

    def on_step_end(self, args, state, control, **kw):
        step = state.global_step
        if step == self.warmup:
            _barrier()
            if torch.cuda.is_available():
                self.ev0 = torch.cuda.Event(enable_timing=True)
                self.ev1 = torch.cuda.Event(enable_timing=True)
                self.ev0.record()
            self.t0 = time.perf_counter()
        elif step == self.warmup + self.steps and self.t0 is not None:
            if self.ev1 is not None:
                self.ev1.record()
            _barrier()
            host_ms = (time.perf_counter() - self.t0) * 1e3
            dev_ms = self.ev0.elapsed_time(self.ev1) if self.ev1 is not None else host_ms
            vals = torch.tensor([dev_ms, host_ms], dtype=torch.float64)
            if torch.distributed.is_available() and torch.distributed.is_initialized():
                if torch.cuda.is_available():
                    vals = vals.cuda()
                torch.distributed.all_reduce(vals, op=torch.distributed.ReduceOp.MAX)   # max over ranks
            rank = int(os.environ.get("RANK", "0"))
            if rank == 0 and self.out:
                peak = torch.cuda.max_memory_allocated() / 1024 ** 3 if torch.cuda.is_available() else 0.0
                with open(self.out, "w") as fh:
                    json.dump({"device_ms": float(vals[0]), "host_ms": float(vals[1]), "steps": self.steps,
                               "warmup": self.warmup, "last_loss": self.last_loss, "peak_mem_gib": peak}, fh)
            control.should_training_stop = True
        return control


class TimingPlugin(BasePlugin):
    def add_callbacks_post_trainer(self, cfg, trainer):
        return [StepTimer()]
