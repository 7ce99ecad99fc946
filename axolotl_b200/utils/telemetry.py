"""Usage telemetry: opt-out, rank 0 only, with path and organisation redaction.

The reference posts a handful of events (config loaded, train start / end, errors with sanitised stack
traces, periodic runtime metrics) to a hosted analytics service (src/axolotl/telemetry/manager.py:99-387,
errors.py, callbacks.py, runtime_metrics.py). The same events are collected here with the same opt-out
switches (``AXOLOTL_DO_NOT_TRACK=1`` / ``DO_NOT_TRACK=1``) and the same redaction rules; the sink is
pluggable: by default events are appended to ``<output_dir>/telemetry.jsonl`` (nothing leaves the
machine), ``AXOLOTL_TELEMETRY_URL`` switches to an HTTP POST per event.
"""
from __future__ import annotations

import atexit
import json
import os
import platform
import re
import time
import traceback
import uuid

FIELDS_WITH_ORGS = ("base_model", "tokenizer_config", "base_model_config", "pretraining_dataset")
PATH_KEYS = ("path", "data_files", "output_dir", "dataset_prepared_path", "resume_from_checkpoint", "lora_model_dir")
KNOWN_ORGS = {"meta-llama", "mistralai", "qwen", "google", "microsoft", "deepseek-ai", "huggingfaceh4", "nousresearch",
              "tiiuae", "allenai", "ibm-granite", "nvidia", "openai", "axolotl-ai-co", "huggingfacetb", "cohereforai"}


def _truthy(name):
    v = os.environ.get(name)
    return v is not None and v.strip().lower() in ("1", "true")


def redact_value(value):
    """``org/name`` stays if the organisation is well known, otherwise the organisation part is hidden;
    filesystem paths are reduced to their last component."""
    if not isinstance(value, str):
        return value
    if value.startswith(("/", "./", "~", "..")) or re.match(r"^[A-Za-z]:\\", value):
        return "<path>/" + os.path.basename(value.rstrip("/\\"))
    if "/" in value:
        org, _, rest = value.partition("/")
        return value if org.lower() in KNOWN_ORGS else "<redacted>/" + rest
    return value


def sanitize_config(cfg: dict) -> dict:
    out = {}
    for k, v in dict(cfg).items():
        if k in FIELDS_WITH_ORGS or k in PATH_KEYS:
            out[k] = redact_value(v) if isinstance(v, str) else ("<set>" if v else v)
        elif k in ("datasets", "test_datasets") and isinstance(v, list):
            out[k] = [{kk: (redact_value(vv) if kk in PATH_KEYS else vv) for kk, vv in d.items()} if isinstance(d, dict) else "<entry>"
                      for d in v]
        elif any(s in k for s in ("token", "api_key", "secret", "password")):
            out[k] = "<redacted>" if v else v
        elif isinstance(v, (str, int, float, bool, type(None))):
            out[k] = v
        elif isinstance(v, (list, dict)):
            try:
                json.dumps(v)
                out[k] = v
            except TypeError:
                out[k] = str(type(v).__name__)
    return out


def sanitize_stack_trace(text: str) -> str:
    """Keeps frames of this package and of well-known libraries, strips directories from every file path."""
    def repl(m):
        p = m.group(1)
        for marker in ("site-packages/", "axolotl_b200/"):
            i = p.rfind(marker)
            if i >= 0:
                return f'File "{p[i + (len(marker) if marker == "site-packages/" else 0):]}"'
        return f'File "<user>/{os.path.basename(p)}"'
    return re.sub(r'File "([^"]+)"', repl, text)


class Telemetry:
    _instance = None

    def __init__(self, output_dir=None):
        rank = int(os.environ.get("RANK", "0"))
        self.enabled = rank == 0 and not (_truthy("AXOLOTL_DO_NOT_TRACK") or _truthy("DO_NOT_TRACK"))
        self.run_id = str(uuid.uuid4())
        self.output_dir = output_dir
        self.url = os.environ.get("AXOLOTL_TELEMETRY_URL")
        self.events = []
        self._sys = None
        if self.enabled:
            atexit.register(self.flush)

    @classmethod
    def get(cls, output_dir=None):
        if cls._instance is None:
            cls._instance = Telemetry(output_dir)
        if output_dir and not cls._instance.output_dir:
            cls._instance.output_dir = output_dir
        return cls._instance

    def system_info(self):
        if self._sys is None:
            info = {"os": platform.system(), "python": platform.python_version(), "cpu_count": os.cpu_count()}
            try:
                import torch

                info["torch"] = torch.__version__
                if torch.cuda.is_available():
                    info["gpu_count"] = torch.cuda.device_count()
                    info["gpu"] = torch.cuda.get_device_name(0)
                    info["cuda"] = torch.version.cuda
            except Exception:   # pragma: no cover
                pass
            self._sys = info
        return self._sys

    def send(self, event: str, properties: dict | None = None):
        if not self.enabled:
            return
        rec = {"event": event, "run_id": self.run_id, "time": time.time(), "properties": properties or {},
               "system": self.system_info()}
        self.events.append(rec)
        if len(self.events) >= 16:
            self.flush()

    def flush(self):
        if not self.enabled or not self.events:
            return
        events, self.events = self.events, []
        try:
            if self.url:
                import urllib.request

                for e in events:
                    req = urllib.request.Request(self.url, data=json.dumps(e).encode(), headers={"Content-Type": "application/json"})
                    urllib.request.urlopen(req, timeout=2)  # nosec B310
            elif self.output_dir:
                os.makedirs(self.output_dir, exist_ok=True)
                with open(os.path.join(self.output_dir, "telemetry.jsonl"), "a") as fh:
                    for e in events:
                        fh.write(json.dumps(e) + "\n")
        except Exception:   # telemetry never breaks a run
            pass

    def send_error(self, exc: BaseException):
        self.send("error", {"type": type(exc).__name__,
                            "stack": sanitize_stack_trace("".join(traceback.format_exception(type(exc), exc, exc.__traceback__)))})


class TelemetryCallback:
    """Trainer callback: train start / end events and runtime metrics every ``every`` logs."""

    def __init__(self, cfg, every=50):
        self.t = Telemetry.get(cfg.get("output_dir"))
        self.cfg, self.every, self.n = cfg, every, 0
        self.t0 = None

    def on_train_begin(self, trainer):
        self.t0 = time.time()
        self.t.send("train-start", {"config": sanitize_config(self.cfg), "world_size": trainer.world_size})

    def on_log(self, trainer, logs):
        self.n += 1
        if self.n % self.every == 0:
            keep = {k: v for k, v in logs.items() if k in ("step", "loss", "learning_rate", "tokens/train_per_sec_per_gpu",
                                                          "memory/max_allocated (GiB)", "grad_norm")}
            self.t.send("train-progress", keep)

    def on_train_end(self, trainer):
        self.t.send("train-end", {"steps": trainer.global_step, "seconds": time.time() - (self.t0 or time.time()),
                                  "tokens": trainer.tokens})
        self.t.flush()

    def on_pre_step(self, trainer): ...
    def on_pre_optimizer_step(self, trainer): ...
    def on_step_end(self, trainer, logs): ...
    def on_save(self, trainer, ckpt_dir): ...
    def on_evaluate(self, trainer, metrics): ...
