"""Remote training backend: the data pipeline runs here, forward / backward / optimizer steps run on a Tinker or
Hatchery service that holds the model and a LoRA adapter.

With the plugin active no model is built locally. The tokenised dataset (chat templates, masking: everything the
``datasets:`` section configures) is turned row by row into the service's *datum* format with the causal shift applied
on the client (inputs ``t[:-1]``, targets ``t[1:]``, a 0/1 weight per target), sent with ``forward_backward`` and
followed by ``optim_step`` once per ``gradient_accumulation_steps`` micro batches. The service returns the SUM of the
per-token losses; the loop logs sum / trained tokens. With a policy-gradient ``loss_fn`` the loop becomes: sample
``num_samples`` completions per prompt from the service, score them with local reward functions, turn rewards into
group-normalised advantages, send (tokens, sampling log-probs, advantages).

Reference: src/axolotl/integrations/hatchery/{plugin.py:22-147, trainer.py:24-327, rl_trainer.py:1-409,
data.py:1-160, args.py:14-62}. The Tinker / Hatchery SDKs are optional imports; ``set_client_factory`` lets a test or
an embedding application supply the client.

YAML::

    plugins: [axolotl.integrations.hatchery.HatcheryPlugin]
    hatchery:
      backend: tinker            # or hatchery (base_url, api_key)
      lora_rank: 32
      loss_fn: cross_entropy     # importance_sampling | ppo | cispo | dro: the RL loop
"""
from __future__ import annotations

import importlib
import inspect
import os
import re
import time
from typing import Any, Callable, Literal, Optional

import numpy as np
from pydantic import BaseModel, Field

from ..utils.logging import get_logger
from .base import BasePlugin

LOG = get_logger(__name__)
RL_LOSSES = ("importance_sampling", "ppo", "cispo", "dro")
_CLIENT_FACTORY: Callable | None = None


class HatcheryConfig(BaseModel):
    backend: Literal["tinker", "hatchery"] = "tinker"
    base_url: Optional[str] = None
    api_key: Optional[str] = None
    project_id: Optional[str] = None
    lora_rank: int = Field(32, ge=1, le=256)
    train_attn: bool = True
    train_mlp: bool = True
    train_unembed: bool = True
    loss_fn: Literal["cross_entropy", "importance_sampling", "ppo", "cispo", "dro"] = "cross_entropy"
    loss_fn_config: Optional[dict[str, Any]] = None
    pipeline: bool = True                  # do not wait for an optimizer step before sending the next batch
    max_sample_tokens: int = 256
    sample_temperature: float = 1.0
    num_samples: int = 4
    reward_funcs: Optional[list[str]] = None
    save_steps: Optional[int] = None
    save_name_prefix: str = "checkpoint"
    future_timeout: float = 600.0


class HatcheryArgs(BaseModel):
    hatchery: Optional[HatcheryConfig] = None


def set_client_factory(factory: Callable | None) -> None:
    """``factory(config, base_model) -> training client`` used instead of the SDK imports (None restores them)."""
    global _CLIENT_FACTORY
    _CLIENT_FACTORY = factory


# ------------------------------------------------------------------------------------------- wire format
_DTYPES = {"float32": "float32", "float64": "float32", "float16": "float16", "int64": "int64", "int32": "int32"}


def tensor_to_wire(values, dtype: str | None = None) -> dict:
    a = np.asarray(values)
    name = dtype or _DTYPES.get(a.dtype.name, "float32")
    return {"dtype": name, "shape": list(a.shape), "data": a.reshape(-1).tolist()}


def make_datum(tokens, loss_fn_inputs: dict) -> dict:
    return {"model_input": {"chunks": [{"type": "encoded_text", "tokens": [int(t) for t in tokens]}]},
            "loss_fn_inputs": {k: tensor_to_wire(v) for k, v in loss_fn_inputs.items()}}


def row_to_datum_sft(input_ids, labels) -> dict:
    """One tokenised row -> a supervised datum with the causal shift."""
    ids, lab = np.asarray(input_ids, dtype=np.int64), np.asarray(labels, dtype=np.int64)
    tgt = lab[1:].copy()
    w = (tgt != -100).astype(np.float32)
    tgt[tgt == -100] = 0
    return make_datum(ids[:-1], {"target_tokens": tgt, "weights": w})


def row_to_datum_rl(tokens, prompt_len, logprobs, advantage) -> dict:
    """prompt + completion -> a policy-gradient datum: sampling log-probs and the sample's advantage on the completion
    positions, zeros on the prompt."""
    ids = np.asarray(tokens, dtype=np.int64)
    n = len(ids)
    lab = np.full(n, -100, dtype=np.int64)
    lab[prompt_len:] = ids[prompt_len:]
    lp = np.zeros(n, dtype=np.float32)
    got = np.asarray(logprobs[: n - prompt_len], dtype=np.float32)
    lp[prompt_len:prompt_len + len(got)] = got
    adv = np.zeros(n, dtype=np.float32)
    adv[prompt_len:] = advantage
    tgt = lab[1:].copy()
    tgt[tgt == -100] = 0
    return make_datum(ids[:-1], {"target_tokens": tgt, "logprobs": lp[1:], "advantages": adv[1:]})


def _to_sdk(datums):
    """Plain-dict datums -> tinker.types.Datum when that SDK is importable (both services accept those); the dicts
    themselves otherwise."""
    try:
        import tinker.types as tt
    except ImportError:
        return datums
    out = []
    for d in datums:
        inputs = {k: tt.TensorData(data=w["data"], dtype=w["dtype"], shape=w["shape"]) for k, w in d["loss_fn_inputs"].items()}
        out.append(tt.Datum(model_input=tt.ModelInput.from_ints(d["model_input"]["chunks"][0]["tokens"]), loss_fn_inputs=inputs))
    return out


def _adam_params(params: dict):
    try:
        import tinker.types as tt

        return tt.AdamParams(**params)
    except ImportError:
        return dict(params)


def _metric(result, *names) -> float:
    metrics = getattr(result, "metrics", None)
    if metrics is None and isinstance(result, dict):
        metrics = result.get("metrics")
    for n in names:
        if metrics and n in metrics:
            return float(metrics[n])
    return 0.0


def create_training_client(hcfg: HatcheryConfig, base_model: str):
    if _CLIENT_FACTORY is not None:
        return _CLIENT_FACTORY(hcfg, base_model)
    kw = dict(base_model=base_model, rank=hcfg.lora_rank, train_mlp=hcfg.train_mlp, train_attn=hcfg.train_attn,
              train_unembed=hcfg.train_unembed)
    if hcfg.backend == "tinker":
        try:
            import tinker
        except ImportError as e:
            raise ImportError("hatchery.backend: tinker needs the `tinker` package") from e
        key = hcfg.api_key or os.environ.get("TINKER_API_KEY")
        if not key:
            raise ValueError("Tinker API key required: set `hatchery.api_key` or the TINKER_API_KEY environment variable")
        os.environ["TINKER_API_KEY"] = key
        return tinker.ServiceClient(project_id=hcfg.project_id).create_lora_training_client(**kw)
    try:
        from hatchery.core.client import HatcheryClient
    except ImportError as e:
        raise ImportError("hatchery.backend: hatchery needs the `hatchery` package") from e
    client = HatcheryClient(base_url=hcfg.base_url or os.environ.get("HATCHERY_URL", "http://127.0.0.1:8420"),
                            token=hcfg.api_key or os.environ.get("HATCHERY_API_KEY", "dev"), timeout=hcfg.future_timeout)
    return client.create_lora_training_client(**kw)


def group_advantages(rewards, group_size: int):
    """(r - mean) / std inside every group of ``group_size`` samples of one prompt; std 1 for a constant group."""
    out = []
    for i in range(0, len(rewards), group_size):
        g = [float(r) for r in rewards[i:i + group_size]]
        mean = sum(g) / len(g)
        var = sum((r - mean) ** 2 for r in g) / len(g)
        std = var ** 0.5 if var > 1e-8 else 1.0
        out.extend((r - mean) / std for r in g)
    return out


def load_reward_func(path: str) -> Callable:
    mod, _, name = path.rpartition(".")
    fn = getattr(importlib.import_module(mod), name)
    if len(inspect.signature(fn).parameters) < 2:
        raise ValueError(f"reward function {path} must accept (prompts, completions)")
    return fn


# ------------------------------------------------------------------------------------------- loops
class RemoteTrainer:
    """Supervised loop against the remote service."""

    def __init__(self, cfg, hcfg: HatcheryConfig, dataset, log_fn: Callable | None = None):
        self.cfg, self.hcfg, self.dataset = cfg, hcfg, dataset
        self.client = None
        self.log_fn = log_fn or (lambda row: LOG.info("%s", row))
        self.optim = {"learning_rate": cfg.get("learning_rate") if cfg.get("learning_rate") is not None else 1e-4,
                      "beta1": cfg.get("adam_beta1") if cfg.get("adam_beta1") is not None else 0.9,
                      "beta2": cfg.get("adam_beta2") if cfg.get("adam_beta2") is not None else 0.95,
                      "eps": cfg.get("adam_epsilon") if cfg.get("adam_epsilon") is not None else 1e-12,
                      "weight_decay": cfg.get("weight_decay") or 0.0,
                      "grad_clip_norm": cfg.get("max_grad_norm") or 0.0}
        self.history = []

    def _client(self):
        if self.client is None:
            if not self.cfg.get("base_model"):
                raise ValueError("hatchery: base_model names the model the service trains")
            self.client = create_training_client(self.hcfg, self.cfg["base_model"])
            LOG.info("remote training session: backend=%s model=%s rank=%d", self.hcfg.backend, self.cfg["base_model"],
                     self.hcfg.lora_rank)
        return self.client

    def save_remote(self, step: int, name: str | None = None):
        ckpt = name or f"{self.hcfg.save_name_prefix}-{step:06d}"
        try:
            self._client().save_state(ckpt).result(timeout=self.hcfg.future_timeout)
            LOG.info("remote checkpoint saved: %s", ckpt)
        except Exception:
            LOG.exception("remote checkpoint %s failed", ckpt)
            if name == "final":
                raise

    def _micro_batches(self):
        mb = int(self.cfg.get("micro_batch_size") or 1)
        n = len(self.dataset)
        for i in range(0, n, mb):
            yield [self.dataset[j] for j in range(i, min(i + mb, n))]

    def train(self):
        h = self.hcfg
        accum = int(self.cfg.get("gradient_accumulation_steps") or 1)
        epochs = int(self.cfg.get("num_epochs") or 1)
        mb = int(self.cfg.get("micro_batch_size") or 1)
        per_epoch = max(((len(self.dataset) + mb - 1) // mb) // accum, 1)
        max_steps = int(self.cfg.get("max_steps") or 0) or per_epoch * epochs
        step, total, t0 = 0, 0.0, time.time()
        pending_optim = None
        for _ in range(epochs):
            pending = []
            for rows in self._micro_batches():
                if step >= max_steps:
                    break
                datums = [row_to_datum_sft(r["input_ids"], r["labels"]) for r in rows]
                active = sum(int((np.asarray(r["labels"])[1:] != -100).sum()) for r in rows)
                fut = self._client().forward_backward(_to_sdk(datums), loss_fn=h.loss_fn, loss_fn_config=h.loss_fn_config)
                pending.append((fut, active))
                if len(pending) < accum:
                    continue
                loss_sum = sum(_metric(f.result(timeout=h.future_timeout), "loss:sum", "loss") for f, _ in pending)
                n_active = sum(a for _, a in pending)
                pending = []
                if pending_optim is not None:          # pipelined: the previous step's result is collected only now
                    pending_optim.result(timeout=h.future_timeout)
                pending_optim = self._client().optim_step(_adam_params(self.optim))
                if not h.pipeline:
                    pending_optim.result(timeout=h.future_timeout)
                    pending_optim = None
                step += 1
                loss = loss_sum / n_active if n_active else loss_sum
                total += loss
                row = {"step": step, "loss": loss, "active_tokens": n_active, "learning_rate": self.optim["learning_rate"]}
                self.history.append(row)
                if step % int(self.cfg.get("logging_steps") or 1) == 0:
                    self.log_fn(row)
                if h.save_steps and step % h.save_steps == 0:
                    self.save_remote(step)
            if step >= max_steps:
                break
        if pending_optim is not None:
            pending_optim.result(timeout=h.future_timeout)
        if step:
            self.save_remote(step, "final")
        return {"global_step": step, "train_loss": total / max(step, 1), "train_runtime": time.time() - t0}


class RemoteRLTrainer(RemoteTrainer):
    """Sample -> reward -> advantage -> policy-gradient step, all model work on the service."""

    def __init__(self, cfg, hcfg, dataset, tokenizer, log_fn=None):
        super().__init__(cfg, hcfg, dataset, log_fn)
        self.tokenizer = tokenizer
        if not hcfg.reward_funcs:
            raise ValueError("hatchery: a policy-gradient loss_fn needs `hatchery.reward_funcs` (module.function paths)")
        self.reward_funcs = [load_reward_func(p) for p in hcfg.reward_funcs]

    def sample(self, prompts_ids):
        h = self.hcfg
        sc = self._client().save_weights_and_get_sampling_client()
        out = []
        for ids in prompts_ids:
            if hasattr(sc, "sampling_session_id"):        # Hatchery's client
                res = sc.sample(list(ids), max_tokens=h.max_sample_tokens, temperature=h.sample_temperature,
                                n=h.num_samples).result(timeout=h.future_timeout)
            else:
                import tinker.types as tt

                res = sc.sample(prompt=tt.ModelInput.from_ints(list(ids)), num_samples=h.num_samples,
                                sampling_params=tt.SamplingParams(max_tokens=h.max_sample_tokens, temperature=h.sample_temperature,
                                                                  top_p=0.95, top_k=-1)).result(timeout=h.future_timeout)
            seqs = res.sequences if hasattr(res, "sequences") else res.get("sequences", [])
            for seq in seqs:
                toks = list(seq.tokens) if hasattr(seq, "tokens") else list(seq.get("tokens", []))
                lps = list(getattr(seq, "logprobs", None) or []) if not isinstance(seq, dict) else list(seq.get("logprobs") or [])
                out.append({"tokens": list(ids) + toks, "completion": toks, "logprobs": lps, "prompt_len": len(ids)})
        return out

    def train(self):
        h, tok = self.hcfg, self.tokenizer
        max_steps = int(self.cfg.get("max_steps") or 0) or 1000
        epochs = int(self.cfg.get("num_epochs") or 1)
        step, total, total_reward, t0 = 0, 0.0, 0.0, time.time()
        for _ in range(epochs):
            for rows in self._micro_batches():
                if step >= max_steps:
                    break
                texts = [tok.decode(r["input_ids"], skip_special_tokens=False) for r in rows]
                # a gold answer embedded for the reward function is not shown to the sampler
                clean = [tok.encode(re.sub(r"<\|gold\|>.*?<\|/gold\|>", "", t), add_special_tokens=False) for t in texts]
                samples = self.sample(clean)
                if not samples:
                    LOG.warning("no samples returned, step skipped")
                    continue
                completions = [tok.decode(s["completion"], skip_special_tokens=False) for s in samples]
                prompts = [t for t in texts for _ in range(h.num_samples)]
                rewards = [0.0] * len(completions)
                for fn in self.reward_funcs:
                    for i, r in enumerate(fn(prompts, completions)):
                        rewards[i] += float(r)
                adv = group_advantages(rewards, h.num_samples)
                loss_sum = 0.0
                for s, a in zip(samples, adv):
                    d = row_to_datum_rl(s["tokens"], s["prompt_len"], s["logprobs"], a)
                    res = self._client().forward_backward(_to_sdk([d]), loss_fn=h.loss_fn, loss_fn_config=h.loss_fn_config)
                    loss_sum += _metric(res.result(timeout=h.future_timeout), "loss:sum")
                fut = self._client().optim_step(_adam_params(self.optim))
                if not h.pipeline:
                    fut.result(timeout=h.future_timeout)
                step += 1
                mean_r = sum(rewards) / len(rewards)
                total += loss_sum
                total_reward += mean_r
                row = {"step": step, "loss": loss_sum, "reward": mean_r, "accuracy": sum(r > 0 for r in rewards) / len(rewards),
                       "mean_abs_advantage": sum(abs(a) for a in adv) / len(adv), "learning_rate": self.optim["learning_rate"]}
                self.history.append(row)
                if step % int(self.cfg.get("logging_steps") or 1) == 0:
                    self.log_fn(row)
                if h.save_steps and step % h.save_steps == 0:
                    self.save_remote(step)
            if step >= max_steps:
                break
        if step:
            self.save_remote(step, "final")
        return {"global_step": step, "train_loss": total / max(step, 1), "train_reward": total_reward / max(step, 1),
                "train_runtime": time.time() - t0}


class HatcheryPlugin(BasePlugin):
    def get_input_args(self):
        return HatcheryArgs

    def register(self, cfg):
        if cfg.get("remove_unused_columns") is None:
            cfg["remove_unused_columns"] = False

    def run_training(self, cfg, dataset_meta, tokenizer=None):
        """Takes the place of the local run: no model is built, nothing is saved locally."""
        raw = cfg.get("hatchery") or {}
        hcfg = raw if isinstance(raw, HatcheryConfig) else HatcheryConfig(**dict(raw))
        if dataset_meta is None or dataset_meta.train is None:
            raise ValueError("hatchery: the remote loop needs a tokenised training dataset (`datasets:`)")
        if hcfg.loss_fn in RL_LOSSES:
            if tokenizer is None:
                raise ValueError("hatchery: the RL loop decodes prompts and completions, a tokenizer is required")
            trainer = RemoteRLTrainer(cfg, hcfg, dataset_meta.train, tokenizer)
        else:
            trainer = RemoteTrainer(cfg, hcfg, dataset_meta.train)
        out = trainer.train()
        LOG.info("hatchery: weights live on the remote service (checkpoint `final`); nothing is saved locally")
        out["history"] = trainer.history
        return out
