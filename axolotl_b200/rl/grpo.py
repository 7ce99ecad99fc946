"""Group-relative policy optimisation (GRPO and its dr_grpo / bnpo / dapo / GSPO variants).

Pipeline per optimizer step: sample ``num_generations`` completions for each prompt with a rollout
engine, score them with the configured reward functions, turn rewards into group-normalised
advantages, pack prompt+completion documents into one varlen row and optimise the clipped
surrogate (rl.losses.grpo_loss) for ``num_iterations`` passes. Rollouts can be produced
ahead of the learner by a background thread (importance ratios against the sampling policy's
log-probs correct the staleness) and zero-signal groups can be swapped for buffered informative
ones. Reference: src/axolotl/core/trainers/grpo/{trainer,async_trainer,replay_buffer,sampler}.py,
which wrap trl's GRPOTrainer and a vLLM server.

Rollout engines:
* ``LocalRollout``: decodes with the training model itself on packed varlen batches (every step
  re-scores the active documents; logits are computed only for each document's last position).
* ``VLLMServerRollout``: HTTP client for an external generation server speaking the
  ``/generate/`` JSON protocol of ``axolotl vllm-serve`` (prompt token ids in, completion token
  ids out); adapter weights are synchronised by writing the adapter to a directory the server
  reloads from.
"""
from __future__ import annotations

import importlib
import json
import queue
import threading

import numpy as np
import torch

from ..ops import functional as Fn
from ..ops.lora import linear
from . import losses as L
from .data import _DocPacker
from .logps import token_logps
from ..models.layers import disable_adapters


# ------------------------------------------------------------------------------- sampling
def sample_from_logits(logits, temperature=1.0, top_p=1.0, top_k=0, generator=None):
    """logits [n, V] fp32 -> token ids [n]; temperature 0 = greedy."""
    if not temperature or temperature <= 0:
        return logits.argmax(-1)
    logits = logits / temperature
    if top_k and top_k > 0:
        kth = logits.topk(min(top_k, logits.shape[-1]), -1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = torch.softmax(logits, -1)
    if top_p is not None and top_p < 1.0:
        sp, si = probs.sort(-1, descending=True)
        keep = sp.cumsum(-1) - sp < top_p
        sp = sp * keep
        probs = torch.zeros_like(probs).scatter_(1, si, sp)
        probs = probs / probs.sum(-1, keepdim=True)
    return torch.multinomial(probs, 1, generator=generator).squeeze(1)


class LocalRollout:
    def __init__(self, model, eos_token_id=None, pad_token_id=0, seed=0):
        self.model, self.eos, self.pad = model, eos_token_id, pad_token_id
        dev = model.embed_tokens.device
        self.gen = torch.Generator(device=dev).manual_seed(seed)

    @torch.no_grad()
    def generate(self, prompts, n, max_new_tokens, temperature=1.0, top_p=1.0, top_k=0):
        """prompts: list of id lists -> list (len(prompts) * n, prompt-major) of completion id lists.
        Decoding is incremental: one packed prefill of all prompts, then one KV-cache step per token."""
        from ..models.kv_cache import generate_cached

        seqs = [list(p) for p in prompts for _ in range(n)]
        return generate_cached(self.model, seqs, max_new_tokens, temperature, top_p, top_k, self.eos, self.gen)

    def sync_weights(self, model, step):   # same weights by construction
        return


class VLLMServerRollout:
    """Client of a generation server. Nothing here imports vllm: the server is a separate process
    (``axolotl vllm-serve``)."""

    def __init__(self, host="127.0.0.1", port=8000, timeout=600.0, adapter_sync_dir=None, save_adapter_fn=None):
        self.url = f"http://{host}:{port}"
        self.timeout, self.sync_dir, self.save_adapter_fn = timeout, adapter_sync_dir, save_adapter_fn

    def generate(self, prompts, n, max_new_tokens, temperature=1.0, top_p=1.0, top_k=0):
        import requests

        r = requests.post(self.url + "/generate/", timeout=self.timeout, json={
            "prompt_ids": [list(map(int, p)) for p in prompts], "n": n, "max_tokens": max_new_tokens,
            "temperature": temperature, "top_p": top_p, "top_k": top_k if top_k else -1})
        r.raise_for_status()
        return r.json()["completion_ids"]

    def sync_weights(self, model, step):
        if self.sync_dir and self.save_adapter_fn:
            import requests

            self.save_adapter_fn(self.sync_dir)
            requests.post(self.url + "/load_adapter/", timeout=self.timeout,
                          json={"path": self.sync_dir, "step": step}).raise_for_status()


# ------------------------------------------------------------------------------- rewards
def load_reward_funcs(names):
    """'pkg.module.func' dotted paths (the reference's ``trl.reward_funcs`` convention); callables
    pass through. A reward function is called as ``f(prompts=..., completions=...,
    completion_ids=..., **dataset_columns)`` and returns one float per completion."""
    out = []
    for n in names or []:
        if callable(n):
            out.append(n)
            continue
        mod, _, fn = n.rpartition(".")
        if not mod:
            raise ValueError(f"reward function '{n}' must be a dotted path module.function")
        out.append(getattr(importlib.import_module(mod), fn))
    if not out:
        raise ValueError("grpo needs at least one reward function (trl.reward_funcs)")
    return out


class ReplayBuffer:
    """Keeps the most informative recent groups (largest reward spread) so that a group whose
    completions all got the same reward (zero advantage, no gradient) can be replaced."""

    def __init__(self, capacity=64):
        self.capacity, self.items = capacity, []

    def add(self, score, group):
        self.items.append((float(score), group))
        self.items.sort(key=lambda t: -t[0])
        del self.items[self.capacity:]

    def pop(self):
        return self.items.pop(0)[1] if self.items else None

    def __len__(self):
        return len(self.items)


# ------------------------------------------------------------------------------- rollout batches
class GRPOSettings:
    def __init__(self, cfg):
        t = dict(cfg.get("trl") or {})
        self.num_generations = t.get("num_generations") or 8
        self.max_completion_length = t.get("max_completion_length") or 256
        self.temperature = t.get("temperature") if t.get("temperature") is not None else 1.0
        self.top_p = t.get("top_p") if t.get("top_p") is not None else 1.0
        self.top_k = t.get("top_k") or 0
        self.beta = t.get("beta") if t.get("beta") is not None else 0.0
        self.epsilon = t.get("epsilon") if t.get("epsilon") is not None else 0.2
        self.epsilon_high = t.get("epsilon_high")
        self.loss_type = t.get("loss_type") or "dapo"
        self.scale_rewards = t.get("scale_rewards") if t.get("scale_rewards") is not None else "group"
        self.num_iterations = t.get("num_iterations") or 1
        self.reward_weights = t.get("reward_weights")
        self.importance_sampling_level = t.get("importance_sampling_level") or "token"
        self.mask_truncated = bool(t.get("mask_truncated_completions"))
        self.use_vllm = bool(t.get("use_vllm"))
        self.host, self.port = t.get("vllm_server_host") or "127.0.0.1", t.get("vllm_server_port") or 8000
        self.async_prefetch = int(t.get("async_prefetch") or 0)
        self.replay_buffer_size = int(t.get("replay_buffer_size") or 0)
        self.multi_objective = cfg.get("rl") == "gdpo"   # GDPO: normalise each reward separately, then combine


class RolloutProducer:
    """Turns prompt records into collated GRPO batches. ``prompts_per_batch`` prompts x
    ``num_generations`` completions form one packed row."""

    def __init__(self, model, engine, reward_funcs, settings: GRPOSettings, prompt_records, prompts_per_batch,
                 tokenizer=None, pad_token_id=0, eos_token_id=None, dp_rank=0, dp_size=1, seed=0):
        self.model, self.engine, self.rf, self.s = model, engine, reward_funcs, settings
        self.records, self.ppb, self.tok = prompt_records, prompts_per_batch, tokenizer
        self.pad, self.eos, self.rank, self.size, self.seed = pad_token_id, eos_token_id, dp_rank, dp_size, seed
        self.replay = ReplayBuffer(settings.replay_buffer_size) if settings.replay_buffer_size else None
        self.stats = {}

    def __len__(self):
        return len(self.records) // (self.ppb * self.size)

    def _rewards(self, recs, completions):
        n = self.s.num_generations
        prompts_rep = [r for r in recs for _ in range(n)]
        texts = [self.tok.decode(c, skip_special_tokens=True) for c in completions] if self.tok is not None else completions
        cols = {k: [r[k] for r in prompts_rep] for k in recs[0] if k not in ("prompt", "prompt_ids")}
        per_fn = []
        for f in self.rf:
            v = f(prompts=[r.get("prompt", r["prompt_ids"]) for r in prompts_rep], completions=texts,
                  completion_ids=completions, prompt_ids=[r["prompt_ids"] for r in prompts_rep], **cols)
            per_fn.append(torch.tensor([float(x) if x is not None else float("nan") for x in v]))
        R = torch.stack(per_fn, 1)                                    # [N, F]
        w = torch.tensor(self.s.reward_weights or [1.0] * len(self.rf))
        return R, w

    def make_batch(self, recs, step=0):
        s = self.s
        n = s.num_generations
        agent = None
        if hasattr(self.engine, "rollouts"):
            # an environment's agents drive the episodes (generation through the served policy, tool calls, several
            # turns) and score them: completions, the mask of policy-written tokens and the reward all come back
            agent = self.engine.rollouts(recs, n, s.max_completion_length, s.temperature, s.top_p)
            completions = [a["completion_ids"] for a in agent]
            env = torch.tensor([float(a["reward"]) for a in agent])
            if self.rf:
                R, w = self._rewards([dict(r, env_reward=None) for r in recs], completions)
                R, w = torch.cat([env[:, None], R], 1), torch.cat([torch.ones(1), w])
            else:
                R, w = env[:, None], torch.ones(1)
        else:
            completions = self.engine.generate([r["prompt_ids"] for r in recs], n, s.max_completion_length,
                                               s.temperature, s.top_p, s.top_k)
            R, w = self._rewards(recs, completions)
        if s.multi_objective:
            adv = sum(w[j] * L.group_advantages(R[:, j].nan_to_num(0.0), n, s.scale_rewards) for j in range(R.shape[1]))
            total = (R.nan_to_num(0.0) * w).sum(1)
        else:
            total = (R.nan_to_num(0.0) * w).sum(1)
            adv = L.group_advantages(total, n, s.scale_rewards)
        groups = []
        for g, r in enumerate(recs):
            sl = slice(g * n, (g + 1) * n)
            grp = {"prompt_ids": r["prompt_ids"], "completions": completions[sl], "adv": adv[sl].clone(),
                   "rewards": total[sl].clone()}
            if agent is not None:      # the agent tokenised the prompt itself (tool schemas, system turns)
                grp["prompts"] = [a["prompt_ids"] for a in agent[sl]]
                grp["masks"] = [a["env_mask"] for a in agent[sl]]
            spread = float(total[sl].std()) if n > 1 else 0.0
            if self.replay is not None:
                if spread > 0:
                    self.replay.add(spread, grp)
                elif len(self.replay):
                    grp = self.replay.pop()
            groups.append(grp)
        self.stats = {"reward": float(total.mean()), "reward_std": float(total.std()) if len(total) > 1 else 0.0,
                      "completion_length": float(np.mean([len(c) for c in completions]))}
        if agent is not None:
            self.stats["num_turns"] = float(np.mean([a.get("num_turns", 1) for a in agent]))
        for f in self.rf:   # model-based rewards report their own breakdown
            self.stats.update(getattr(f, "last_metrics", None) or {})
        return self.collate(groups)

    def collate(self, groups):
        s = self.s
        pk = _DocPacker()
        advs, trunc = [], []
        for g in groups:
            for i, (c, a) in enumerate(zip(g["completions"], g["adv"])):
                empty = not len(c)
                c = list(c) if not empty else [self.eos if self.eos is not None else self.pad]
                if "masks" in g and not empty:
                    pk.add(g["prompts"][i], c, g["masks"][i])
                else:
                    pk.add(g["prompt_ids"], c)
                advs.append(float(a))
                trunc.append(len(c) >= s.max_completion_length and (self.eos is None or c[-1] != self.eos))
        aux = {"advantages": torch.tensor(advs, dtype=torch.float32)}
        if s.mask_truncated:
            aux["keep_seq"] = torch.tensor([not t for t in trunc])
        b = pk.finish(self.pad, 64, aux, {"grpo": True})
        return b

    @torch.no_grad()
    def attach_policy_logps(self, b_dev):
        """Log-probs of the sampling policy (needed when a batch is optimised more than once or
        was generated ahead of the learner) and of the reference (when beta > 0)."""
        was = self.model.training
        self.model.eval()
        if self.s.num_iterations > 1 or self.s.async_prefetch:
            b_dev["old_logps"] = token_logps(self.model, b_dev)[0].detach()
        if self.s.beta:
            with disable_adapters():
                b_dev["ref_logps_tok"] = token_logps(self.model, b_dev)[0].detach()
        self.model.train(was)
        return b_dev

    def __call__(self, epoch):
        idx = np.arange(len(self.records))
        np.random.default_rng(self.seed + epoch).shuffle(idx)
        per = self.ppb * self.size
        batches = (idx[b * per + self.rank * self.ppb: b * per + (self.rank + 1) * self.ppb]
                   for b in range(len(idx) // per))
        if self.s.async_prefetch > 0:
            yield from self._prefetched(batches)
            return
        for step, mine in enumerate(batches):
            self.engine.sync_weights(self.model, step)
            b = self.make_batch([self.records[i] for i in mine], step)
            for _ in range(self.s.num_iterations):
                yield b

    def _prefetched(self, batches):
        """Producer thread generates up to ``async_prefetch`` batches ahead of the learner."""
        q: queue.Queue = queue.Queue(maxsize=self.s.async_prefetch)
        stop = object()
        err = []

        def work():
            try:
                for step, mine in enumerate(batches):
                    q.put(self.make_batch([self.records[i] for i in mine], step))
            except Exception as exc:   # surfaced on the consumer side
                err.append(exc)
            finally:
                q.put(stop)

        th = threading.Thread(target=work, daemon=True)
        th.start()
        step = 0
        while True:
            b = q.get()
            if b is stop:
                break
            for _ in range(self.s.num_iterations):
                yield b
            step += 1
            self.engine.sync_weights(self.model, step)
        th.join()
        if err:
            raise err[0]


class GRPOObjective:
    needs_reference = False

    def __init__(self, settings: GRPOSettings, producer: RolloutProducer | None = None):
        self.s, self.producer = settings, producer
        self.last_metrics = {}

    def __call__(self, model, b, n_items):
        s = self.s
        if self.producer is not None and "old_logps" not in b and "_logps_attached" not in b:
            self.producer.attach_policy_logps(b)
            b["_logps_attached"] = True
        lab = b["labels"].reshape(-1)
        ent = torch.zeros(lab.numel(), dtype=torch.float32, device=lab.device)
        tok, out = token_logps(model, b, entropy_out=ent)
        sid = b["seq_ids"].reshape(-1)
        mask = lab != -100
        if "keep_seq" in b:
            mask = mask & b["keep_seq"][sid.clamp(min=0).long()]
        loss, m = L.grpo_loss(tok, b.get("old_logps"), b.get("ref_logps_tok"), b["advantages"], sid, int(b["n_seq"]),
                              mask, beta=s.beta, epsilon=s.epsilon, epsilon_high=s.epsilon_high, loss_type=s.loss_type,
                              max_completion_length=s.max_completion_length,
                              importance_sampling_level=s.importance_sampling_level, num_items=n_items)
        coef = getattr(model.config, "router_aux_loss_coef", 0.0)
        ga = b.get("ga_steps", 1)
        if out.aux_loss is not None and coef:
            loss = loss + (coef / ga) * out.aux_loss.to(loss.dtype)
        m["entropy"] = (ent * mask).sum() / mask.sum().clamp(min=1)   # mean policy entropy of completion tokens
        self.last_metrics = {k: float(v) for k, v in m.items()}
        if self.producer is not None:
            self.last_metrics.update(self.producer.stats)
        return loss if s.loss_type == "dapo" else loss / ga


def load_prompt_records(cfg, tokenizer, split="train"):
    """Prompt datasets for online RL: rows with ``prompt`` (string, or a list of chat messages
    rendered through the chat template) or ``prompt_ids``; other columns reach the reward functions."""
    from ..data.loading import _shard, read_raw

    recs = []
    for d in cfg.get("datasets" if split == "train" else "test_datasets") or []:
        for r in _shard(read_raw(dict(d)), dict(d)):
            r = dict(r)
            if "prompt_ids" not in r:
                p = r["prompt"]
                if isinstance(p, (list, tuple)):
                    r["prompt_ids"] = list(tokenizer.apply_chat_template(list(p), tokenize=True, add_generation_prompt=True))
                else:
                    ids = list(tokenizer(p, add_special_tokens=False)["input_ids"])
                    if tokenizer.bos_token_id is not None:
                        ids = [tokenizer.bos_token_id] + ids
                    r["prompt_ids"] = ids
            mp = cfg.get("max_prompt_len")
            if mp and len(r["prompt_ids"]) > mp:
                r["prompt_ids"] = r["prompt_ids"][-mp:]
            recs.append(r)
    return recs
