"""NeMo-Gym environments as GRPO reward sources (single-turn mode).

A NeMo-Gym deployment has a head server that publishes the deployment's configuration and one
"resources server" per environment with a ``/verify`` endpoint: given the prompt and the model's
answer in the OpenAI *Responses* wire format it returns ``{"reward": float}``. Dataset rows name
their environment (``resources_server_ref: {name: ...}``) and may carry extra verifier fields
(``verify_extra``); both columns reach the reward function through the rollout producer.
Reference: src/axolotl/integrations/nemo_gym/{plugin.py:135-700, rewards.py, args.py}.

Multi-turn mode (``nemo_gym_multi_turn: true``): the deployment's AGENT servers run the episodes. For every sample
the trainer POSTs the dataset row to an agent's ``/run`` endpoint; the agent generates through the policy's
generation server (``axolotl vllm-serve``, kept in sync by the usual adapter hand-over), executes tool calls, feeds
their results back for further turns and scores the episode. The answer lists the turns with their token ids and
sampling log-probs; turns are stitched into one completion in which the tokens an environment inserted (tool
results) stay in the context but are masked out of the loss, and the episode reward takes the place of reward
functions (reference: multi_turn.py:31-329, data_producer.py:32-279, server.py:170-199). Starting / cloning the Gym
servers from the trainer is not implemented: the servers are expected to be running.

YAML::

    plugins: [axolotl.integrations.nemo_gym.NemoGymPlugin]
    nemo_gym_enabled: true
    nemo_gym_head_port: 11000
    rl: grpo
    trl:
      reward_funcs: [axolotl_b200.plugins.nemo_gym.reward_nemo_gym_verify]
"""
from __future__ import annotations

import threading

from pydantic import BaseModel

from ..utils.logging import get_logger
from .base import BasePlugin

LOG = get_logger(__name__)
_STATE = {"head": "http://127.0.0.1:11000", "verify_timeout": 30, "urls": None}
_LOCK = threading.Lock()


class NemoGymArgs(BaseModel):
    nemo_gym_enabled: bool | None = None
    nemo_gym_dir: str | None = None
    nemo_gym_auto_clone: bool | None = None
    nemo_gym_config_paths: list[str] | None = None
    nemo_gym_head_port: int | None = 11000
    nemo_gym_head_host: str | None = "127.0.0.1"
    nemo_gym_server_timeout: int | None = 360
    nemo_gym_verify_timeout: int | None = 30
    nemo_gym_run_timeout: int | None = None
    nemo_gym_datasets: list[dict] | None = None
    nemo_gym_auto_start: bool | None = None
    nemo_gym_model_name: str | None = None
    nemo_gym_multi_turn: bool | None = None
    nemo_gym_max_turns: int | None = None


def discover_verify_urls(head_url: str | None = None, timeout: float = 5.0, refresh: bool = False) -> dict:
    """{environment name: verify URL} from the head server's published configuration (cached)."""
    import requests
    import yaml

    with _LOCK:
        if _STATE["urls"] is not None and not refresh:
            return _STATE["urls"]
        urls = {}
        try:
            text = requests.get(f"{(head_url or _STATE['head']).rstrip('/')}/global_config_dict_yaml", timeout=timeout).text
            conf = yaml.safe_load(text)
            if isinstance(conf, str):      # the endpoint may wrap the YAML document in a YAML string
                conf = yaml.safe_load(conf)
            for block in (conf or {}).values():
                if not isinstance(block, dict):
                    continue
                for name, srv in (block.get("resources_servers") or {}).items():
                    if isinstance(srv, dict) and "host" in srv and "port" in srv:
                        urls[name] = f"http://{srv['host']}:{srv['port']}/verify"
        except Exception as exc:   # the trainer keeps going with zero rewards, as the reference does
            LOG.warning("NeMo-Gym head server not reachable: %s", exc)
        _STATE["urls"] = urls
        return urls


def _text(x):
    if isinstance(x, (list, tuple)):       # chat-format prompt / completion
        return x[0].get("content", "") if x and isinstance(x[0], dict) else ""
    return x if isinstance(x, str) else ""


def _verify_request(prompt, answer, extra):
    req = {k: v for k, v in (extra or {}).items() if v is not None}
    req["responses_create_params"] = {"input": [{"role": "user", "content": prompt}]}
    req["response"] = {
        "id": "resp", "created_at": 0, "model": "axolotl_b200", "object": "response",
        "output": [{"id": "msg", "role": "assistant", "type": "message", "status": "completed",
                    "content": [{"type": "output_text", "text": answer, "annotations": []}]}],
        "parallel_tool_calls": True, "tool_choice": "auto", "tools": [],
    }
    return req


def reward_nemo_gym_verify(completions, prompts=None, resources_server_ref=None, verify_extra=None, **kwargs):
    """One ``/verify`` call per completion; 0.0 when the row names no known environment or the call fails."""
    import requests

    urls = discover_verify_urls()
    out = []
    for i, c in enumerate(completions):
        ref = resources_server_ref[i] if resources_server_ref and i < len(resources_server_ref) else None
        name = ref.get("name", "") if isinstance(ref, dict) else (ref or "")
        url = urls.get(name)
        if not url:
            out.append(0.0)
            continue
        prompt = _text(prompts[i]) if prompts and i < len(prompts) else ""
        extra = verify_extra[i] if verify_extra and i < len(verify_extra) else None
        try:
            r = requests.post(url, json=_verify_request(prompt, _text(c), extra), timeout=_STATE["verify_timeout"])
            out.append(float(r.json().get("reward", 0.0)) if r.ok else 0.0)
        except Exception as exc:
            LOG.warning("verify request to %s failed: %s", url, exc)
            out.append(0.0)
    return out


def discover_agent_servers(head_url: str | None = None, timeout: float = 5.0) -> dict:
    """{top-level config name: agent URL} for every block of the head server's configuration that declares
    ``responses_api_agents`` (dataset rows name their agent by that top-level name in ``agent_ref.name``)."""
    import requests
    import yaml

    agents = {}
    try:
        conf = yaml.safe_load(requests.get(f"{(head_url or _STATE['head']).rstrip('/')}/global_config_dict_yaml", timeout=timeout).text)
        if isinstance(conf, str):
            conf = yaml.safe_load(conf)
        for top, block in (conf or {}).items():
            if not isinstance(block, dict):
                continue
            for acfg in (block.get("responses_api_agents") or {}).values():
                if isinstance(acfg, dict) and acfg.get("port"):
                    agents[top] = f"http://{acfg.get('host', '127.0.0.1')}:{acfg['port']}"
    except Exception as exc:
        LOG.warning("NeMo-Gym head server not reachable: %s", exc)
    return agents


def parse_agent_response(response, eos_token_id: int) -> dict:
    """One ``/run`` answer -> prompt ids, one stitched completion, the mask of policy-written tokens, sampling
    log-probs, reward, number of turns. A failed or empty episode becomes a one-token masked sample that keeps its
    reward (the group statistics still see it, the loss does not)."""
    blank = {"prompt_ids": [eos_token_id], "completion_ids": [eos_token_id], "env_mask": [0], "logprobs": [0.0],
             "reward": 0.0, "num_turns": 0}
    if not isinstance(response, dict) or "error" in response:
        return blank
    turns = (response.get("response") or {}).get("output") or []
    blank["reward"] = float(response.get("reward", 0.0))

    def says_something(item):
        if item.get("type") == "function_call":
            return True
        return item.get("type") == "message" and any(
            isinstance(c, dict) and c.get("type") == "output_text" and (c.get("text") or "").strip() for c in item.get("content") or [])
    if not any(says_something(t) for t in turns):
        return blank
    first, seen = None, []
    completion, mask, logps, n_turns = [], [], [], 0
    for t in turns:
        gen = list(t.get("generation_token_ids") or [])
        if not gen:
            continue
        ctx = list(t.get("prompt_token_ids") or [])
        n_turns += 1
        if first is None:
            first = ctx
        elif len(ctx) > len(seen):           # what the environment appended since the last turn: context, not policy
            extra = ctx[len(seen):]
            completion += extra
            mask += [0] * len(extra)
            logps += [0.0] * len(extra)
        lp = [float(v) for v in (t.get("generation_log_probs") or [])][: len(gen)]
        completion += gen
        mask += [1] * len(gen)
        logps += lp + [0.0] * (len(gen) - len(lp))
        seen = ctx + gen
    if first is None:
        return blank
    return {"prompt_ids": first, "completion_ids": completion, "env_mask": mask, "logprobs": logps,
            "reward": blank["reward"], "num_turns": n_turns}


class AgentRollout:
    """Rollout source of the multi-turn mode: one ``/run`` request per sample, in parallel."""

    def __init__(self, inner, agent_servers: dict, eos_token_id: int, timeout: float = 10800.0, max_workers: int = 64):
        self.inner, self.agents, self.eos, self.timeout, self.max_workers = inner, dict(agent_servers), eos_token_id, timeout, max_workers
        if not self.agents:
            raise ValueError("nemo_gym_multi_turn: the head server lists no agent server (`responses_api_agents`)")

    def sync_weights(self, model, step):      # the agents sample from the generation server the inner engine talks to
        return self.inner.sync_weights(model, step)

    def _request(self, rec, max_len, temperature, top_p):
        item = dict(rec.get("verify_extra") or {})
        if not item:
            prompt = rec.get("prompt")
            text = prompt[-1].get("content", "") if isinstance(prompt, list) and prompt and isinstance(prompt[-1], dict) else (prompt or "")
            item = {"responses_create_params": {"input": [{"role": "user", "content": text}]}}
        if "agent_ref" not in item and rec.get("agent_ref"):
            item["agent_ref"] = rec["agent_ref"]
        params = item.setdefault("responses_create_params", {})
        params = item["responses_create_params"] = dict(params)
        params.setdefault("max_output_tokens", max_len)
        params["temperature"], params["top_p"] = temperature, (top_p if top_p and top_p < 1.0 else 0.999)
        name = (item.get("agent_ref") or {}).get("name", "")
        return self.agents.get(name) or next(iter(self.agents.values())), item

    def _run(self, url, body):
        import requests

        try:
            r = requests.post(f"{url}/run", json=body, timeout=self.timeout)
            if r.status_code == 200:
                return r.json()
            return {"error": f"HTTP {r.status_code}: {r.text[:200]}"}
        except Exception as exc:   # noqa: BLE001 - a lost episode must not stop the step
            LOG.warning("agent /run failed: %s", exc)
            return {"error": str(exc)}

    def rollouts(self, recs, n, max_len, temperature=1.0, top_p=1.0):
        """Prompt-major list of len(recs) * n parsed episodes."""
        from concurrent.futures import ThreadPoolExecutor

        jobs = [self._request(r, max_len, temperature, top_p) for r in recs for _ in range(n)]
        with ThreadPoolExecutor(max_workers=min(self.max_workers, max(len(jobs), 1))) as ex:
            answers = list(ex.map(lambda j: self._run(*j), jobs))
        return [parse_agent_response(a, self.eos) for a in answers]


def reward_env(completions, env_reward=None, **kwargs):
    """Passthrough of a reward an environment already attached to the sample (``env_reward`` column)."""
    if env_reward is None:
        return [0.0] * len(completions)
    if isinstance(env_reward, (list, tuple)):
        return [float(r) for r in env_reward]
    return [float(env_reward)] * len(completions)


class NemoGymPlugin(BasePlugin):
    def get_input_args(self):
        return NemoGymArgs

    def register(self, cfg):
        if not cfg.get("nemo_gym_enabled"):
            return
        if cfg.get("nemo_gym_multi_turn") and not (cfg.get("trl") or {}).get("use_vllm"):
            raise ValueError("nemo_gym_multi_turn: the agents generate through a served policy, set trl.use_vllm "
                             "(and start `axolotl vllm-serve`)")
        _STATE["head"] = f"http://{cfg.get('nemo_gym_head_host') or '127.0.0.1'}:{cfg.get('nemo_gym_head_port') or 11000}"
        _STATE["verify_timeout"] = cfg.get("nemo_gym_verify_timeout") or 30
        _STATE["urls"] = None

    def wrap_rollout_engine(self, cfg, engine):
        if not (cfg.get("nemo_gym_enabled") and cfg.get("nemo_gym_multi_turn")):
            return None
        eos = cfg.get("eos_token_id")
        return AgentRollout(engine, discover_agent_servers(), int(eos if eos is not None else 0),
                            timeout=float(cfg.get("nemo_gym_run_timeout") or 10800))

    def pre_model_load(self, cfg):
        self.register(cfg)
        if cfg.get("nemo_gym_enabled"):
            LOG.info("NeMo-Gym environments: %s", sorted(discover_verify_urls(refresh=True)) or "none reachable")
