"""NeMo-Gym environments as GRPO reward sources (single-turn mode).

A NeMo-Gym deployment has a head server that publishes the deployment's configuration and one
"resources server" per environment with a ``/verify`` endpoint: given the prompt and the model's
answer in the OpenAI *Responses* wire format it returns ``{"reward": float}``. Dataset rows name
their environment (``resources_server_ref: {name: ...}``) and may carry extra verifier fields
(``verify_extra``); both columns reach the reward function through the rollout producer.
Reference: src/axolotl/integrations/nemo_gym/{plugin.py:135-700, rewards.py, args.py}. The
multi-turn mode (agent ``/run`` rollouts replacing local generation) and starting / cloning the
Gym servers from the trainer are not implemented: the servers are expected to be running.

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
        if cfg.get("nemo_gym_multi_turn"):
            raise ValueError("nemo_gym_multi_turn (agent /run rollouts) is not implemented; single-turn /verify rewards are")
        _STATE["head"] = f"http://{cfg.get('nemo_gym_head_host') or '127.0.0.1'}:{cfg.get('nemo_gym_head_port') or 11000}"
        _STATE["verify_timeout"] = cfg.get("nemo_gym_verify_timeout") or 30
        _STATE["urls"] = None

    def pre_model_load(self, cfg):
        self.register(cfg)
        if cfg.get("nemo_gym_enabled"):
            LOG.info("NeMo-Gym environments: %s", sorted(discover_verify_urls(refresh=True)) or "none reachable")
