"""``load_cfg``: YAML (path, directory chooser or https URL) -> CLI overrides -> plugin
registration -> schema + cross-field validation -> normalisation -> DictDefault
(flow of src/axolotl/cli/config.py:233-341)."""
from __future__ import annotations

import os
import tempfile
from pathlib import Path

import yaml

from ..utils.logging import get_logger
from .dict import DictDefault
from .normalize import normalize
from .schema import AxolotlConfig, check_keys
from .validation import validate

LOG = get_logger(__name__)
_SECRET_KEYS = ("wandb_api_key", "comet_api_key", "hf_token", "hub_token")


def coerce_value(v):
    """CLI strings -> bool/int/float/None/list where unambiguous."""
    if not isinstance(v, str):
        return v
    low = v.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    try:
        return int(v)
    except ValueError:
        pass
    try:
        return float(v)
    except ValueError:
        pass
    if v.startswith("[") or v.startswith("{"):
        try:
            return yaml.safe_load(v)
        except yaml.YAMLError:
            return v
    return v


def apply_overrides(raw: dict, overrides: dict) -> dict:
    """``parent__child=value`` addresses nested keys (same convention as the reference CLI)."""
    for k, v in overrides.items():
        if v is None:
            continue
        v = coerce_value(v)
        parts = k.split("__")
        d = raw
        for p in parts[:-1]:
            if not isinstance(d.get(p), dict):
                d[p] = {}
            d = d[p]
        d[parts[-1]] = v
    return raw


def fetch_config(path: str) -> str:
    if path.startswith(("http://", "https://")):
        import requests

        r = requests.get(path, timeout=30)
        r.raise_for_status()
        tmp = tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False)
        tmp.write(r.text)
        tmp.close()
        return tmp.name
    p = Path(path)
    if p.is_dir():
        cands = sorted(list(p.glob("*.yml")) + list(p.glob("*.yaml")))
        if not cands:
            raise FileNotFoundError(f"no YAML config found in {path}")
        if len(cands) > 1:
            LOG.warning("several configs in %s, using %s", path, cands[0].name)
        return str(cands[0])
    return str(p)


def gpu_capabilities() -> dict:
    import torch

    if not torch.cuda.is_available():
        return {"bf16": True, "tf32": False, "fp8": False, "n_gpu": 0, "compute_capability": None}
    major, minor = torch.cuda.get_device_capability()
    return {"bf16": major >= 8, "tf32": major >= 8, "fp8": major >= 9, "n_gpu": torch.cuda.device_count(),
            "compute_capability": f"sm_{major}{minor}"}


def redact(cfg: dict) -> dict:
    return {k: ("***" if any(s in k for s in _SECRET_KEYS) and v else v) for k, v in cfg.items()}


def validate_config(raw: dict, capabilities: dict | None = None) -> DictDefault:
    raw = dict(raw)
    inert = check_keys(raw)
    warnings = validate(raw, capabilities)
    model = AxolotlConfig(**raw)
    out = model.model_dump(exclude_none=True)
    for k in inert:
        LOG.info("config key '%s' has no effect on axolotl_b200", k)
    for m in warnings:
        LOG.warning(m)
    return DictDefault(out)


def load_cfg(config: str | dict, **overrides) -> DictDefault:
    if isinstance(config, dict):
        raw = dict(config)
        path = None
    else:
        path = fetch_config(config)
        with open(path) as fh:
            raw = yaml.safe_load(fh) or {}
    raw = apply_overrides(raw, overrides)
    if path:
        raw["axolotl_config_path"] = path
    if raw.get("plugins"):
        from ..plugins.base import PluginManager

        pm = PluginManager.get_instance()
        for name in raw["plugins"]:
            pm.register(name)
        # plugin-contributed keys are validated by the plugins' own pydantic models
        extra = pm.get_input_keys()
        plugin_vals = {k: raw.pop(k) for k in list(raw) if k in extra}
        plugin_vals = pm.validate_input(plugin_vals)
    else:
        plugin_vals = {}
    cfg = validate_config(raw, gpu_capabilities())
    cfg.update(plugin_vals)
    normalize(cfg)
    LOG.debug("config: %s", redact(cfg))
    return cfg
