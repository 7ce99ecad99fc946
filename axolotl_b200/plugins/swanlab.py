"""SwanLab experiment tracking (reference: src/axolotl/integrations/swanlab/plugins.py:18,
callbacks.py, args.py). The ``swanlab`` package is optional: without it the plugin validates the
config, warns once and logs nothing."""
from __future__ import annotations

import os

from pydantic import BaseModel, field_validator, model_validator

from ..train.trainer import Callback
from ..utils.logging import get_logger
from .base import BasePlugin

LOG = get_logger(__name__)
_MODES = ("cloud", "local", "offline", "disabled")


class SwanLabArgs(BaseModel):
    use_swanlab: bool | None = None
    swanlab_project: str | None = None
    swanlab_experiment_name: str | None = None
    swanlab_description: str | None = None
    swanlab_mode: str | None = None
    swanlab_workspace: str | None = None
    swanlab_api_key: str | None = None
    swanlab_log_model: bool | None = None
    swanlab_web_host: str | None = None
    swanlab_api_host: str | None = None
    swanlab_lark_webhook_url: str | None = None
    swanlab_lark_secret: str | None = None
    swanlab_log_completions: bool | None = None
    swanlab_completion_log_interval: int | None = None
    swanlab_completion_max_buffer: int | None = None

    @field_validator("swanlab_mode")
    @classmethod
    def _mode(cls, v):
        if v is not None and v not in _MODES:
            raise ValueError(f"swanlab_mode must be one of {_MODES}, got '{v}'")
        return v

    @field_validator("swanlab_project")
    @classmethod
    def _project(cls, v):
        if v is not None and not v.strip():
            raise ValueError("swanlab_project must not be empty")
        return v

    @model_validator(mode="after")
    def _needs_project(self):
        if self.use_swanlab and not self.swanlab_project:
            raise ValueError("use_swanlab: true requires swanlab_project")
        return self


class SwanLabCallback(Callback):
    def __init__(self, cfg):
        self.cfg, self.run, self.swanlab = cfg, None, None
        self.completions = []

    def on_train_begin(self, trainer):
        if trainer.rank != 0:
            return
        try:
            import swanlab
        except ImportError:
            LOG.warning("use_swanlab is set but the swanlab package is not installed: nothing is logged")
            return
        cfg = self.cfg
        for key, env in (("swanlab_api_key", "SWANLAB_API_KEY"), ("swanlab_web_host", "SWANLAB_WEB_HOST"),
                         ("swanlab_api_host", "SWANLAB_API_HOST"), ("swanlab_mode", "SWANLAB_MODE")):
            if cfg.get(key):
                os.environ[env] = str(cfg[key])
        self.swanlab = swanlab
        self.run = swanlab.init(project=cfg.get("swanlab_project"), experiment_name=cfg.get("swanlab_experiment_name"),
                                description=cfg.get("swanlab_description"), workspace=cfg.get("swanlab_workspace"),
                                mode=cfg.get("swanlab_mode"),
                                config={k: v for k, v in dict(cfg).items() if isinstance(v, (int, float, str, bool))})

    def on_log(self, trainer, logs):
        if self.swanlab is not None:
            self.swanlab.log({k: v for k, v in logs.items() if isinstance(v, (int, float))}, step=logs.get("step"))

    on_evaluate = on_log

    def on_train_end(self, trainer):
        if self.swanlab is not None:
            self.swanlab.finish()


class SwanLabPlugin(BasePlugin):
    def get_input_args(self):
        return SwanLabArgs

    def add_callbacks_post_trainer(self, cfg, trainer):
        if not cfg.get("use_swanlab") or cfg.get("swanlab_mode") == "disabled":
            return []
        return [SwanLabCallback(cfg)]
