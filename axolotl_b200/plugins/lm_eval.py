"""Post-training evaluation hook (reference: src/axolotl/integrations/lm_eval/__init__.py:13).
The lm-evaluation-harness package is not bundled; when it is importable the plugin shells out to
its CLI on the trained model, otherwise it logs how to run it."""
from __future__ import annotations

import shutil
import subprocess

from pydantic import BaseModel

from ..utils.logging import get_logger
from .base import BasePlugin

LOG = get_logger(__name__)


class LMEvalArgs(BaseModel):
    lm_eval_tasks: list[str] | None = None
    lm_eval_batch_size: int | None = 8
    lm_eval_post_train: bool | None = True


def build_command(cfg):
    tasks = ",".join(cfg.get("lm_eval_tasks") or [])
    model_args = f"pretrained={cfg['output_dir']}"
    return ["lm_eval", "--model", "hf", "--model_args", model_args, "--tasks", tasks,
            "--batch_size", str(cfg.get("lm_eval_batch_size") or 8), "--output_path", f"{cfg['output_dir']}/lm_eval"]


class LMEvalPlugin(BasePlugin):
    def get_input_args(self):
        return LMEvalArgs

    def post_train(self, cfg, model):
        if not cfg.get("lm_eval_tasks") or cfg.get("lm_eval_post_train") is False:
            return
        cmd = build_command(cfg)
        if shutil.which("lm_eval") is None:
            LOG.warning("lm_eval is not installed; run: %s", " ".join(cmd))
            return
        subprocess.run(cmd, check=False)
