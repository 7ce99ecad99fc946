"""Plugin system: lifecycle hooks around config loading, model building, trainer creation and
training (the hook set of the reference's BasePlugin / PluginManager,
src/axolotl/integrations/base.py:54-760). YAML: ``plugins: [package.module.ClassName]``; the
short names of the bundled plugins (``grokfast``, ``spectrum``, ``lm_eval`` ...) also resolve.
"""
from __future__ import annotations

import importlib

from ..utils.logging import get_logger

LOG = get_logger(__name__)


class BasePlugin:
    """Override what you need; every hook has a no-op default."""

    def register(self, cfg): ...
    def get_input_args(self):  # -> pydantic model class or None (extra config keys)
        return None
    def get_input_keys(self):
        m = self.get_input_args()
        return set(m.model_fields) if m is not None else set()
    def load_datasets(self, cfg, preprocess=False):
        return None
    def pre_model_load(self, cfg): ...
    def post_model_build(self, cfg, model): ...
    def pre_lora_load(self, cfg, model): ...
    def post_lora_load(self, cfg, model): ...
    def post_model_load(self, cfg, model): ...
    def get_trainer_cls(self, cfg):
        return None
    def get_collator_cls_and_kwargs(self, cfg, is_eval=False):
        return None
    def create_optimizer(self, cfg, trainer_or_model):
        return None
    def create_lr_scheduler(self, cfg, optimizer, num_training_steps):
        return None
    def add_callbacks_pre_trainer(self, cfg, model):
        return []
    def add_callbacks_post_trainer(self, cfg, trainer):
        return []
    def post_trainer_create(self, cfg, trainer): ...
    def compute_loss(self, cfg):
        """Optional replacement for the trainer's loss: callable(model, device_batch, num_items) -> loss."""
        return None
    def wrap_rollout_engine(self, cfg, engine):
        """Online-RL runs: a plugin may put its own rollout source in front of the generation engine."""
        return None
    def run_training(self, cfg, dataset_meta, tokenizer=None):
        """A plugin that trains somewhere else (a remote service) returns its result dict here; the local run (model
        build, trainer, saving) is then skipped. None = train locally."""
        return None
    def post_train(self, cfg, model): ...
    def post_train_unload(self, cfg): ...


_BUNDLED = {
    "grokfast": "axolotl_b200.plugins.grokfast.GrokfastPlugin",
    "spectrum": "axolotl_b200.plugins.spectrum.SpectrumPlugin",
    "lm_eval": "axolotl_b200.plugins.lm_eval.LMEvalPlugin",
    "kd": "axolotl_b200.plugins.kd.KDPlugin",
    "mora": "axolotl_b200.plugins.compat.MoraPlugin",
    "diffusion": "axolotl_b200.plugins.diffusion.DiffusionPlugin",
    "densemixer": "axolotl_b200.plugins.compat.DenseMixerPlugin",
    "nemo_gym": "axolotl_b200.plugins.nemo_gym.NemoGymPlugin",
    "llm_compressor": "axolotl_b200.plugins.sparse_ft.LLMCompressorPlugin",
    "swanlab": "axolotl_b200.plugins.swanlab.SwanLabPlugin",
    "hatchery": "axolotl_b200.plugins.hatchery.HatcheryPlugin",
    "liger": "axolotl_b200.plugins.compat.NativeKernelsPlugin",
    "cut_cross_entropy": "axolotl_b200.plugins.compat.NativeKernelsPlugin",
    "kernels": "axolotl_b200.plugins.compat.NativeKernelsPlugin",
    "expert_parallel": "axolotl_b200.plugins.compat.ExpertParallelPlugin",
}
# reference plugin class paths that map onto native functionality
_ALIASES = {
    "axolotl.integrations.liger.LigerPlugin": "liger",
    "axolotl.integrations.cut_cross_entropy.CutCrossEntropyPlugin": "cut_cross_entropy",
    "axolotl.integrations.kernels.KernelsPlugin": "kernels",
    "axolotl.integrations.expert_parallel.ExpertParallelPlugin": "expert_parallel",
    "axolotl.integrations.grokfast.GrokfastPlugin": "grokfast",
    "axolotl.integrations.spectrum.SpectrumPlugin": "spectrum",
    "axolotl.integrations.lm_eval.LMEvalPlugin": "lm_eval",
    "axolotl.integrations.kd.KDPlugin": "kd",
    "axolotl.integrations.mora.MoraPlugin": "mora",
    "axolotl.integrations.diffusion.DiffusionPlugin": "diffusion",
    "axolotl.integrations.densemixer.DenseMixerPlugin": "densemixer",
    "axolotl.integrations.nemo_gym.NemoGymPlugin": "nemo_gym",
    "axolotl.integrations.llm_compressor.LLMCompressorPlugin": "llm_compressor",
    "axolotl.integrations.swanlab.SwanLabPlugin": "swanlab",
    "axolotl.integrations.hatchery.HatcheryPlugin": "hatchery",
}


def load_plugin(name: str) -> BasePlugin:
    name = _ALIASES.get(name, name)
    path = _BUNDLED.get(name, name)
    mod, _, cls = path.rpartition(".")
    if not mod:
        raise ImportError(f"plugin '{name}' is neither a bundled plugin nor a module.Class path")
    obj = getattr(importlib.import_module(mod), cls)
    inst = obj()
    if not isinstance(inst, BasePlugin):
        raise TypeError(f"{path} does not derive from BasePlugin")
    return inst


class PluginManager:
    _instance = None

    def __init__(self):
        self.plugins: dict[str, BasePlugin] = {}

    @classmethod
    def get_instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    @classmethod
    def reset(cls):
        cls._instance = None

    def register(self, name):
        if name in self.plugins:
            return self.plugins[name]
        p = load_plugin(name)
        self.plugins[name] = p
        LOG.info("registered plugin %s", name)
        return p

    def get_input_keys(self):
        keys = set()
        for p in self.plugins.values():
            keys |= p.get_input_keys()
        return keys

    def validate_input(self, values: dict) -> dict:
        """Runs every plugin's args model over its own keys (type coercion, validators); keys the
        user did not give stay absent."""
        out = dict(values)
        for p in self.plugins.values():
            model = p.get_input_args()
            if model is None:
                continue
            mine = {k: v for k, v in values.items() if k in model.model_fields}
            checked = model(**mine).model_dump(exclude_unset=True)
            out.update({k: checked[k] for k in mine if k in checked})
        return out

    def _each(self, hook, *args, **kw):
        out = []
        for p in self.plugins.values():
            r = getattr(p, hook)(*args, **kw)
            if r is not None:
                out.append(r)
        return out

    def first(self, hook, *args, **kw):
        for p in self.plugins.values():
            r = getattr(p, hook)(*args, **kw)
            if r is not None:
                return r
        return None

    def call(self, hook, *args, **kw):
        self._each(hook, *args, **kw)

    def collect_callbacks(self, hook, *args):
        cbs = []
        for r in self._each(hook, *args):
            cbs.extend(r)
        return cbs
