"""Compatibility shims for reference plugins whose job is done natively here: Liger / cut-CE /
kernels plugins swap PyTorch modules for Triton kernels in the reference; on this framework the
hand-written kernels are always on, so these plugins only accept their config keys."""
from __future__ import annotations

from pydantic import BaseModel

from .base import BasePlugin


class NativeKernelArgs(BaseModel):
    liger_rope: bool | None = None
    liger_rms_norm: bool | None = None
    liger_layer_norm: bool | None = None
    liger_glu_activation: bool | None = None
    liger_cross_entropy: bool | None = None
    liger_fused_linear_cross_entropy: bool | None = None
    cut_cross_entropy: bool | None = None
    use_kernels: bool | None = None
    use_scattermoe: bool | None = None
    use_sonicmoe: bool | None = None


class NativeKernelsPlugin(BasePlugin):
    def get_input_args(self):
        return NativeKernelArgs


class ExpertParallelArgs(BaseModel):
    expert_parallel_size: int | None = None
    expert_parallel_capacity_factor: float | None = None
    expert_parallel_local_kernel: str | None = None


class ExpertParallelPlugin(BasePlugin):
    def get_input_args(self):
        return ExpertParallelArgs


class MoraBlock(BaseModel):
    use_mora: bool = True
    mora_type: str | int = "rope"      # `sharing` (1) or `rope` (6)


class MoraArgs(BaseModel):
    mora: MoraBlock | None = None


class MoraPlugin(BasePlugin):
    """Enables the nested ``mora:`` block for ``adapter: mora`` (reference:
    src/axolotl/integrations/mora/plugin.py:44-97). The operators themselves are part of the model
    (``models/mora.py``); no PEFT fork is involved."""

    def get_input_args(self):
        return MoraArgs

    def pre_model_load(self, cfg):
        if cfg.get("adapter") == "mora":
            from ..models.mora import mora_type_id

            mora_type_id((cfg.get("mora") or {}).get("mora_type", "rope"))   # raises on an unknown variant


class DenseMixerArgs(BaseModel):
    dense_mixer: bool | None = True


class DenseMixerPlugin(BasePlugin):
    """DenseMixer: a more precise router gradient for sparse MoE layers at the price of evaluating
    every expert on every token in the backward pass (reference:
    src/axolotl/integrations/densemixer/plugin.py:11-42, which patches OLMoE / Qwen2-MoE / Qwen3-MoE
    through the external ``densemixer`` package). Here it is a switch on ``models.moe.SparseMoE``."""

    SUPPORTED = ("olmoe", "qwen2_moe", "qwen3_moe")

    def get_input_args(self):
        return DenseMixerArgs

    def post_model_build(self, cfg, model):
        if cfg.get("dense_mixer") is False:
            return
        if model.config.model_type not in self.SUPPORTED:
            raise ValueError(f"dense_mixer supports {self.SUPPORTED}, not '{model.config.model_type}'")
        if (cfg.get("expert_parallel_size") or 1) > 1:
            raise ValueError("dense_mixer cannot be combined with expert parallelism")
        n = 0
        for m in model.modules():
            if hasattr(m, "dense_mixer"):
                m.dense_mixer = True
                n += 1
        from ..utils.logging import get_logger

        get_logger(__name__).info("DenseMixer router gradient enabled on %d MoE layers", n)
