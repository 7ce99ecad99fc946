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
