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
    """Accepts the kernel-selection flags of the reference's Liger / cut-cross-entropy / kernels plugins and reports
    which native kernel serves each request (they are always on; a flag set to false cannot switch one off)."""

    NATIVE = {"liger_rope": "rope_qk_kernel", "liger_rms_norm": "rmsnorm_fwd/bwd_kernel", "liger_layer_norm": "rmsnorm_fwd/bwd_kernel",
              "liger_glu_activation": "GLU epilogues of gemm_bf16_pair_kernel / glu_fwd/bwd_kernel",
              "liger_cross_entropy": "ce_fwd_bwd_kernel", "liger_fused_linear_cross_entropy": "chunked lm-head GEMM + ce_fwd_bwd_kernel",
              "cut_cross_entropy": "chunked lm-head GEMM + ce_fwd_bwd_kernel", "use_kernels": "all native kernels",
              "use_scattermoe": "grouped_gemm_kernel / grouped_w4a16_kernel", "use_sonicmoe": "grouped_gemm_kernel / grouped_w4a16_kernel"}

    def get_input_args(self):
        return NativeKernelArgs

    def pre_model_load(self, cfg):
        from ..utils.logging import get_logger

        log = get_logger(__name__)
        for key, kernel in self.NATIVE.items():
            if cfg.get(key) is True:
                log.info("%s: served by %s", key, kernel)
            elif cfg.get(key) is False:
                log.warning("%s: false has no effect, %s is always used", key, kernel)


class ExpertParallelArgs(BaseModel):
    expert_parallel_size: int | None = None
    expert_parallel_capacity_factor: float | None = None
    expert_parallel_local_kernel: str | None = None


class ExpertParallelPlugin(BasePlugin):
    """``expert_parallel_size`` is read by the parallel runtime; ``expert_parallel_capacity_factor`` bounds the rows a
    rank may receive per layer call in the device-built routing plan (parallel/ep.py); ``expert_parallel_local_kernel``
    names a reference kernel choice that the grouped tcgen05 kernels replace."""

    def get_input_args(self):
        return ExpertParallelArgs

    def pre_model_load(self, cfg):
        import os

        cf = cfg.get("expert_parallel_capacity_factor")
        if cf is not None:
            if float(cf) <= 0:
                raise ValueError("expert_parallel_capacity_factor must be positive")
            os.environ["AXB_EP_CAPACITY"] = str(float(cf))
        if cfg.get("expert_parallel_local_kernel"):
            from ..utils.logging import get_logger

            get_logger(__name__).info("expert_parallel_local_kernel=%s: the local expert pass always runs the grouped tcgen05 "
                                      "GEMM kernels", cfg["expert_parallel_local_kernel"])


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
