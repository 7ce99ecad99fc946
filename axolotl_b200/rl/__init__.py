"""Preference optimisation and RL objectives on packed token streams.

Every objective here is a ``compute_loss(model, batch, n_items)`` callable plugged into the same
``Trainer`` that runs SFT: chosen/rejected (or prompt/completion, or sampled) sequences are packed
as documents of one varlen row, one forward pass of the flash-varlen model scores all of them,
per-token log-probabilities come from the chunked lm-head + cross-entropy kernels, and the
reference policy of an adapter run is the same model with adapters switched off.
"""
from .losses import cpo_loss, dpo_loss, grpo_loss, kto_loss, orpo_loss  # noqa: F401
from .logps import sequence_logps  # noqa: F401
