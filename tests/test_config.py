import os

import pytest
import yaml

from axolotl_b200.config.dict import DictDefault
from axolotl_b200.config.load import apply_overrides, coerce_value, load_cfg, validate_config
from axolotl_b200.config.normalize import normalize
from axolotl_b200.config.schema import check_keys

BASE = {"model_preset": "tiny-llama", "datasets": [{"type": "_synthetic", "length": 10}], "sequence_len": 256,
        "learning_rate": "2e-4", "micro_batch_size": 2}


def test_dictdefault_missing_is_none_and_nested():
    d = DictDefault({"a": {"b": 1}, "l": [{"c": 2}]})
    assert d.a.b == 1 and d.zzz is None and d.l[0].c == 2 and d.a.q is None
    d.x = {"y": 3}
    assert d.x.y == 3 and d.to_dict()["x"] == {"y": 3}


def test_minimal_config_validates_and_normalises():
    cfg = load_cfg(dict(BASE, gradient_accumulation_steps=4))
    assert cfg.learning_rate == pytest.approx(2e-4)
    assert cfg.batch_size == 8 and cfg.gradient_accumulation_steps == 4 and cfg.eval_batch_size == 2
    assert cfg.save_total_limit == 4 and cfg.seed == 42 and cfg.max_grad_norm == 1.0
    assert cfg.is_llama_derived_model is True and cfg.model_config_type == "llama"


def test_batch_size_derives_grad_accum():
    cfg = load_cfg(dict(BASE, batch_size=8))
    assert cfg.gradient_accumulation_steps == 4
    with pytest.raises(ValueError):
        load_cfg(dict(BASE, batch_size=8, gradient_accumulation_steps=2))


def test_world_size_scaling_excludes_tp_and_cp(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "8")
    assert load_cfg(dict(BASE, gradient_accumulation_steps=1)).batch_size == 16
    assert load_cfg(dict(BASE, gradient_accumulation_steps=1, tensor_parallel_size=2)).batch_size == 8
    assert load_cfg(dict(BASE, gradient_accumulation_steps=1, context_parallel_size=4, micro_batch_size=1)).batch_size == 2
    assert load_cfg(dict(BASE, gradient_accumulation_steps=1, expert_parallel_size=8)).batch_size == 16


@pytest.mark.parametrize("patch,msg", [
    ({"foo_bar": 1}, "unknown config key"),
    ({"lora_rr": 8}, "did you mean 'lora_r'"),
    ({"deepspeed": "zero3.json"}, "unsupported"),
    ({"bf16": True, "fp16": True}, "mutually exclusive"),
    ({"adapter": "lora"}, "lora_r"),
    ({"adapter": "lora", "lora_r": 8, "lora_alpha": 16}, "no LoRA targets"),
    ({"adapter": "qlora", "lora_r": 8, "lora_alpha": 16, "lora_target_linear": True}, "load_in_4bit"),
    ({"sample_packing": True, "group_by_length": True}, "group_by_length"),
    ({"warmup_steps": 3, "warmup_ratio": 0.1}, "only one of"),
    ({"save_steps": 5, "saves_per_epoch": 2}, "only one of"),
    ({"optimizer": "adamw_bnb_8bit"}, "bitsandbytes"),
    ({"rl": "grpo"}, "reward_funcs"),
    ({"rl": "ebft"}, "ebft"),
    ({"tensor_parallel_size": 2, "expert_parallel_size": 2}, "expert parallelism"),
    ({"context_parallel_size": 2, "sample_packing": True, "micro_batch_size": 2}, "micro_batch_size: 1"),
    ({"val_set_size": 0.1, "test_datasets": [{"type": "_synthetic"}]}, "mutually exclusive"),
    ({"datasets": None}, "no `datasets`"),
    ({"max_packed_sequence_len": 2048}, "removed"),
    ({"early_stopping_patience": 3}, "periodic evaluation"),
])
def test_validation_errors(patch, msg):
    raw = dict(BASE)
    raw.update(patch)
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(Exception) as ei:
        load_cfg(raw)
    assert msg in str(ei.value)


def test_deprecated_and_legacy_spellings_are_mapped():
    cfg = load_cfg(dict(BASE, flash_attention=True, sequence_parallel_degree=1, evaluation_strategy="no",
                        sample_packing=True))
    assert cfg.attn_implementation == "flash_attention_2" and cfg.context_parallel_size == 1
    assert cfg.eval_strategy == "no" and cfg.pad_to_sequence_len is True
    with pytest.raises(ValueError):
        load_cfg(dict(BASE, flash_attention=True, attn_implementation="sdpa"))


def test_inert_reference_keys_are_accepted():
    raw = dict(BASE, liger_rope=True, torch_compile_backend="inductor", gc_collect_steps=2)
    assert set(check_keys(raw)) == {"liger_rope", "torch_compile_backend", "gc_collect_steps"}
    load_cfg(raw)


def test_saves_per_epoch_and_eval_cadence():
    cfg = load_cfg(dict(BASE, saves_per_epoch=2, num_epochs=2, val_set_size=0.1, evals_per_epoch=4))
    assert cfg.save_steps == pytest.approx(0.25) and cfg.save_strategy == "steps"
    assert cfg.eval_steps == pytest.approx(0.125) and cfg.eval_strategy == "steps"
    cfg2 = load_cfg(dict(BASE))
    assert cfg2.eval_strategy == "no"
    # one save per epoch of a one-epoch run is "save at the end", not "after every step"
    cfg3 = load_cfg(dict(BASE, saves_per_epoch=1, num_epochs=1, val_set_size=0.1, evals_per_epoch=1))
    assert not cfg3.save_steps and not cfg3.eval_steps
    cfg4 = load_cfg(dict(BASE, saves_per_epoch=2))          # num_epochs unset counts as 1
    assert cfg4.save_steps == pytest.approx(0.5)


def test_rank_and_alpha_patterns_match_like_peft():
    from axolotl_b200.io.merge import _adapter_rank, _adapter_scale

    cfg = {"r": 8, "lora_alpha": 16, "rank_pattern": {"q_proj": 4, r"layers\.1\.mlp\.down_proj": 2},
           "alpha_pattern": {"q_proj": 32}}
    assert _adapter_rank(cfg, "model.layers.0.self_attn.q_proj") == 4
    assert _adapter_rank(cfg, "model.layers.0.self_attn.qq_proj") == 8        # no module boundary before the key
    assert _adapter_rank(cfg, "model.layers.0.self_attn.q_proj_extra") == 8   # suffix rule, not a substring search
    assert _adapter_rank(cfg, "model.layers.1.mlp.down_proj") == 2
    assert _adapter_rank(cfg, "model.layers.11.mlp.down_proj") == 8
    assert _adapter_scale(cfg, "model.layers.0.self_attn.q_proj") == 32 / 4


def test_cli_style_overrides_and_yaml_file(tmp_path):
    assert coerce_value("true") is True and coerce_value("3") == 3 and coerce_value("1e-3") == 1e-3
    assert coerce_value("none") is None and coerce_value("[1, 2]") == [1, 2] and coerce_value("abc") == "abc"
    raw = apply_overrides({"fsdp_config": {"a": 1}}, {"fsdp_config__reshard_after_forward": "true", "lora_r": "16"})
    assert raw["fsdp_config"] == {"a": 1, "reshard_after_forward": True} and raw["lora_r"] == 16
    p = tmp_path / "c.yaml"
    p.write_text(yaml.safe_dump(BASE))
    cfg = load_cfg(str(p), micro_batch_size="4", output_dir=str(tmp_path / "o"))
    assert cfg.micro_batch_size == 4 and cfg.axolotl_config_path == str(p)
    assert load_cfg(str(tmp_path)).micro_batch_size == 2   # directory chooser


def test_fsdp_config_prefix_stripping():
    cfg = load_cfg(dict(BASE, fsdp_config={"fsdp_version": 2, "fsdp_reshard_after_forward": True,
                                           "fsdp_state_dict_type": "FULL_STATE_DICT"}))
    assert cfg.fsdp_config.reshard_after_forward is True and cfg.fsdp_version == 2


def test_plugins_contribute_keys():
    from axolotl_b200.plugins.base import PluginManager

    PluginManager.reset()
    cfg = load_cfg(dict(BASE, plugins=["axolotl.integrations.liger.LigerPlugin", "grokfast"], liger_rope=True,
                        grokfast_alpha=0.9))
    assert cfg.grokfast_alpha == 0.9
    PluginManager.reset()


def test_architecture_registry_checks():
    from axolotl_b200.models import registry as R
    from axolotl_b200.models.config import SUPPORTED_MODEL_TYPES, ModelConfig, preset

    # every model type the config reader accepts has a descriptor (the training entry point validates against it)
    for mt in SUPPORTED_MODEL_TYPES:
        assert R.get_model_support(mt) is not None, mt
    assert isinstance(R.support_for("llama").capabilities[R.EP], R.Unsupported)
    with pytest.raises(ValueError, match="no model graph"):
        R.support_for("mllama")
    with pytest.raises(ValueError, match="expert parallelism needs"):
        R.validate_cfg({"expert_parallel_size": 2}, preset("tiny-llama"))
    with pytest.raises(ValueError, match="cannot be split"):
        R.validate_cfg({"expert_parallel_size": 3}, preset("tiny-qwen3-moe"))
    with pytest.raises(ValueError, match="tensor parallelism is not supported for model_type=qwen3_moe"):
        R.validate_cfg({"tensor_parallel_size": 2}, preset("tiny-qwen3-moe"))
    assert R.validate_cfg({"sample_packing": True}, preset("tiny-llama")) == []
    # wide heads pass the head-width check (their own kernels), and say why context parallelism is closed
    gemma = preset("tiny-gemma2")
    assert R.validate_cfg({"sample_packing": True, "adapter": "lora"}, gemma)
    with pytest.raises(ValueError, match="head widths 64 and 128"):
        R.validate_cfg({"context_parallel_size": 2}, gemma)
    qn = ModelConfig.from_hf_dict(dict(model_type="qwen3_next", vocab_size=64, hidden_size=32, intermediate_size=32,
                                       num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1, head_dim=16,
                                       linear_num_value_heads=2, linear_num_key_heads=1, linear_key_head_dim=8,
                                       linear_value_head_dim=8, num_experts=0))
    with pytest.raises(ValueError, match="Gated DeltaNet"):
        R.validate_cfg({"context_parallel_size": 2}, qn)


def test_model_support_registration_and_experimental_warning(caplog):
    import logging

    from axolotl_b200.models import registry as R

    @R.register_model_support
    class Toy(R.ModelSupport):
        model_types = ("toy_arch",)
        capabilities = {R.CP: R.Experimental("Only tried at two ranks."), R.TP: R.Unsupported("No sharding rule.")}

        def validate_cfg(self, cfg, model_cfg):
            if cfg.get("sequence_len", 0) > 8:
                raise ValueError("toy_arch: sequence_len above 8")

    try:
        sup = R.get_model_support("toy_arch")
        with caplog.at_level(logging.WARNING):
            R.check_capability(sup, R.CP, "toy_arch", feature="context parallelism")
            R.check_capability(sup, R.CP, "toy_arch", feature="context parallelism")      # said once
        assert sum("experimental for model_type=toy_arch" in r.getMessage() for r in caplog.records) == 1
        with pytest.raises(ValueError, match="No sharding rule"):
            R.check_capability(sup, R.TP, "toy_arch")
        R.check_capability(sup, "something_unknown", "toy_arch")                          # unknown: generic path

        class MC:
            model_type, num_experts, head_dim = "toy_arch", 0, 32
        with pytest.raises(ValueError, match="above 8"):
            R.validate_cfg({"sequence_len": 16}, MC())
        with pytest.raises(ValueError):
            type("Bad", (R.ModelSupport,), {}) and R.register_model_support(type("Bad", (R.ModelSupport,), {}))
    finally:
        R._REGISTRY.pop("toy_arch", None)


def test_compat_plugins_act_on_their_keys(monkeypatch, caplog):
    import logging

    from axolotl_b200.plugins.compat import ExpertParallelPlugin, NativeKernelsPlugin
    monkeypatch.delenv("AXB_EP_CAPACITY", raising=False)
    ExpertParallelPlugin().pre_model_load({"expert_parallel_size": 2, "expert_parallel_capacity_factor": 1.25})
    import os
    assert os.environ["AXB_EP_CAPACITY"] == "1.25"
    with pytest.raises(ValueError):
        ExpertParallelPlugin().pre_model_load({"expert_parallel_capacity_factor": 0})
    with caplog.at_level(logging.INFO):
        NativeKernelsPlugin().pre_model_load({"liger_rms_norm": True, "cut_cross_entropy": False})
    text = " ".join(r.getMessage() for r in caplog.records)
    assert "rmsnorm" in text and "always used" in text


def test_blocked_attention_for_head_widths_without_a_kernel_matches_the_reference():
    """The blocked path that serves head widths outside the kernels' set (documents, windows, soft cap, bidirectional)."""
    import torch

    from axolotl_b200.ops import functional as Fn

    torch.manual_seed(0)
    Hq, Hk, D, Dv = 4, 2, 48, 32
    lens = [300, 77, 513]
    T = sum(lens)
    cu = [0, 300, 377, 890]
    qkv = torch.randn(T, (Hq + Hk) * D + Hk * Dv, requires_grad=True)
    for causal, window, softcap in [(True, 0, 0.0), (True, 100, 0.0), (False, 0, 0.0), (True, 0, 5.0)]:
        meta = Fn.AttnMeta(cu, "cpu", causal=causal, window=window or None)
        q = qkv[:, : Hq * D].reshape(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D)
        v = qkv[:, (Hq + Hk) * D:].reshape(T, Hk, Dv)
        ref = Fn._attn_ref(q, k, v, cu, 0.2, causal, window, softcap).reshape(T, Hq * Dv)
        got = Fn._blocked_attention(qkv, meta, Hq, Hk, D, Dv, 0.2, softcap)
        g1, = torch.autograd.grad((got ** 2).sum(), qkv, retain_graph=True)
        g2, = torch.autograd.grad((ref ** 2).sum(), qkv)
        assert (got - ref).abs().max() < 1e-5
        assert (g1 - g2).abs().max() < 1e-3


def test_every_example_config_passes_validation():
    """The YAML files under examples/ are what a new user copies: each one must load through the schema and the
    cross-field rules (model weights are not touched)."""
    import glob
    import os

    import yaml

    from axolotl_b200.config.load import load_cfg

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    files = sorted(glob.glob(os.path.join(root, "**", "*.yaml"), recursive=True))
    assert len(files) >= 25
    for f in files:
        with open(f) as fh:
            raw = yaml.safe_load(fh)
        cfg = load_cfg(raw)
        assert cfg["sequence_len"] > 0 and cfg["output_dir"], f


def test_xielu_and_gated_pool_reference_paths():
    import torch

    from axolotl_b200.ops import functional as Fn

    x = torch.tensor([-3.0, -1e-7, 0.0, 0.5, 2.0])
    y = Fn.xielu(x, torch.tensor([0.8]), torch.tensor([0.8]), 0.5, -1e-6)
    want = torch.where(x > 0, 0.8 * x * x + 0.5 * x, 0.8 * (torch.expm1(torch.clamp(x, max=-1e-6)) - x) + 0.5 * x)
    assert torch.allclose(y, want)
    kv, gate = torch.randn(2, 5, 4, 7), torch.randn(2, 5, 4, 7)
    assert torch.allclose(Fn.gated_softmax_pool(kv, gate), (kv * gate.softmax(-2)).sum(-2), atol=1e-6)


def test_hyperconnection_mixer_reference_properties():
    """The plain form of the DeepSeek-V4 hyper-connection mixer: pre / post ranges, a (nearly) doubly stochastic stream
    mixer after the Sinkhorn chain, and the collapse of the streams."""
    import torch

    from axolotl_b200.ops import functional as Fn

    torch.manual_seed(0)
    M, hc, H = 9, 4, 32
    mixes = torch.randn(M, hc * (2 + hc)) * 2
    scale, base = torch.tensor([0.7, 1.3, 0.9]), torch.randn(hc * (2 + hc)) * 0.3
    pre, post, comb = Fn.sinkhorn_mix(mixes, scale, base)
    assert pre.shape == (M, 4) and post.shape == (M, 4) and comb.shape == (M, 4, 4)
    assert (pre > 0).all() and (pre < 1.001).all() and (post >= 0).all() and (post <= 2).all()
    assert torch.allclose(comb.sum(1), torch.ones(M, 4), atol=1e-4) and torch.allclose(comb.sum(2), torch.ones(M, 4), atol=2e-2)
    streams = torch.randn(2, 5, hc, H)
    fn = torch.randn(hc * (2 + hc), hc * H) * 0.05
    post2, comb2, collapsed = Fn.hyperconnection_forward(streams, fn, base, scale)
    assert post2.shape == (2, 5, 4) and comb2.shape == (2, 5, 4, 4) and collapsed.shape == (2, 5, H)
    flat = streams.reshape(-1, hc * H)
    mixes2 = (flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + 1e-6)) @ fn.t()
    pre3, _, _ = Fn.sinkhorn_mix_ref(mixes2, scale, base)
    want = (pre3[:, :, None] * streams.reshape(-1, hc, H)).sum(1)
    assert torch.allclose(collapsed.reshape(-1, H), want, atol=1e-5)
