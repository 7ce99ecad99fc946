"""Format-preserving LoRA merge into quantised checkpoints (block-fp8, MXFP8, MXFP4, NVFP4 with reused or fresh block
scales) and the NF4 round-trip image of a base weight."""
import json
import os

import pytest
import torch

from axolotl_b200.io import quant_formats as qf
from axolotl_b200.io import safetensors_io as st
from axolotl_b200.io.merge import merge_lora_sharded
from axolotl_b200.ops.nvfp4 import quantize_nvfp4


def _scales_like(fmt, w):
    *lead, N, K = w.shape
    if fmt == "block_fp8":
        return {"_scale_inv": torch.ones(*lead, N // 32, K // 32)}
    if fmt in ("mxfp8", "mxfp4"):
        return {"_scale": torch.zeros(*lead, N, K // 32, dtype=torch.uint8)}
    q, sc, pts = quantize_nvfp4(w)
    return {"_scale": sc, "_scale_2": pts}


@pytest.mark.parametrize("fmt,tol", [("block_fp8", 0.04), ("mxfp8", 0.08), ("mxfp4", 0.5), ("nvfp4", 0.2)])
def test_requantise_then_dequantise_stays_on_the_formats_grid(fmt, tol):
    torch.manual_seed(0)
    w = torch.randn(64, 128) * 0.1
    q = qf.requantize(fmt, w, _scales_like(fmt, w), nvfp4_scale_mode="fresh")
    shard = {"k" + suf: t for suf, t in q.items()}
    got_fmt, scales = qf.detect_format("k", shard["k"], shard)
    assert got_fmt == fmt
    d = qf.dequantize(fmt, shard["k"], scales)
    assert d.shape == w.shape and float((d - w).abs().max() / w.abs().max()) < tol
    # quantising the expansion again changes nothing: the expansion is on the grid
    q2 = qf.requantize(fmt, d, scales, nvfp4_scale_mode="reuse")
    assert torch.equal(q2[""].view(torch.uint8), shard["k"].view(torch.uint8))
    assert qf.detect_format("k", w, {}) == (None, {})


def test_nvfp4_reuse_mode_changes_only_codes_the_delta_moves():
    torch.manual_seed(1)
    w = torch.randn(3, 32, 64) * 0.1
    qd, sc, pts = quantize_nvfp4(w)
    base = qf.dequantize("nvfp4", qd, {"_scale": sc, "_scale_2": pts})
    delta = torch.zeros_like(base)
    delta[1, 5, :16] = base[1, 5, :16].abs().max() * 0.6          # one block of one expert
    out = qf.requantize("nvfp4", base + delta, {"_scale": sc, "_scale_2": pts}, nvfp4_scale_mode="reuse")
    assert torch.equal(out["_scale"].view(torch.uint8), sc.view(torch.uint8)) and torch.equal(out["_scale_2"], pts)
    changed = (out[""] != qd).nonzero()
    assert len(changed) > 0 and set(changed[:, 0].tolist()) == {1} and set(changed[:, 1].tolist()) == {5}
    assert int(changed[:, 2].max()) < 8                             # 16 values = 8 packed bytes
    fresh = qf.requantize("nvfp4", base + delta, {"_scale": sc, "_scale_2": pts}, nvfp4_scale_mode="fresh")
    assert not torch.equal(fresh["_scale"].view(torch.uint8), sc.view(torch.uint8))


@pytest.mark.parametrize("fmt", ["block_fp8", "mxfp8", "mxfp4", "nvfp4"])
def test_merge_into_a_quantised_checkpoint_keeps_its_format(tmp_path, fmt):
    torch.manual_seed(2)
    N, K, r = 64, 128, 4
    w = torch.randn(N, K) * 0.1
    q = qf.requantize(fmt, w, _scales_like(fmt, w), nvfp4_scale_mode="fresh")
    name = "model.layers.0.self_attn.q_proj.weight"
    base = {name + suf: t for suf, t in q.items()}
    base["model.norm.weight"] = torch.ones(K)
    os.makedirs(tmp_path / "base")
    st.save_file(base, str(tmp_path / "base" / "model.safetensors"), {"format": "pt"})
    with open(tmp_path / "base" / "config.json", "w") as fh:
        json.dump({"model_type": "llama"}, fh)
    A, B = torch.randn(r, K) * 0.3, torch.randn(N, r) * 0.3
    os.makedirs(tmp_path / "ad")
    st.save_file({"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": A,
                  "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": B},
                 str(tmp_path / "ad" / "adapter_model.safetensors"), {"format": "pt"})
    with open(tmp_path / "ad" / "adapter_config.json", "w") as fh:
        json.dump({"r": r, "lora_alpha": 8, "target_modules": ["q_proj"], "peft_type": "LORA"}, fh)
    res = merge_lora_sharded(str(tmp_path / "base"), str(tmp_path / "ad"), str(tmp_path / "out"), nvfp4_scale_mode="fresh")
    assert res["merged"] == 1 and res["unmatched"] == []
    out = st.load_file(str(tmp_path / "out" / "model.safetensors"))
    assert set(out) == set(base)
    for k in base:
        assert out[k].dtype == base[k].dtype and out[k].shape == base[k].shape, k
    got_fmt, scales = qf.detect_format(name, out[name], out)
    assert got_fmt == fmt
    merged = qf.dequantize(fmt, out[name], scales)
    want = qf.dequantize(fmt, base[name], {s: base[name + s] for s in scales}) + 2.0 * (B @ A)
    tol = {"block_fp8": 0.05, "mxfp8": 0.08, "mxfp4": 0.5, "nvfp4": 0.25}[fmt]
    assert float((merged - want).abs().max() / want.abs().max()) < tol
    assert float((merged - want).norm() / want.norm()) < tol * 0.6


def test_nf4_roundtrip_image_is_what_qlora_trained_against():
    from axolotl_b200.ops.nf4 import dequantize_nf4, quantize_nf4
    torch.manual_seed(3)
    w = (torch.randn(64, 96) * 0.05).bfloat16()
    img = qf.simulate_nf4_roundtrip(w)
    q, state = quantize_nf4(w)
    assert img.dtype == w.dtype and torch.equal(img, dequantize_nf4(q, state, dtype=torch.float32).reshape(w.shape).to(w.dtype))
    assert not torch.equal(img, w) and float((img.float() - w.float()).abs().max()) < 0.04
    odd = torch.randn(7, 9)
    assert qf.simulate_nf4_roundtrip(odd) is odd


def test_gpt_oss_mxfp4_checkpoint_loads_as_bf16(tmp_path):
    """The released gpt-oss layout (packed blocks + e8m0 scales per expert weight) expands on load to the same model
    as the bf16 checkpoint of the expanded values."""
    from axolotl_b200.io import hf as hf_io
    from axolotl_b200.models.config import ModelConfig
    from axolotl_b200.models.transformer import CausalLM
    d = dict(model_type="gpt_oss", vocab_size=200, hidden_size=64, intermediate_size=64, num_hidden_layers=1,
             num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_local_experts=2, num_experts_per_tok=1,
             sliding_window=8, layer_types=["full_attention"], tie_word_embeddings=False, max_position_embeddings=128)
    cfg = ModelConfig.from_hf_dict(d)
    model = CausalLM(cfg, dtype=torch.float32).init_weights(5)
    sd = hf_io.hf_state_dict(model)
    packed = {}
    for k in list(sd):
        if k.endswith("experts.gate_up_proj") or k.endswith("experts.down_proj"):
            w = sd.pop(k).transpose(1, 2).contiguous()                       # [E, out, in]
            q = qf.requantize("mxfp4", w, {"_scale": torch.zeros(1, dtype=torch.uint8)})
            E, rows = w.shape[:2]
            packed[k + "_blocks"] = q[""].reshape(E, rows, -1, 16)
            packed[k + "_scales"] = q["_scale"].reshape(E, rows, -1)
            # the bf16 twin holds exactly the values the packed form expands to
            sd[k] = qf.dequantize("mxfp4", q[""], {"_scale": q["_scale"]}).transpose(1, 2).contiguous()
    ref = CausalLM(cfg, dtype=torch.float32)
    hf_io.load_state_into(ref, sd.items())
    got = CausalLM(cfg, dtype=torch.float32)
    hf_io.load_state_into(got, {**{k: v for k, v in sd.items() if "experts.gate_up_proj" != k[-20:] and not k.endswith("experts.down_proj")
                                    and not k.endswith("experts.gate_up_proj")}, **packed}.items())
    ids = torch.randint(3, 200, (1, 24))
    with torch.no_grad():
        assert torch.allclose(got(ids, return_logits=True).logits, ref(ids, return_logits=True).logits, atol=1e-5)
