"""Our model definitions must be numerically interchangeable with the Hugging Face ones: same
weights (round-tripped through safetensors files) -> same logits and loss on CPU fp32."""
import numpy as np
import pytest
import torch

from axolotl_b200.io import hf as hf_io
from axolotl_b200.models.config import ModelConfig, preset
from axolotl_b200.models.transformer import CausalLM

transformers = pytest.importorskip("transformers")


def _packed_inputs(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.cat([torch.randint(3, vocab, (l,), generator=g) for l in lens])[None]
    pos = torch.cat([torch.arange(l) for l in lens])[None].to(torch.int32)
    return ids, pos


def _hf_docwise_logits(hf_model, ids, lens):
    outs, s = [], 0
    for l in lens:
        with torch.no_grad():
            outs.append(hf_model(input_ids=ids[:, s:s + l]).logits)
        s += l
    return torch.cat(outs, 1)


def test_llama_logits_match_hf_and_packing_isolates_documents(tmp_path):
    cfg = preset("tiny-llama", vocab_size=512, num_hidden_layers=2)
    ours = CausalLM(cfg, dtype=torch.float32).init_weights(1)
    hf_io.save_pretrained(ours, str(tmp_path / "m"))
    hf_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), torch_dtype=torch.float32)
    hf_model.eval()
    lens = [37, 64, 19]
    ids, pos = _packed_inputs(512, lens)
    ours.eval()
    with torch.no_grad():
        got = ours(ids, pos, return_logits=True).logits
    ref = _hf_docwise_logits(hf_model, ids, lens)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (got - ref).abs().max()
    # reload through our loader as well
    again = hf_io.load_pretrained(str(tmp_path / "m"), dtype=torch.float32)
    with torch.no_grad():
        got2 = again(ids, pos, return_logits=True).logits
    assert torch.equal(got, got2)


def test_llama_loss_matches_hf_single_document(tmp_path):
    cfg = preset("tiny-llama", vocab_size=300, num_hidden_layers=1)
    ours = CausalLM(cfg, dtype=torch.float32).init_weights(2)
    hf_io.save_pretrained(ours, str(tmp_path / "m"))
    hf_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), torch_dtype=torch.float32)
    ids, pos = _packed_inputs(300, [50])
    labels = ids.clone()
    labels[:, :12] = -100
    loss = ours(ids, pos, labels).loss
    ref = hf_model(input_ids=ids, labels=labels).loss
    assert abs(loss.item() - ref.item()) < 1e-4


def test_qwen3_qk_norm_matches_hf(tmp_path):
    cfg = ModelConfig(model_type="qwen3", vocab_size=400, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6)
    ours = CausalLM(cfg, dtype=torch.float32).init_weights(3)
    with torch.no_grad():
        for l in ours.layers:
            l.self_attn.q_norm.weight.uniform_(0.5, 1.5)
            l.self_attn.k_norm.weight.uniform_(0.5, 1.5)
    hf_io.save_pretrained(ours, str(tmp_path / "m"))
    hf_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), torch_dtype=torch.float32)
    ids, pos = _packed_inputs(400, [33])
    with torch.no_grad():
        got = ours(ids, pos, return_logits=True).logits
        ref = hf_model(input_ids=ids).logits
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (got - ref).abs().max()


def test_qwen3_moe_matches_hf(tmp_path):
    cfg = preset("tiny-qwen3-moe", vocab_size=300)
    ours = CausalLM(cfg, dtype=torch.float32).init_weights(4)
    hf_io.save_pretrained(ours, str(tmp_path / "m"), per_expert=False)
    try:
        hf_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), torch_dtype=torch.float32)
    except Exception as exc:  # older transformers want per-expert tensors
        hf_io.save_pretrained(ours, str(tmp_path / "m2"), per_expert=True)
        hf_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m2"), torch_dtype=torch.float32)
    ids, pos = _packed_inputs(300, [41])
    ours.eval()
    with torch.no_grad():
        got = ours(ids, pos, return_logits=True).logits
        ref = hf_model(input_ids=ids).logits
    assert torch.allclose(got, ref, atol=3e-4, rtol=1e-3), (got - ref).abs().max()
