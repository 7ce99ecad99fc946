"""Multimodal fine-tuning through the training entry point: a LLaVA checkpoint (CLIP tower, projector, Llama language model),
conversations with images rendered by the family's processor, padding-free batches, adapters on the language model."""
import json
import os

import pytest
import torch

from axolotl_b200.data import multimodal as mm
from axolotl_b200.io import hf as hf_io
from axolotl_b200.models.config import ModelConfig
from axolotl_b200.models.transformer import CausalLM

IMG = 299


class Tok:
    """Whitespace tokenizer over a tiny closed vocabulary."""
    pad_token_id, eos_token_id, unk_token_id, chat_template = 0, 2, 1, None
    words = ["<pad>", "<unk>", "</s>", "USER:", "ASSISTANT:", "what", "is", "this", "a", "red", "square", "blue", "circle", "describe"]

    def __init__(self):
        self.vocab = {w: i for i, w in enumerate(self.words)}
        self.vocab["<image>"] = IMG

    def __len__(self):
        return 300

    def encode(self, text, add_special_tokens=False):
        return [self.vocab.get(w, 1) for w in text.split()]

    def __call__(self, text, add_special_tokens=False, **kw):
        return {"input_ids": self.encode(text)}

    def convert_tokens_to_ids(self, name):
        return self.vocab.get(name, 1)

    def decode(self, ids, **kw):
        inv = {i: w for w, i in self.vocab.items()}
        return " ".join(inv.get(int(i), "?") for i in ids)


class Processor:
    """Stands in for LlavaProcessor: four placeholder tokens per image, pixel tensors in row order."""
    image_token = "<image>"

    def __init__(self):
        self.tokenizer = Tok()

    def apply_chat_template(self, conversations, add_generation_prompt=False, tokenize=True, return_tensors="pt",
                            return_dict=True, chat_template=None, processor_kwargs=None):
        rows, pixels = [], []
        for msgs in conversations:
            ids = []
            for m in msgs:
                ids += self.tokenizer.encode("USER:" if m["role"] == "user" else "ASSISTANT:")
                for part in m["content"]:
                    if part["type"] == "image":
                        ids += [IMG] * 4
                        g = torch.Generator().manual_seed(len(str(part.get("image"))))
                        pixels.append(torch.randn(3, 28, 28, generator=g))
                    else:
                        ids += self.tokenizer.encode(part["text"])
                if m["role"] == "assistant":
                    ids.append(2)
            rows.append(ids)
        L = max(len(r) for r in rows)
        ids = torch.tensor([r + [0] * (L - len(r)) for r in rows])
        out = {"input_ids": ids, "attention_mask": (ids != 0).long()}
        if pixels:
            out["pixel_values"] = torch.stack(pixels)
        return out


def _checkpoint(path):
    vc = dict(model_type="clip_vision_model", hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              image_size=28, patch_size=14, num_channels=3, hidden_act="quick_gelu", projection_dim=16)
    tc = dict(model_type="llama", vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=256, tie_word_embeddings=False)
    cfg = ModelConfig.from_hf_dict(dict(model_type="llava", text_config=tc, vision_config=vc, image_token_id=IMG))
    model = CausalLM(cfg, dtype=torch.float32).init_weights(3)
    hf_io.save_pretrained(model, path)
    return model


def test_unpad_batch_packs_rows_and_keeps_media():
    ids = torch.tensor([[5, 6, 7, 0, 0], [8, 9, 10, 11, 12]])
    b = mm.unpad_batch({"input_ids": ids, "labels": ids.clone(), "attention_mask": (ids != 0).long(), "pixel_values": torch.zeros(1, 3, 4, 4)})
    assert b["input_ids"].tolist() == [[5, 6, 7, 8, 9, 10, 11, 12]] and b["position_ids"].tolist() == [[0, 1, 2, 0, 1, 2, 3, 4]]
    assert b["cu_seqlens"].tolist() == [0, 3, 8] and b["aux_tensors"]["pixel_values"].shape == (1, 3, 4, 4)


def test_llava_lora_training_through_the_entry_point(tmp_path, monkeypatch):
    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.plugins.base import PluginManager
    from axolotl_b200.train.run import train

    PluginManager.reset()
    base = str(tmp_path / "base")
    _checkpoint(base)
    rows = []
    for i in range(12):
        shape = ("red square", "blue circle")[i % 2]
        rows.append({"messages": [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "what is this"}]},
                                  {"role": "assistant", "content": [{"type": "text", "text": f"a {shape}"}]}],
                     "images": [f"img{'x' * (i % 2)}"]})
    rows.append({"messages": [{"role": "user", "content": "describe a square"}, {"role": "assistant", "content": "a red square"}]})
    data = tmp_path / "train.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in rows))
    monkeypatch.setattr(mm, "load_processor", lambda cfg, tokenizer=None: Processor())
    monkeypatch.setattr(mm, "_load_image", lambda v: v)
    cfg = load_cfg({
        "base_model": base, "device": "cpu", "processor_type": "AutoProcessor", "adapter": "lora", "lora_r": 4, "lora_alpha": 8,
        "lora_target_modules": ["q_proj", "v_proj"], "datasets": [{"path": str(data), "type": "chat_template"}],
        "role_boundaries": [{"role": "assistant", "start": "ASSISTANT:", "end": "</s>"}],
        "sequence_len": 64, "sample_packing": False, "micro_batch_size": 2, "gradient_accumulation_steps": 1,
        "learning_rate": 5e-3, "max_steps": 6, "logging_steps": 1, "seed": 0, "output_dir": str(tmp_path / "out"),
        "skip_prepare_dataset": True, "remove_unused_columns": False})
    train(cfg)
    out = tmp_path / "out"
    logs = [json.loads(l) for l in open(out / "train_log.jsonl")]
    losses = [l["loss"] for l in logs if "loss" in l]
    assert len(losses) == 6 and losses[-1] < losses[0]
    assert os.path.exists(out / "adapter_model.safetensors")
    # the loss saw assistant words only: 2 words + eos per row, never the placeholder tokens
    per_step = [l["tokens/trainable"] for l in logs if "tokens/trainable" in l]
    assert per_step[0] == 8 and per_step[-1] == 48          # (a, colour, shape, eos) x 2 conversations per step, cumulative


def test_multimodal_entry_refuses_language_only_checkpoints(tmp_path, monkeypatch):
    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.plugins.base import PluginManager
    from axolotl_b200.train.run import train

    PluginManager.reset()
    tc = dict(model_type="llama", vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=256)
    base = str(tmp_path / "base")
    hf_io.save_pretrained(CausalLM(ModelConfig.from_hf_dict(tc), dtype=torch.float32).init_weights(1), base)
    data = tmp_path / "t.jsonl"
    data.write_text(json.dumps({"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "a"}]}))
    monkeypatch.setattr(mm, "load_processor", lambda cfg, tokenizer=None: Processor())
    cfg = load_cfg({"base_model": base, "device": "cpu", "processor_type": "AutoProcessor", "datasets": [{"path": str(data), "type": "chat_template"}],
                           "sequence_len": 64, "micro_batch_size": 1, "gradient_accumulation_steps": 1, "learning_rate": 1e-3, "max_steps": 1,
                           "output_dir": str(tmp_path / "out"), "skip_prepare_dataset": True, "remove_unused_columns": False})
    with pytest.raises(ValueError, match="image front end"):
        train(cfg)


def test_llava_adapter_keys_and_sharded_merge(tmp_path):
    """Adapters of a LLaVA checkpoint are named as PEFT names them on the HF graph (``model.language_model.layers...``) and
    the shard-by-shard merge finds their base tensors."""
    import safetensors.torch as sft

    from axolotl_b200.io.merge import merge_lora_sharded
    from axolotl_b200.models.lora import LoraSpec, inject_lora, save_adapter

    model = _checkpoint(str(tmp_path / "base"))
    spec = LoraSpec(r=4, lora_alpha=8, target_modules=["q_proj", "down_proj"])
    inject_lora(model, spec)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "lora_B" in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
        for _, m in model.fused_linears():
            if getattr(m, "lora_B", None) is not None:
                keep = torch.zeros_like(m.lora_B)
                for (r0, rows, c0, r) in m.lora_blocks:
                    keep[r0:r0 + rows, c0:c0 + r] = 1
                m.lora_B.mul_(keep)
    save_adapter(model, spec, str(tmp_path / "ad"))
    keys = list(sft.load_file(str(tmp_path / "ad" / "adapter_model.safetensors")))
    assert "base_model.model.model.language_model.layers.0.self_attn.q_proj.lora_A.weight" in keys
    pixels = torch.randn(1, 3, 28, 28)
    ids = torch.tensor([[3, 4, IMG, IMG, IMG, IMG, 5, 6, 7]])
    model.eval()
    with torch.no_grad():
        want = model(ids, pixel_values=pixels, return_logits=True).logits
    res = merge_lora_sharded(str(tmp_path / "base"), str(tmp_path / "ad"), str(tmp_path / "merged"))
    assert res["unmatched"] == []
    merged = hf_io.load_pretrained(str(tmp_path / "merged"), dtype=torch.float32)
    merged.eval()
    with torch.no_grad():
        got = merged(ids, pixel_values=pixels, return_logits=True).logits
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()


def test_generate_with_images_matches_stepwise_greedy(tmp_path):
    """``generate(pixel_values=...)``: the tower runs once, every pass merges its features into the prompt's embeddings."""
    model = _checkpoint(str(tmp_path / "b"))
    ids = torch.tensor([[3, 4, IMG, IMG, IMG, IMG, 5, 6]])
    pixels = torch.randn(1, 3, 28, 28)
    out = model.generate(ids, max_new_tokens=4, pixel_values=pixels)
    assert type(model.vision).__name__ == "VisionFrontEnd"        # the stand-in used while generating is gone again
    model.eval()
    cur = ids.clone()
    with torch.no_grad():
        for _ in range(4):
            nxt = model(cur, pixel_values=pixels, return_logits=True).logits[0, -1].argmax()
            cur = torch.cat([cur, nxt.reshape(1, 1)], 1)
    assert torch.equal(cur, out)
