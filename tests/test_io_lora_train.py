import json
import math
import os

import numpy as np
import pytest
import torch

from axolotl_b200.io import hf as hf_io
from axolotl_b200.io import safetensors_io as st
from axolotl_b200.io.merge import merge_lora_sharded, merge_sharded_fsdp_weights
from axolotl_b200.models.config import preset
from axolotl_b200.models.lora import (ALL_LINEAR, LoraSpec, get_peft_state_dict, inject_lora, load_adapter,
                                      merge_and_unload, save_adapter)
from axolotl_b200.models.transformer import CausalLM
from axolotl_b200.ops.nvfp4 import dequantize_nvfp4, quantize_nvfp4
from axolotl_b200.train.optimizer import (FlatAdamW, build_param_groups, default_warmup_steps, make_lr_lambda)
from axolotl_b200.train.trainer import TrainArgs, Trainer, find_last_checkpoint


def _tiny(seed=0, **kw):
    cfg = preset("tiny-llama", vocab_size=256, num_hidden_layers=2, **kw)
    return CausalLM(cfg, dtype=torch.float32).init_weights(seed)


def _randomise_lora(model, seed=5):
    g = torch.Generator().manual_seed(seed)
    for _, m in model.fused_linears():
        if m.lora_A is None:
            continue
        with torch.no_grad():
            for (r0, rows, c0, r) in m.lora_blocks:
                m.lora_B[r0:r0 + rows, c0:c0 + r] = torch.randn(rows, r, generator=g) * 0.05


def test_safetensors_roundtrip_and_interop(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b.c": torch.arange(7, dtype=torch.int64), "h": torch.randn(4, 4).bfloat16(),
               "q": torch.randint(0, 255, (6,), dtype=torch.uint8), "e": torch.zeros(0)}
    p = str(tmp_path / "x.safetensors")
    st.save_file(tensors, p, {"format": "pt"})
    back = st.load_file(p)
    assert all(torch.equal(back[k], v) for k, v in tensors.items())
    safetensors = pytest.importorskip("safetensors.torch")
    theirs = safetensors.load_file(p)
    assert all(torch.equal(theirs[k], v) for k, v in tensors.items())
    safetensors.save_file({k: v for k, v in tensors.items()}, str(tmp_path / "y.safetensors"))
    mine = st.load_file(str(tmp_path / "y.safetensors"))
    assert all(torch.equal(mine[k], v) for k, v in tensors.items())
    names = st.save_sharded({f"w{i}": torch.randn(100, 100) for i in range(6)}, str(tmp_path / "sh"), max_shard_bytes=90_000)
    assert len(names) == 3 and os.path.exists(tmp_path / "sh" / "model.safetensors.index.json")
    assert len(dict(st.iter_checkpoint(str(tmp_path / "sh")))) == 6


def test_peft_adapter_format_and_reload(tmp_path):
    model = _tiny()
    spec = LoraSpec(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj", "down_proj"])
    n = inject_lora(model, spec)
    H, I = 256, 688
    per_layer = 4 * (H + 256) + 4 * (H + 128) + 4 * (I + H)
    assert n == 2 * per_layer
    assert all(not p.requires_grad for k, p in model.named_parameters() if "lora_" not in k)
    _randomise_lora(model)
    sd = get_peft_state_dict(model)
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in sd
    assert sd["base_model.model.model.layers.1.mlp.down_proj.lora_B.weight"].shape == (H, 4)
    assert not any("k_proj" in k or "gate_proj" in k for k in sd)
    save_adapter(model, spec, str(tmp_path / "ad"))
    conf = json.load(open(tmp_path / "ad" / "adapter_config.json"))
    assert conf["peft_type"] == "LORA" and conf["r"] == 4 and conf["target_modules"] == ["down_proj", "q_proj", "v_proj"]
    other = _tiny()
    inject_lora(other, spec)
    load_adapter(other, str(tmp_path / "ad"))
    ids = torch.randint(3, 256, (1, 40))
    with torch.no_grad():
        assert torch.allclose(model(ids, return_logits=True).logits, other(ids, return_logits=True).logits, atol=1e-6)


def test_merge_lora_matches_adapter_forward(tmp_path):
    model = _tiny(1)
    hf_io.save_pretrained(model, str(tmp_path / "base"), max_shard_bytes=2_000_000)  # force several shards
    assert len(st.checkpoint_files(str(tmp_path / "base"))) > 1
    spec = LoraSpec(r=4, lora_alpha=16, target_modules=list(ALL_LINEAR), use_rslora=True)
    inject_lora(model, spec)
    _randomise_lora(model)
    save_adapter(model, spec, str(tmp_path / "ad"))
    ids = torch.randint(3, 256, (1, 48))
    with torch.no_grad():
        want = model(ids, return_logits=True).logits
    res = merge_lora_sharded(str(tmp_path / "base"), str(tmp_path / "ad"), str(tmp_path / "merged"))
    assert res["unmatched"] == [] and res["merged"] == 2 * 7
    merged = hf_io.load_pretrained(str(tmp_path / "merged"), dtype=torch.float32)
    with torch.no_grad():
        got = merged(ids, return_logits=True).logits
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()
    assert os.path.exists(tmp_path / "merged" / "config.json")
    assert os.path.exists(tmp_path / "merged" / "model.safetensors.index.json")
    # in-memory merge agrees too
    merge_and_unload(model)
    with torch.no_grad():
        assert torch.allclose(model(ids, return_logits=True).logits, want, atol=1e-4)


def test_expert_lora_layout_and_merge(tmp_path):
    cfg = preset("tiny-qwen3-moe", vocab_size=256)
    model = CausalLM(cfg, dtype=torch.float32).init_weights(2)
    hf_io.save_pretrained(model, str(tmp_path / "base"))
    spec = LoraSpec(r=2, lora_alpha=4, target_modules=["q_proj"], target_parameters=["mlp.experts.gate_up_proj", "mlp.experts.down_proj"])
    inject_lora(model, spec)
    ex = model.layers[0].mlp.experts
    E, r = ex.E, 2
    assert ex.lora["gate_up_A"].shape == (E * r, 256) and ex.lora["gate_up_B"].shape == (2 * 128, r * E)
    with torch.no_grad():
        for l in model.layers:
            for k in ("gate_up_B", "down_B"):
                l.mlp.experts.lora[k].normal_(0, 0.05)
    A, B = ex.expert_lora("down", 3)
    assert torch.equal(A, ex.lora["down_A"][3 * r:4 * r]) and torch.equal(B, ex.lora["down_B"].view(256, r, E)[:, :, 3])
    save_adapter(model, spec, str(tmp_path / "ad"))
    keys = st.SafeFile(str(tmp_path / "ad" / "adapter_model.safetensors")).keys()
    assert "base_model.model.model.layers.0.mlp.experts.gate_up_proj.lora_A.weight" in keys
    ids = torch.randint(3, 256, (1, 32))
    model.eval()
    with torch.no_grad():
        want = model(ids, return_logits=True).logits
    merge_lora_sharded(str(tmp_path / "base"), str(tmp_path / "ad"), str(tmp_path / "m"))
    merged = hf_io.load_pretrained(str(tmp_path / "m"), dtype=torch.float32).eval()
    with torch.no_grad():
        got = merged(ids, return_logits=True).logits
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()


def test_nvfp4_quantisation_roundtrip_and_grid():
    torch.manual_seed(0)
    w = torch.randn(4, 32, 64)
    q, s, pts = quantize_nvfp4(w)
    assert q.shape == (4, 32, 32) and q.dtype == torch.uint8 and s.shape == (4, 32, 4) and s.dtype == torch.float8_e4m3fn
    d = dequantize_nvfp4(q, s, pts, dtype=torch.float32)
    rel = ((d - w).norm() / w.norm()).item()
    assert rel < 0.12
    # values already on the grid survive exactly; nibble order: low = even k
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0, 0.0])
    x = grid.repeat(2, 1)
    q2, s2, p2 = quantize_nvfp4(x, pts=torch.tensor(1.0))
    assert torch.equal(dequantize_nvfp4(q2, s2, p2, dtype=torch.float32), x)
    assert (q2[0, 0] & 0xF) == 0 and (q2[0, 0] >> 4) == 1
    q3, s3, p3 = quantize_nvfp4(dequantize_nvfp4(q, s, pts, dtype=torch.float32), pts=pts)
    assert torch.equal(q3, q)   # requantising with the same scales is idempotent


def test_nvfp4_expert_loading_reconciles_scales():
    from axolotl_b200.io.nvfp4_loading import fuse_nvfp4_experts, is_nvfp4_parts

    torch.manual_seed(1)
    parts, ref = {}, {}
    for e in range(2):
        for sub, shape, scale in (("gate_proj", (16, 32), 1.0), ("up_proj", (16, 32), 3.0), ("down_proj", (32, 16), 1.0)):
            w = torch.randn(*shape) * scale
            q, s, p = quantize_nvfp4(w)
            parts[(e, sub, "weight")] = q
            parts[(e, sub, "weight_scale")] = s
            parts[(e, sub, "weight_scale_2")] = p
            ref[(e, sub)] = dequantize_nvfp4(q, s, p, dtype=torch.float32)
    assert is_nvfp4_parts(parts)
    fused = fuse_nvfp4_experts(parts, 2)
    gu = dequantize_nvfp4(fused["gate_up"]["qdata"], fused["gate_up"]["scale"], fused["gate_up"]["pts"], dtype=torch.float32)
    for e in range(2):
        want = torch.cat([ref[(e, "gate_proj")], ref[(e, "up_proj")]], 0)
        assert ((gu[e] - want).norm() / want.norm()).item() < 0.08
        assert torch.equal(gu[e][16:], ref[(e, "up_proj")])   # the larger scale is kept exactly


def test_flat_adamw_matches_torch_and_param_groups():
    torch.manual_seed(0)
    lin = torch.nn.Linear(16, 8)
    ref = torch.nn.Linear(16, 8)
    ref.load_state_dict(lin.state_dict())
    groups = build_param_groups(lin.named_parameters(), weight_decay=0.1)
    assert {g["name"]: g["weight_decay"] for g in groups} == {"decay": 0.1, "no_decay": 0.0}
    opt = FlatAdamW(groups, lr=1e-2, max_grad_norm=0.5)
    ro = torch.optim.AdamW([{"params": [ref.weight], "weight_decay": 0.1}, {"params": [ref.bias], "weight_decay": 0.0}], lr=1e-2)
    for _ in range(4):
        x = torch.randn(5, 16)
        lin(x).pow(2).sum().backward()
        ref(x).pow(2).sum().backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        opt.step()
        opt.zero_grad()
        ro.step()
        ro.zero_grad()
    assert torch.allclose(lin.weight, ref.weight, atol=1e-6) and torch.allclose(lin.bias, ref.bias, atol=1e-6)
    g2 = build_param_groups([("model.embed_tokens", torch.nn.Parameter(torch.zeros(4, 4))),
                             ("x.lora_B", torch.nn.Parameter(torch.zeros(4, 4))),
                             ("x.lora_A", torch.nn.Parameter(torch.zeros(4, 4)))], embedding_lr_scale=0.5, loraplus_lr_ratio=16, lr=1e-3)
    assert {g["name"]: g["lr_scale"] for g in g2} == {"embeddings": 0.5, "lora_B": 16, "decay": 1.0}


def test_schedules_and_warmup_defaults():
    f = make_lr_lambda("cosine", 100, 10)
    assert f(0) == 0 and f(5) == 0.5 and f(10) == 1.0 and abs(f(55) - 0.5) < 1e-6 and f(100) < 1e-6
    m = make_lr_lambda("cosine_with_min_lr", 100, 0, min_lr_ratio=0.1)
    assert abs(m(100) - 0.1) < 1e-9 and m(0) == 1.0
    assert make_lr_lambda("linear", 10, 0)(5) == 0.5 and make_lr_lambda("constant", 10, 0)(7) == 1.0
    assert make_lr_lambda("constant_with_warmup", 10, 4)(2) == 0.5
    q = make_lr_lambda("cosine_with_quadratic_warmup", 100, 10)
    assert q(5) == 0.25
    r = make_lr_lambda("rex", 100, 0)
    assert r(0) == 1.0 and 0 < r(50) < 1 and r(100) == 0
    with pytest.raises(ValueError):
        make_lr_lambda("nope", 10, 0)
    assert default_warmup_steps(1000) == 30 and default_warmup_steps(10000) == 100
    assert default_warmup_steps(1000, warmup_ratio=0.001) == 2 and default_warmup_steps(1000, warmup_steps=7) == 7


def _make_trainer(tmp, max_steps, resume=None, seed=0):
    from axolotl_b200.data.collator import PackedCollator
    from axolotl_b200.data.synthetic import synthetic_varlen

    torch.manual_seed(seed)
    model = _tiny(3)
    inject_lora(model, LoraSpec(r=4, lora_alpha=8, target_modules=list(ALL_LINEAR)))
    _randomise_lora(model)
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=5e-3, max_grad_norm=1.0)
    ds = synthetic_varlen(64, 20, 60, 3, 256, 0.25, seed=1)
    coll = PackedCollator()

    def batches(epoch):
        for i in range(0, 64, 2):
            yield coll([[ds[i], ds[i + 1]]])

    spec = LoraSpec(r=4, lora_alpha=8, target_modules=list(ALL_LINEAR))
    args = TrainArgs(output_dir=str(tmp), max_steps=max_steps, gradient_accumulation_steps=2, learning_rate=5e-3,
                     save_steps=3, save_strategy="steps", save_total_limit=2, resume_from_checkpoint=resume)
    tr = Trainer(model, opt, make_lr_lambda("linear", 8, 2), args, batches, total_steps=8,
                 save_fn=lambda t, d: save_adapter(model, spec, d))
    if resume:
        load_adapter(model, resume)
    return tr, model, opt


def test_trainer_checkpoint_resume_is_exact(tmp_path):
    tr, model, opt = _make_trainer(tmp_path / "a", 8)
    hist = tr.train()
    full = [h["loss"] for h in hist if "loss" in h]
    assert len(full) == 8
    cks = sorted(os.listdir(tmp_path / "a"))
    assert "checkpoint-6" in cks and "checkpoint-3" in cks
    ck = tmp_path / "a" / "checkpoint-6"
    for f in ("adapter_model.safetensors", "adapter_config.json", "optimizer.pt", "rng_state.pth", "trainer_state.json", "tokens_state.json"):
        assert os.path.exists(ck / f), f
    assert find_last_checkpoint(str(tmp_path / "a")).endswith("checkpoint-6")
    tr2, model2, _ = _make_trainer(tmp_path / "a", 8, resume=str(ck))
    hist2 = tr2.train()
    tail = [h["loss"] for h in hist2 if "loss" in h and h["step"] > 6]
    assert tail == pytest.approx(full[6:], rel=1e-5)
    assert tr2.tokens["trainable"] == tr.tokens["trainable"]
    a = torch.cat([p.detach().reshape(-1) for p in model.parameters() if p.requires_grad])
    b = torch.cat([p.detach().reshape(-1) for p in model2.parameters() if p.requires_grad])
    assert torch.allclose(a, b, atol=1e-6)


def _epoch_trainer(tmp, *, num_epochs, max_steps=-1, resume=None, save_strategy="steps", save_steps=2):
    """12 micro-batches per epoch whose ORDER depends on the epoch, gradient accumulation 2 -> 6 steps per epoch."""
    from axolotl_b200.data.collator import PackedCollator
    from axolotl_b200.data.synthetic import synthetic_varlen

    torch.manual_seed(0)
    model = _tiny(3)
    spec = LoraSpec(r=4, lora_alpha=8, target_modules=list(ALL_LINEAR))
    inject_lora(model, spec)
    _randomise_lora(model)
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=5e-3, max_grad_norm=1.0)
    ds = synthetic_varlen(24, 20, 60, 3, 256, 0.25, seed=1)
    coll = PackedCollator()

    def batches(epoch):
        order = np.random.default_rng(100 + epoch).permutation(12)
        for i in order:
            yield coll([[ds[2 * i], ds[2 * i + 1]]])

    args = TrainArgs(output_dir=str(tmp), max_steps=max_steps, num_epochs=num_epochs, gradient_accumulation_steps=2,
                     learning_rate=5e-3, save_steps=save_steps, save_strategy=save_strategy, save_total_limit=20,
                     resume_from_checkpoint=resume)
    tr = Trainer(model, opt, make_lr_lambda("constant", 100, 0), args, batches, total_steps=6 * num_epochs,
                 save_fn=lambda t, d: save_adapter(model, spec, d))
    if resume:
        load_adapter(model, resume)
    return tr, model


def test_resume_from_a_checkpoint_in_a_later_epoch(tmp_path):
    """A checkpoint taken inside epoch 1 of a 3-epoch run: the resumed run skips only the batches
    of THAT epoch which were already consumed, and ends exactly like the uninterrupted run."""
    tr, model = _epoch_trainer(tmp_path / "a", num_epochs=3)
    full = [h["loss"] for h in tr.train() if "loss" in h]
    assert len(full) == 18 and tr.epoch == 2
    ck = tmp_path / "a" / "checkpoint-10"       # step 10 = epoch 1, 4 of its 6 steps done
    state = json.load(open(ck / "trainer_state.json"))
    assert state["epoch"] == 1 and state["batches_in_epoch"] == 8
    tr2, model2 = _epoch_trainer(tmp_path / "a", num_epochs=3, resume=str(ck))
    hist2 = tr2.train()
    tail = [h["loss"] for h in hist2 if "loss" in h and h["step"] > 10]
    assert len(tail) == 8 and tr2.global_step == 18
    assert tail == pytest.approx(full[10:], rel=1e-5)
    a = torch.cat([p.detach().reshape(-1) for p in model.parameters() if p.requires_grad])
    b = torch.cat([p.detach().reshape(-1) for p in model2.parameters() if p.requires_grad])
    assert torch.allclose(a, b, atol=1e-6)


def test_epoch_save_strategy_and_max_steps_beyond_the_data(tmp_path):
    tr, _ = _epoch_trainer(tmp_path / "e", num_epochs=2, save_strategy="epoch", save_steps=None)
    tr.train()
    assert sorted(os.listdir(tmp_path / "e")) == ["checkpoint-12", "checkpoint-6"]
    # max_steps larger than num_epochs x steps-per-epoch: the data is cycled until the steps are done
    tr2, _ = _epoch_trainer(tmp_path / "m", num_epochs=1, max_steps=9, save_strategy="no", save_steps=None)
    tr2.train()
    assert tr2.global_step == 9 and tr2.epoch == 1


def test_loss_decreases_on_learnable_data():
    from axolotl_b200.data.collator import PackedCollator

    torch.manual_seed(0)
    model = _tiny(4)
    inject_lora(model, LoraSpec(r=8, lora_alpha=16, target_modules=list(ALL_LINEAR)))
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=1e-2, max_grad_norm=1.0)
    seq = np.tile(np.arange(3, 35), 4)
    batch = PackedCollator()([[{"input_ids": seq, "labels": seq}]])
    tr = Trainer(model, opt, make_lr_lambda("constant", 100, 0), TrainArgs(max_steps=30, learning_rate=1e-2), lambda e: [batch])
    losses = [float(tr.training_step([batch]).item()) for _ in range(30)]
    assert losses[-1] < 0.85 * losses[0] and losses[-1] < losses[10] < losses[0]


def test_merge_sharded_fsdp_weights(tmp_path):
    full = {"w": torch.randn(8, 4), "b": torch.randn(4)}
    os.makedirs(tmp_path / "s")
    for r in range(2):
        st.save_file({"w": full["w"][r * 4:(r + 1) * 4].contiguous(), "b": full["b"]}, str(tmp_path / "s" / f"shard_rank{r}.safetensors"))
    json.dump({"world_size": 2, "sharded": ["w"]}, open(tmp_path / "s" / "shard_index.json", "w"))
    merge_sharded_fsdp_weights(str(tmp_path / "s"), str(tmp_path / "o"), dtype=torch.float32)
    back = st.load_file(str(tmp_path / "o" / "model.safetensors"))
    assert torch.equal(back["w"], full["w"]) and torch.equal(back["b"], full["b"])


def test_nf4_roundtrip_and_qlora_training(tmp_path):
    """NF4 quantise/dequantise error bounds, double-quant storage, and a QLoRA run through the
    run builder that learns with frozen 4-bit projections."""
    import torch

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.models.layers import FusedLinear
    from axolotl_b200.ops.nf4 import dequantize_nf4, quantize_nf4
    from axolotl_b200.train.run import train

    torch.manual_seed(0)
    w = torch.randn(128, 256) * 0.02
    for dq in (False, True):
        q, st = quantize_nf4(w, double_quant=dq)
        assert q.dtype == torch.uint8 and q.numel() == w.numel() // 2
        err = (dequantize_nf4(q, st, dtype=torch.float32) - w).norm() / w.norm()
        assert err < 0.11
    # absmax maps to code 15 (or 0) exactly
    blk = torch.zeros(64); blk[3] = 2.0; blk[7] = -1.0
    q, st = quantize_nf4(blk, double_quant=False)
    d = dequantize_nf4(q, st, dtype=torch.float32)
    assert d[3] == 2.0 and abs(d[7] + 1.0) < 0.11 and float(d[0]) == 0.0

    lin = FusedLinear(256, [128], ["x"], dtype=torch.float32)
    with torch.no_grad():
        lin.weight.copy_(w)
    x = torch.randn(5, 256)
    y_ref = x @ w.t()
    lin.quantize_nf4_()
    assert lin.weight.dtype == torch.uint8 and lin.weight.shape == (128, 128)
    assert ((lin(x) - y_ref).norm() / y_ref.norm()) < 0.12

    cfg = load_cfg({"model_preset": "tiny-llama", "adapter": "qlora", "load_in_4bit": True, "lora_r": 8, "lora_alpha": 16,
                    "lora_target_linear": True, "sequence_len": 256, "micro_batch_size": 2, "gradient_accumulation_steps": 1,
                    "max_steps": 12, "learning_rate": 2e-3, "optimizer": "adamw_torch", "lr_scheduler": "constant",
                    "output_dir": str(tmp_path / "q"), "device": "cpu", "logging_steps": 1, "sample_packing": True,
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 64, "min_length": 32,
                                  "max_length": 128, "max_input_id": 400}]})
    model, _, trainer = train(cfg)
    assert all(getattr(m.weight, "_axb_quant", None) is not None for n, m in model.fused_linears() if n.startswith("layers."))
    losses = [l["loss"] for l in trainer.log_history if "loss" in l]
    assert losses[-1] < losses[0]
    assert (tmp_path / "q" / "adapter_model.safetensors").exists()


def test_dora_matches_definition_saves_and_merges(tmp_path):
    import torch

    from axolotl_b200.io.merge import merge_tensor
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.lora import LoraSpec, get_peft_state_dict, inject_lora, merge_and_unload, set_peft_state_dict
    from axolotl_b200.models.transformer import CausalLM

    torch.manual_seed(0)
    cfg = preset("tiny-llama", num_hidden_layers=1, vocab_size=128)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(0)
    spec = LoraSpec(r=4, lora_alpha=8, target_modules=["q_proj", "down_proj"], use_dora=True)
    ids = torch.randint(0, 128, (1, 24))
    base_logits = model(ids, return_logits=True).logits
    inject_lora(model, spec)
    assert torch.allclose(model(ids, return_logits=True).logits, base_logits, atol=1e-5)   # identity at init
    lin = model.layers[0].self_attn.qkv_proj
    with torch.no_grad():
        for _, m in model.fused_linears():
            if m.lora_A is not None:
                mask = torch.zeros_like(m.lora_B)
                for (r0, rows, c0, r) in m.lora_blocks:
                    mask[r0:r0 + rows, c0:c0 + r] = 1
                m.lora_B.copy_(torch.randn_like(m.lora_B) * 0.05 * mask)
                m.dora_magnitude.mul_(1.0 + 0.1 * torch.rand_like(m.dora_magnitude))
    x = torch.randn(3, cfg.hidden_size)
    W = lin.weight + lin.scaling * lin.lora_B @ lin.lora_A
    q0, q1 = lin.row_range("q_proj")
    want = x @ W.t()
    want[:, q0:q1] *= (lin.dora_magnitude / W.norm(dim=1))[q0:q1]
    assert torch.allclose(lin(x), want, atol=1e-5)
    # gradient reaches the magnitude of adapted rows only
    lin(x).sum().backward()
    assert lin.dora_magnitude.grad[q0:q1].abs().sum() > 0 and lin.dora_magnitude.grad[q1:].abs().sum() == 0
    sd = get_peft_state_dict(model)
    key = "base_model.model.model.layers.0.self_attn.q_proj"
    assert sd[key + ".lora_magnitude_vector"].shape == (q1 - q0,)
    # the offline merge tool reproduces the layer
    pairs = {"model.layers.0.self_attn.q_proj": {"A": sd[key + ".lora_A.weight"].float(), "B": sd[key + ".lora_B.weight"].float(),
                                                  "M": sd[key + ".lora_magnitude_vector"].float()}}
    merged = merge_tensor("model.layers.0.self_attn.q_proj.weight", lin.weight[q0:q1].detach(), spec.to_peft_dict(), pairs)
    assert torch.allclose(x @ merged.t(), want[:, q0:q1], atol=1e-5)
    # reload into a fresh model, then merge in place
    logits = model(ids, return_logits=True).logits
    model2 = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(0)
    inject_lora(model2, spec)
    set_peft_state_dict(model2, {k: v.clone() for k, v in sd.items()})
    assert torch.allclose(model2(ids, return_logits=True).logits, logits, atol=1e-5)
    merge_and_unload(model2)
    assert torch.allclose(model2(ids, return_logits=True).logits, logits, atol=1e-4)


def test_relora_restart_and_jagged_schedule():
    import torch

    from axolotl_b200.models.config import preset
    from axolotl_b200.models.lora import LoraSpec, inject_lora
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.train.callbacks import ReLoRACallback
    from axolotl_b200.train.optimizer import FlatAdamW, build_param_groups, jagged_restarts, make_lr_lambda

    f = jagged_restarts(make_lr_lambda("constant", 100, 0), restart_steps=10, warmup_steps=4, anneal_steps=2)
    assert f(0) == 1.0 and f(7) == 1.0 and f(9) < 1.0 and f(10) < 0.01 and f(12) < f(13) <= 1.0 and f(15) == 1.0

    cfg = preset("tiny-llama", num_hidden_layers=1, vocab_size=128)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(0)
    inject_lora(model, LoraSpec(r=4, lora_alpha=8, target_modules="all-linear"))
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=1e-2)
    lin = model.layers[0].mlp.down_proj
    with torch.no_grad():
        lin.lora_B.normal_(0, 0.05)
    for g in opt.groups:
        g["exp_avg"].fill_(1.0)
    ids = torch.randint(0, 128, (1, 16))
    before = model(ids, return_logits=True).logits
    w0 = lin.weight.clone()

    class T:
        global_step = 10
    T.model, T.opt = model, opt
    ReLoRACallback(10, prune_ratio=1.0).on_step_end(T, {})
    assert float(lin.lora_B.detach().abs().max()) == 0.0 and not torch.equal(lin.weight, w0)
    assert torch.allclose(model(ids, return_logits=True).logits, before, atol=1e-5)   # function preserved
    assert all(float(g["exp_avg"][o:o + k].abs().max()) == 0.0 for g in opt.groups for n, p, o, k in g["entries"] if "lora" in n)


def test_neftune_only_in_training():
    import torch

    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM

    model = CausalLM(preset("tiny-llama", num_hidden_layers=1, vocab_size=64), dtype=torch.float32, device="cpu").init_weights(0)
    ids = torch.randint(0, 64, (1, 16))
    model.eval()
    a = model(ids, return_logits=True).logits
    model.neftune_noise_alpha = 5.0
    assert torch.allclose(model(ids, return_logits=True).logits, a, atol=1e-6)
    model.train()
    assert (model(ids, return_logits=True).logits - a).abs().max() > 1e-4


def test_tiled_mlp_matches_untiled_and_trace_analyzer(tmp_path):
    import json

    import torch

    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.utils.analyze_profile import compare, summarize

    cfg = preset("tiny-llama", num_hidden_layers=2, vocab_size=128)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(0)
    model.train()
    ids = torch.randint(0, 128, (1, 96))
    out = model(ids, labels=ids)
    out.loss.backward()
    g0 = model.layers[0].mlp.down_proj.weight.grad.clone()
    model.zero_grad()
    for l in model.layers:
        l.mlp.tile_rows = 32
    out2 = model(ids, labels=ids)
    out2.loss.backward()
    assert torch.allclose(out.loss, out2.loss, atol=1e-6)
    assert torch.allclose(model.layers[0].mlp.down_proj.weight.grad, g0, atol=1e-5)

    ev = [{"ph": "X", "cat": "kernel", "name": "gemm_bf16_tcgen05_kernel<256, false, false>", "dur": 300.0},
          {"ph": "X", "cat": "kernel", "name": "flash_bwd_kernel<128>", "dur": 100.0},
          {"ph": "X", "cat": "kernel", "name": "adamw_kernel", "dur": 10.0},
          {"ph": "X", "cat": "kernel", "name": "some_library_kernel", "dur": 5.0},
          {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "dur": 999.0}]
    p = tmp_path / "t.json"
    p.write_text(json.dumps({"traceEvents": ev}))
    agg, steps, lines = summarize(str(p))
    assert steps == 1 and agg["gemm (tcgen05)"][1] == 300.0 and agg["attention bwd"][0] == 1
    assert agg["library / other"][1] == 5.0 and any("gemm" in l for l in lines)
    assert any("attention bwd" in l for l in compare(str(p), str(p)))


def test_sample_generation_callback_writes_rows(tmp_path):
    import json

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.train.run import train

    cfg = load_cfg({"model_preset": "tiny-llama", "adapter": "lora", "lora_r": 8, "lora_alpha": 16, "lora_target_linear": True,
                    "sequence_len": 128, "micro_batch_size": 2, "gradient_accumulation_steps": 1, "max_steps": 4,
                    "learning_rate": 1e-3, "optimizer": "adamw_torch", "output_dir": str(tmp_path / "g"), "device": "cpu",
                    "generate_samples": True, "num_generation_samples": 2, "generation_max_new_tokens": 5,
                    "generation_do_sample": False, "save_steps": 2, "save_strategy": "steps", "sample_packing": True,
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 24, "min_length": 16,
                                  "max_length": 48, "max_input_id": 300}]})
    train(cfg)
    rows = [json.loads(l) for l in open(tmp_path / "g" / "generations.jsonl")]
    assert len(rows) == 4 and rows[0]["step"] == 2 and rows[-1]["step"] == 4
    assert len(rows[0]["generation"]) <= 5 and len(rows[0]["prompt"]) >= 1


def test_lisa_trains_only_sampled_layers(tmp_path):
    import torch

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.train.run import train

    cfg = load_cfg({"model_preset": "tiny-llama", "sequence_len": 128, "micro_batch_size": 2, "gradient_accumulation_steps": 1,
                    "max_steps": 4, "learning_rate": 1e-3, "optimizer": "adamw_torch", "lr_scheduler": "constant",
                    "output_dir": str(tmp_path / "l"), "device": "cpu", "lisa_n_layers": 1, "lisa_step_interval": 100,
                    "sample_packing": True, "save_strategy": "no", "weight_decay": 0.0,
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 24, "min_length": 16,
                                  "max_length": 48, "max_input_id": 300}]})
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM
    ref = CausalLM(preset("tiny-llama"), dtype=torch.float32, device="cpu").init_weights(cfg.get("seed") or 42)
    model, _, trainer = train(cfg)
    changed = []
    for i, (a, b) in enumerate(zip(model.layers, ref.layers)):
        d = max(float((p.detach() - q.detach()).abs().max()) for p, q in zip(a.parameters(), b.parameters()))
        changed.append(d > 0)
    assert sum(changed) == 1, changed                      # exactly the sampled layer moved
    assert float((model.embed_tokens.detach() - ref.embed_tokens.detach()).abs().max()) > 0   # embeddings always train


def test_sparse_finetuning_keeps_zero_pattern(tmp_path):
    import torch

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.io import hf as hf_io
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM
    from axolotl_b200.plugins.base import PluginManager
    from axolotl_b200.plugins.sparse_ft import recipe_targets
    from axolotl_b200.train.run import train

    base = CausalLM(preset("tiny-llama"), dtype=torch.float32, device="cpu").init_weights(3)
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for layer in base.layers:   # 2:4-like pruning of q_proj and down_proj; k/v/o/gate/up stay dense
            q0, q1 = layer.self_attn.qkv_proj.row_range("q_proj")
            w = layer.self_attn.qkv_proj.weight
            w[q0:q1] *= (torch.rand(w[q0:q1].shape, generator=g) > 0.5)
            d = layer.mlp.down_proj.weight
            d *= (torch.rand(d.shape, generator=g) > 0.5)
    hf_io.save_pretrained(base, str(tmp_path / "sparse"))
    recipe = {"finetuning_stage": {"finetuning_modifiers": {"ConstantPruningModifier": {
        "targets": ["re:.*q_proj.weight", "re:.*down_proj.weight"], "start": 0}}}}
    assert recipe_targets(recipe) == ["re:.*q_proj.weight", "re:.*down_proj.weight"]
    PluginManager.reset()
    cfg = load_cfg({"base_model": str(tmp_path / "sparse"), "plugins": ["axolotl.integrations.llm_compressor.LLMCompressorPlugin"],
                    "llmcompressor": {"recipe": recipe}, "sequence_len": 128, "micro_batch_size": 2,
                    "gradient_accumulation_steps": 1, "max_steps": 3, "learning_rate": 1e-3, "optimizer": "adamw_torch",
                    "lr_scheduler": "constant", "output_dir": str(tmp_path / "o"), "device": "cpu", "sample_packing": True,
                    "save_strategy": "no", "weight_decay": 0.01,
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 24, "min_length": 16,
                                  "max_length": 48, "max_input_id": 300}]})
    model, _, _ = train(cfg)
    PluginManager.reset()
    for a, b in zip(model.layers, base.layers):
        q0, q1 = a.self_attn.qkv_proj.row_range("q_proj")
        wa, wb = a.self_attn.qkv_proj.weight.detach().float(), b.self_attn.qkv_proj.weight.detach().float()
        zeros = wb[q0:q1] == 0
        assert bool((wa[q0:q1][zeros] == 0).all())                  # pruned entries stayed zero
        assert float((wa[q0:q1][~zeros] - wb[q0:q1][~zeros]).abs().max()) > 0   # the others trained
        assert float((wa[q1:] - wb[q1:]).abs().max()) > 0           # k/v rows of the same fused weight are untouched by the mask
        da, db = a.mlp.down_proj.weight.detach().float(), b.mlp.down_proj.weight.detach().float()
        assert bool((da[db == 0] == 0).all())


def test_mora_operators_training_save_and_merge(tmp_path):
    import torch

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.models.mora import ROPE, SHARING, mora_delta, mora_dense_delta, mora_rank
    from axolotl_b200.plugins.base import PluginManager
    from axolotl_b200.train.run import train

    # operators against a direct transcription of their definition
    torch.manual_seed(0)
    in_f, out_f, r = 96, 160, 4
    rh = mora_rank(in_f, out_f, r)
    assert rh == 32 and rh * rh <= (in_f + out_f) * r + rh
    M = torch.randn(rh, rh)
    x = torch.randn(5, in_f)
    # sharing: sum of chunks -> M -> tiled
    ref = torch.cat([(x.reshape(5, 3, rh).sum(1) @ M.t())] * 5, -1)[:, :out_f]
    assert torch.allclose(mora_delta(x, M, out_f, SHARING), ref, atol=1e-5)
    # rope: linear in x, so it must equal its own dense form; chunks are distinguishable
    W = mora_dense_delta(M, in_f, out_f, ROPE)
    assert W.shape == (out_f, in_f)
    assert torch.allclose(mora_delta(x, M, out_f, ROPE), x @ W.t(), atol=1e-4)
    x2 = x.clone()
    x2[:, :rh], x2[:, rh:2 * rh] = x[:, rh:2 * rh], x[:, :rh]
    assert not torch.allclose(mora_delta(x2, M, out_f, ROPE)[:, :rh], mora_delta(x, M, out_f, ROPE)[:, rh:2 * rh], atol=1e-3)

    PluginManager.reset()
    cfg = load_cfg({"model_preset": "tiny-llama", "plugins": ["axolotl.integrations.mora.MoraPlugin"], "adapter": "mora",
                    "mora": {"use_mora": True, "mora_type": "rope"}, "lora_r": 8, "lora_target_modules": ["q_proj", "down_proj"],
                    "sequence_len": 128, "micro_batch_size": 2, "gradient_accumulation_steps": 1, "max_steps": 6,
                    "learning_rate": 5e-3, "optimizer": "adamw_torch", "lr_scheduler": "constant", "logging_steps": 1,
                    "output_dir": str(tmp_path / "m"), "device": "cpu", "sample_packing": True,
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 24, "min_length": 16,
                                  "max_length": 48, "max_input_id": 300}]})
    model, _, trainer = train(cfg)
    PluginManager.reset()
    losses = [l["loss"] for l in trainer.log_history if "loss" in l]
    assert losses[-1] < losses[0]
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("mora_M" in n for n in trainable)
    import json
    from axolotl_b200.io.safetensors_io import load_file
    from axolotl_b200.models.lora import merge_and_unload
    sd = load_file(str(tmp_path / "m" / "adapter_model.safetensors"))
    k = "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"
    assert k in sd and sd[k].shape[0] == sd[k].shape[1] and float(sd[k].abs().max()) > 0
    assert json.load(open(tmp_path / "m" / "adapter_config.json"))["use_mora"] is True
    ids = torch.randint(3, 300, (1, 40))
    pos = torch.arange(40, dtype=torch.int32)[None]
    model.eval()
    with torch.no_grad():
        before = model(ids, pos, return_logits=True).logits
        merge_and_unload(model)
        after = model(ids, pos, return_logits=True).logits
    assert torch.allclose(before, after, atol=2e-3, rtol=1e-3)


def test_embedding_lora_matches_definition_saves_and_merges(tmp_path):
    import torch

    from axolotl_b200.io.safetensors_io import load_file
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.lora import LoraSpec, inject_lora, load_adapter, merge_and_unload, save_adapter
    from axolotl_b200.models.transformer import CausalLM

    cfg = preset("tiny-llama", vocab_size=200, num_hidden_layers=1, tie_word_embeddings=False)
    model = CausalLM(cfg, dtype=torch.float32).init_weights(0)
    spec = LoraSpec(r=8, lora_alpha=16, target_modules=["embed_tokens", "q_proj"])
    inject_lora(model, spec)
    assert model.embed_lora_At.shape == (200, 8) and model.embed_lora_At.requires_grad and not model.embed_tokens.requires_grad
    ids = torch.randint(0, 200, (1, 24))
    base = model(ids, return_logits=True).logits
    with torch.no_grad():
        model.embed_lora_At.normal_(0, 0.3)
    out = model(ids, labels=ids)
    out.loss.backward()
    gA = model.embed_lora_At.grad if model.embed_lora_At.grad is not None else model.embed_lora_At._axb_grad
    used = torch.zeros(200, dtype=torch.bool)
    used[ids.reshape(-1)] = True
    assert float(gA[used].abs().sum()) > 0 and float(gA[~used].abs().sum()) == 0   # only looked-up rows get gradient
    model.eval()
    with torch.no_grad():
        adapted = model(ids, return_logits=True).logits
        assert (adapted - base).abs().max() > 1e-3
        # definition: E' = E + s * A^T B^T
        E2 = model.embed_tokens + 2.0 * model.embed_lora_At @ model.embed_lora_B.t()
    save_adapter(model, spec, str(tmp_path / "a"))
    sd = load_file(str(tmp_path / "a" / "adapter_model.safetensors"))
    assert sd["base_model.model.model.embed_tokens.lora_embedding_A"].shape == (8, 200)
    assert sd["base_model.model.model.embed_tokens.lora_embedding_B"].shape == (cfg.hidden_size, 8)
    fresh = CausalLM(cfg, dtype=torch.float32).init_weights(0)
    inject_lora(fresh, spec)
    load_adapter(fresh, str(tmp_path / "a"))
    fresh.eval()
    with torch.no_grad():
        assert torch.allclose(fresh(ids, return_logits=True).logits, adapted, atol=1e-5)
        merge_and_unload(model)
        assert torch.allclose(model.embed_tokens, E2, atol=1e-5)
        assert torch.allclose(model(ids, return_logits=True).logits, adapted, atol=1e-4)


def test_kv_cache_generation_equals_full_recompute():
    import torch

    from axolotl_b200.models.config import preset
    from axolotl_b200.models.kv_cache import generate_cached
    from axolotl_b200.models.transformer import CausalLM

    for name in ("tiny-llama", "tiny-qwen3-moe"):
        m = CausalLM(preset(name, vocab_size=97), dtype=torch.float32).init_weights(0)
        prompts = [[1, 5, 9, 12, 40], [3, 4], [7, 8, 9]]
        outs = generate_cached(m, prompts, 6)
        ref = [m.generate(torch.tensor(p), max_new_tokens=6, use_cache=False)[0, len(p):].tolist() for p in prompts]
        assert outs == ref
    # EOS ends a sequence while the others go on; sampled decoding is reproducible under a seeded generator
    first = outs[0][0]
    stopped = generate_cached(m, prompts, 6, eos_token_id=first)
    assert stopped[0] == [first] and len(stopped[1]) >= 1
    g1 = generate_cached(m, prompts, 5, temperature=1.0, top_p=0.9, generator=torch.Generator().manual_seed(3))
    g2 = generate_cached(m, prompts, 5, temperature=1.0, top_p=0.9, generator=torch.Generator().manual_seed(3))
    assert g1 == g2


def test_trainable_token_rows_and_fix_untrained_tokens(tmp_path):
    import torch

    from axolotl_b200.io.safetensors_io import load_file
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.lora import LoraSpec, inject_lora, load_adapter, merge_and_unload, save_adapter
    from axolotl_b200.models.transformer import CausalLM

    cfg = preset("tiny-llama", vocab_size=200, num_hidden_layers=1, tie_word_embeddings=False)
    model = CausalLM(cfg, dtype=torch.float32).init_weights(0)
    with torch.no_grad():
        model.embed_tokens[190:] = 0          # "new" tokens the base model never saw
        model.lm_head[195:] = 0
    assert model.fix_untrained_tokens() == 10 + 5
    assert torch.allclose(model.embed_tokens[199], model.embed_tokens[:190].mean(0), atol=1e-6)
    spec = LoraSpec(r=8, lora_alpha=16, target_modules=["q_proj"], trainable_token_indices=[190, 3, 199])
    inject_lora(model, spec)
    assert model.token_rows.shape == (3, cfg.hidden_size) and model.token_rows.requires_grad
    ids = torch.tensor([[3, 5, 190, 7, 199, 3, 8, 9]])
    before = model.embed_tokens.detach().clone()
    out = model(ids, labels=ids)
    out.loss.backward()
    g = model.token_rows.grad if model.token_rows.grad is not None else model.token_rows._axb_grad
    assert float(g.abs().sum()) > 0 and model.embed_tokens.grad is None
    with torch.no_grad():
        model.token_rows.add_(0.5)
    model.eval()
    with torch.no_grad():
        adapted = model(ids, return_logits=True).logits
    save_adapter(model, spec, str(tmp_path / "a"))
    sd = load_file(str(tmp_path / "a" / "adapter_model.safetensors"))
    assert sd["base_model.model.model.embed_tokens.token_adapter.trainable_tokens_delta"].shape == (3, cfg.hidden_size)
    fresh = CausalLM(cfg, dtype=torch.float32).init_weights(0)
    fresh.load_state_dict({k: v for k, v in model.state_dict().items() if k in fresh.state_dict()}, strict=False)
    with torch.no_grad():
        fresh.embed_tokens.copy_(before)
        fresh.lm_head.copy_(model.lm_head)
    inject_lora(fresh, spec)
    load_adapter(fresh, str(tmp_path / "a"))
    fresh.eval()
    with torch.no_grad():
        assert torch.allclose(fresh(ids, return_logits=True).logits, adapted, atol=1e-5)
        merge_and_unload(model)
        assert torch.allclose(model.embed_tokens[3], before[3] + 0.5, atol=1e-6)
        assert torch.equal(model.embed_tokens[5], before[5])
        assert torch.allclose(model(ids, return_logits=True).logits, adapted, atol=1e-4)


def test_muon_and_came_optimizers():
    import torch

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.train.optimizers_extra import CAME, Muon, newton_schulz_orthogonalize
    from axolotl_b200.train.run import train

    # Newton-Schulz drives the singular values towards 1 (it is an approximate polar factor)
    torch.manual_seed(0)
    G = torch.randn(48, 96)
    O = newton_schulz_orthogonalize(G, steps=8)
    sv = torch.linalg.svdvals(O)
    assert 0.6 < float(sv.min()) and float(sv.max()) < 1.3
    U, _, Vh = torch.linalg.svd(G, full_matrices=False)
    assert torch.nn.functional.cosine_similarity((U @ Vh).flatten(), O.flatten(), dim=0) > 0.98
    assert newton_schulz_orthogonalize(G.t().contiguous(), 5).shape == (96, 48)

    # both optimizers minimise a least-squares problem
    for make in (lambda ps: Muon(ps, lr=0.02, weight_decay=0.0), lambda ps: CAME(ps, lr=0.02)):
        torch.manual_seed(1)
        W = torch.nn.Parameter(torch.randn(16, 32) * 0.1)
        b = torch.nn.Parameter(torch.zeros(16))
        X, Y = torch.randn(256, 32), torch.randn(256, 16)
        opt = make([W, b])
        first = None
        for _ in range(60):
            loss = ((X @ W.t() + b - Y) ** 2).mean()
            first = first if first is not None else float(loss)
            opt.zero_grad()
            loss.backward()
            opt.step()
        assert float(loss) < 0.85 * first, (type(opt).__name__, first, float(loss))

    # through the run builder
    cfg = load_cfg({"model_preset": "tiny-llama", "sequence_len": 128, "micro_batch_size": 2, "gradient_accumulation_steps": 1,
                    "max_steps": 8, "learning_rate": 2e-3, "optimizer": "muon", "lr_scheduler": "constant", "logging_steps": 1,
                    "output_dir": "/tmp/axb_muon_test", "device": "cpu", "sample_packing": True, "save_strategy": "no",
                    "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 24, "min_length": 16,
                                  "max_length": 48, "max_input_id": 300}]})
    _, _, trainer = train(cfg)
    losses = [l["loss"] for l in trainer.log_history if "loss" in l]
    assert losses[-1] < losses[0]


def test_every_torch_optimizer_steps_through_the_run_builder(tmp_path):
    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.train.run import train

    for name in ("sgd", "lion_pytorch", "adopt_adamw", "sinkgd", "came_pytorch", "adafactor"):
        cfg = load_cfg({"model_preset": "tiny-llama", "sequence_len": 128, "micro_batch_size": 2, "gradient_accumulation_steps": 1,
                        "max_steps": 2, "learning_rate": 1e-3, "optimizer": name, "lr_scheduler": "constant", "logging_steps": 1,
                        "output_dir": str(tmp_path / name), "device": "cpu", "sample_packing": True, "save_strategy": "no",
                        "adapter": "lora", "lora_r": 8, "lora_alpha": 16, "lora_target_linear": True,
                        "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 8, "min_length": 16,
                                      "max_length": 48, "max_input_id": 300}]})
        _, _, trainer = train(cfg)
        assert trainer.global_step == 2, name


def test_densemixer_router_gradient_is_the_dense_mixture_gradient():
    import torch

    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM

    cfg = preset("tiny-qwen3-moe", vocab_size=97, num_hidden_layers=1)
    cfg.norm_topk_prob = False
    model = CausalLM(cfg, dtype=torch.float32).init_weights(0)
    moe = model.layers[0].mlp
    x = torch.randn(6, cfg.hidden_size)
    dy = torch.randn(6, cfg.hidden_size)
    model.train()

    def router_grad(dense):
        moe.dense_mixer = dense
        moe.gate.grad = None
        y, _ = moe(x)
        (y * dy).sum().backward()
        return moe.gate.grad.clone()

    g_sparse, g_dense = router_grad(False), router_grad(True)
    assert (g_sparse - g_dense).abs().max() > 1e-4
    # reference: dense mixture y = sum_e p_e O_e(x), gradient w.r.t. the router weight only
    gate = moe.gate.detach().clone().requires_grad_(True)
    probs = torch.softmax(x @ gate.t(), -1)
    with torch.no_grad():
        outs = []
        for e in range(moe.E):
            counts = [0] * moe.E
            counts[e] = 6
            outs.append(moe.experts(x, counts))
        O = torch.stack(outs, 1)                                  # [T, E, H]
    ((probs[:, :, None] * O).sum(1) * dy).sum().backward()
    assert torch.allclose(g_dense, gate.grad, atol=1e-4, rtol=1e-3), (g_dense - gate.grad).abs().max()
    moe.dense_mixer = False


def test_sharded_state_dict_roundtrip_through_the_merge_tool(tmp_path):
    """Row-sharded fused weights (as FSDP holds them) -> per-rank shard files under HF names -> merged checkpoint
    equal to the unsharded model's."""
    from types import SimpleNamespace

    from axolotl_b200.io import hf as hf_io
    from axolotl_b200.models.layers import FusedLinear

    world = 2
    ref = _tiny(2)
    want = {k: v.clone() for k, v in hf_io.hf_state_dict(ref).items()}
    for rank in range(world):
        m = _tiny(2)
        m.load_state_dict(ref.state_dict())
        for mod in m.modules():
            if isinstance(mod, FusedLinear) and mod.weight.shape[0] % world == 0:
                N, K = mod.weight.shape
                rows = N // world
                shard = torch.nn.Parameter(mod.weight.detach()[rank * rows:(rank + 1) * rows].clone(), requires_grad=False)
                shard._axb_shard = SimpleNamespace(rows=N, cols=K, world=world, rank=rank)
                mod.weight = shard
        d = hf_io.save_sharded_state(m, str(tmp_path / "out"), rank, world)
    idx = json.load(open(os.path.join(d, "shard_index.json")))
    assert idx["world_size"] == 2 and any(k.endswith("q_proj.weight") for k in idx["sharded"])
    part1 = st.load_file(os.path.join(d, "shard_rank1.safetensors"))
    assert any(v.shape[0] == 0 for v in part1.values())          # q_proj lies entirely in rank 0's rows
    assert "model.embed_tokens.weight" not in part1               # unsharded tensors live in rank 0's file only
    merge_sharded_fsdp_weights(d, str(tmp_path / "merged"), dtype=torch.float32)
    back = st.load_checkpoint(str(tmp_path / "merged")) if hasattr(st, "load_checkpoint") else st.load_file(str(tmp_path / "merged" / "model.safetensors"))
    assert set(back) == set(want)
    for k in want:
        assert torch.equal(back[k].float(), want[k].float()), k
