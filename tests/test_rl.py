"""Preference / RL objectives on CPU: op numerics vs autograd, loss formulas vs hand-written
references, and short learning runs on synthetic preferences."""
import math

import pytest
import torch
import torch.nn.functional as F

from axolotl_b200.models.config import preset
from axolotl_b200.models.lora import LoraSpec, inject_lora
from axolotl_b200.models.transformer import CausalLM
from axolotl_b200.ops.functional import linear_token_logps
from axolotl_b200.rl import losses as L
from axolotl_b200.rl.data import KTOCollator, PairwiseCollator, synthetic_preference
from axolotl_b200.rl.logps import sequence_logps
from axolotl_b200.rl.objectives import add_score_head, build_objective, precompute_reference_logps
from axolotl_b200.rl.strategies import load_preference_transform
from axolotl_b200.train.optimizer import FlatAdamW, build_param_groups, make_lr_lambda
from axolotl_b200.train.trainer import TrainArgs, Trainer, to_device_batch


def test_token_logps_match_autograd():
    torch.manual_seed(0)
    T, H, V = 37, 32, 101
    h = torch.randn(T, H, requires_grad=True)
    w = torch.randn(V, H, requires_grad=True)
    lab = torch.randint(0, V, (T,))
    lab[::5] = -100
    g = torch.randn(T)
    lp = linear_token_logps(h, w, lab, chunk_rows=16)
    (lp * g).sum().backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    ref = torch.log_softmax(h2 @ w2.t(), -1).gather(1, lab.clamp(min=0)[:, None]).squeeze(1) * (lab != -100)
    (ref * g).sum().backward()
    assert torch.allclose(lp, ref, atol=1e-5)
    assert torch.allclose(h.grad, h2.grad, atol=1e-5)
    assert torch.allclose(w.grad, w2.grad, atol=1e-4)


def test_dpo_loss_variants_against_formulas():
    torch.manual_seed(1)
    pc, pr, rc, rr = (torch.randn(6) for _ in range(4))
    beta = 0.25
    x = (pc - rc) - (pr - rr)
    loss, m = L.dpo_loss(pc, pr, rc, rr, beta, "sigmoid")
    assert torch.allclose(loss, -F.logsigmoid(beta * x).mean())
    assert 0.0 <= float(m["rewards/accuracies"]) <= 1.0
    loss, _ = L.dpo_loss(pc, pr, rc, rr, beta, "ipo")
    assert torch.allclose(loss, ((x - 1 / (2 * beta)) ** 2).mean())
    loss, _ = L.dpo_loss(pc, pr, rc, rr, beta, "hinge")
    assert torch.allclose(loss, torch.relu(1 - beta * x).mean())
    ls = 0.1
    loss, _ = L.dpo_loss(pc, pr, rc, rr, beta, "sigmoid", ls)
    assert torch.allclose(loss, (-F.logsigmoid(beta * x) * (1 - ls) - F.logsigmoid(-beta * x) * ls).mean())
    for lt in L.DPO_LOSS_TYPES:
        l, _ = L.dpo_loss(pc, pr, rc, rr, beta, lt, 0.05)
        assert torch.isfinite(l)
    with pytest.raises(ValueError):
        L.dpo_loss(pc, pr, rc, rr, beta, "nope")


def test_orpo_simpo_kto_formulas():
    torch.manual_seed(2)
    ac, ar = -torch.rand(5) - 0.1, -torch.rand(5) - 0.1
    nll = -ac.mean()
    loss, m = L.orpo_loss(ac, ar, nll, beta=0.2)
    odds = lambda p: p - torch.log1p(-torch.exp(p))
    want = nll - 0.2 * F.logsigmoid(odds(ac) - odds(ar)).mean()
    assert torch.allclose(loss, want, atol=1e-6)
    loss, _ = L.cpo_loss(ac, ar, nll, beta=2.0, loss_type="simpo", cpo_alpha=0.0, simpo_gamma=1.0)
    assert torch.allclose(loss, -F.logsigmoid(2.0 * (ac - ar - 0.5)).mean(), atol=1e-6)
    pol, ref = torch.randn(6), torch.randn(6)
    des = torch.tensor([1, 0, 1, 0, 1, 1], dtype=torch.bool)
    kl = torch.tensor(0.3)
    loss, _ = L.kto_loss(pol, ref, des, kl, beta=0.1, desirable_weight=1.0, undesirable_weight=2.0)
    r = pol - ref
    want = torch.where(des, 1 - torch.sigmoid(0.1 * (r - kl)), 2.0 * (1 - torch.sigmoid(0.1 * (kl - r)))).mean()
    assert torch.allclose(loss, want, atol=1e-6)


def test_grpo_loss_on_policy_gradient_is_reinforce():
    torch.manual_seed(3)
    T, n_seq = 12, 3
    lp = (-torch.rand(T)).requires_grad_()
    sid = torch.tensor([0] * 4 + [1] * 4 + [2] * 4)
    mask = torch.tensor([0, 1, 1, 1] * 3, dtype=torch.bool)
    adv = torch.tensor([1.0, -0.5, 0.25])
    loss, m = L.grpo_loss(lp, None, None, adv, sid, n_seq, mask, loss_type="grpo")
    loss.backward()
    want = -(adv[sid] * mask.float()) / 3 / 3     # d/dlp of -ratio*A, mean over 3 tokens and 3 sequences
    assert torch.allclose(lp.grad, want, atol=1e-6)
    assert float(m["clip_ratio"]) == 0.0
    a = L.group_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0]), 2)
    assert torch.allclose(a[:2], torch.tensor([1.0, -1.0]) * (0.5 / (math.sqrt(0.5) + 1e-4)), atol=1e-5)
    assert torch.allclose(a[4:], torch.zeros(2))


def test_pairwise_collator_layout():
    recs = [{"prompt": [5, 6, 7], "chosen": [8, 9], "rejected": [10]},
            {"prompt": [11], "chosen": [12, 13, 14], "rejected": [15, 16]}]
    b = PairwiseCollator(pad_to_multiple_of=8)(recs)
    ids, lab, sid = b["input_ids"][0].tolist(), b["labels"][0].tolist(), b["aux_tensors"]["seq_ids"][0].tolist()
    assert ids[:5] == [5, 6, 7, 8, 9] and lab[:5] == [-100, -100, 8, 9, -100]
    assert ids[5:9] == [5, 6, 7, 10] and lab[5:9] == [-100, -100, 10, -100]
    assert sid[:9] == [0] * 5 + [1] * 4
    assert b["meta"]["n_seq"] == 4 and b["cu_seqlens"].tolist()[:5] == [0, 5, 9, 13, 16]
    assert b["n_trainable"] == 2 + 1 + 3 + 2
    assert len(ids) == 16
    b3 = PairwiseCollator(pad_to_multiple_of=8)(recs[:1])
    assert b3["input_ids"].shape[1] == 16 and b3["aux_tensors"]["seq_ids"][0, -1] == -1 and b3["cu_seqlens"].tolist() == [0, 5, 9, 16]
    k = KTOCollator(pad_to_multiple_of=8)([{"prompt": [1, 2], "completion": [3], "label": True},
                                          {"prompt": [4], "completion": [5, 6], "label": False}])
    assert k["meta"]["n_seq"] == 4 and k["aux_tensors"]["is_desirable"].tolist() == [True, False]
    assert k["input_ids"][0].tolist()[:11] == [1, 2, 3, 4, 5, 6, 1, 2, 5, 6, 4]


def test_strategy_transforms():
    f = load_preference_transform("chatml.intel", "dpo")
    o = f({"system": "S", "question": "Q", "chosen": "A", "rejected": "B"})
    assert o["prompt"] == "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nQ<|im_end|>\n<|im_start|>assistant\n"
    assert o["chosen"] == "A<|im_end|>" and o["rejected"] == "B<|im_end|>"
    f = load_preference_transform("llama3.ultra", "dpo")
    o = f({"prompt": "Q", "chosen": [{"content": "Q"}, {"content": "A"}], "rejected": [{"content": "Q"}, {"content": "B"}]})
    assert o["prompt"].endswith("<|start_header_id|>assistant<|end_header_id|>\n\n") and o["chosen"] == "A<|eot_id|>"
    f = load_preference_transform("chatml.argilla_chat", "dpo")
    o = f({"chosen": [{"content": "Q"}, {"content": "A"}], "rejected": [{"content": "Q"}, {"content": "B"}]})
    assert "user\nQ" in o["prompt"] and o["rejected"] == "B<|im_end|>"
    f = load_preference_transform("zephyr.nectar", "dpo")
    o = f({"prompt": "Q", "answers": [{"rank": 2, "answer": "x"}, {"rank": 1, "answer": "y"}, {"rank": 3, "answer": "z"}]})
    assert o["chosen"] == "z" and o["rejected"] == "x"
    f = load_preference_transform({"field_prompt": "q", "prompt_format": "[{system}] {prompt} ->",
                                   "field_chosen": "good", "field_rejected": "bad"}, "dpo")
    o = f({"q": "Q", "system": "S", "good": "A", "bad": "B"})
    assert o == {"prompt": "[S] Q ->", "chosen": "A", "rejected": "B"}
    f = load_preference_transform("chatml.argilla", "kto")
    o = f({"instruction": "Q", "completion": "A", "label": False})
    assert o["completion"] == "A<|im_end|>" and o["label"] is False


def _tiny(seed=0, lora=True):
    cfg = preset("tiny-llama", num_hidden_layers=2, vocab_size=256, hidden_size=64, intermediate_size=128,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(seed)
    if lora:
        inject_lora(model, LoraSpec(r=8, lora_alpha=16, target_modules="all-linear"))
    return model


def _train(model, cfg_d, recs, steps=30, lr=5e-3, mbs=8):
    obj = build_objective(cfg_d)
    coll = obj.collator()
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=lr, max_grad_norm=1.0)
    opt.bind_model_shadows(model)
    tr = Trainer(model, opt, make_lr_lambda("constant", 100, 0), TrainArgs(max_steps=steps, learning_rate=lr),
                 lambda e: [], device=torch.device("cpu"), compute_loss=obj)
    hist = []
    for s in range(steps):
        chunk = [recs[(s * mbs + j) % len(recs)] for j in range(mbs)]
        loss = float(tr.training_step([coll(chunk)]))
        hist.append((loss, dict(obj.last_metrics)))
    return hist


@pytest.mark.parametrize("rl", ["dpo", "ipo", "simpo", "orpo"])
def test_pairwise_objectives_learn(rl):
    model = _train_model = _tiny()
    recs = synthetic_preference(32, 6, 6, 256, seed=1)
    hist = _train(model, {"rl": rl, "rl_beta": 0.5 if rl != "simpo" else 2.0}, recs, steps=25)
    assert hist[-1][0] < hist[0][0]
    assert hist[-1][1]["rewards/accuracies"] >= 0.9
    if rl == "dpo":   # with B = 0 the policy equals the reference: loss starts at log 2
        assert abs(hist[0][0] - math.log(2)) < 1e-4


def test_dpo_precomputed_reference_matches_online():
    model = _tiny()
    recs = synthetic_preference(8, 5, 5, 256, seed=2)
    obj = build_objective({"rl": "dpo", "rl_beta": 0.3})
    coll = obj.collator()
    # make the policy differ from the reference
    with torch.no_grad():
        for _, m in model.fused_linears():
            m.lora_B.normal_(0, 0.05)
            mask = torch.zeros_like(m.lora_B)
            for (r0, rows, c0, r) in m.lora_blocks:
                mask[r0:r0 + rows, c0:c0 + r] = 1
            m.lora_B.mul_(mask)
    b = to_device_batch(coll(recs[:4]), torch.device("cpu"))
    l_online = float(obj(model, b, 1).detach())
    precompute_reference_logps(model, recs, coll, torch.device("cpu"), micro_batch_size=4)
    b2 = to_device_batch(coll(recs[:4]), torch.device("cpu"))
    assert "ref_logps" in b2
    assert abs(float(obj(model, b2, 1).detach()) - l_online) < 1e-5
    assert l_online != pytest.approx(math.log(2), abs=1e-3)


def test_sequence_logps_equal_unpacked():
    """Packing documents into one row must not change any document's log-prob."""
    model = _tiny(lora=False)
    recs = synthetic_preference(3, 7, 5, 256, seed=5)
    coll = PairwiseCollator(pad_to_multiple_of=8)
    b = to_device_batch(coll(recs), torch.device("cpu"))
    packed, counts, _ = sequence_logps(model, b)
    for i, r in enumerate(recs):
        for j, key in enumerate(("chosen", "rejected")):
            ids = torch.tensor([r["prompt"] + r[key]])
            logits = model(ids, return_logits=True).logits[0].float()
            lp = torch.log_softmax(logits[:-1], -1).gather(1, ids[0, 1:, None]).squeeze(1)
            want = lp[len(r["prompt"]) - 1:].sum()
            assert abs(float(packed[2 * i + j]) - float(want)) < 1e-3
            assert int(counts[2 * i + j]) == len(r[key])


def test_kto_learns():
    model = _tiny()
    recs = synthetic_preference(32, 6, 6, 256, kto=True, seed=3)
    hist = _train(model, {"rl": "kto", "rl_beta": 0.5}, recs, steps=25)
    assert hist[-1][0] < hist[0][0]
    assert hist[-1][1]["rewards/chosen"] > hist[-1][1]["rewards/rejected"]


def test_reward_model_learns():
    model = _tiny()
    add_score_head(model, 1)
    recs = synthetic_preference(32, 6, 6, 256, seed=4)
    hist = _train(model, {"reward_model": True}, recs, steps=30)
    assert hist[-1][0] < hist[0][0]
    assert hist[-1][1]["accuracy"] >= 0.9


def _reward_low_tokens(prompts, completions, completion_ids, **kw):
    return [sum(1.0 for t in c if t < 32) / max(len(c), 1) for c in completion_ids]


def test_grpo_improves_reward():
    from axolotl_b200.rl import grpo as G

    cfg = preset("tiny-llama", num_hidden_layers=2, vocab_size=64, hidden_size=64, intermediate_size=128,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(0)
    inject_lora(model, LoraSpec(r=8, lora_alpha=16, target_modules="all-linear"))
    st = G.GRPOSettings({"rl": "grpo", "trl": {"num_generations": 8, "max_completion_length": 6, "beta": 0.01,
                                               "loss_type": "grpo", "num_iterations": 1, "replay_buffer_size": 8}})
    recs = [{"prompt_ids": [3, 4, 5, 6 + i % 5]} for i in range(256)]
    prod = G.RolloutProducer(model, G.LocalRollout(model, seed=0), [_reward_low_tokens], st, recs, 4)
    obj = G.GRPOObjective(st, prod)
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=5e-2, max_grad_norm=1.0)
    opt.bind_model_shadows(model)
    tr = Trainer(model, opt, make_lr_lambda("constant", 100, 0), TrainArgs(max_steps=50, learning_rate=5e-2),
                 lambda e: [], device=torch.device("cpu"), compute_loss=obj)
    rewards = []
    it = prod(0)
    for _ in range(50):
        tr.training_step([next(it)])
        rewards.append(obj.last_metrics["reward"])
    assert sum(rewards[-8:]) / 8 > sum(rewards[:8]) / 8 + 0.05, rewards
    assert "kl" in obj.last_metrics and "clip_ratio" in obj.last_metrics


def test_grpo_async_prefetch_yields_same_shapes():
    from axolotl_b200.rl import grpo as G

    model = _tiny()
    st = G.GRPOSettings({"rl": "grpo", "trl": {"num_generations": 2, "max_completion_length": 3, "async_prefetch": 2}})
    recs = [{"prompt_ids": [3, 4, 5]} for _ in range(8)]
    prod = G.RolloutProducer(model, G.LocalRollout(model, seed=1), [_reward_low_tokens], st, recs, 2)
    batches = list(prod(0))
    assert len(batches) == 4
    for b in batches:
        assert b["meta"]["n_seq"] == 4 and b["aux_tensors"]["advantages"].shape == (4,)


def test_dpo_cli_run(tmp_path):
    """``rl: dpo`` through the run builder with a synthetic preference dataset."""
    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.train.run import train

    cfg = load_cfg({"model_preset": "tiny-llama", "rl": "dpo", "rl_beta": 0.5, "adapter": "lora", "lora_r": 8,
                    "lora_alpha": 16, "lora_target_linear": True, "sequence_len": 64, "micro_batch_size": 4,
                    "gradient_accumulation_steps": 2, "num_epochs": 1, "learning_rate": 5e-3, "optimizer": "adamw_torch",
                    "lr_scheduler": "constant", "output_dir": str(tmp_path / "out"), "device": "cpu", "logging_steps": 1,
                    "datasets": [{"path": "synthetic", "type": "_synthetic_pref", "length": 64, "prompt_len": 6,
                                  "completion_len": 6, "max_input_id": 500}]})
    model, _, trainer = train(cfg)
    logs = [l for l in trainer.log_history if "rewards/accuracies" in l]
    assert trainer.global_step == 8 and logs
    assert logs[-1]["loss"] < logs[0]["loss"]
    assert (tmp_path / "out" / "adapter_model.safetensors").exists()


def test_kd_plugin_loss_matches_definition_and_learns(tmp_path):
    import json

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.plugins.base import PluginManager
    from axolotl_b200.plugins.kd import KDCollator, KDObjective
    from axolotl_b200.train.run import train

    torch.manual_seed(0)
    model = _tiny(lora=False)
    V, K, n = 256, 4, 10
    rows = []
    g = torch.Generator().manual_seed(1)
    for i in range(24):
        ids = torch.randint(3, V, (n,), generator=g)
        top = torch.stack([ids.roll(-0)] + [torch.randint(3, V, (n,), generator=g) for _ in range(K - 1)], 1)
        lp = torch.log_softmax(torch.tensor([3.0] + [0.0] * (K - 1)).repeat(n, 1), -1)
        rows.append({"input_ids": ids.tolist(), "labels": ids.tolist(), "target_token_ids": top.tolist(),
                     "target_logprobs": lp.tolist()})
    coll = KDCollator(top_k=K, pad_to_multiple_of=8)
    b = to_device_batch(coll([rows[:2]]), torch.device("cpu"))
    obj = KDObjective({"kd_alpha": 1.0, "kd_ce_alpha": 0.0, "kd_temperature": 1.0})
    loss = obj(model, b, 1)
    # definition: forward KL over the teacher's top-k tokens at every supervised position
    logits = model(b["input_ids"], b["position_ids"], attn_meta=b["attn_meta"], return_logits=True).logits[0].float()
    slp = torch.log_softmax(logits, -1).gather(1, b["target_token_ids"][0])
    m = b["target_mask"][0]
    want = (b["target_logprobs"][0].exp() * (b["target_logprobs"][0] - slp) * m).sum() / (m.sum(1) > 0).sum()
    assert abs(float(loss.detach()) - float(want)) < 1e-4
    loss.backward()   # gradients flow through the hand-written chunk backward
    assert model.embed_tokens.grad is not None or getattr(model.embed_tokens, "_axb_grad", None) is not None

    data = tmp_path / "kd.jsonl"
    with open(data, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")
    PluginManager.reset()
    cfg = load_cfg({"model_preset": "tiny-llama", "plugins": ["kd"], "kd_trainer": True, "kd_alpha": 0.9, "kd_ce_alpha": 0.1,
                    "adapter": "lora", "lora_r": 8, "lora_alpha": 16, "lora_target_linear": True, "sequence_len": 64,
                    "micro_batch_size": 4, "gradient_accumulation_steps": 1, "num_epochs": 3, "learning_rate": 1e-2,
                    "optimizer": "adamw_torch", "lr_scheduler": "constant", "output_dir": str(tmp_path / "o"), "device": "cpu",
                    "logging_steps": 1, "datasets": [{"path": str(data), "ds_type": "json"}]})
    _, _, trainer = train(cfg)
    PluginManager.reset()
    logs = [l for l in trainer.log_history if "kd_loss" in l]
    assert logs and logs[-1]["kd_loss"] < logs[0]["kd_loss"]


def test_diffusion_plugin_noising_loss_and_generation(tmp_path):
    import torch

    from axolotl_b200.config.load import load_cfg
    from axolotl_b200.ops import functional as Fn
    from axolotl_b200.plugins.base import PluginManager
    from axolotl_b200.plugins.diffusion import forward_process, generate
    from axolotl_b200.train.run import train

    # noising: only trainable, non-first, non-special tokens are masked; rate follows each document's t
    cu = torch.tensor([0, 400, 1000], dtype=torch.int32)
    ids = torch.randint(5, 200, (1, 1000))
    lab = ids.clone()
    lab[0, :100] = -100
    g = torch.Generator().manual_seed(1)
    noisy, masked, p_tok, doc = forward_process(ids, lab, cu, 299, 1e-3, special_ids=(7,), generator=g)
    assert not masked[:100].any() and not masked[400] and not (masked & (ids.reshape(-1) == 7)).any()
    assert bool((noisy.reshape(-1)[masked] == 299).all()) and bool((noisy.reshape(-1)[~masked] == ids.reshape(-1)[~masked]).all())
    for d, (s, e) in enumerate(((100, 400), (401, 1000))):
        rate = masked[s:e].float().mean().item()
        assert abs(rate - float(p_tok[s])) < 0.12, (d, rate, float(p_tok[s]))

    PluginManager.reset()
    cfg = load_cfg({"model_preset": "tiny-llama", "plugins": ["axolotl.integrations.diffusion.DiffusionPlugin"],
                    "diffusion": {"mask_token_id": 511, "generate_samples": False}, "sequence_len": 128,
                    "micro_batch_size": 2, "gradient_accumulation_steps": 1, "max_steps": 30, "learning_rate": 3e-3,
                    "optimizer": "adamw_torch", "lr_scheduler": "constant", "logging_steps": 1, "save_strategy": "no",
                    "output_dir": str(tmp_path / "d"), "device": "cpu", "sample_packing": True,
                    "num_epochs": 8, "datasets": [{"path": "synthetic", "type": "_synthetic", "length": 40, "min_length": 24,
                                  "max_length": 48, "max_input_id": 300}]})
    model, _, trainer = train(cfg)
    PluginManager.reset()
    logs = [l for l in trainer.log_history if "ce_loss" in l]
    assert logs and "mask_ratio" in logs[0]
    first, last = sum(l["ce_loss"] for l in logs[:5]) / 5, sum(l["ce_loss"] for l in logs[-5:]) / 5
    assert last < first, (first, last)
    out = generate(model, torch.tensor([1, 5, 9, 12]), 12, 511, steps=4)
    assert out.shape == (16,) and not bool((out == 511).any()) and out[:4].tolist() == [1, 5, 9, 12]


def test_ebft_feature_rewards_and_training_raises_alignment():
    from axolotl_b200.rl import grpo as G
    from axolotl_b200.rl.ebft import FeatureMatchingReward, feature_rewards, pool_features

    # reward arithmetic against the definition
    torch.manual_seed(0)
    gen, gt = torch.randn(6, 16), torch.randn(2, 16)
    r, m = feature_rewards(gen, gt, 3, alignment_coef=1.0, diversity_coef=0.5)
    gn, tn = torch.nn.functional.normalize(gen, dim=-1), torch.nn.functional.normalize(gt, dim=-1)
    want0 = 2 * (gn[0] @ tn[0]) - 0.5 * 2 * ((gn[0] @ gn[1]) + (gn[0] @ gn[2])) / 2
    assert abs(float(r[0]) - float(want0)) < 1e-5 and set(m) >= {"ebft/alignment", "ebft/diversity", "ebft/cfm_loss"}
    rw, _ = feature_rewards(gen, gt, 3, use_whitening=True)
    assert rw.shape == (6,) and torch.isfinite(rw).all()
    h = torch.arange(40, dtype=torch.float32).reshape(10, 4)
    assert torch.equal(pool_features(h, "last_token", 3), h[-1])
    assert torch.allclose(pool_features(h, "completion_mean", 6), h[6:].mean(0))
    assert pool_features(h, "concat", 0).shape == (12,) and torch.equal(pool_features(h, "concat", 0)[:4], h[2])

    # the hidden states captured for the reward follow the HF numbering
    cfg = preset("tiny-llama", num_hidden_layers=4, vocab_size=64, hidden_size=64, intermediate_size=128,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu").init_weights(0)
    ids = torch.randint(3, 60, (1, 12))
    out = model(ids, return_logits=False, capture_hidden=[0, 2, 4])
    assert set(out.captured) == {0, 2, 4} and torch.equal(out.captured[4].reshape(-1), out.hidden_states.reshape(-1))
    two = CausalLM(preset("tiny-llama", num_hidden_layers=2, vocab_size=64, hidden_size=64, intermediate_size=128,
                          num_attention_heads=4, num_key_value_heads=2, head_dim=16), dtype=torch.float32, device="cpu")
    two.load_state_dict({k: v for k, v in model.state_dict().items() if k in two.state_dict()}, strict=False)
    h2 = two(ids, return_logits=False, capture_hidden=[2]).captured[2]      # after the final norm of the 2-layer model
    mid = out.captured[2]
    normed = mid * torch.rsqrt(mid.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * two.norm.weight
    assert torch.allclose(h2.reshape(-1, 64), normed.reshape(-1, 64), atol=1e-4)

    # GRPO with the feature reward: completions drift towards the ground truth's features
    inject_lora(model, LoraSpec(r=8, lora_alpha=16, target_modules="all-linear"))
    st = G.GRPOSettings({"rl": "ebft", "trl": {"num_generations": 6, "max_completion_length": 5, "loss_type": "grpo"}})
    recs = [{"prompt_ids": [3, 4, 5, 6 + i % 4], "ground_truth": [9, 9, 9, 9, 9]} for i in range(256)]
    rf = FeatureMatchingReward(model, None, {"feature_layers": [0.5, 1.0], "embed_method": "completion_mean",
                                             "diversity_coef": 0.0}, st.num_generations)
    prod = G.RolloutProducer(model, G.LocalRollout(model, seed=0), [rf], st, recs, 4)
    obj = G.GRPOObjective(st, prod)
    opt = FlatAdamW(build_param_groups(model.named_parameters()), lr=3e-2, max_grad_norm=1.0)
    opt.bind_model_shadows(model)
    tr = Trainer(model, opt, make_lr_lambda("constant", 100, 0), TrainArgs(max_steps=40, learning_rate=3e-2),
                 lambda e: [], device=torch.device("cpu"), compute_loss=obj)
    align = []
    it = prod(0)
    for _ in range(40):
        tr.training_step([next(it)])
        align.append(obj.last_metrics["ebft/alignment"])
    assert sum(align[-8:]) / 8 > sum(align[:8]) / 8 + 0.02, align


def test_ebft_strided_records_and_rloo_baseline():
    from axolotl_b200.rl.ebft import strided_records

    recs = strided_records([list(range(100, 130))], stride=8, context_length=6, generate_max_len=4, bos_token_id=1)
    assert [r["prompt_ids"][1:] for r in recs[:2]] == [list(range(100, 106)), list(range(108, 114))]
    assert all(r["prompt_ids"][0] == 1 and len(r["ground_truth"]) == 4 for r in recs)
    assert recs[0]["ground_truth"] == [106, 107, 108, 109] and recs[-1]["ground_truth"][-1] <= 129
    r = torch.tensor([1.0, 2.0, 6.0, 0.0, 0.0, 3.0])
    a = L.group_advantages(r, 3, "rloo")
    assert torch.allclose(a, torch.tensor([1 - 4.0, 2 - 3.5, 6 - 1.5, 0 - 1.5, 0 - 1.5, 3 - 0.0]))


def test_nemo_gym_verify_rewards_against_a_fake_environment_server():
    import json
    import http.server
    import threading

    from axolotl_b200.plugins import nemo_gym as NG

    seen = []

    class Env(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            seen.append(body)
            answer = body["response"]["output"][0]["content"][0]["text"]
            reward = 1.0 if answer.strip() == str(body.get("expected")) else 0.25
            data = json.dumps({"reward": reward}).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    env = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Env)
    env_port = env.server_address[1]

    class Head(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            doc = f"math_env:\n  resources_servers:\n    math:\n      host: 127.0.0.1\n      port: {env_port}\n"
            data = doc.encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    head = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Head)
    for srv in (env, head):
        threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        plug = NG.NemoGymPlugin()
        plug.register({"nemo_gym_enabled": True, "nemo_gym_head_port": head.server_address[1], "nemo_gym_verify_timeout": 5})
        assert NG.discover_verify_urls(refresh=True) == {"math": f"http://127.0.0.1:{env_port}/verify"}
        r = NG.reward_nemo_gym_verify(completions=["4", "5", "x"], prompts=["2+2?", "2+2?", "?"],
                                      resources_server_ref=[{"name": "math"}, {"name": "math"}, {"name": "unknown"}],
                                      verify_extra=[{"expected": 4}, {"expected": 4}, None])
        assert r == [1.0, 0.25, 0.0]
        assert seen[0]["responses_create_params"]["input"][0]["content"] == "2+2?" and seen[0]["expected"] == 4
        assert NG.reward_env(["a", "b"], env_reward=[0.5, 2]) == [0.5, 2.0]
        with pytest.raises(ValueError):      # the agents need a served policy to sample from
            plug.register({"nemo_gym_enabled": True, "nemo_gym_multi_turn": True})
    finally:
        env.shutdown()
        head.shutdown()
        NG._STATE["urls"] = None


def test_nemo_gym_multi_turn_agent_rollouts_feed_grpo_with_masked_tool_tokens():
    """Agents run the episodes: turns are stitched into one completion, tokens the environment inserted between turns
    stay in the context without being targets, the episode reward drives the advantages."""
    import http.server
    import json
    import threading

    from axolotl_b200.plugins import nemo_gym as NG
    from axolotl_b200.rl import grpo as G

    calls = []

    class Agent(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            calls.append(body)
            k = len(calls)
            prompt = [11, 12, 13]
            turn1 = {"type": "function_call", "prompt_token_ids": prompt, "generation_token_ids": [21, 22],
                     "generation_log_probs": [-0.5, -0.25]}
            # second turn: the context grew by the first generation AND two tool-result tokens (91, 92)
            turn2 = {"type": "message", "content": [{"type": "output_text", "text": "done"}],
                     "prompt_token_ids": prompt + [21, 22, 91, 92], "generation_token_ids": [31, 2],
                     "generation_log_probs": [-0.125]}
            data = json.dumps({"response": {"output": [turn1, turn2]}, "reward": float(k % 2)}).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    agent = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Agent)

    class Head(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            doc = (f"tool_env:\n  responses_api_agents:\n    simple_agent:\n      host: 127.0.0.1\n"
                   f"      port: {agent.server_address[1]}\n").encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(doc)))
            self.end_headers()
            self.wfile.write(doc)

    head = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Head)
    for srv in (agent, head):
        threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        plug = NG.NemoGymPlugin()
        cfg = {"nemo_gym_enabled": True, "nemo_gym_multi_turn": True, "nemo_gym_head_port": head.server_address[1],
               "trl": {"use_vllm": True}, "eos_token_id": 2, "nemo_gym_run_timeout": 5}
        plug.register(cfg)
        assert NG.discover_agent_servers() == {"tool_env": f"http://127.0.0.1:{agent.server_address[1]}"}

        class Inner:
            synced = []

            def sync_weights(self, model, step):
                self.synced.append(step)

        engine = plug.wrap_rollout_engine(cfg, Inner())
        engine.sync_weights(None, 3)
        assert Inner.synced == [3]
        one = NG.parse_agent_response({"response": {"output": []}, "reward": 0.7}, 2)
        assert one["env_mask"] == [0] and one["reward"] == 0.7          # an empty episode keeps its reward, trains nothing

        st = G.GRPOSettings({"trl": {"num_generations": 2, "max_completion_length": 16}})
        recs = [{"prompt": "use the tool", "prompt_ids": [5, 6], "agent_ref": {"name": "tool_env"},
                 "verify_extra": {"responses_create_params": {"input": [{"role": "user", "content": "use the tool"}]}, "expected": 4}}]
        prod = G.RolloutProducer(None, engine, [], st, recs, 1, None, 0, 2)
        b = prod.make_batch(recs)
        assert len(calls) == 2 and calls[0]["expected"] == 4 and calls[0]["agent_ref"] == {"name": "tool_env"}
        assert calls[0]["responses_create_params"]["max_output_tokens"] == 16
        ids, lab = b["input_ids"][0].tolist(), b["labels"][0].tolist()
        doc = [11, 12, 13, 21, 22, 91, 92, 31, 2]                        # the agent's own prompt ids, stitched turns
        assert ids[:9] == doc and ids[9:18] == doc
        # shifted targets: policy tokens 21 22 | tool tokens masked | 31 2
        assert lab[:9] == [-100, -100, 21, 22, -100, -100, 31, 2, -100]
        adv = b["aux_tensors"]["advantages"].tolist()
        assert adv[0] == -adv[1] and adv[0] != 0                           # rewards 1.0 and 0.0 inside the group
        assert prod.stats["num_turns"] == 2.0
    finally:
        agent.shutdown()
        head.shutdown()
        NG._STATE["urls"] = None
