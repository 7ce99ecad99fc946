import json
import os

import pytest
import yaml
from click.testing import CliRunner

from axolotl_b200.cli.main import _extra_to_overrides, cli
from axolotl_b200.cli.sweeps import generate_sweep_configs
from axolotl_b200.parallel.mesh import MeshSpec


def test_mesh_axis_order_and_groups():
    m = MeshSpec.from_cfg(8, tensor_parallel_size=2, dp_shard_size=None)
    assert m.shape == (1, 1, 4, 1, 2) and m.data_parallel_size == 4
    assert m.coords(5) == {"ep": 0, "dp_replicate": 0, "dp_shard": 2, "cp": 0, "tp": 1}
    assert m.group_ranks(5, "tp") == [4, 5] and m.group_ranks(5, "dp_shard") == [1, 3, 5, 7]
    assert m.all_groups("tp") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    m2 = MeshSpec.from_cfg(8, context_parallel_size=2, dp_replicate_size=2)
    assert m2.shape == (1, 2, 2, 2, 1) and m2.group_ranks(0, ("dp_shard", "cp")) == [0, 1, 2, 3]
    m3 = MeshSpec.from_cfg(8, expert_parallel_size=8)
    assert m3.data_parallel_size == 8 and m3.dp_shard == 1
    with pytest.raises(ValueError):
        MeshSpec.from_cfg(8, tensor_parallel_size=3)
    with pytest.raises(ValueError):
        MeshSpec.from_cfg(8, tensor_parallel_size=2, dp_shard_size=8)


def test_cli_flag_parsing():
    ov = _extra_to_overrides(["--lora_r", "16", "--bf16", "--no-sample_packing", "--learning-rate=1e-4",
                              "--fsdp_config__reshard_after_forward", "false"])
    assert ov == {"lora_r": "16", "bf16": True, "sample_packing": False, "learning_rate": "1e-4",
                  "fsdp_config__reshard_after_forward": "false"}


def test_sweep_expansion():
    out = generate_sweep_configs({"a": 1, "lr": 0}, {"lr": [1, 2], "r": [8, 16], "_": [{"x": 1, "y": 2}, {"x": 3, "y": 4}]})
    assert len(out) == 8 and {(c["lr"], c["r"], c["x"]) for c in out} == {(l, r, x) for l in (1, 2) for r in (8, 16) for x in (1, 3)}


def test_cli_preprocess_train_merge_roundtrip(tmp_path):
    cfg = {"model_preset": "tiny-llama", "overrides_of_model_config": {"vocab_size": 512, "num_hidden_layers": 1},
           "reinit_weights": True, "float32": True, "bf16": False, "device": "cpu", "adapter": "lora", "lora_r": 4,
           "lora_alpha": 8, "lora_target_linear": True,
           "datasets": [{"type": "_synthetic", "length": 40, "min_length": 30, "max_length": 100, "min_input_id": 3,
                         "max_input_id": 512, "mask_prefix_fraction": 0.2, "seed": 0}],
           "sequence_len": 256, "sample_packing": True, "multipack_real_batches": True, "micro_batch_size": 2,
           "gradient_accumulation_steps": 1, "learning_rate": 1e-3, "max_steps": 3, "save_steps": 2, "seed": 0,
           "val_set_size": 0.1, "eval_steps": 2,
           "output_dir": str(tmp_path / "out"), "dataset_prepared_path": str(tmp_path / "prep")}
    p = tmp_path / "c.yaml"
    p.write_text(yaml.safe_dump(cfg))
    r = CliRunner()
    res = r.invoke(cli, ["preprocess", str(p)])
    assert res.exit_code == 0, res.output
    assert "prepared 36 training samples" in res.output  # 10% validation split
    res = r.invoke(cli, ["train", str(p), "--launcher", "python", "--logging_steps", "1"])
    assert res.exit_code == 0, res.output + str(res.exception)
    out = tmp_path / "out"
    for f in ("adapter_model.safetensors", "adapter_config.json", "config.json", "README.md", "train_log.jsonl", "checkpoint-2"):
        assert os.path.exists(out / f), f
    logs = [json.loads(l) for l in open(out / "train_log.jsonl")]
    assert [l["step"] for l in logs if "loss" in l] == [1, 2, 3] and any("eval_loss" in l for l in logs)
    res = r.invoke(cli, ["evaluate", str(p), "--lora_model_dir", str(out)])
    assert res.exit_code == 0 and "eval_loss" in res.output
    res = r.invoke(cli, ["config-schema"])
    assert res.exit_code == 0 and "lora_target_linear" in res.output
    res = r.invoke(cli, ["merge-lora", str(p)])
    assert res.exit_code != 0 and "local HF checkpoint" in res.output
    res = r.invoke(cli, ["vllm-serve", str(p)])
    assert res.exit_code != 0


def test_chat_session_commands_and_turns(tmp_path):
    import torch

    from axolotl_b200.cli.chat import ChatSession
    from axolotl_b200.models.config import preset
    from axolotl_b200.models.transformer import CausalLM

    class Tok:
        eos_token_id = 2
        chat_template = None

        def __call__(self, text):
            return {"input_ids": [3 + (ord(c) % 40) for c in text][-48:]}

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(i) for i in ids)

    model = CausalLM(preset("tiny-llama", num_hidden_layers=1, vocab_size=64), dtype=torch.float32, device="cpu").init_weights(0)
    s = ChatSession(model, Tok(), max_new_tokens=4, temperature=0.0)
    assert s.command("hello") is None
    assert "set" in s.command("/system be brief") and s.system == "be brief"
    r1 = s.say("hi")
    assert isinstance(r1, str) and len(s.history) == 2 and s.history[1]["role"] == "assistant"
    assert s.say("hi again") and len(s.history) == 4
    s.command("/undo")
    assert len(s.history) == 2
    s.command(f"/save {tmp_path / 'c.json'}")
    import json
    assert json.load(open(tmp_path / "c.json"))[0]["role"] == "system"
    assert s.command("/max 7") and s.max_new_tokens == 7
    s.command("/reset")
    assert s.history == []
