"""The reference arm of bench.py, driven against a stand-in ``axolotl`` package: the harness must
write a loadable config / dataset / model directory, call ``axolotl.cli.train.do_cli``, get its timing
callback registered through the plugin list and print a well-formed bench line."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAKE_TRAIN = '''
import importlib, json, yaml
from types import SimpleNamespace


def do_cli(config, **kw):
    cfg = yaml.safe_load(open(config))
    assert cfg["adapter"] == "lora" and cfg["lora_r"] == 16 and cfg["lora_alpha"] == 32 and cfg["lora_target_linear"]
    assert cfg["sample_packing"] and cfg["reinit_weights"] and cfg["micro_batch_size"] == 1
    arch = json.load(open(cfg["base_model"] + "/config.json"))
    assert arch["num_hidden_layers"] >= 1
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(cfg["base_model"])
    assert tok.pad_token == "<pad>"
    rows = [json.loads(l) for l in open(cfg["datasets"][0]["path"])]
    assert all(set(r) == {"input_ids", "attention_mask", "labels"} for r in rows)
    assert min(len(r["input_ids"]) for r in rows) >= 256 and max(len(r["input_ids"]) for r in rows) <= 4096
    assert sum(len(r["input_ids"]) for r in rows) >= cfg["max_steps"] * cfg["sequence_len"]
    callbacks = []
    for name in cfg["plugins"]:
        mod, cls = name.rsplit(".", 1)
        callbacks += getattr(importlib.import_module(mod), cls)().add_callbacks_post_trainer(cfg, None)
    state, control = SimpleNamespace(global_step=0), SimpleNamespace(should_training_stop=False)
    for step in range(cfg["max_steps"]):
        state.global_step = step + 1
        for cb in callbacks:
            cb.on_log(None, state, control, logs={"loss": 10.0 - step})
            cb.on_step_end(None, state, control)
        if control.should_training_stop:
            break
    print("fake reference trained", state.global_step, "steps")
'''


def _fake_reference(tmp_path):
    pkg = tmp_path / "fake_ref" / "axolotl"
    (pkg / "cli").mkdir(parents=True)
    (pkg / "integrations").mkdir()
    (pkg / "__init__.py").write_text("")
    (pkg / "cli" / "__init__.py").write_text("")
    (pkg / "cli" / "train.py").write_text(FAKE_TRAIN)
    (pkg / "integrations" / "__init__.py").write_text("")
    (pkg / "integrations" / "base.py").write_text("class BasePlugin:\n    pass\n")
    return str(tmp_path / "fake_ref")


def test_reference_harness_against_a_stand_in_package(tmp_path):
    fake = _fake_reference(tmp_path)
    script = tmp_path / "drive.py"
    script.write_text(textwrap.dedent(f"""
        import json, sys
        sys.path.insert(0, {os.path.join(ROOT, 'baseline')!r})
        import ref_harness
        arch = dict(ref_harness.LLAMA3_8B, num_hidden_layers=2, hidden_size=64, vocab_size=512)
        res = ref_harness.run_reference(1, 3, 2, ref_path={fake!r}, required=(), arch=arch, seq_len=8192,
                                        work_dir={str(tmp_path / 'work')!r})
        assert "axolotl_b200" not in sys.modules
        print("LINE " + json.dumps(res))
    """))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    res = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("LINE ")][0][5:])
    assert line["impl"] == "reference" and "unavailable" not in line
    assert line["steps"] == 3 and line["warmup"] == 2 and line["n_gpus"] == 1
    assert line["metric"].startswith("train tokens/s/box") and line["unit"] == "tokens/s"
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["e2e"]["value"] > 0
    assert line["config"]["seq_len"] == 8192 and line["config"]["lora_r"] == 16
    assert line["e2e"]["last_loss"] == 10.0 - 4      # the loss logged at the last timed step


def test_reference_arm_reports_missing_dependencies():
    """On a box without peft / accelerate / trl the arm answers `unavailable` with the module list."""
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, timeout=300, env=env)
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import ref_harness

    if ref_harness.missing_modules() or not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "axolotl")):
        assert "unavailable" in line
