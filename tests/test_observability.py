"""Telemetry (opt-out, redaction, local sink), optional reporters behind fake modules, CLI helper commands."""
import json
import os
import sys
import types

import pytest


def test_telemetry_redaction_and_opt_out(tmp_path, monkeypatch):
    from axolotl_b200.utils import telemetry as T

    assert T.redact_value("meta-llama/Llama-3-8B") == "meta-llama/Llama-3-8B"
    assert T.redact_value("secret-lab/internal-model") == "<redacted>/internal-model"
    assert T.redact_value("/home/alice/models/m1") == "<path>/m1"
    cfg = {"base_model": "secret-lab/m", "output_dir": "/data/alice/out", "hf_token": "abc", "learning_rate": 1e-4,
           "datasets": [{"path": "/data/alice/d.jsonl", "type": "alpaca"}], "wandb_api_key": "k"}
    clean = T.sanitize_config(cfg)
    assert clean["base_model"] == "<redacted>/m" and clean["output_dir"] == "<path>/out" and clean["hf_token"] == "<redacted>"
    assert clean["datasets"][0]["path"] == "<path>/d.jsonl" and clean["learning_rate"] == 1e-4 and clean["wandb_api_key"] == "<redacted>"
    trace = 'File "/home/alice/proj/train.py", line 3\n  File "/x/site-packages/torch/nn/modules/module.py", line 9'
    out = T.sanitize_stack_trace(trace)
    assert "alice" not in out and 'File "<user>/train.py"' in out and 'File "torch/nn/modules/module.py"' in out
    monkeypatch.delenv("AXOLOTL_DO_NOT_TRACK", raising=False)
    monkeypatch.delenv("DO_NOT_TRACK", raising=False)
    monkeypatch.delenv("AXOLOTL_TELEMETRY_URL", raising=False)
    monkeypatch.setenv("RANK", "0")
    t = T.Telemetry(str(tmp_path))
    assert t.enabled
    t.send("train-start", {"config": clean})
    try:
        raise ValueError("boom")
    except ValueError as exc:
        t.send_error(exc)
    t.flush()
    rows = [json.loads(l) for l in open(tmp_path / "telemetry.jsonl")]
    assert [r["event"] for r in rows] == ["train-start", "error"] and rows[1]["properties"]["type"] == "ValueError"
    assert all(r["run_id"] == t.run_id for r in rows) and "python" in rows[0]["system"]
    monkeypatch.setenv("AXOLOTL_DO_NOT_TRACK", "1")
    off = T.Telemetry(str(tmp_path / "off"))
    off.send("x")
    off.flush()
    assert not off.enabled and not os.path.exists(tmp_path / "off")
    monkeypatch.delenv("AXOLOTL_DO_NOT_TRACK")
    monkeypatch.setenv("RANK", "1")
    assert not T.Telemetry(str(tmp_path)).enabled       # only rank 0 reports


class _Trainer:
    rank, global_step, world_size = 0, 3, 1
    tokens = {"total": 10, "trainable": 5}


def test_comet_and_trackio_reporters_with_stand_in_modules(monkeypatch):
    calls = []
    comet = types.ModuleType("comet_ml")

    class Exp:
        def log_parameters(self, p): calls.append(("params", sorted(p)[:1]))
        def log_metrics(self, m, step=None): calls.append(("comet", m, step))
        def end(self): calls.append(("end",))

    comet.start = lambda **kw: (calls.append(("start", kw)), Exp())[1]
    trackio = types.ModuleType("trackio")
    trackio.init = lambda **kw: calls.append(("tinit", kw["project"]))
    trackio.log = lambda m: calls.append(("tlog", m))
    trackio.finish = lambda: calls.append(("tfinish",))
    monkeypatch.setitem(sys.modules, "comet_ml", comet)
    monkeypatch.setitem(sys.modules, "trackio", trackio)
    from axolotl_b200.train.callbacks import build_callbacks

    cbs = build_callbacks({"output_dir": "/tmp/x", "use_comet": True, "comet_project_name": "p", "comet_workspace": "w",
                           "trackio_project_name": "tp"})
    names = [type(c).__name__ for c in cbs]
    assert "CometReporter" in names and "TrackioReporter" in names and "TelemetryCallback" in names
    for c in cbs:
        if type(c).__name__ in ("CometReporter", "TrackioReporter"):
            c.on_log(_Trainer(), {"step": 3, "loss": 1.5, "note": "x"})
            c.on_train_end(_Trainer())
    assert ("start", {"workspace": "w", "project_name": "p"}) in calls
    assert ("comet", {"step": 3, "loss": 1.5}, 3) in calls and ("tlog", {"step": 3, "loss": 1.5}) in calls
    assert ("end",) in calls and ("tfinish",) in calls and ("tinit", "tp") in calls


def test_cli_helper_commands(tmp_path):
    from click.testing import CliRunner

    from axolotl_b200.cli.main import cli

    r = CliRunner()
    out = r.invoke(cli, ["agent-docs", "--list"])
    assert out.exit_code == 0 and "overview" in out.output and "grpo" in out.output
    out = r.invoke(cli, ["agent-docs", "sft"])
    assert out.exit_code == 0 and "roles_to_train" in out.output
    assert r.invoke(cli, ["agent-docs", "nope"]).exit_code != 0
    out = r.invoke(cli, ["config-schema", "--field", "ADAPTER", "--format", "yaml"])
    assert out.exit_code == 0 and "adapter" in out.output
    assert r.invoke(cli, ["config-schema", "--field", "not_a_field"]).exit_code != 0
    f = tmp_path / "opts.json"
    assert r.invoke(cli, ["generate-cli-config-options", "--output", str(f)]).exit_code == 0
    opts = json.load(open(f))
    assert opts["learning_rate"]["option"] == "--learning-rate" and opts["sample_packing"]["type"] == "bool"
    assert r.invoke(cli, ["generate-cli-config-options", "--output", str(f), "--check"]).exit_code == 0
    f.write_text("{}")
    assert r.invoke(cli, ["generate-cli-config-options", "--output", str(f), "--check"]).exit_code != 0
    assert "Llama-4" in r.invoke(cli, ["delinearize-llama4", "a", "b"]).output
