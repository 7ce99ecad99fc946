"""Remote-training plugin against a stand-in service client: wire format, loss normalisation, accumulation,
pipelining, remote checkpoints, the policy-gradient loop."""
import numpy as np
import pytest

from axolotl_b200.data.loading import TokenizedDataset, TrainDatasetMeta
from axolotl_b200.plugins import hatchery as H
from axolotl_b200.plugins.base import PluginManager


class _Future:
    def __init__(self, value, log, tag):
        self.value, self.log, self.tag = value, log, tag

    def result(self, timeout=None):
        self.log.append(("result", self.tag))
        return self.value


class _Sampler:
    sampling_session_id = "s1"

    def __init__(self, log):
        self.log = log

    def sample(self, ids, max_tokens, temperature, n):
        self.log.append(("sample", tuple(ids), n))
        seqs = [{"tokens": [7 + i, 8 + i, 9], "logprobs": [-0.1 * (i + 1), -0.2, -0.3]} for i in range(n)]
        return _Future({"sequences": seqs}, self.log, "sample")


class _Client:
    def __init__(self):
        self.log = []
        self.fb = []

    def forward_backward(self, datums, loss_fn, loss_fn_config=None):
        self.fb.append((datums, loss_fn))
        self.log.append(("fb", len(datums)))
        loss = sum(sum(d["loss_fn_inputs"].get("weights", {"data": [1.0]})["data"]) * 2.0 for d in datums)   # 2.0 per trained token
        return _Future({"metrics": {"loss:sum": loss}}, self.log, "fb")

    def optim_step(self, params):
        self.log.append(("optim", dict(params)))
        return _Future({}, self.log, "optim")

    def save_state(self, name):
        self.log.append(("save", name))
        return _Future({}, self.log, "save")

    def save_weights_and_get_sampling_client(self):
        return _Sampler(self.log)


@pytest.fixture
def client():
    c = _Client()
    H.set_client_factory(lambda hcfg, base: c)
    yield c
    H.set_client_factory(None)


def _rows():
    return [{"input_ids": [1, 5, 6, 7, 2], "labels": [-100, -100, 6, 7, 2]},
            {"input_ids": [1, 9, 2], "labels": [-100, 9, 2]},
            {"input_ids": [1, 4, 4, 2], "labels": [-100, 4, 4, 2]},
            {"input_ids": [1, 3, 2], "labels": [-100, -100, 2]}]


def test_supervised_datum_applies_the_causal_shift_on_the_client():
    d = H.row_to_datum_sft([1, 5, 6, 7, 2], [-100, -100, 6, 7, 2])
    assert d["model_input"]["chunks"][0]["tokens"] == [1, 5, 6, 7]
    assert d["loss_fn_inputs"]["target_tokens"]["data"] == [0, 6, 7, 2]
    assert d["loss_fn_inputs"]["weights"]["data"] == [0.0, 1.0, 1.0, 1.0]
    assert d["loss_fn_inputs"]["target_tokens"]["dtype"] == "int64" and d["loss_fn_inputs"]["weights"]["dtype"] == "float32"


def test_remote_supervised_loop_accumulates_normalises_and_checkpoints(client):
    cfg = {"base_model": "meta-llama/Llama-3.1-8B", "micro_batch_size": 1, "gradient_accumulation_steps": 2, "num_epochs": 1,
           "learning_rate": 3e-4, "max_grad_norm": 1.0, "hatchery": {"save_steps": 1, "pipeline": False}}
    tr = H.RemoteTrainer(cfg, H.HatcheryConfig(**cfg["hatchery"]), TokenizedDataset.from_rows(_rows()))
    out = tr.train()
    assert out["global_step"] == 2
    # the service returns the SUM over trained tokens (2.0 each here): the logged loss is per trained token
    assert [round(r["loss"], 6) for r in tr.history] == [2.0, 2.0]
    assert [r["active_tokens"] for r in tr.history] == [3 + 2, 3 + 1]
    kinds = [e[0] for e in client.log]
    assert kinds.count("fb") == 4 and kinds.count("optim") == 2
    assert [e[1] for e in client.log if e[0] == "save"] == ["checkpoint-000001", "checkpoint-000002", "final"]
    opt = [e[1] for e in client.log if e[0] == "optim"][0]
    assert opt["learning_rate"] == 3e-4 and opt["beta2"] == 0.95 and opt["grad_clip_norm"] == 1.0


def test_pipelined_loop_collects_the_optimizer_result_one_step_late(client):
    cfg = {"base_model": "m", "micro_batch_size": 2, "gradient_accumulation_steps": 1, "hatchery": {"pipeline": True}}
    H.RemoteTrainer(cfg, H.HatcheryConfig(pipeline=True), TokenizedDataset.from_rows(_rows())).train()
    order = [e for e in client.log if e[0] in ("optim", "fb") or e == ("result", "optim")]
    # step 1: fb, optim (not awaited); step 2: fb, THEN the first optimizer result, optim; the last one at the end
    assert [e[0] if e[0] != "result" else "await" for e in order] == ["fb", "optim", "fb", "await", "optim", "await"]


def test_policy_gradient_loop_samples_scores_and_sends_advantages(client, monkeypatch):
    import sys
    import types

    mod = types.ModuleType("hatchery_test_rewards")
    mod.length_reward = lambda prompts, completions: [float(len(c)) for c in completions]
    monkeypatch.setitem(sys.modules, "hatchery_test_rewards", mod)

    class Tok:
        def decode(self, ids, skip_special_tokens=False):
            return " ".join(str(int(i)) for i in ids)

        def encode(self, text, add_special_tokens=False):
            return [int(t) for t in text.split()]

    hcfg = H.HatcheryConfig(loss_fn="importance_sampling", num_samples=2, reward_funcs=["hatchery_test_rewards.length_reward"])
    cfg = {"base_model": "m", "micro_batch_size": 1, "max_steps": 1}
    tr = H.RemoteRLTrainer(cfg, hcfg, TokenizedDataset.from_rows(_rows()[:1]), Tok())
    out = tr.train()
    assert out["global_step"] == 1 and ("sample", (1, 5, 6, 7, 2), 2) in client.log
    assert len(client.fb) == 2 and all(loss == "importance_sampling" for _, loss in client.fb)
    d0, d1 = client.fb[0][0][0], client.fb[1][0][0]
    assert d0["model_input"]["chunks"][0]["tokens"] == [1, 5, 6, 7, 2, 7, 8]           # prompt + completion, last dropped
    assert d0["loss_fn_inputs"]["target_tokens"]["data"] == [0, 0, 0, 0, 7, 8, 9]
    np.testing.assert_allclose(d0["loss_fn_inputs"]["logprobs"]["data"], [0, 0, 0, 0, -0.1, -0.2, -0.3], atol=1e-6)
    # two samples, rewards len("7 8 9") = 5 and len("8 9 9") = 5 -> a constant group: zero advantages
    assert set(d0["loss_fn_inputs"]["advantages"]["data"]) == {0.0} and set(d1["loss_fn_inputs"]["advantages"]["data"]) == {0.0}
    assert H.group_advantages([1.0, 3.0, 2.0, 2.0], 2) == [-1.0, 1.0, 0.0, 0.0]


def test_plugin_takes_over_the_run_without_building_a_model(client, tmp_path, monkeypatch):
    from axolotl_b200.train import run as run_mod

    PluginManager.reset()
    pm = PluginManager.get_instance()
    pm.register("axolotl.integrations.hatchery.HatcheryPlugin")
    monkeypatch.setattr(run_mod, "build_model", lambda *a, **k: (_ for _ in ()).throw(AssertionError("no local model")))
    cfg = {"base_model": "some/remote-model", "output_dir": str(tmp_path / "out"), "micro_batch_size": 2,
           "gradient_accumulation_steps": 1, "num_epochs": 1, "device": "cpu", "hatchery": {"lora_rank": 8}}
    try:
        out = run_mod.train(cfg, TrainDatasetMeta(train=TokenizedDataset.from_rows(_rows())))
    finally:
        PluginManager.reset()
    assert out["global_step"] == 2 and len(out["history"]) == 2
    assert ("save", "final") in client.log
