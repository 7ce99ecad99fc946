"""Ray and cloud launchers against stand-in SDK modules (neither `ray` nor `modal` is needed to test the wiring)."""
import sys
import types

import pytest

from axolotl_b200.cli import launchers


def _fake_ray(calls):
    ray = types.ModuleType("ray")
    train = types.ModuleType("ray.train")
    torch_mod = types.ModuleType("ray.train.torch")

    class ScalingConfig:
        def __init__(self, **kw):
            self.kw = kw

    class RunConfig:
        def __init__(self, **kw):
            self.kw = kw

    class TorchTrainer:
        def __init__(self, fn, train_loop_config, scaling_config, run_config):
            calls["fn"], calls["loop"], calls["scaling"], calls["run"] = fn, train_loop_config, scaling_config.kw, run_config.kw

        def fit(self):
            calls["fit"] = True
            return "result"

    train.ScalingConfig, train.RunConfig, torch_mod.TorchTrainer = ScalingConfig, RunConfig, TorchTrainer
    ray.train = train
    return {"ray": ray, "ray.train": train, "ray.train.torch": torch_mod}


def test_ray_launcher_builds_the_trainer_from_the_config(monkeypatch, tmp_path):
    calls = {}
    for k, v in _fake_ray(calls).items():
        monkeypatch.setitem(sys.modules, k, v)
    cfg = {"use_ray": True, "ray_num_workers": 4, "ray_run_name": "run7", "output_dir": str(tmp_path / "out"),
           "base_model": "m", "micro_batch_size": 1}
    assert launchers.train_with_ray(cfg, raw=dict(cfg, learning_rate=1e-4)) == "result"
    assert calls["fit"] and calls["fn"] is launchers.ray_worker
    assert calls["scaling"] == {"num_workers": 4, "resources_per_worker": {"GPU": 1}, "use_gpu": True}
    assert calls["run"]["name"] == "run7" and calls["run"]["storage_path"].endswith("/out")
    assert "use_ray" not in calls["loop"]["cfg"] and calls["loop"]["cfg"]["learning_rate"] == 1e-4


def test_ray_launcher_without_ray_names_the_missing_package(monkeypatch):
    for k in ("ray", "ray.train", "ray.train.torch"):
        monkeypatch.setitem(sys.modules, k, None)
    with pytest.raises(RuntimeError, match="ray"):
        launchers.train_with_ray({"use_ray": True})


class _FakeModal:
    """Records what the launcher asks of the SDK."""

    def __init__(self):
        self.log = []
        sdk = self

        class Image:
            def __init__(self, tag):
                self.tag, self.cmds, self.envs, self.dirs = tag, [], {}, {}

            @classmethod
            def from_registry(cls, tag):
                return cls(tag)

            def dockerfile_commands(self, cmds):
                self.cmds = list(cmds)
                return self

            def env(self, e):
                self.envs = dict(e)
                return self

            def add_local_dir(self, local, mount):
                self.dirs[mount] = local
                return self

        class Volume:
            def __init__(self, name):
                self.name = name

            @classmethod
            def from_name(cls, name, create_if_missing=False):
                sdk.log.append(("volume", name, create_if_missing))
                return cls(name)

        class Secret:
            @staticmethod
            def from_dict(d):
                return ("secret", dict(d))

        class _Ctx:
            def __enter__(self):
                return self

            def __exit__(self, *a):
                return False

        class App:
            def function(self, **kw):
                sdk.log.append(("function", kw))

                def wrap(fn):
                    class Remote:
                        @staticmethod
                        def remote(*a, **k):
                            sdk.log.append(("remote", fn.__name__, a, k))
                            return "ok"
                    return Remote
                return wrap

            def run(self, detach=False):
                sdk.log.append(("run", detach))
                return _Ctx()

        self.Image, self.Volume, self.Secret, self.App = Image, Volume, Secret, App
        self.enable_output = lambda: _Ctx()


def test_modal_cloud_train_and_preprocess(monkeypatch, tmp_path):
    sdk = _FakeModal()
    monkeypatch.setenv("HF_TOKEN", "tok")
    monkeypatch.delenv("WANDB_API_KEY", raising=False)
    cloud = launchers.ModalCloud({"gpu": "B200", "gpu_count": 8, "memory": 64, "timeout": 100, "docker_tag": "t1",
                                  "volumes": [{"name": "ckpt", "mount": "/workspace/out"}], "branch": "dev",
                                  "env": ["HF_TOKEN", {"A": 1}], "secrets": ["HF_TOKEN", "WANDB_API_KEY"]}, sdk=sdk)
    assert cloud.gpu() == "B200:8" and ("volume", "ckpt", True) in sdk.log
    assert cloud.train("base_model: x\n", launcher="torchrun", launcher_args=["--foo"], local_dirs={"/workspace/mounts": str(tmp_path)},
                       num_processes=8) == "ok"
    fn_kw = [e[1] for e in sdk.log if e[0] == "function"][-1]
    assert fn_kw["gpu"] == "B200:8" and fn_kw["memory"] == 64 * 1024 and fn_kw["timeout"] == 100
    assert fn_kw["secrets"] == [("secret", {"HF_TOKEN": "tok"})] and list(fn_kw["volumes"]) == ["/workspace/out"]
    img = fn_kw["image"]
    assert img.tag == "axolotl-b200:t1" and img.envs["A"] == "1" and img.envs["HF_TOKEN"] == "tok" and "dev" in img.cmds[-1]
    assert img.dirs == {"/workspace/mounts": str(tmp_path)}
    name, args, kw = [e[1:] for e in sdk.log if e[0] == "remote"][-1]
    assert name == "_remote_train" and args == ("base_model: x\n",) and kw["launcher_args"] == ["--foo"] and kw["num_processes"] == 8
    cloud.preprocess("base_model: x\n")
    fn_kw = [e[1] for e in sdk.log if e[0] == "function"][-1]
    assert "gpu" not in fn_kw and fn_kw["timeout"] == 3 * 3600 and fn_kw["ephemeral_disk"] > 0
    with pytest.raises(ValueError, match="GPU family"):
        launchers.ModalCloud({"gpu": "tpu"}, sdk=sdk).gpu()
    with pytest.raises(ValueError, match="provider"):
        launchers.cloud_for({"provider": "nimbus"})


def test_remote_commands_go_through_this_packages_cli(monkeypatch, tmp_path):
    ran = []
    monkeypatch.setattr(launchers, "run_cmd", lambda cmd, folder, volumes=None: ran.append((cmd, folder)))
    monkeypatch.setattr(launchers, "_write_run_config", lambda text, run_folder=str(tmp_path): str(tmp_path / "config.yaml"))
    launchers._remote_train("a: 1", launcher="torchrun", launcher_args=["--x", "1"], num_processes=4)
    launchers._remote_preprocess("a: 1")
    assert ran[0][0] == f"axolotl train {tmp_path}/config.yaml --launcher torchrun --num-processes 4 --x 1"
    assert ran[1][0].startswith("axolotl preprocess") and ran[1][0].endswith("--no-cloud")


def test_baseten_provider_writes_the_job_directory_and_pushes_it(tmp_path):
    import os

    import yaml

    seen = {}

    def runner(cmd, cwd):
        seen["cmd"] = cmd
        seen["files"] = {f: open(os.path.join(cwd, f), encoding="utf-8").read() for f in sorted(os.listdir(cwd))}
        return 0

    cloud = launchers.cloud_for({"provider": "baseten", "gpu": "h100", "gpu_count": 8, "node_count": 2,
                                 "project_name": "tune", "secrets": ["HF_TOKEN"]}, runner=runner)
    assert cloud.train("base_model: x\n", launcher="torchrun", launcher_args=["--nnodes=2"]) == 0
    assert seen["cmd"] == ["truss", "train", "push", "train_job.py"]
    assert set(seen["files"]) == {"cloud.yaml", "run.sh", "train.yaml", "train_job.py"}
    written = yaml.safe_load(seen["files"]["cloud.yaml"])
    assert written["launcher"] == "torchrun" and written["launcher_args"] == ["--nnodes=2"] and written["gpu_count"] == 8
    assert seen["files"]["train.yaml"] == "base_model: x\n"
    assert "axolotl train train.yaml --launcher ${AXOLOTL_LAUNCHER}" in seen["files"]["run.sh"]
    compile(seen["files"]["train_job.py"], "train_job.py", "exec")            # the job definition is valid Python
    with pytest.raises(NotImplementedError):
        cloud.preprocess("x")
    with pytest.raises(ValueError, match="modal, baseten"):
        launchers.cloud_for({"provider": "nowhere"})


def test_gradio_interface_streams_generated_text(monkeypatch):
    import torch

    import axolotl_b200.train.evaluate  # noqa: F401  (imported before the builders below are replaced)
    from axolotl_b200.cli import gradio_ui

    class Tok:
        eos_token_id = 2
        chat_template = None

        def __call__(self, text):
            return {"input_ids": [5, 6, 7]}

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(i) for i in ids)

    class Model:
        calls = 0

        def eval(self):
            return self

        def generate(self, ids, max_new_tokens, temperature, top_p, eos_token_id):
            Model.calls += 1
            new = [10 + Model.calls] * max_new_tokens if Model.calls < 3 else [2]       # third piece ends with EOS
            return torch.cat([ids, torch.tensor([new])], 1)

    fn = gradio_ui.build_generator({"gradio_max_new_tokens": 10, "gradio_temperature": 0.5}, Model(), Tok(), "cpu", piece=4)
    pieces = list(fn("hello"))
    assert pieces == ["11 11 11 11", "11 11 11 11 12 12 12 12", "11 11 11 11 12 12 12 12 2"]
    assert list(fn("")) == []

    class FakeGradio:
        class Interface:
            def __init__(self, fn, inputs, outputs, title):
                FakeGradio.built = (inputs, outputs, title)

            def launch(self, **kw):
                FakeGradio.launched = kw
                return "served"

    monkeypatch.setattr("axolotl_b200.data.tokenizer.load_tokenizer", lambda cfg: Tok())
    monkeypatch.setattr("axolotl_b200.train.run.build_model", lambda cfg, dev: Model())
    monkeypatch.setattr("axolotl_b200.train.run.setup_adapter", lambda cfg, model: None)
    out = gradio_ui.launch({"device": "cpu", "gradio_title": "demo", "gradio_share": False, "gradio_server_port": 7861}, gr=FakeGradio)
    assert out == "served" and FakeGradio.built == ("textbox", "text", "demo")
    assert FakeGradio.launched == {"share": False, "server_name": "127.0.0.1", "server_port": 7861}
