"""Launchers beyond local torchrun: Ray Train (``use_ray: true``) and cloud runs (``--cloud cloud.yaml``, Modal).

Both SDKs are optional and imported on use. The Ray path hands the validated config to a ``TorchTrainer`` whose
workers (one per GPU) re-normalise it against their own device and run the ordinary training entry; Ray's torch
back end sets the process-group environment. The cloud path builds an image, named volumes and secrets from the
cloud YAML and runs ``preprocess`` / ``train`` / ``lm-eval`` remotely through this package's own CLI, with the run's
config written into the run folder on a volume.

Behaviour of the reference's launchers (src/axolotl/cli/train.py:117-202, src/axolotl/cli/cloud/__init__.py:17-74,
src/axolotl/cli/cloud/modal_.py:18-316).
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

import yaml

from ..utils.logging import get_logger

LOG = get_logger(__name__)


# --------------------------------------------------------------------------------------------- Ray
def ray_worker(kwargs: dict):
    """Runs on every Ray Train worker: the config travels as a plain dict and is validated again here, where the
    training device is attached."""
    from ..config.load import load_cfg
    from ..train.run import train as run_train

    return run_train(load_cfg(dict(kwargs["cfg"])))


def train_with_ray(cfg: dict, raw: dict | None = None):
    """``use_ray: true``: ``ray_num_workers`` workers with ``resources_per_worker`` (default one GPU each); results and
    checkpoints of the Ray run go under ``output_dir``."""
    try:
        from ray.train import RunConfig, ScalingConfig
        from ray.train.torch import TorchTrainer
    except ImportError as e:
        raise RuntimeError("use_ray needs the `ray[train]` package, which is not installed") from e
    resources = cfg.get("resources_per_worker") or {"GPU": 1}
    if hasattr(resources, "to_dict"):
        resources = resources.to_dict()
    # the workers validate the user's own keys again (the normalised config carries derived values)
    plain = {k: v for k, v in dict(raw if raw is not None else cfg).items() if k != "use_ray"}
    trainer = TorchTrainer(
        ray_worker,
        train_loop_config={"cfg": plain},
        scaling_config=ScalingConfig(num_workers=int(cfg.get("ray_num_workers") or 1), resources_per_worker=dict(resources),
                                     use_gpu=True),
        run_config=RunConfig(name=cfg.get("ray_run_name"), storage_path=Path(cfg.get("output_dir") or "./outputs").absolute().as_posix()),
    )
    return trainer.fit()


# --------------------------------------------------------------------------------------------- cloud
def load_cloud_cfg(path) -> dict:
    with open(path, encoding="utf-8") as fh:
        cfg = yaml.safe_load(fh) or {}
    if not isinstance(cfg, dict):
        raise ValueError(f"{path}: a cloud config is a YAML mapping")
    return cfg


def run_cmd(cmd: str, run_folder: str, volumes=None):
    """Runs one shell command inside the remote container; volumes are reloaded before and committed after so that
    other containers see the files."""
    for v in (volumes or {}).values():
        v.reload()
    code = subprocess.call(cmd.split(), cwd=run_folder, env=dict(os.environ, PYTHONUNBUFFERED="1"))
    if code:
        raise SystemExit(code)
    for v in (volumes or {}).values():
        v.commit()


def _write_run_config(config_yaml: str, run_folder="/workspace/mounts") -> str:
    os.makedirs(run_folder, exist_ok=True)
    path = os.path.join(run_folder, "config.yaml")
    with open(path, "w", encoding="utf-8") as fh:
        fh.write(config_yaml)
    return path


def _remote_preprocess(config_yaml: str, volumes=None):
    path = _write_run_config(config_yaml)
    run_cmd(f"axolotl preprocess {path} --no-cloud", os.path.dirname(path), volumes)


def _remote_train(config_yaml: str, launcher="torchrun", launcher_args=None, volumes=None, **kw):
    path = _write_run_config(config_yaml)
    extra = " ".join(launcher_args or [])
    n = kw.get("num_processes")
    cmd = f"axolotl train {path} --launcher {launcher}" + (f" --num-processes {n}" if n else "") + (f" {extra}" if extra else "")
    run_cmd(cmd, os.path.dirname(path), volumes)


def _remote_lm_eval(config_yaml: str, volumes=None):
    path = _write_run_config(config_yaml)
    run_cmd(f"axolotl lm-eval {path}", os.path.dirname(path), volumes)


GPU_FAMILIES = {"l40s": "L40S", "a100": "A100-40GB", "a100-40gb": "A100-40GB", "a100-80gb": "A100-80GB", "a10": "A10G",
                "a10g": "A10G", "h100": "H100", "h200": "H200", "b200": "B200", "t4": "T4", "l4": "L4"}


class ModalCloud:
    """Cloud YAML keys: ``provider`` (modal), ``docker_tag`` / ``image``, ``dockerfile_commands``, ``branch``, ``env``
    (names copied from the local environment, or ``{NAME: value}``), ``secrets`` (same forms), ``volumes``
    (``[{name, mount}]``), ``gpu``, ``gpu_count``, ``memory`` / ``memory_preprocess`` (GiB), ``timeout`` /
    ``timeout_preprocess`` (seconds)."""

    def __init__(self, config: dict, app=None, sdk=None):
        if sdk is None:
            try:
                import modal as sdk
            except ImportError as e:
                raise RuntimeError("cloud runs on Modal need the `modal` package, which is not installed") from e
        self.modal, self.config = sdk, config
        self.app = app or sdk.App()
        self.volumes = {}
        for vc in config.get("volumes") or []:
            self.volumes[vc["mount"]] = sdk.Volume.from_name(vc["name"], create_if_missing=True)

    def _pairs(self, key):
        out = {}
        for item in self.config.get(key) or []:
            if isinstance(item, str):
                if os.environ.get(item):
                    out[item] = os.environ[item]
            elif isinstance(item, dict):
                out.update({k: str(v) for k, v in item.items()})
        return out

    def env(self) -> dict:
        base = {"HF_DATASETS_CACHE": "/workspace/data/huggingface-cache/datasets",
                "HF_HUB_CACHE": "/workspace/data/huggingface-cache/hub"}
        base.update(self._pairs("env"))
        return base

    def image(self, local_dirs=None):
        tag = self.config.get("image") or f"axolotl-b200:{self.config.get('docker_tag') or 'latest'}"
        img = self.modal.Image.from_registry(tag)
        cmds = list(self.config.get("dockerfile_commands") or [])
        if self.config.get("branch"):
            cmds.append(f"RUN cd /workspace/axolotl_b200 && git fetch && git checkout {self.config['branch']} && git pull")
        if cmds:
            img = img.dockerfile_commands(cmds)
        img = img.env(self.env())
        for mount, local in (local_dirs or {}).items():
            img = img.add_local_dir(local, mount)
        return img

    def secrets(self):
        return [self.modal.Secret.from_dict({k: v}) for k, v in self._pairs("secrets").items()]

    def gpu(self) -> str:
        fam = str(self.config.get("gpu") or "b200").lower()
        if fam not in GPU_FAMILIES:
            raise ValueError(f"unsupported GPU family {fam!r} (known: {sorted(GPU_FAMILIES)})")
        return f"{GPU_FAMILIES[fam]}:{int(self.config.get('gpu_count') or 1)}"

    def _memory(self, *keys):
        gib = 128
        for k in keys:
            if self.config.get(k):
                gib = int(self.config[k])
        return 1024 * gib

    def _function(self, fn, gpu=None, cpu=8.0, memory=None, timeout=None, local_dirs=None):
        kw = dict(image=self.image(local_dirs), volumes=dict(self.volumes), cpu=cpu, memory=memory, timeout=timeout,
                  secrets=self.secrets())
        if gpu:
            kw["gpu"] = gpu
        else:
            kw["ephemeral_disk"] = 1000 * 525
        return self.app.function(**kw)(fn)

    def _call(self, fn, *args, **kw):
        with self.modal.enable_output():
            with self.app.run(detach=True):
                return fn.remote(*args, volumes=dict(self.volumes), **kw)

    def preprocess(self, config_yaml: str):
        fn = self._function(_remote_preprocess, memory=self._memory("memory", "memory_preprocess"),
                            timeout=int(self.config.get("timeout_preprocess") or 3 * 3600))
        return self._call(fn, config_yaml)

    def train(self, config_yaml: str, launcher="torchrun", launcher_args=None, local_dirs=None, **kw):
        fn = self._function(_remote_train, gpu=self.gpu(), cpu=16.0, memory=self._memory("memory"),
                            timeout=int(self.config.get("timeout") or 24 * 3600), local_dirs=local_dirs)
        return self._call(fn, config_yaml, launcher=launcher, launcher_args=launcher_args, **kw)

    def lm_eval(self, config_yaml: str):
        fn = self._function(_remote_lm_eval, gpu=self.gpu(), cpu=16.0, memory=self._memory("memory"),
                            timeout=int(self.config.get("timeout") or 24 * 3600))
        return self._call(fn, config_yaml)


_BASETEN_RUN_SH = """#!/bin/bash
set -eux
# multi-node jobs: keep NCCL off the container bridge and the loopback device
export NCCL_SOCKET_IFNAME="^docker0,lo"
export NCCL_TIMEOUT=1800000
axolotl preprocess train.yaml
axolotl train train.yaml --launcher ${AXOLOTL_LAUNCHER} ${AXOLOTL_LAUNCHER_ARGS}
"""

_BASETEN_JOB_PY = """# Training-job definition pushed with `truss train push`; reads cloud.yaml written next to it.
import yaml
from truss.base import truss_config
from truss_train import definitions

cloud = yaml.safe_load(open("cloud.yaml"))
launcher_args = cloud.get("launcher_args") or []
env = {"AXOLOTL_LAUNCHER": cloud.get("launcher") or "torchrun",
       "AXOLOTL_LAUNCHER_ARGS": ("-- " + " ".join(launcher_args)) if launcher_args else ""}
for name in cloud.get("secrets") or []:
    env[name] = definitions.SecretReference(name=name)
accelerator = getattr(truss_config.Accelerator, str(cloud.get("gpu") or "h100").upper())
job = definitions.TrainingJob(
    image=definitions.Image(base_image=cloud.get("image") or cloud.get("docker_tag") or "{image}"),
    compute=definitions.Compute(node_count=int(cloud.get("node_count") or 1),
                                accelerator=truss_config.AcceleratorSpec(accelerator=accelerator, count=int(cloud.get("gpu_count") or 1))),
    runtime=definitions.Runtime(start_commands=["/bin/sh -c 'chmod +x ./run.sh && ./run.sh'"], environment_variables=env))
project = definitions.TrainingProject(name=cloud.get("project_name") or "axolotl-project", job=job)
"""


class BasetenCloud:
    """Training jobs on Baseten: a temporary directory receives the cloud settings, the training YAML, a start script
    and the job definition, and is pushed with the `truss` command line tool. Cloud YAML keys: ``provider: baseten``,
    ``gpu``, ``gpu_count``, ``node_count``, ``project_name``, ``secrets``, ``image``. Preprocessing runs inside the
    training job (reference: src/axolotl/cli/cloud/baseten/__init__.py:14-48 and its template directory)."""

    default_image = "axolotlai/axolotl:main-latest"

    def __init__(self, config: dict, runner=None):
        self.config = dict(config)
        self.runner = runner or (lambda cmd, cwd: subprocess.run(cmd, cwd=cwd, check=False))

    def preprocess(self, config_yaml: str, *a, **kw):
        raise NotImplementedError("Baseten has no separate preprocessing step: it happens at the start of the training job")

    def lm_eval(self, config_yaml: str, *a, **kw):
        raise NotImplementedError("lm-eval is not available on the Baseten provider")

    def train(self, config_yaml: str, launcher: str = "torchrun", launcher_args=None, **kw):
        import tempfile

        import yaml

        with tempfile.TemporaryDirectory() as tmp:
            cloud = dict(self.config, launcher=launcher, launcher_args=list(launcher_args or []))
            with open(os.path.join(tmp, "cloud.yaml"), "w", encoding="utf-8") as fh:
                yaml.safe_dump(cloud, fh)
            with open(os.path.join(tmp, "train.yaml"), "w", encoding="utf-8") as fh:
                fh.write(config_yaml)
            with open(os.path.join(tmp, "run.sh"), "w", encoding="utf-8") as fh:
                fh.write(_BASETEN_RUN_SH)
            with open(os.path.join(tmp, "train_job.py"), "w", encoding="utf-8") as fh:
                fh.write(_BASETEN_JOB_PY.replace("{image}", self.default_image))
            return self.runner(["truss", "train", "push", "train_job.py"], tmp)


def cloud_for(cloud_cfg: dict, **kw):
    provider = cloud_cfg.get("provider") or "modal"
    if provider == "modal":
        return ModalCloud(cloud_cfg, **kw)
    if provider == "baseten":
        return BasetenCloud(cloud_cfg, **kw)
    raise ValueError(f"unsupported cloud provider {provider!r} (supported: modal, baseten)")


def run_in_cloud(command: str, cloud_config, config, **kw):
    """``axolotl <preprocess|train|lm-eval> config.yaml --cloud cloud.yaml``."""
    cloud = cloud_for(load_cloud_cfg(cloud_config))
    with open(config, encoding="utf-8") as fh:
        text = fh.read()
    if command == "preprocess":
        return cloud.preprocess(text)
    if command == "train":
        return cloud.train(text, **kw)
    if command in ("lm-eval", "lm_eval"):
        return cloud.lm_eval(text)
    raise ValueError(f"`{command}` cannot run in the cloud")
