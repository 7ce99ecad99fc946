"""Hyper-parameter sweeps: a YAML of ``key: [values]`` (and ``_: [ {k: v, ...}, ... ]`` for
paired settings) expands to the cartesian product of temporary config files
(src/axolotl/cli/utils/sweeps.py:9, src/axolotl/cli/utils/train.py:69-106)."""
from __future__ import annotations

import itertools
import tempfile

import yaml


def generate_sweep_configs(base: dict, sweep: dict) -> list[dict]:
    paired = sweep.get("_", [None])
    keys = [k for k in sweep if k != "_"]
    out = []
    for combo in itertools.product(*[sweep[k] for k in keys]) if keys else [()]:
        for pair in paired:
            c = dict(base)
            c.update(dict(zip(keys, combo)))
            if pair:
                c.update(pair)
            out.append(c)
    return out


def expand_sweep(config_path: str, sweep_path: str) -> list[str]:
    with open(config_path) as fh:
        base = yaml.safe_load(fh)
    with open(sweep_path) as fh:
        sweep = yaml.safe_load(fh)
    paths = []
    for i, c in enumerate(generate_sweep_configs(base, sweep)):
        if "output_dir" in c:
            c["output_dir"] = f"{c['output_dir']}/sweep-{i}"
        f = tempfile.NamedTemporaryFile("w", suffix=f"-sweep{i}.yaml", delete=False)
        yaml.safe_dump(c, f)
        f.close()
        paths.append(f.name)
    return paths
