"""Self-contained safetensors reader / writer (format: u64 header length, JSON header, raw
little-endian tensor bytes) with lazy per-tensor access through mmap and sharded-checkpoint
helpers (``model.safetensors.index.json``). Interoperable with the ``safetensors`` package and
therefore with ``transformers`` / ``peft`` checkpoints.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterable

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    items = sorted(tensors.items())
    for name, t in items:
        if t.dtype not in _NAMES:
            raise TypeError(f"dtype {t.dtype} of '{name}' cannot be stored in safetensors")
        n = _nbytes(t)
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(hb)))
        fh.write(hb)
        for _, t in items:
            c = t.detach().to("cpu").contiguous()
            fh.write(c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    os.replace(tmp, path)


class SafeFile:
    """Lazy reader: ``keys()``, ``get_tensor(name)``, ``shape(name)``; tensors are copied out of the
    mapping so the file can be closed."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        self.header = json.loads(self._fh.read(hlen))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(path) else None

    def keys(self):
        return list(self.header.keys())

    def shape(self, name):
        return tuple(self.header[name]["shape"])

    def dtype(self, name):
        return _DTYPES[self.header[name]["dtype"]]

    def get_tensor(self, name) -> torch.Tensor:
        info = self.header[name]
        a, b = info["data_offsets"]
        dt = _DTYPES[info["dtype"]]
        if b == a:
            return torch.zeros(info["shape"], dtype=dt)
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=b - a, offset=self._base + a).copy()
        return torch.from_numpy(raw).view(dt).reshape(info["shape"])

    def close(self):
        if self._mm is not None:
            self._mm.close()
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def load_file(path: str, device="cpu") -> dict:
    with SafeFile(path) as f:
        return {k: f.get_tensor(k).to(device) for k in f.keys()}


# ------------------------------------------------------------------------ sharded checkpoints
def checkpoint_files(model_dir: str) -> list[str]:
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as fh:
            files = sorted(set(json.load(fh)["weight_map"].values()))
        return [os.path.join(model_dir, f) for f in files]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(single):
        return [single]
    found = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors") and not f.startswith("adapter"))
    return [os.path.join(model_dir, f) for f in found]


def iter_checkpoint(model_dir: str) -> Iterable[tuple[str, torch.Tensor]]:
    for f in checkpoint_files(model_dir):
        with SafeFile(f) as sf:
            for k in sf.keys():
                yield k, sf.get_tensor(k)


def save_sharded(tensors: dict, out_dir: str, max_shard_bytes: int = 5 * 1024 ** 3, metadata=None) -> list[str]:
    """HF layout: one ``model.safetensors`` or ``model-0000i-of-0000n.safetensors`` + index."""
    os.makedirs(out_dir, exist_ok=True)
    shards, cur, cur_b = [], {}, 0
    for k in sorted(tensors):
        n = _nbytes(tensors[k])
        if cur and cur_b + n > max_shard_bytes:
            shards.append(cur)
            cur, cur_b = {}, 0
        cur[k] = tensors[k]
        cur_b += n
    if cur:
        shards.append(cur)
    meta = {"format": "pt"}
    meta.update(metadata or {})
    if len(shards) == 1:
        save_file(shards[0], os.path.join(out_dir, "model.safetensors"), meta)
        return ["model.safetensors"]
    names, wmap, total = [], {}, 0
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(out_dir, fn), meta)
        names.append(fn)
        for k, t in sh.items():
            wmap[k] = fn
            total += _nbytes(t)
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as fh:
        json.dump({"metadata": {"total_size": total}, "weight_map": wmap}, fh, indent=2)
    return names
