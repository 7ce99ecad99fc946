"""In-tree native build: compiles every ``csrc/*.cu`` for sm_100a with nvcc and links them into
``axolotl_b200/lib/libaxb200.so``; host-only C++ (the multipack packer) goes to
``libaxb200_host.so`` so CPU-only environments can load it without a CUDA runtime.

The libraries export a plain C ABI and are loaded with ctypes (``axolotl_b200.ops._lib``): no
torch headers are involved, so a full rebuild takes seconds per file and cross-compiles on a
machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA kernels of axolotl_b200 cannot be built")
    return cand


def _stamp(src: Path, flags: list[str]) -> str:
    h = hashlib.sha1()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool, extra: list[str], tag: str = "") -> Path:
    obj = OBJ / (src.stem + tag + ".o")
    stamp_file = OBJ / (src.stem + tag + ".stamp")
    flags = NVCC_FLAGS + extra
    stamp = _stamp(src, flags)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, flush=True)
    stamp_file.write_text(stamp)
    return obj


def _build_checked(cu_sources, verbose: bool) -> Path:
    """The bounds-check variant (``libaxb200_checked.so``, loaded instead of the regular library when
    ``AXB_BOUNDS_CHECK=1``): same sources with ``-DAXB_BOUNDS_CHECK`` and relocatable device code, so that one
    device record is shared by all kernels."""
    extra = ["-DAXB_BOUNDS_CHECK", "-rdc=true"]
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(cu_sources)))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, extra, tag="_checked"), cu_sources))
    out = LIB / "libaxb200_checked.so"
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", str(out),
               *map(str, objs), "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link of the bounds-check library failed:\n{res.stdout}\n{res.stderr}")
    return out


def build(verbose: bool = False, ptxas_info: bool = False, force: bool = False) -> dict[str, Path]:
    """Build both shared libraries; returns their paths. Incremental (content-hashed)."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    if force:
        for f in OBJ.glob("*.stamp"):
            f.unlink()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    cu_sources = sorted(CSRC.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(cu_sources)))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose or ptxas_info, extra), cu_sources))
    out = LIB / "libaxb200.so"
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    _build_checked(cu_sources, verbose)
    host_out = LIB / "libaxb200_host.so"
    cpp_sources = sorted(CSRC.glob("*.cpp"))
    if cpp_sources:
        newest_src = max(s.stat().st_mtime for s in cpp_sources)
        if not host_out.exists() or host_out.stat().st_mtime < newest_src:
            cxx = shutil.which("g++") or "g++"
            cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-o", str(host_out), *map(str, cpp_sources), "-lpthread"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"host link failed:\n{res.stdout}\n{res.stderr}")
    return {"cuda": out, "checked": LIB / "libaxb200_checked.so", "host": host_out}


if __name__ == "__main__":
    paths = build(verbose=True, ptxas_info="--ptxas" in sys.argv, force="--force" in sys.argv)
    for k, v in paths.items():
        print(k, v)
