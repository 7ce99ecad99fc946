"""Launches tests/dist_checks.py under torchrun: gloo ranks on CPU here, NCCL ranks on GPUs."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, extra, port):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = env.get("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dist_checks.py"), *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + "\n" + res.stderr[-6000:]
    return res.stdout


def test_data_parallel_gloo_world2():
    out = _run(2, ["cpu"], 29611)
    assert "rank-0 loading ok" in out
    assert "dp training equivalence ok (collective)" in out
    assert "dp training equivalence ok (collective, two groups)" in out
    assert "dp training equivalence ok (collective, full fine-tune)" in out
    assert "dp training equivalence ok (collective, replicated)" in out
    for line in ("tensor parallel ok", "context parallel ok", "context parallel state-space ok", "expert parallel ok"):
        assert line in out, out[-2000:]


def test_tp_x_cp_gloo_world4():
    out = _run(4, ["cpu", "tpcp", "cpssm"], 29613)
    assert "tp x cp ok" in out
    assert "context parallel state-space ok" in out      # a document that crosses three chunk borders


@pytest.mark.gpu
def test_fused_multi_gpu():
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    out = _run(2, [], 29612)
    for line in ("gather-gemm ok", "fused rs+adamw+ag ok (multimem=on)", "fused rs+adamw+ag ok (multimem=off)",
                 "dp training equivalence ok (fused)", "dp training equivalence ok (fused, two groups)",
                 "dp training equivalence ok (fused, full fine-tune)",
                 "dp training equivalence ok (collective)", "dp training equivalence ok (fused, replicated)",
                 "tensor parallel ok", "context parallel ok", "context parallel state-space ok", "expert parallel ok"):
        assert line in out, (line, out[-3000:])
