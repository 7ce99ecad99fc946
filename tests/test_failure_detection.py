"""Failure detection without faulting anything: host-side heartbeats between gloo ranks, the loss
watchdog, a corrupted checkpoint, and (GPU) a bounded device wait that runs out and reports through
the status word while the context stays usable."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_heartbeat_monitor_detects_leaving_and_silent_peers():
    from axolotl_b200.parallel.health import HeartbeatMonitor, PeerFailure

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self[k]

    st = Store()
    a = HeartbeatMonitor(st, rank=0, world=2, timeout_s=50.0)
    with pytest.raises(PeerFailure, match="no heartbeat"):
        a.check()
    b = HeartbeatMonitor(st, rank=1, world=2, timeout_s=50.0)
    a.check()
    b.beat(3)
    a.check()
    # a heartbeat that is too old
    st["axb_hb/1"] = b"3:1.000:alive"
    with pytest.raises(PeerFailure, match="heartbeat is"):
        a.check()
    b.beat(4)
    b.leave("dataloader raised")
    with pytest.raises(PeerFailure, match="left the job .dataloader raised"):
        a.check()


def test_rank_exit_between_steps_is_seen_before_the_next_collective(tmp_path):
    """Two gloo ranks; rank 1 raises in its 'dataloader' after step 2 and leaves between steps. Rank 0
    must stop with PeerFailure at its next pre-step check instead of entering a collective."""
    script = tmp_path / "ranks.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, time, datetime
        sys.path.insert(0, {ROOT!r})
        import torch, torch.distributed as dist
        from axolotl_b200.parallel.health import HeartbeatMonitor, PeerFailure
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
        rank = dist.get_rank()
        mon = HeartbeatMonitor(timeout_s=5.0)
        dist.barrier()
        try:
            for step in range(6):
                mon.check()                       # nothing in flight here
                t = torch.ones(4); dist.all_reduce(t)
                mon.beat(step)
                if rank == 1 and step == 1:       # fails while preparing the next step's data
                    raise ValueError("dataloader worker failed")
                time.sleep(0.5)                   # the survivors' next check comes after the notice
            print(f"rank {{rank}} finished", flush=True)
        except PeerFailure as exc:
            print(f"rank {{rank}} detected: {{exc}} at step {{step}}", flush=True)
            sys.exit(0)
        except ValueError as exc:
            mon.leave(str(exc))
            print(f"rank {{rank}} leaving: {{exc}}", flush=True)
            sys.exit(0)
    """))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=120, cwd=ROOT)
    out = res.stdout + res.stderr
    assert "rank 1 leaving: dataloader worker failed" in out, out[-2000:]
    assert "rank 0 detected: rank 1 left the job (dataloader worker failed)" in out, out[-2000:]
    assert "rank 0 finished" not in out


def test_loss_watchdog_stops_training():
    from axolotl_b200.train.callbacks import LossWatchdogCallback

    class T:
        should_stop = False
        global_step = 0

    cb, t = LossWatchdogCallback(threshold=5.0, patience=2), T()
    for loss in (1.0, 9.0, 2.0, 9.0, 9.5):
        t.global_step += 1
        cb.on_log(t, {"loss": loss})
    assert t.should_stop


def test_corrupt_checkpoint_is_reported(tmp_path):
    from axolotl_b200.io.safetensors_io import load_file, save_file

    p = tmp_path / "a.safetensors"
    save_file({"w": torch.arange(12.0).reshape(3, 4)}, str(p))
    raw = p.read_bytes()
    p.write_bytes(raw[: len(raw) - 17])           # truncated while being written
    with pytest.raises(Exception):
        load_file(str(p))
    p.write_bytes(b"\\xff" * 8 + raw[8:])         # header length corrupted
    with pytest.raises(Exception):
        load_file(str(p))


@pytest.mark.gpu
def test_bounded_device_wait_reports_timeout_and_context_survives():
    """A barrier whose partner never signals (a flag that nothing sets): the kernel gives up after its
    budget, records the timeout in the status word and returns; later kernels run normally."""
    import ctypes as C

    from axolotl_b200.ops import _lib
    import axolotl_b200.parallel.symm  # noqa: F401  (registers the kernel signatures)

    dev = torch.device("cuda", 0)
    pads = torch.zeros(2, 4096, dtype=torch.int32, device=dev)      # own pad + a fake peer's pad
    ptrs = (C.c_uint64 * 8)(pads[0].data_ptr(), pads[1].data_ptr(), 0, 0, 0, 0, 0, 0)
    lib = _lib.cuda_lib()
    _lib.check_status(dev)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.axb_peer_barrier(ptrs, 0, 2, 1, 1, _lib.status_word(dev).data_ptr(), 200_000_000, _lib.stream_ptr())
    t1.record()
    assert rc == 0
    with pytest.raises(_lib.KernelTimeoutError):
        _lib.check_status(dev)
    assert 100.0 < t0.elapsed_time(t1) < 2000.0                      # waited its 0.2 s budget, not forever
    _lib.check_status(dev)                                           # the word was cleared
    x = torch.randn(256, 256, device=dev, dtype=torch.bfloat16)
    from axolotl_b200.ops.gemm import gemm
    y = gemm(x, x)
    assert torch.isfinite(y.float()).all()
    _lib.check_status(dev)
