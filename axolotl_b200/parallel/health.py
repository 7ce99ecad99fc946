"""Host-side failure detection between steps.

Every rank publishes a heartbeat (step counter + wall-clock time) in the process group's
key-value store after each optimizer step and checks its peers' heartbeats BEFORE launching the
next step. A peer that announced that it is leaving, or whose heartbeat is older than the timeout,
raises ``PeerFailure`` on the survivors while none of their kernels or collectives is in flight,
so they can save a checkpoint and exit instead of hanging in a collective until the NCCL watchdog
fires (the reference relies on that watchdog alone: ``AXOLOTL_NCCL_TIMEOUT`` / ``ddp_timeout``,
src/axolotl/utils/distributed.py:53-55). Device-side waits are bounded separately and report through
the kernels' status word (``ops._lib.check_status``).
"""
from __future__ import annotations

import time

import torch.distributed as dist

from ..train.trainer import Callback


class PeerFailure(RuntimeError):
    pass


class HeartbeatMonitor:
    def __init__(self, store=None, rank=None, world=None, timeout_s=300.0, prefix="axb_hb"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.timeout, self.prefix = float(timeout_s), prefix
        self.beat(-1)

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, step):
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}:alive")

    def leave(self, reason="exit"):
        """Announce an orderly or failed exit (call between steps, with nothing in flight)."""
        self.store.set(self._key(self.rank), f"-1:{time.time():.3f}:left:{reason}")

    def check(self):
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                raw = self.store.get(self._key(r)).decode()
            except Exception as exc:
                raise PeerFailure(f"rank {r} has no heartbeat: {exc}") from exc
            parts = raw.split(":")
            if parts[2] == "left":
                raise PeerFailure(f"rank {r} left the job ({':'.join(parts[3:]) or 'no reason given'})")
            age = now - float(parts[1])
            if age > self.timeout:
                raise PeerFailure(f"rank {r} heartbeat is {age:.0f} s old (limit {self.timeout:.0f} s)")


class HeartbeatCallback(Callback):
    """Beats after every step and checks the peers before the next one starts. A peer failure
    raises ``PeerFailure`` out of ``Trainer.train``; the trainer first writes a collective-free dump
    of this rank's optimizer state and counters (``Trainer.save_local_state``)."""

    def __init__(self, monitor: HeartbeatMonitor):
        self.mon = monitor

    def on_step_end(self, trainer, logs):
        self.mon.beat(trainer.global_step)

    def on_pre_step(self, trainer):
        self.mon.check()
