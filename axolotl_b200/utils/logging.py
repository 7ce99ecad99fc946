"""Logging: rank-aware logger (INFO on the main process, WARNING elsewhere unless
AXOLOTL_LOG_LEVEL overrides) and an output tee to ``<output_dir>/debug.log``
(reference: src/axolotl/logging_config.py:71-175, src/axolotl/utils/tee.py:90-166)."""
from __future__ import annotations

import logging
import os
import sys

_configured = False


class _StderrHandler(logging.StreamHandler):
    """Always writes to the *current* ``sys.stderr`` (so output tees and test harnesses that swap
    the stream keep working)."""

    def __init__(self):
        logging.Handler.__init__(self)

    @property
    def stream(self):
        return sys.stderr

    @stream.setter
    def stream(self, value):
        pass


def configure(level=None):
    global _configured
    if _configured:
        return
    rank = int(os.environ.get("RANK", "0"))
    lvl = level or os.environ.get("AXOLOTL_LOG_LEVEL") or ("INFO" if rank == 0 else "WARNING")
    h = _StderrHandler()
    h.setFormatter(logging.Formatter(f"[%(asctime)s] [%(levelname)s] [%(name)s] [rank{rank}] %(message)s",
                                     "%Y-%m-%d %H:%M:%S"))
    root = logging.getLogger("axolotl_b200")
    root.handlers[:] = [h]
    root.setLevel(getattr(logging, str(lvl).upper(), logging.INFO))
    root.propagate = False
    _configured = True


def get_logger(name):
    configure()
    short = name.split("axolotl_b200.")[-1]
    return logging.getLogger("axolotl_b200").getChild(short)


class Tee:
    """Duplicates a text stream into a file (used for stdout/stderr -> debug.log)."""

    def __init__(self, stream, fh):
        self.stream, self.fh = stream, fh

    def write(self, s):
        self.stream.write(s)
        try:
            self.fh.write(s)
            self.fh.flush()
        except ValueError:
            pass
        return len(s)

    def flush(self):
        self.stream.flush()

    def __getattr__(self, k):
        return getattr(self.stream, k)


_tee_state = {}


def start_debug_log(output_dir, append=False):
    if _tee_state or int(os.environ.get("RANK", "0")) != 0:
        return None
    os.makedirs(output_dir, exist_ok=True)
    path = os.path.join(output_dir, "debug.log")
    fh = open(path, "a" if append else "w")
    _tee_state.update(fh=fh, out=sys.stdout, err=sys.stderr)
    sys.stdout, sys.stderr = Tee(sys.stdout, fh), Tee(sys.stderr, fh)
    return path


def stop_debug_log():
    if not _tee_state:
        return
    sys.stdout, sys.stderr = _tee_state["out"], _tee_state["err"]
    _tee_state["fh"].close()
    _tee_state.clear()
