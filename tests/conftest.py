import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

_CUDA_FATAL = ("device-side assert", "illegal memory access", "misaligned address",
               "illegal instruction", "unspecified launch failure")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.hookimpl(hookwrapper=True)
def pytest_runtest_makereport(item, call):
    # A poisoned CUDA context makes every later test fail with noise: stop the session instead.
    outcome = yield
    rep = outcome.get_result()
    if rep.failed and call.excinfo is not None:
        text = str(call.excinfo.value).lower()
        if any(m in text for m in _CUDA_FATAL):
            pytest.exit(f"CUDA context is unusable after {item.nodeid}: aborting the session", 3)
