import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    try:
        from helpers import CROSS, WORST
    except Exception:
        return
    for dtype, (diff, what) in sorted(CROSS.items()):
        terminalreporter.write_line(f"largest difference between two ways of cutting the same request, {dtype}: "
                                    f"{diff:.2e} of the largest logit"
                                    + (f" = {diff / 2 ** -24:.0f} float32 ulp" if dtype == "float32" else "") + f" ({what})")
    for dtype, (ratio, what) in sorted(WORST.items()):
        terminalreporter.write_line(f"largest error / tolerance against the plain implementation, {dtype}: "
                                    f"{ratio:.2f} ({what})")
