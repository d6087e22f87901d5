"""pytest configuration: markers and shared helpers."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name):
    """Load tests/golden/<name>.npz as a plain dict."""
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def golden_cases(d):
    """Group 'case.key' entries of a golden dict into {case: {key: array}}."""
    out = {}
    for full, val in d.items():
        if "." not in full:
            continue
        case, key = full.rsplit(".", 1)
        out.setdefault(case, {})[key] = val
    return out


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle

    _oracle.build()
    return _oracle


EMULATED = os.environ.get("BITTORCH_B200_EMULATED") == "1"      # GPU-marked tests run against tests/emu on the CPU
needs_real_gpu = pytest.mark.skipif(EMULATED, reason="checks the CUDA library itself, not host logic")


@pytest.fixture
def tuning():
    """Kernel-selection overrides (bt_set_tuning) that are undone when the test ends."""
    from bittorch_b200 import _C

    touched = []

    def set_knob(knob: int, value: int) -> None:
        touched.append(knob)
        _C.set_tuning(knob, value)

    yield set_knob
    for knob in touched:
        _C.set_tuning(knob, -1)
