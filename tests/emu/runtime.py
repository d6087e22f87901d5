"""Runs host-side code of the package against the host emulation of the C ABI.  TEST INFRASTRUCTURE ONLY.

``activate()`` must be called in a fresh process before ``bittorch_b200`` is imported.  It

* builds ``tests/emu/libbt_emu.so`` (gcc, seconds) and points ``BITTORCH_B200_LIB`` at it, so the ctypes binding
  loads the emulation instead of the CUDA library;
* makes CPU tensors pass for device tensors: the binding's "must be CUDA" checks, ``Tensor.is_cuda``, the current
  stream, ``torch.cuda.device`` / ``synchronize`` / ``set_device`` become harmless on the CPU.

Nothing of this is reachable from the package itself: the package has no CPU path, and these patches live only in
the child processes the tests start (``python -m tests.emu.runtime <script> [args]`` or an explicit ``activate()``).
"""

from __future__ import annotations

import contextlib
import os
import runpy
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.path.join(HERE, "libbt_emu.so")
_SOURCES = [os.path.join(HERE, "bt_emu.c"), os.path.join(ROOT, "oracle", "bt_oracle.c"),
            os.path.join(ROOT, "include", "bittorch_b200.h")]


def build(force: bool = False) -> str:
    stale = force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in _SOURCES)
    if stale:
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-Wall",
                               "-o", LIB, _SOURCES[0], "-lm"])
    return LIB


class _FakeStream:
    cuda_stream = 0

    def wait_stream(self, other) -> None:
        pass

    def synchronize(self) -> None:
        pass


def activate() -> None:
    """Patch torch and the package for emulated runs (see the module docstring)."""
    if "bittorch_b200" in sys.modules:
        raise RuntimeError("activate() must run before bittorch_b200 is imported")
    os.environ["BITTORCH_B200_LIB"] = build()
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import torch

    torch.Tensor.is_cuda = property(lambda self: True)
    stream = _FakeStream()
    torch.cuda.current_stream = lambda device=None: stream
    torch.cuda.device = lambda device=None: contextlib.nullcontext()
    torch.cuda.synchronize = lambda device=None: None
    torch.cuda.set_device = lambda device=None: None
    torch.cuda.is_available = lambda: True
    torch.cuda.empty_cache = lambda: None
    torch.cuda.is_current_stream_capturing = lambda: False

    import bittorch_b200  # noqa: F401  (loads the emulation through BITTORCH_B200_LIB)
    from bittorch_b200 import _C

    assert os.path.samefile(_C.LIB_PATH, LIB), _C.LIB_PATH
    _C._stream = lambda t: 0


def main() -> None:
    """python -m tests.emu.runtime <script.py> [args...]: run a script under the emulation."""
    activate()
    script = sys.argv[1]
    sys.argv = sys.argv[1:]
    runpy.run_path(script, run_name="__main__")


if __name__ == "__main__":
    main()
