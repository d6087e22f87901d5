"""Runs GPU-marked test files on the CPU against the host emulation of the C ABI.  TEST INFRASTRUCTURE ONLY.

    python tests/emu/run_pytest.py <pytest arguments>

This checks the TESTS (their oracle comparisons, shapes, bookkeeping) and the host-side code they drive, not the
kernels: `.cuda()` / `.to("cuda")` keep tensors on the CPU and the library is tests/emu/libbt_emu.so.
"""

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests.emu import runtime  # noqa: E402

runtime.activate()

import torch  # noqa: E402


def _is_cuda(x):
    return (isinstance(x, str) and x.startswith("cuda")) or (isinstance(x, torch.device) and x.type == "cuda")


def _strip(args, kwargs):
    args = tuple("cpu" if _is_cuda(a) else a for a in args)
    kwargs = {k: ("cpu" if _is_cuda(v) else v) for k, v in kwargs.items()}
    return args, kwargs


_tensor_to, _module_to = torch.Tensor.to, torch.nn.Module.to


def tensor_to(self, *args, **kwargs):
    args, kwargs = _strip(args, kwargs)
    return _tensor_to(self, *args, **kwargs)


def module_to(self, *args, **kwargs):
    args, kwargs = _strip(args, kwargs)
    return _module_to(self, *args, **kwargs)


class _CpuFactories(torch.overrides.TorchFunctionMode):
    """device="cuda" in factory calls (torch.randn(..., device="cuda")) becomes the CPU."""

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if _is_cuda(kwargs.get("device")):
            kwargs = dict(kwargs, device="cpu")
        return func(*args, **kwargs)


_CpuFactories().__enter__()
torch.Tensor.to = tensor_to
torch.nn.Module.to = module_to
torch.Tensor.cuda = lambda self, *a, **k: self
torch.nn.Module.cuda = lambda self, *a, **k: self
torch.cuda.current_device = lambda: 0
os.environ["BITTORCH_B200_EMULATED"] = "1"

import bittorch_b200.utils.decoder as _decoder  # noqa: E402


class _Replayable:
    def __init__(self, fn):
        self.replay = fn


def _fake_capture(step_fn, reset, warm=3):
    """Stands in for the CUDA-graph capture of the greedy loop: the same warm-up protocol, replay = call."""
    for _ in range(warm):
        step_fn()
        reset()
    return _Replayable(step_fn)


_decoder._capture_cuda_graph = _fake_capture

if __name__ == "__main__":
    import pytest

    sys.exit(pytest.main(sys.argv[1:]))
