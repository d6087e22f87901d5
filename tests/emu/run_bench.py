"""Runs bench.py's GPU arm on the CPU against the host emulation of the C ABI.  TEST INFRASTRUCTURE ONLY.

    python tests/emu/run_bench.py [bench.py arguments]              (one process)
    python -m torch.distributed.run --nproc-per-node 2 ... tests/emu/run_bench.py --gpus 2     (gloo ranks)

Everything that is CUDA plumbing in bench.py is replaced by a host stand-in (graph capture = calling the function
again, CUDA events = perf_counter, pinned memory = plain memory, NCCL = gloo, nvidia-smi = a canned sampler, child
processes = in-process calls) and the workloads are shrunk to sizes the emulation finishes in seconds.  What is left
is the bench's own logic: which kernels are enqueued on which buffers, the sharded chain with its gathers, the
bookkeeping of bytes and launches, and the JSON line.
"""

import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests.emu import runtime  # noqa: E402

runtime.activate()

import torch  # noqa: E402

import bench  # noqa: E402


class FakeEvent:
    def __init__(self, enable_timing=True):
        self.t = None

    def record(self):
        self.t = time.perf_counter()

    def elapsed_time(self, other):
        return max((other.t - self.t) * 1e3, 1e-6)


class FakeGraph:
    def __init__(self, fn):
        self.fn = fn
        self.replays = 0

    def replay(self):
        self.replays += 1
        self.fn()

    def reset(self):
        self.fn = None


def fake_capture(step_fn, warm=3):
    for _ in range(warm):
        step_fn()
    return FakeGraph(step_fn), step_fn()


class FakeSampler(bench.ClockSampler):
    """The real parser and window logic on canned nvidia-smi output: one line per 5 ms while the bench runs."""

    def start(self):
        self.t0 = time.time()
        return self

    def stop(self):
        import datetime

        lines, t = [], self.t0
        while t < time.time():
            stamp = datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
            lines.append(f"{stamp}, 1965, 1965, Not Active, Not Active, Not Active, Active")
            t += 0.005
        self.proc = type("P", (), {"terminate": lambda s: None, "communicate": lambda s, timeout=None: ("\n".join(lines), "")})()
        return super().stop()


torch.cuda.Event = FakeEvent
bench.capture = fake_capture
bench.pin = lambda t: t
bench.ClockSampler = FakeSampler
bench.DIST_BACKEND = "gloo"
bench.device_of = lambda local_rank: torch.device("cpu")
bench.init_kwargs = lambda dev: {}
bench.int8_peak_proxy_tops = lambda: 3000.0
bench.MIN_TIMED_S = 0.05
bench.ROTATE_BYTES = 40e3
bench.run_leg_child = lambda name, local_rank, timeout_s=600: bench.run_leg(
    name, torch.device("cpu"), bench.Ranks(1, 0, None, torch.device("cpu")))
bench.cpu_reference_layer_seconds = lambda budget_s=0.2, min_reps=2, f=bench.cpu_reference_layer_seconds: f(0.2, 2)
bench.cpu_packed_port_layer_seconds = lambda budget_s=0.2, f=bench.cpu_packed_port_layer_seconds: f(0.2)
bench.C5.update({"hidden": 256, "ffn": 512, "q_heads": 4, "kv_heads": 2, "head_dim": 64, "blocks": 2, "model_blocks": 80})
bench.C3.update({"k": 256, "n_small": 128, "n": 320, "layers": 3, "m_list": (1, 4, 16, 40)})
bench.C2.update({"vocab": 65, "dim": 64, "layers": 2, "heads": 2, "ffn": 128, "ctx": 16, "batch": 3, "new_tokens": 8})
bench.C4.update({"vocab": 50, "dim": 128, "layers": 2, "heads": 2, "ffn": 256, "prefill": 8, "decode": 4,
                 "batches": (1, 3), "prefill_rows": 16})
bench.SHARDED_BATCHES = (1, 5, 16)

if __name__ == "__main__":
    bench.main()
