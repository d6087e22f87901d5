"""Benchmark of the packed ternary linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-sweep]

Headline workload, the SAME global job at every N ("config5-decode-chain"): one decode token (M = 1, bf16
activations) through the projections of 8 Llama-70B-shaped blocks (hidden 8192, FFN 28672, 64 query / 8 key-value
heads): per block q+kv fused 8192 -> 10240, o 8192 -> 8192, gate+up fused 8192 -> 57344, down 28672 -> 8192, random
ternary weights (N(0, sigma) masters, threshold 0.05 max|w|, per-channel fp32 scale).  A block is 214 MB of 2-bit
weights, the chain 1.7 GB, so every step streams from HBM (at 8 GPUs a rank still holds 214 MB > the 126 MB L2).
Each projection is ONE kernel (activation quantizer fused into the GEMV); the next projection reads the first K
columns of the previous output.  With --gpus N > 1 every projection is column-sharded over the N ranks
(rank r owns columns [rN/p, (r+1)N/p)) and followed by one NCCL all-gather of the [M, N/p] outputs: strong
scaling.  A step is replayed from a CUDA graph whose kernels are chained with programmatic dependent launch.

Metric: achieved HBM GB/s on ALGORITHMIC bytes of the whole (unsharded) job: per projection
ceil(K/4)*N + 4N + 2MK + 2MN.

Timing: `steps` graph replays form one block, timed with CUDA events on the launching stream; blocks repeat until
at least MIN_TIMED_S seconds have been timed (so that clocks can be sampled), the reported `ms_per_step` is the
median block / steps, max over ranks.

The one JSON line also carries `roofline` (the chain's kernel, collectives taken out), `e2e` (host buffers through
the public modules), `sharded` (N > 1: kernel time and gather time per projection, batches 1 / 16 / 64, and the
single-GPU chain timed in the same run), and at N = 1: `rooflines` (single shapes), `roofline_gemm` (prefill,
tensor cores), `sweep` (config-3 cells), `config3_stack`, `tokens_per_s` (configs 2 and 4 through the decoder
harness) and `cpu_baseline`.
"""

from __future__ import annotations

import argparse
import datetime
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "packed_ternary_gemv_hbm_gbs"
MIN_TIMED_S = 2.0                  # shortest timed region of the headline (clock samples need wall time)
MAX_TIMED_BLOCKS = 400
DIST_BACKEND = "nccl"
ROTATE_BYTES = 280e6               # packed weights a rotating stack must hold: more than twice the 126 MB L2

# config 5: Llama-70B-shaped projections; `blocks` distinct blocks rotate the weights past L2
C5 = {"hidden": 8192, "ffn": 28672, "q_heads": 64, "kv_heads": 8, "head_dim": 128, "blocks": 8, "model_blocks": 80}
# config 3: the sweep shapes and the 32-layer decode stack
C3 = {"k": 4096, "n_small": 4096, "n": 11008, "layers": 32, "m_list": (1, 4, 16, 256, 2048)}
# config 2: tiny char-LM; config 4: BitNet-b1.58-2B-like stack
C2 = {"vocab": 65, "dim": 256, "layers": 4, "heads": 4, "ffn": 1024, "ctx": 128, "batch": 8, "new_tokens": 128}
C4 = {"vocab": 32000, "dim": 2560, "layers": 30, "heads": 20, "ffn": 6912, "prefill": 2048, "decode": 256,
      "batches": (1, 32), "prefill_rows": 4096}
SHARDED_BATCHES = (1, 16, 64)


def workload_name(c=None) -> str:
    c = c or C5
    shapes = ", ".join(f"{name} {k}->{n}" for name, k, n in c5_projections(c))
    return (f"config5-decode-chain: M=1 bf16 through the projections of {c['blocks']} Llama-70B-shaped blocks "
            f"({shapes}), packed ternary")


def algorithmic_bytes(m: int, k: int, n: int, bias: bool = False) -> int:
    """Bytes one layer call must move: packed W + fp32 scale (+ bias) + bf16 x + bf16 y."""
    return ((k + 3) // 4) * n + 4 * n + (4 * n if bias else 0) + 2 * m * k + 2 * m * n


def c5_projections(c=None):
    """(name, K, N) of the four fused projections of one block."""
    c = c or C5
    kv = c["kv_heads"] * c["head_dim"]
    return [("qkv", c["hidden"], c["q_heads"] * c["head_dim"] + 2 * kv), ("o", c["hidden"], c["hidden"]),
            ("gate_up", c["hidden"], 2 * c["ffn"]), ("down", c["ffn"], c["hidden"])]


def chain_bytes(m: int, c=None) -> int:
    """Algorithmic bytes of one pass over the whole chain (all blocks, unsharded)."""
    c = c or C5
    return c["blocks"] * sum(algorithmic_bytes(m, k, n) for _, k, n in c5_projections(c))


def master_std(k: int) -> float:
    """Keeps activations O(1) through a chain of layers: y ~ sqrt(0.85 K) * x * scale with scale ~ 4 sigma.
    Ternary codes do not depend on it."""
    return 1.0 / (4.0 * math.sqrt(0.85 * k))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_traffic_ratio():
    """dram bytes / algorithmic bytes of one decode GEMV launch, from the committed summary of the ncu capture
    (profiles/gemv_tiled_decode_k4096_n11008.json).  Traffic grows in proportion to the packed weight bytes, so
    other shapes scale it by their algorithmic bytes."""
    path = os.path.join(ROOT, "profiles", "gemv_tiled_decode_k4096_n11008.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return (float(d["dram_bytes_read"]) + float(d["dram_bytes_write"])) / float(d["algorithmic_bytes"]), os.path.basename(path)
    except (OSError, KeyError, ValueError):
        return None, None


# ---------------------------------------------------------------------------------------
# Clocks
# ---------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi (every 100 ms) from `start()` on; `result`
    keeps the samples whose time stamps fall between `mark_begin()` and `mark_end()` (the timed region)."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int, command=None):
        self.index = index
        self.command = command or ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                   "--format=csv,noheader,nounits", "-lms", "100"]
        self.proc = None
        self.t_begin = self.t_end = None
        self.error = None

    def start(self):
        try:
            self.proc = subprocess.Popen(self.command, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError as exc:
            self.proc, self.error = None, f"cannot start nvidia-smi: {exc}"
        return self

    def mark_begin(self):
        self.t_begin = datetime.datetime.now()

    def mark_end(self):
        self.t_end = datetime.datetime.now()

    @staticmethod
    def parse(text: str):
        """[(datetime | None, sm MHz, max MHz, [active reasons])] from nvidia-smi's csv lines."""
        rows = []
        for line in text.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm, mx = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
            except ValueError:
                stamp = None
            active = [name for name, val in zip(ClockSampler.REASONS, parts[3:7]) if val.lower().startswith("active")]
            rows.append((stamp, sm, mx, active))
        return rows

    def stop(self):
        """Ends the sampler; returns (clocks dict | None, reason | None)."""
        if self.proc is None:
            return None, self.error or "sampler was not started"
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = self.parse(out)
        if not rows:
            return None, "nvidia-smi printed no samples"
        inside = [r for r in rows if r[0] is not None and self.t_begin is not None and self.t_end is not None
                  and self.t_begin <= r[0] <= self.t_end]
        used, window = (inside, "timed region") if len(inside) >= 3 else (rows, "whole run (too few stamped samples)")
        return {"sm_mhz": statistics.median(r[1] for r in used), "sm_max_mhz": max(r[2] for r in used),
                "reasons": sorted({name for r in used for name in r[3]}), "samples": len(used),
                "samples_total": len(rows), "window": window}, None


# ---------------------------------------------------------------------------------------
# Graph capture and timing (CUDA events on the launching stream)
# ---------------------------------------------------------------------------------------

def capture(step_fn, warm: int = 3):
    """Runs step_fn a few times eagerly on a side stream, then captures it into a CUDA graph.
    Returns (graph, what step_fn returned during capture)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warm):
            step_fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step_fn()
    return graph, out


def pin(t: torch.Tensor) -> torch.Tensor:
    return t.pin_memory()


class Ranks:
    """The process group as the timing code needs it (a single process when world == 1)."""

    def __init__(self, world: int, rank: int, group=None, device=None):
        self.world, self.rank, self.group, self.device = world, rank, group, device

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)

    def max_over_ranks(self, values):
        """Element-wise maximum of a list of floats over the ranks."""
        if self.world == 1:
            return list(values)
        import torch.distributed as dist
        t = torch.tensor(list(values), dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return [float(v) for v in t.tolist()]


def time_blocks(replay, steps: int, warmup: int, ranks: Ranks, min_s: float = 0.0, on_begin=None, on_end=None):
    """Times blocks of `steps` calls of `replay` until `min_s` seconds are covered (at least one block, the same
    number on every rank).  Barrier + synchronize on both sides of the timed region, one CUDA-event pair per block.
    Returns (median block ms [max over ranks], blocks timed)."""
    for _ in range(warmup):
        replay()
    torch.cuda.synchronize()

    def one_region(n_blocks: int):
        ranks.barrier()
        torch.cuda.synchronize()
        if on_begin is not None:
            on_begin()
        events = []
        for _ in range(n_blocks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                replay()
            e1.record()
            events.append((e0, e1))
        torch.cuda.synchronize()
        if on_end is not None:
            on_end()
        ranks.barrier()
        return ranks.max_over_ranks([a.elapsed_time(b) for a, b in events])

    if min_s <= 0.0:
        return one_region(1)[0], 1
    probe = one_region(1)[0]                                   # sizes the region; not reported
    n_blocks = int(min(MAX_TIMED_BLOCKS, max(1, math.ceil(min_s * 1e3 / max(probe, 1e-3)))))
    n_blocks = int(ranks.max_over_ranks([float(n_blocks)])[0])
    times = one_region(n_blocks)
    return statistics.median(times), n_blocks


# ---------------------------------------------------------------------------------------
# Device-side workloads
# ---------------------------------------------------------------------------------------

class Layer:
    """One packed ternary layer K -> N on this rank: its column shard [n0, n1) as tiled weights + scales."""

    def __init__(self, k: int, n: int, device, rank: int, world: int, gen, keep_packed: bool = False):
        from bittorch_b200 import _C
        from bittorch_b200.parallel import column_range

        self.k, self.n = k, n
        self.n0, self.n1 = column_range(n, rank, world)
        self.n_local = self.n1 - self.n0
        w = torch.randn(n, k, generator=gen, device=device) * master_std(k)      # same masters on every rank
        out = _C.quantize_pack(w[self.n0:self.n1], 0.05, want_packed=True)
        del w
        self.tiled = _C.retile(out["packed_T"], k)
        self.scale = out["scale"]
        self.packed = out["packed_T"] if keep_packed else None


class LayerStack:
    """`layers` distinct layers of one shape K -> N (the config-3 stack and the single-shape roofline cases)."""

    def __init__(self, layers: int, k: int, n: int, device, seed: int = 0, keep_packed: bool = False):
        gen = torch.Generator(device=device).manual_seed(seed)
        self.k, self.n, self.n_local = k, n, n
        self.layers = [Layer(k, n, device, 0, 1, gen, keep_packed) for _ in range(layers)]
        torch.cuda.synchronize()


class ProjectionChain:
    """The config-5 chain on this rank: blocks x (qkv, o, gate_up, down), each column-sharded over `world`."""

    def __init__(self, device, rank: int, world: int, seed: int = 0, keep_packed: bool = False, c=None):
        self.c = c or C5
        self.rank, self.world = rank, world
        gen = torch.Generator(device=device).manual_seed(seed)
        self.names = [name for name, _, _ in c5_projections(self.c)]
        self.layers = []                                       # in execution order
        for _ in range(self.c["blocks"]):
            for _, k, n in c5_projections(self.c):
                self.layers.append(Layer(k, n, device, rank, world, gen, keep_packed))
        torch.cuda.synchronize()

    def local_bytes(self, m: int) -> int:
        return sum(algorithmic_bytes(m, l.k, l.n_local) for l in self.layers)


def launch_linear(layer: Layer, m: int, x: torch.Tensor, ldx: int, y: torch.Tensor, scratch) -> int:
    """Enqueues y[m, n_local] = layer(x[m, :k]) on the current stream.  M <= DECODE_MAX_M: one kernel (activation
    quantizer fused into the GEMV); above: the quantizer kernel, then the tensor-core kernel.  Returns launches."""
    from bittorch_b200 import _C

    lib, st = _C._lib, _C._stream(x)
    if m <= _C.DECODE_MAX_M:
        _C._check(lib.bt_gemv_tiled(x.data_ptr(), _C.BT_BF16, m, layer.k, ldx, layer.tiled.data_ptr(), layer.n_local,
                                    layer.scale.data_ptr(), None, y.data_ptr(), _C.BT_BF16, y.stride(0),
                                    None, None, None, _C.LAUNCH_DEFAULT, st))
        return 1
    xq, sx, xsum = scratch
    _C._check(lib.bt_act_quant_i8(x.data_ptr(), _C.BT_BF16, m, layer.k, ldx, xq.data_ptr(), sx.data_ptr(),
                                  xsum.data_ptr(), st))
    _C._check(lib.bt_gemm_tiled_i8(xq.data_ptr(), sx.data_ptr(), xsum.data_ptr(), m, layer.k, layer.tiled.data_ptr(),
                                   layer.n_local, layer.scale.data_ptr(), None, y.data_ptr(), _C.BT_BF16, y.stride(0),
                                   None, st))
    return 2


def make_chain_step(layers, m: int, x0: torch.Tensor, ranks: Ranks, gather: bool = True, published: bool = False):
    """Returns (step_fn, launches per step) for a chain of layers: the next layer reads the first K columns of the
    previous output.  `published` (one GPU, decode kernel): every layer publishes its output rows' maxima and the
    next layer takes its quantization scale from them (bt_gemv_tiled_chained; one memset of the maxima per step).
    world > 1 and `gather`: each layer's [M, N/p] shard outputs are all-gathered (NCCL) into [p][M][N/p] and, for
    M > 1, transposed into [M, N] by one copy.  world > 1 and not `gather`: the same kernels
    with the collective taken out (each layer reads a fixed input), which is what the gathers' cost is measured
    against.  Buffers are allocated once; step_fn only enqueues."""
    import torch.distributed as dist

    dev = x0.device
    world = ranks.world
    kmax = max(l.k for l in layers)
    scratch = (torch.empty((m, kmax), dtype=torch.int8, device=dev), torch.empty((m,), dtype=torch.float32, device=dev),
               torch.empty((m,), dtype=torch.int32, device=dev))
    y_loc = [torch.empty((m, l.n_local), dtype=torch.bfloat16, device=dev) for l in layers]
    y_all = x_full = x_fixed = None
    if world > 1 and gather:
        y_all = [torch.empty((world * m, l.n_local), dtype=torch.bfloat16, device=dev) for l in layers]
        if m > 1:
            x_full = [torch.empty((m, l.n), dtype=torch.bfloat16, device=dev) for l in layers]
    elif world > 1:
        g = torch.Generator(device=dev).manual_seed(11)
        x_fixed = torch.randn(m, kmax, generator=g, device=dev).to(torch.bfloat16)
    launches = sum(1 if m <= _decode_max_m() else 2 for _ in layers)
    if published:
        from bittorch_b200 import _C
        if world != 1 or m > _C.DECODE_MAX_M:
            raise ValueError("published row maxima need the decode kernel on one GPU")
        amax = _C.new_amax_buffer(len(layers), m, dev)

    def step_published():
        lib, st = _C._lib, _C._stream(x0)
        amax.fill_(0)          # a fill kernel rather than a memset: the chain stays kernel -> kernel inside the graph
        x, ldx = x0, x0.stride(0)
        for i, l in enumerate(layers):
            next_k = layers[i + 1].k if i + 1 < len(layers) else l.n_local
            _C._check(lib.bt_gemv_tiled_chained(
                x.data_ptr(), _C.BT_BF16, m, l.k, ldx, l.tiled.data_ptr(), l.n_local, l.scale.data_ptr(), None,
                y_loc[i].data_ptr(), _C.BT_BF16, l.n_local, amax[i - 1].data_ptr() if i > 0 else None,
                amax[i].data_ptr(), min(next_k, l.n_local), _C.LAUNCH_DEFAULT, st))
            x, ldx = y_loc[i], l.n_local
        return x

    if published:
        return step_published, launches

    def step():
        x, ldx = x0, x0.stride(0)
        for i, l in enumerate(layers):
            launch_linear(l, m, x, ldx, y_loc[i], scratch)
            if world == 1:
                x, ldx = y_loc[i], l.n_local
            elif not gather:
                x, ldx = x_fixed, kmax
            else:
                dist.all_gather_into_tensor(y_all[i], y_loc[i], group=ranks.group)       # rank-major [p][m][N/p]
                if m == 1:
                    x, ldx = y_all[i], l.n                     # [p][1][N/p] is the full row already
                else:
                    x_full[i].view(m, world, l.n_local).copy_(y_all[i].view(world, m, l.n_local).permute(1, 0, 2))
                    x, ldx = x_full[i], l.n
        return x

    return step, launches


def _decode_max_m() -> int:
    from bittorch_b200 import _C
    return _C.DECODE_MAX_M


def time_chain(layers, m: int, x0, ranks: Ranks, gather: bool, steps: int, warmup: int, min_s: float = 0.0,
               on_begin=None, on_end=None, published: bool = False):
    """Captures the chain and times it.  Returns dict(ms_per_step, blocks, launches_per_step, graph)."""
    step, launches = make_chain_step(layers, m, x0, ranks, gather, published)
    graph, _ = capture(step)
    ms_block, blocks = time_blocks(graph.replay, steps, warmup, ranks, min_s, on_begin, on_end)
    return {"ms_per_step": ms_block / steps, "blocks": blocks, "launches_per_step": launches, "graph": graph}


def rotating_kernel_us(stack: LayerStack, m: int, reps: int, ranks: Ranks, float_activations: bool = False,
                       path: str = None) -> float:
    """Average duration (us) of one linear-layer call over the rotating stack (every call reads the same input, so
    launches are independent).  `path`: "fused" = the decode kernel with its quantizer inside (bt_gemv_tiled),
    "int8_rows" = the decode kernel on rows quantized beforehand (bt_gemv_tiled_i8), "tensor_core" = the tcgen05
    kernel on rows quantized beforehand (bt_gemm_tiled_i8), "float" = the float-activation decode kernel
    (bt_gemv_tiled_float).  Default: what the modules run, "fused" up to DECODE_MAX_M rows and "tensor_core" above."""
    from bittorch_b200 import _C

    if path is None:
        path = "float" if float_activations else ("fused" if m <= _C.DECODE_MAX_M else "tensor_core")
    dev = stack.layers[0].tiled.device
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(m, stack.k, generator=g, device=dev).to(torch.bfloat16)
    y = torch.empty((m, stack.n_local), dtype=torch.bfloat16, device=dev)
    lib = _C._lib
    if path in ("int8_rows", "tensor_core"):
        xq, sx, xsum = _C.act_quant_i8(x, want_sum=True)

    def run():
        st = _C._stream(x)
        for l in stack.layers:
            if path == "float":
                _C._check(lib.bt_gemv_tiled_float(x.data_ptr(), _C.BT_BF16, m, stack.k, stack.k, l.tiled.data_ptr(), l.n_local,
                                                  l.scale.data_ptr(), None, y.data_ptr(), _C.BT_BF16, l.n_local,
                                                  _C.LAUNCH_DEFAULT, st))
            elif path == "fused":
                _C._check(lib.bt_gemv_tiled(x.data_ptr(), _C.BT_BF16, m, stack.k, stack.k, l.tiled.data_ptr(), l.n_local,
                                            l.scale.data_ptr(), None, y.data_ptr(), _C.BT_BF16, l.n_local,
                                            None, None, None, _C.LAUNCH_DEFAULT, st))
            elif path == "int8_rows":
                _C._check(lib.bt_gemv_tiled_i8(xq.data_ptr(), sx.data_ptr(), m, stack.k, l.tiled.data_ptr(), l.n_local,
                                               l.scale.data_ptr(), None, y.data_ptr(), _C.BT_BF16, l.n_local, None,
                                               _C.LAUNCH_DEFAULT, st))
            else:
                _C._check(lib.bt_gemm_tiled_i8(xq.data_ptr(), sx.data_ptr(), xsum.data_ptr(), m, stack.k,
                                               l.tiled.data_ptr(), l.n_local, l.scale.data_ptr(), None, y.data_ptr(),
                                               _C.BT_BF16, l.n_local, None, st))
        return y

    graph, _ = capture(run)
    ms, _ = time_blocks(graph.replay, reps, 3, ranks)
    graph.reset()
    return ms * 1e3 / (reps * len(stack.layers))


def act_quant_us(m: int, k: int, reps: int, ranks: Ranks, dev) -> float:
    """Average duration (us) of the stand-alone activation quantizer on [m, k] bf16 rows (32 calls per replay)."""
    from bittorch_b200 import _C

    x = torch.randn(m, k, generator=torch.Generator(device=dev).manual_seed(2), device=dev).to(torch.bfloat16)
    xq = torch.empty((m, k), dtype=torch.int8, device=dev)
    sx = torch.empty((m,), dtype=torch.float32, device=dev)
    xsum = torch.empty((m,), dtype=torch.int32, device=dev)
    calls = 32

    def run():
        st = _C._stream(x)
        for _ in range(calls):
            _C._check(_C._lib.bt_act_quant_i8(x.data_ptr(), _C.BT_BF16, m, k, k, xq.data_ptr(), sx.data_ptr(), xsum.data_ptr(), st))

    graph, _ = capture(run)
    ms, _ = time_blocks(graph.replay, reps, 3, ranks)
    graph.reset()
    return ms * 1e3 / (reps * calls)


# ---------------------------------------------------------------------------------------
# End to end through the public modules: host buffers in, host buffers out
# ---------------------------------------------------------------------------------------

def build_e2e(chain: ProjectionChain, m: int, ranks: Ranks):
    """The call a user makes: the chain as TernaryLinearInference modules (one GPU) or
    ColumnParallelTernaryLinear modules (column shards + all-gather), captured in a CUDA graph, fed from pinned
    host memory and read back to pinned host memory every step.  Returns (step_fn, h2d bytes, d2h bytes)."""
    from bittorch_b200.nn import TernaryLinearInference
    from bittorch_b200.parallel import ColumnParallelTernaryLinear

    dev = chain.layers[0].tiled.device
    mods = []
    for l in chain.layers:
        if ranks.world == 1:
            mods.append(TernaryLinearInference(l.k, l.n, l.packed, l.scale))
        else:
            mods.append(ColumnParallelTernaryLinear(l.k, l.n, l.packed, l.scale, None, ranks.group))
    k0, n_last = chain.layers[0].k, chain.layers[-1].n
    x_host = pin(torch.randn(m, k0, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16))
    y_host = pin(torch.empty((m, n_last), dtype=torch.bfloat16))
    x_dev = torch.empty((m, k0), dtype=torch.bfloat16, device=dev)

    def forward():
        x = x_dev
        for i, mod in enumerate(mods):
            y = mod(x)
            if i + 1 < len(mods):
                x = y[:, :chain.layers[i + 1].k]
        return y

    with torch.no_grad():
        graph, y_dev = capture(forward)

    def step():
        x_dev.copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(y_dev, non_blocking=True)

    return step, x_host.numel() * 2, y_host.numel() * 2, graph


# ---------------------------------------------------------------------------------------
# CPU baseline: the reference's python backend, restated (oracle/), on the host cores
# ---------------------------------------------------------------------------------------

def cpu_sample_name(c=None) -> str:
    h = (c or C5)["hidden"]
    return (f"one o-projection of the chain (K={h}->N={h}, M=1, bf16) per step with the eager restatement of the "
            "reference's python backend: fp32 master re-quantized and straight-through rewrite on every call, "
            "dense F.linear")


def cpu_sample_tensors(c=None):
    c = c or C5
    g = torch.Generator().manual_seed(0)
    h = c["hidden"]
    w = torch.randn(h, h, generator=g) * master_std(h)
    x = torch.randn(1, h, generator=g).to(torch.bfloat16)
    return x, w


def cpu_reference_layer_seconds(budget_s: float = 15.0, min_reps: int = 3):
    """Median seconds of one sample layer with the eager restatement of the reference's CPU python backend, all
    host threads.  Returns (seconds, reps, threads)."""
    import oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, w = cpu_sample_tensors()
    for _ in range(2):
        oracle.ref_python_forward(x, w)
    samples, t_begin = [], time.perf_counter()
    while len(samples) < min_reps or (time.perf_counter() - t_begin < budget_s and len(samples) < 200):
        t0 = time.perf_counter()
        oracle.ref_python_forward(x, w)
        samples.append(time.perf_counter() - t0)
    return statistics.median(samples), len(samples), threads


def cpu_packed_port_layer_seconds(budget_s: float = 8.0):
    """The packed inference path on the CPU (C oracle: activation quantizer + integer contraction from packed
    bytes), all host threads, the same sample layer."""
    import oracle

    threads = os.cpu_count() or 1
    x, w = cpu_sample_tensors()
    codes, scale = oracle.ternarize(w.numpy(), 0.05)
    packed = oracle.pack_transposed(codes)
    k = w.shape[1]
    xf = x.float().numpy()
    oracle.packed_forward_i8_threaded(xf, packed, k, scale, None, threads)
    samples, t_begin = [], time.perf_counter()
    while len(samples) < 3 or (time.perf_counter() - t_begin < budget_s and len(samples) < 200):
        t0 = time.perf_counter()
        oracle.packed_forward_i8_threaded(xf, packed, k, scale, None, threads)
        samples.append(time.perf_counter() - t0)
    return statistics.median(samples), len(samples), threads


def base_config(world: int):
    return {"workload": workload_name(), "M": 1, "blocks": C5["blocks"],
            "projections": [{"name": n, "K": k, "N": nn} for n, k, nn in c5_projections()],
            "l2": f"weights rotate over {C5['blocks']} blocks ({chain_bytes(1) / 1e6:.0f} MB, "
                  f"{chain_bytes(1) / 1e6 / max(world, 1):.0f} MB per GPU), larger than the 126 MB L2",
            "parallelism": "single GPU" if world == 1 else
            f"column-parallel x{world} (rank r owns columns [rN/p,(r+1)N/p) of every projection) + one NCCL "
            "all-gather per projection",
            "prefill_not_sharded": "a 4096-token prefill gathers 2*M*N/p = 29 MB per rank and projection at p=8 "
                                   "(~0.23 ms at 900 GB/s) against ~0.11 ms of sharded GEMM: sharding pays only where "
                                   "packed-weight bytes >> gathered bytes, i.e. M << K/(8p)",
            "launch": "CUDA graph replay, kernels chained by programmatic dependent launch"}


def run_reference_arm(args) -> None:
    """--impl reference: the reference's CPU implementation of the path (eager restatement of its python backend,
    oracle/), all host threads; a step is one sample layer of the chain."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, w = cpu_sample_tensors()
    for _ in range(max(args.warmup, 1)):
        oracle.ref_python_forward(x, w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.ref_python_forward(x, w)
    per_layer = (time.perf_counter() - t0) / args.steps
    gbs = algorithmic_bytes(1, w.shape[1], w.shape[0]) / per_layer / 1e9
    config = base_config(args.gpus)
    config["sample"] = cpu_sample_name()
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": cpu_sample_name()},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
# Secondary legs (N = 1): single-shape rooflines, config-3 stack and sweep, tokens/s
# ---------------------------------------------------------------------------------------

def int8_peak_proxy_tops() -> float:
    """Measured yardstick for the int8 tensor-core peak: torch._int_mm 8192^3, best of 5."""
    try:
        a = torch.randint(-127, 128, (8192, 8192), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (8192, 8192), device="cuda", dtype=torch.int8)
        for _ in range(2):
            torch._int_mm(a, b)
        best = float("inf")
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192**3 / (best * 1e-3) / 1e12
    except Exception:      # noqa: BLE001  (a yardstick only)
        return float("nan")


def gemv_roofline(us: float, m: int, k: int, n: int, peaks, traffic_ratio, traffic_source, note: str = ""):
    b = algorithmic_bytes(m, k, n)
    achieved = b / us / 1e3
    return {"bound": "hbm", "kernel": f"gemv_tiled_kernel<{m},fused>", "K": k, "N": n, "M": m, "achieved": achieved,
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_source": peaks["source"], "frac_of_nominal_8tbs": achieved / 8000.0, "us_per_launch": us,
            "algorithmic_bytes_per_launch": b,
            "traffic": None if traffic_ratio is None else int(round(b * traffic_ratio)),
            "traffic_source": traffic_source, **({"note": note} if note else {})}


def run_config3(peaks, dev, ranks: Ranks, traffic):
    """Config-3 cells: kernel-only times over weights rotated past L2, the 32-layer decode stack as a chain, and
    the prefill GEMM's roofline object."""
    rows, out = [], {}
    int8_proxy = int8_peak_proxy_tops()
    for n in (C3["n_small"], C3["n"]):
        k = C3["k"]
        layers = max(C3["layers"], int(math.ceil(ROTATE_BYTES / (k // 4 * n))))          # >= 2 x L2 of packed weights
        stack = LayerStack(layers, k, n, dev, seed=k + n)
        for m in C3["m_list"]:
            us = rotating_kernel_us(stack, m, 10 if m <= 16 else 3, ranks)
            row = {"K": k, "N": n, "M": m, "us": us}
            if m <= 16:     # decode sizes are measured in bytes streamed
                gbs = algorithmic_bytes(m, k, n) / us / 1e3
                row.update({"kernel": "gemv_tiled" if m <= _decode_max_m() else "gemm_tcgen05", "gbs": gbs,
                            "frac_hbm_measured": gbs / peaks["hbm_gbs"], "frac_hbm_nominal_8tbs": gbs / 8000.0})
            if m > _decode_max_m():       # tensor-core sizes on integer operations
                tops = 2.0 * m * n * k / us / 1e6
                row.update({"kernel": "gemm_tcgen05", "int8_tops": tops, "frac_int8_nominal_4500": tops / 4500.0,
                            "frac_int8_mm_proxy": tops / int8_proxy if int8_proxy == int8_proxy else None})
            rows.append(row)
        if n == C3["n"]:
            # the 32-layer stack as a dependent chain (each layer reads the first K columns of the previous output)
            x0 = torch.randn(1, k, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(dev)
            r = time_chain(stack.layers[:C3["layers"]], 1, x0, ranks, False, 50, 5)
            r.pop("graph").reset()
            b = C3["layers"] * algorithmic_bytes(1, k, n)
            out["config3_stack"] = {"workload": f"M=1 bf16, {C3['layers']} layers of K={k}->N={n}, dependent chain",
                                    "ms_per_step": r["ms_per_step"], "gbs": b / r["ms_per_step"] / 1e6,
                                    "frac_hbm_measured": b / r["ms_per_step"] / 1e6 / peaks["hbm_gbs"]}
        del stack
        torch.cuda.empty_cache()
    cell = next(r for r in rows if r["M"] == max(C3["m_list"]) and r["N"] == C3["n"])
    measured_peak = 2.0 * peaks["bf16_tflops"]
    out["roofline_gemm"] = {
        "bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel (tcgen05.mma.cta_group::2.kind::i8)",
        "M": cell["M"], "K": cell["K"], "N": cell["N"], "achieved": cell["int8_tops"], "unit": "TOP/s",
        "peak": measured_peak, "peak_source": f"2 x bf16_tflops ({peaks['source']}; int8 issues at twice the bf16 rate)",
        "frac": cell["int8_tops"] / measured_peak, "peak_nominal": 4500.0, "frac_of_nominal": cell["int8_tops"] / 4500.0,
        "int8_mm_proxy_tops": int8_proxy if int8_proxy == int8_proxy else None, "us_per_launch": cell["us"],
        "algorithmic_ops_per_launch": 2 * cell["M"] * cell["K"] * cell["N"],
        "tensor_pipe_active_pct_ncu": _gemm_profile_pct(), "traffic": None}
    out["sweep"] = rows
    return out


def _gemm_profile_pct():
    """Tensor-pipe activity of the prefill GEMM from the committed ncu summary (profiles/*.json)."""
    try:
        with open(os.path.join(ROOT, "profiles", "gemm_tcgen05_prefill_m2048_k4096_n11008.json")) as f:
            return json.load(f).get("tensor_pipe_active_pct_of_elapsed")
    except (OSError, ValueError):
        return None


def run_single_shape_rooflines(peaks, dev, ranks: Ranks, traffic):
    """M = 1 decode GEMV alone on single shapes, weights rotated past L2."""
    ratio, src = traffic
    out = []
    for k, n in ((C3["k"], C3["n"]), (C5["hidden"], C5["ffn"]), (C5["hidden"], 2 * C5["ffn"])):
        layers = max(4, int(math.ceil(ROTATE_BYTES / (k // 4 * n))))
        stack = LayerStack(layers, k, n, dev, seed=k + n + 1)
        us = rotating_kernel_us(stack, 1, 10, ranks)
        out.append(gemv_roofline(us, 1, k, n, peaks, ratio, src, "independent launches over rotating weights"))
        if (k, n) == (C3["k"], C3["n"]):
            # the same layer with floating-point activations (four digit planes through the same pipeline)
            us_f = rotating_kernel_us(stack, 1, 10, ranks, float_activations=True)
            entry = gemv_roofline(us_f, 1, k, n, peaks, None, None, "float activations (bt_gemv_tiled_float), same weights")
            entry["kernel"] = "gemv_tiled_kernel<4,planes>"
            entry["relative_to_int8_path"] = us / us_f
            out.append(entry)
        del stack
        torch.cuda.empty_cache()
    return out


def run_decode_batch_paths(peaks, dev, ranks: Ranks):
    """Where a small batch should run: for M = 1 .. 32 rows on two layer shapes, the kernel-only time of the decode
    kernel with its quantizer inside, the decode kernel on int8 rows (plus the stand-alone quantizer, which fused
    elementwise producers make unnecessary) and the tensor-core kernel on int8 rows, weights rotated past L2.  The
    table is what the DECODE_MAX_M switch-over of the modules rests on."""
    from bittorch_b200 import _C

    out = {"decode_max_m_in_use": _C.DECODE_MAX_M, "shapes": []}
    for k, n in ((C3["k"], C3["n"]), (C5["hidden"], C5["ffn"])):
        layers = max(4, int(math.ceil(ROTATE_BYTES / (k // 4 * n))))
        stack = LayerStack(layers, k, n, dev, seed=k + n + 2)
        rows = []
        for m in (1, 2, 4, 8, 16, 32):
            row = {"M": m, "act_quant_us": act_quant_us(m, k, 10, ranks, dev)}
            for path in ("fused", "int8_rows", "tensor_core"):
                if (path == "tensor_core" and m < 4) or (path != "tensor_core" and m > _C.GEMV_MAX_M):
                    continue
                try:
                    us = rotating_kernel_us(stack, m, 10, ranks, path=path)
                    row[path + "_us"] = us
                    row[path + "_frac_hbm_measured"] = algorithmic_bytes(m, k, n) / us / 1e3 / peaks["hbm_gbs"]
                except Exception as exc:      # noqa: BLE001  (a refused shape costs its cell only)
                    row[path + "_error"] = f"{type(exc).__name__}: {exc}"[:200]
                    torch.cuda.synchronize()
            # all-in cost from floating-point rows / from int8 rows a fused producer already wrote
            from_float = {p_: row[p_ + "_us"] + (0.0 if p_ == "fused" else row["act_quant_us"])
                          for p_ in ("fused", "int8_rows", "tensor_core") if p_ + "_us" in row}
            from_int8 = {p_: row[p_ + "_us"] for p_ in ("int8_rows", "tensor_core") if p_ + "_us" in row}
            row["fastest_from_float_rows"] = min(from_float, key=from_float.get) if from_float else None
            row["fastest_from_int8_rows"] = min(from_int8, key=from_int8.get) if from_int8 else None
            rows.append(row)
        out["shapes"].append({"K": k, "N": n, "rows": rows})
        del stack
        torch.cuda.empty_cache()
    return out


def _decoder_tools(dev):
    """Helpers of the two tokens/s legs: model builder, event timer, capture hook for the greedy loop."""
    from bittorch_b200.nn import verify_weight_contents
    from bittorch_b200.utils.decoder import DecoderConfig, TernaryDecoder

    def build(vocab, dim, layers, heads, ffn, max_seq, dtype):
        cfg = DecoderConfig(vocab_size=vocab, dim=dim, n_layers=layers, n_heads=heads, ffn_dim=ffn, max_seq_len=max_seq,
                            backend="cuda")
        torch.manual_seed(0)
        with torch.device(dev):
            model = TernaryDecoder(cfg)
        model = model.to(dtype).eval()
        model.to_inference()                                   # random-init masters -> packed ternary layers
        verify_weight_contents(model, False)                   # final weights: no host read-back per eager forward
        torch.cuda.empty_cache()
        return model

    def timed(fn) -> float:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3

    def capture_loop(step_fn, reset):
        for _ in range(3):
            step_fn()
            reset()
        torch.cuda.synchronize()
        return capture(step_fn, warm=0)[0]

    return build, timed, capture_loop


def tokens_config2(dev, ranks: Ranks):
    """Config 2 through the decoder harness in its packed inference form: batch 8, one random prompt token per
    sequence, 128 greedy tokens (positions 0..127 = the context), one CUDA-graph launch per token."""
    from bittorch_b200.utils.decoder import GreedyDecodeGraph

    build, timed, capture_loop = _decoder_tools(dev)
    c = C2
    model = build(c["vocab"], c["dim"], c["layers"], c["heads"], c["ffn"], c["ctx"], torch.float32)
    first = torch.randint(0, c["vocab"], (c["batch"], 1), generator=torch.Generator().manual_seed(3)).to(dev)
    loop = GreedyDecodeGraph(model, c["batch"], capture=capture_loop)
    loop.start(first, 0)
    loop.run(c["new_tokens"])                                  # warm replay of the whole generation
    loop.start(first, 0)
    sec = timed(lambda: loop.run(c["new_tokens"]))
    loop.graph.reset()
    return {"workload": f"{c['layers']}-layer decoder d={c['dim']}, {c['heads']} heads, FFN {c['ffn']}, vocab {c['vocab']}, "
                        f"batch {c['batch']}, {c['new_tokens']} greedy tokens, fp32 activations, random-init ternary weights",
            "decode_tokens_per_s": c["batch"] * c["new_tokens"] / sec, "ms_per_token_step": sec * 1e3 / c["new_tokens"],
            "launch": "one CUDA graph replay per token"}


def tokens_config4(dev, ranks: Ranks):
    """Config 4 through the decoder harness: prefill 2048 tokens (eager, at most `prefill_rows` rows per pass) and
    256 greedy tokens (one CUDA-graph launch per token), batch 1 and 32, bf16."""
    from bittorch_b200.utils.decoder import GreedyDecodeGraph

    build, timed, capture_loop = _decoder_tools(dev)
    c = C4
    model = build(c["vocab"], c["dim"], c["layers"], c["heads"], c["ffn"], c["prefill"] + c["decode"], torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    rows = []
    for batch in c["batches"]:
        prompt = torch.randint(0, c["vocab"], (batch, c["prefill"]), generator=g).to(dev)
        cache = model.new_cache(batch)
        per_pass = max(1, c["prefill_rows"] // c["prefill"])      # sequences per prefill pass
        last = torch.empty((batch, 1), dtype=torch.long, device=dev)

        @torch.no_grad()
        def prefill():
            for b0 in range(0, batch, per_pass):
                b1 = min(batch, b0 + per_pass)
                view = [(kc[b0:b1], vc[b0:b1]) for kc, vc in cache]
                logits = model(prompt[b0:b1], view, 0, last_only=True)      # a prefill needs the last position's logits
                last[b0:b1] = logits[:, -1].argmax(dim=-1, keepdim=True)

        prefill()                                              # warm-up (builds the layers' derived buffers)
        t_prefill = timed(prefill)
        loop = GreedyDecodeGraph(model, batch, cache=cache, capture=capture_loop)
        loop.start(last, c["prefill"])
        loop.run(min(8, c["decode"]))                          # warm replays
        loop.start(last, c["prefill"])
        t_decode = timed(lambda: loop.run(c["decode"]))
        rows.append({"batch": batch, "prefill_tokens_per_s": batch * c["prefill"] / t_prefill,
                     "decode_tokens_per_s": batch * c["decode"] / t_decode,
                     "ms_per_decode_step": t_decode * 1e3 / c["decode"], "prefill_ms": t_prefill * 1e3,
                     "prefill_sequences_per_pass": per_pass})
        loop.graph.reset()
        del loop, cache
        torch.cuda.empty_cache()
    return {"workload": f"{c['layers']}-layer decoder hidden {c['dim']}, FFN {c['ffn']} gated, {c['heads']} heads, "
                        f"vocab {c['vocab']}, prefill {c['prefill']} + decode {c['decode']}, bf16, random-init ternary weights",
            "rows": rows, "launch": "prefill eager, decode one CUDA graph replay per token"}


def selftest_published(dev) -> dict:
    """The chain with published row maxima against the plain chain on a small stack: every layer's output must be
    the same bits.  Run in a child process before the headline uses that path."""
    from bittorch_b200 import _C

    ranks = Ranks(1, 0, None, dev)
    ok = True
    for (k, n, count, m) in ((C3["k"], C3["k"], 3, 1), (C3["k"], C3["n"], 2, 1), (1024, 2560, 3, 4)):
        stack = LayerStack(count, k, n, dev, seed=k + n + m)
        x0 = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).to(dev)
        plain = make_chain_step(stack.layers, m, x0, ranks, False, False)[0]().clone()
        chained = make_chain_step(stack.layers, m, x0, ranks, False, True)[0]().clone()
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(plain.view(torch.int16), chained.view(torch.int16)))
        del stack
    # and one block of the headline chain itself: its four shapes, the long-row branch (K = 28672) included
    block = ProjectionChain(dev, 0, 1, seed=3, c=dict(C5, blocks=2))
    x0 = torch.randn(1, block.layers[0].k, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(dev)
    plain = make_chain_step(block.layers, 1, x0, ranks, False, False)[0]().clone()
    chained = make_chain_step(block.layers, 1, x0, ranks, False, True)[0]().clone()
    torch.cuda.synchronize()
    ok = ok and bool(torch.equal(plain.view(torch.int16), chained.view(torch.int16)))
    return {"ok": ok and _C.device_status(dev) == 0}


LEGS = ("rooflines", "config3", "decode_batch_paths", "tokens_config2", "tokens_config4")


def run_leg(name: str, dev, ranks: Ranks):
    """One secondary leg on this process's GPU; returns its JSON-able result."""
    peaks, traffic = load_peaks(), load_traffic_ratio()
    if name == "rooflines":
        return run_single_shape_rooflines(peaks, dev, ranks, traffic)
    if name == "config3":
        return run_config3(peaks, dev, ranks, traffic)
    if name == "decode_batch_paths":
        return run_decode_batch_paths(peaks, dev, ranks)
    if name == "selftest_published":
        return selftest_published(dev)
    if name == "tokens_config2":
        return tokens_config2(dev, ranks)
    if name == "tokens_config4":
        return tokens_config4(dev, ranks)
    raise ValueError(f"unknown leg {name!r}")


def run_leg_child(name: str, local_rank: int, timeout_s: int = 600):
    """Runs `python bench.py --leg name` on the same GPU and returns its result (or {"error": ...})."""
    env = dict(os.environ, LOCAL_RANK=str(local_rank), RANK="0", WORLD_SIZE="1")
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--leg", name], capture_output=True, text=True,
                             timeout=timeout_s, env=env, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"error": f"leg {name} did not finish in {timeout_s} s"}
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    if out.returncode != 0 or not lines:
        tail = (out.stderr or out.stdout).strip().splitlines()[-1:] or [""]
        return {"error": f"leg {name} exited {out.returncode}: {tail[0][:300]}"}
    return json.loads(lines[-1])["result"]


def leg_main(name: str) -> None:
    from bittorch_b200 import _C

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = device_of(local_rank)
    result = run_leg(name, dev, Ranks(1, 0, None, dev))
    print(json.dumps({"leg": name, "result": result, "device_status": _C.device_status(dev)}), flush=True)


def run_case(case: str, m, k, n) -> None:
    """A few eager launches of one kernel (3 warm-up + 6), sized for a profiler capture: inputs past L2 where the
    kernel is bandwidth-bound, well under 1 GB on the device."""
    from bittorch_b200 import _C

    dev = device_of(0)
    torch.cuda.set_device(0)
    k = k or C3["k"]
    n = n or C3["n"]
    if case in ("gemv", "gemm"):
        m = m or (1 if case == "gemv" else 2048)
        layers = max(2, int(math.ceil(0.6 * ROTATE_BYTES / (k // 4 * n)))) if case == "gemv" else 2
        stack = LayerStack(layers, k, n, dev, seed=0)
        g = torch.Generator(device=dev).manual_seed(1)
        xq = torch.randint(-127, 128, (m, k), generator=g, device=dev, dtype=torch.int8)
        sx = torch.full((m,), 0.01, device=dev)
        x = torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16)
        for i in range(9):
            l = stack.layers[i % len(stack.layers)]
            if case == "gemv":      # the bench's dominant kernel: fused quantizer + GEMV
                _C.gemv_tiled(x, l.tiled, k, n, l.scale, None)
            else:
                _C.gemm_tiled_i8(xq, sx, l.tiled, k, n, l.scale, None, torch.bfloat16)
    elif case == "quantize":
        g = torch.Generator(device=dev).manual_seed(1)
        ws = [torch.randn(n, k, generator=g, device=dev) for _ in range(3)]
        for i in range(9):
            _C.quantize_pack(ws[i % 3], 0.05, want_packed=True)
    else:
        m = m or 2048
        g = torch.Generator(device=dev).manual_seed(1)
        xs = [torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
        for i in range(9):
            _C.act_quant_i8(xs[i % 3])
    torch.cuda.synchronize()
    print(json.dumps({"case": case, "m": m, "k": k, "n": n, "device_status": _C.device_status(dev)}))


# ---------------------------------------------------------------------------------------
# Main
# ---------------------------------------------------------------------------------------

def sharded_section(dev, ranks: Ranks, chain: ProjectionChain, steps: int, warmup: int, headline):
    """N > 1: for decode batches 1 / 16 / 64 the sharded chain with and without its all-gathers, and the unsharded
    chain on one GPU (every rank times its own copy at once).  Times are per block (4 projections), max over ranks."""
    blocks, nproj = chain.c["blocks"], len(chain.names)
    full = ProjectionChain(dev, 0, 1, seed=0, c=chain.c)
    solo = Ranks(1, 0, None, dev)
    rows, graphs = [], []
    for m in SHARDED_BATCHES:
        x0 = torch.randn(m, chain.layers[0].k, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(dev)
        row = {"M": m}
        try:
            if m == 1:
                with_gather = headline
            else:
                with_gather = time_chain(chain.layers, m, x0, ranks, True, steps, warmup)
                graphs.append(with_gather.pop("graph"))
            no_gather = time_chain(chain.layers, m, x0, ranks, False, steps, warmup)
            no_gather.pop("graph").reset()
            ranks.barrier()
            single = time_chain(full.layers, m, x0, solo, False, steps, warmup)
            single.pop("graph").reset()
            single_ms = ranks.max_over_ranks([single["ms_per_step"]])[0]
            # the sharded chain's last output (gathered) against the unsharded chain's, bit for bit
            y_sharded = make_chain_step(chain.layers, m, x0, ranks, True)[0]().reshape(m, -1).clone()
            y_single = make_chain_step(full.layers, m, x0, solo, False)[0]().reshape(m, -1)
            torch.cuda.synchronize()
            row["matches_single_gpu"] = bool(torch.equal(y_sharded, y_single))
            us = lambda r: r * 1e3 / blocks                     # noqa: E731  per block
            row.update({
                "us_per_block_sharded": us(with_gather["ms_per_step"]),
                "us_per_block_kernels_only": us(no_gather["ms_per_step"]),
                "us_per_block_gathers": us(with_gather["ms_per_step"] - no_gather["ms_per_step"]),
                "us_per_gather": us(with_gather["ms_per_step"] - no_gather["ms_per_step"]) / nproj,
                "us_per_block_single_gpu": us(single_ms),
                "speedup_vs_single_gpu": single_ms / with_gather["ms_per_step"],
                "speedup_kernels_only": single_ms / no_gather["ms_per_step"],
                "tokens_per_s_projections_of_an_80_block_model":
                    m / (us(with_gather["ms_per_step"]) * 1e-6 * chain.c["model_blocks"]),
                "gather_bytes_per_rank_and_block": sum(2 * m * l.n_local for l in chain.layers[:nproj]),
            })
        except Exception as exc:      # noqa: BLE001  (a secondary row must not take the headline with it)
            if m == 1:
                raise
            row["error"] = f"{type(exc).__name__}: {exc}"[:300]
        rows.append(row)
    del full
    torch.cuda.empty_cache()
    return {"workload": "config-5 chain column-sharded; per block = 4 projections; kernels_only = the same launches "
                        "with the all-gathers taken out (each projection reads a fixed input)",
            "rows": rows}, graphs


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--plain-chain", action="store_true",
                    help="one GPU: do not let layers publish their row maxima (bt_gemv_tiled instead of bt_gemv_tiled_chained)")
    ap.add_argument("--no-sweep", action="store_true",
                    help="headline only: skip the single-shape rooflines, the config-3 cells, tokens/s and the CPU baseline")
    ap.add_argument("--case", default=None, choices=["gemv", "gemm", "quantize", "actquant"],
                    help="profiling aid: a few eager launches of one kernel on a small case, then exit")
    ap.add_argument("--leg", default=None, choices=list(LEGS) + ["selftest_published"], help="run one secondary leg and print its result")
    ap.add_argument("--case-m", type=int, default=None, help="rows of X for --case")
    ap.add_argument("--case-k", type=int, default=None, help="in_features for --case")
    ap.add_argument("--case-n", type=int, default=None, help="out_features for --case")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)
    if args.case is not None:
        run_case(args.case, args.case_m, args.case_k, args.case_n)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.leg is not None:
        leg_main(args.leg)
        return

    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU path")
    from bittorch_b200 import _C   # fails loudly when the library is missing

    torch.cuda.set_device(local_rank)
    dev = device_of(local_rank)
    group = None
    if world > 1:
        dist.init_process_group(DIST_BACKEND, timeout=datetime.timedelta(seconds=180), **init_kwargs(dev))
        group = dist.group.WORLD
    ranks = Ranks(world, rank, group, dev)
    peaks = load_peaks()
    traffic = load_traffic_ratio()

    chain = ProjectionChain(dev, rank, world, seed=0, keep_packed=True)
    x0 = torch.randn(1, chain.layers[0].k, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(dev)

    # One GPU: layers hand their row maxima to the next layer (bt_gemv_tiled_chained) once that path has reproduced
    # the plain chain bit for bit in a child process on this GPU; the plain chain is timed beside it.
    published, published_note = False, None
    if world == 1 and not args.plain_chain:
        res = run_leg_child("selftest_published", local_rank, 300)
        published = res.get("ok") is True
        if not published:
            published_note = res.get("error", "outputs differ from the plain chain")
    sampler = ClockSampler(local_rank).start()                 # before every warm-up of the timed chains
    quick = {}
    if published:                                              # a short run of each; the headline takes the faster
        try:
            for name, flag in (("plain", False), ("published_row_maxima", True)):
                r = time_chain(chain.layers, 1, x0, ranks, True, args.steps, args.warmup, 0.3, published=flag)
                r.pop("graph").reset()
                quick[name] = r["ms_per_step"]
            published = quick["published_row_maxima"] <= quick["plain"]
        except Exception as exc:      # noqa: BLE001  (the plain chain is the fallback, not an error of the bench)
            published, published_note = False, f"{type(exc).__name__}: {exc}"[:300]
            torch.cuda.synchronize()

    # ---- headline: the chain (with its all-gathers when sharded), >= MIN_TIMED_S of timed replays -------------
    head = time_chain(chain.layers, 1, x0, ranks, True, args.steps, args.warmup, MIN_TIMED_S,
                      sampler.mark_begin, sampler.mark_end, published)
    clocks, clocks_reason = sampler.stop()
    ms_per_step = head["ms_per_step"]
    job_bytes = chain_bytes(1)
    value = job_bytes / ms_per_step / 1e6
    gpu_launches = head["launches_per_step"] * args.steps * head["blocks"] * world
    keep_graphs = [head["graph"]]

    # ---- the chain's kernel alone (collectives taken out): the roofline object ----------------------------------
    if world == 1:
        kern_ms = ms_per_step
    else:
        r = time_chain(chain.layers, 1, x0, ranks, False, args.steps, args.warmup, 0.5)
        r.pop("graph").reset()
        kern_ms = r["ms_per_step"]
    local_bytes = chain.local_bytes(1)
    us_launch = kern_ms * 1e3 / head["launches_per_step"]
    achieved = local_bytes / kern_ms / 1e6
    ratio, ratio_src = traffic
    roofline = {"bound": "hbm", "kernel": "gemv_tiled_kernel<1,fused>" + (" (row maxima published)" if published else ""),
                "scope": f"average over the chain's {head['launches_per_step']} launches per step on one rank "
                         "(4 shapes), dependent launches, collectives taken out",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": peaks["source"], "frac_of_nominal_8tbs": achieved / 8000.0, "us_per_launch": us_launch,
                "algorithmic_bytes_per_launch": local_bytes / head["launches_per_step"],
                "traffic": None if ratio is None else int(round(local_bytes / head["launches_per_step"] * ratio)),
                "traffic_source": None if ratio is None else
                f"{ratio_src}: dram bytes / algorithmic bytes = {ratio:.4f} on the 4096x11008 capture, scaled by bytes"}

    # ---- end to end: host buffers through the public modules ------------------------------------------------------
    e2e_step, h2d, d2h, e2e_graph = build_e2e(chain, 1, ranks)
    keep_graphs.append(e2e_graph)
    e_ms, _ = time_blocks(e2e_step, args.steps, args.warmup, ranks, 0.5)
    e_ms_step = e_ms / args.steps
    e2e = {"value": job_bytes / e_ms_step / 1e6, "unit": "GB/s", "ms_per_step": e_ms_step,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "api": "TernaryLinearInference chain" if world == 1 else "ColumnParallelTernaryLinear chain"}

    config = base_config(world)
    chain_variants = None
    if world == 1:
        config["row_maxima"] = ("published by the producing layer (bt_gemv_tiled_chained), one memset per step"
                                if published else "reduced by the consuming layer (bt_gemv_tiled)")
        chain_variants = {"headline": "published_row_maxima" if published else "plain"}
        for name, ms in quick.items():
            chain_variants[name] = {"ms_per_step": ms, "gbs": job_bytes / ms / 1e6}
        if published_note is not None:
            chain_variants["published_row_maxima_not_used"] = published_note
    config["timed_region"] = (f"{head['blocks']} blocks of {args.steps} graph replays (>= {MIN_TIMED_S} s), "
                              "median block, max over ranks")
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
        "frac_of_measured_hbm": value / (peaks["hbm_gbs"] * world),
        "tokens_per_s_projections_of_an_80_block_model": 1.0 / (ms_per_step * 1e-3 / C5["blocks"] * C5["model_blocks"]),
        "roofline": roofline, "e2e": e2e, "gpu_launches": gpu_launches, "timed_blocks": head["blocks"],
        "clocks": clocks,
    }
    if clocks is None:
        line["clocks_reason"] = clocks_reason
    if chain_variants is not None:
        line["chain_variants"] = chain_variants

    if world > 1:
        line["sharded"], graphs = sharded_section(dev, ranks, chain, args.steps, args.warmup, head)
        keep_graphs += graphs
    line["device_status"] = _C.device_status(dev)

    if rank == 0 and world == 1 and not args.no_sweep:
        # Secondary legs run one after the other in child processes of their own (this process keeps its weights
        # and graphs): a leg that fails, or runs out of memory, costs its own entry and nothing else.
        for name in LEGS:
            res = run_leg_child(name, local_rank)
            if "error" in res:
                line[name + "_error"] = res["error"]
            elif name == "config3":
                line.update(res)
            elif name.startswith("tokens_"):
                line.setdefault("tokens_per_s", {})[name[len("tokens_"):]] = res
            else:
                line[name] = res
        sec, reps, threads = cpu_reference_layer_seconds()
        h = C5["hidden"]
        cpu_gbs = algorithmic_bytes(1, h, h) / sec / 1e9
        psec, _, _ = cpu_packed_port_layer_seconds()
        line["cpu_baseline"] = {
            "value": cpu_gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{cpu_sample_name()}; median of {reps} forwards ({sec * 1e3:.1f} ms per layer)",
            "packed_int8_port_gbs": algorithmic_bytes(1, h, h) / psec / 1e9,
            "packed_int8_port_ms_per_layer": psec * 1e3,
        }
    if rank == 0:
        print(json.dumps(line), flush=True)
    leave(world, keep_graphs)


def device_of(local_rank: int):
    return torch.device("cuda", local_rank)


def init_kwargs(dev):
    return {"device_id": dev}


def leave(world: int, graphs) -> None:
    """Tearing an NCCL communicator down while CUDA graphs that captured its collectives are alive blocks forever:
    drop the graphs, synchronise, and leave without the (optional) destroy_process_group."""
    if world == 1:
        return
    import torch.distributed as dist
    try:
        torch.cuda.synchronize()
        dist.barrier()
        for g in graphs:
            g.reset()
    except Exception:             # noqa: BLE001  (leaving anyway)
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
