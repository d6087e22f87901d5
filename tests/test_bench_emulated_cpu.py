"""bench.py's GPU arm, run on the CPU against the host emulation of the C ABI (tests/emu/): the whole line at one
"GPU" and at two gloo ranks, on shrunken workloads.  Checks the bench's own logic - the chain's data flow through the
real entry points' signatures, the sharded chain against the unsharded one bit for bit, launch and byte bookkeeping,
the clock record, every secondary leg - not performance."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "tests", "emu", "run_bench.py")


def _line(cmd, timeout=600):
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-3000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_one_gpu_line_has_every_contract_key_and_every_leg():
    d = _line([sys.executable, RUNNER, "--steps", "3", "--warmup", "3"])
    assert d["metric"] == "packed_ternary_gemv_hbm_gbs" and d["unit"] == "GB/s" and d["n_gpus"] == 1
    assert d["steps"] == 3 and d["warmup"] == 3 and d["higher_is_better"] is True and d["scaling"] == "strong"
    assert d["vs_baseline"] is None and d["dtype"] == "int8" and d["data"] == "synthetic"
    assert d["value"] > 0 and d["ms_per_step"] > 0 and "workload" in d["config"] and "model" not in d["config"]
    # 2 blocks x 4 projections, one fused launch each, per replay; timed_blocks blocks of 3 replays
    assert d["gpu_launches"] == 8 * 3 * d["timed_blocks"] and d["timed_blocks"] >= 1
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-12
    assert abs(r["achieved"] - d["value"]) < 1e-9 * max(1.0, d["value"])          # one GPU: the chain is the kernel
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] == 2 * 256 and e["d2h_bytes_per_step"] == 2 * 256
    c = d["clocks"]
    assert c["samples"] >= 3 and c["window"] == "timed region" and c["reasons"] == ["sw_power_cap"]
    assert d["device_status"] == 0
    v = d["chain_variants"]                                     # both chains were timed; the headline is one of them
    assert v["headline"] in ("plain", "published_row_maxima") and v["plain"]["gbs"] > 0 and v["published_row_maxima"]["gbs"] > 0
    assert not [k for k in d if k.endswith("_error")], [d[k] for k in d if k.endswith("_error")]
    assert len(d["rooflines"]) == 4 and all(x["frac"] > 0 for x in d["rooflines"])      # three shapes + the float-activation kernel
    assert d["rooflines"][1]["kernel"] == "gemv_tiled_kernel<4,planes>" and d["rooflines"][1]["relative_to_int8_path"] > 0
    g = d["roofline_gemm"]
    assert g["bound"] == "tensor" and g["unit"] == "TOP/s" and abs(g["frac"] - g["achieved"] / g["peak"]) < 1e-12
    assert len(d["sweep"]) == 8 and d["config3_stack"]["gbs"] > 0
    paths = d["decode_batch_paths"]                             # the table the decode / tensor-core switch-over rests on
    assert paths["decode_max_m_in_use"] >= 1 and len(paths["shapes"]) == 2
    for shape in paths["shapes"]:
        assert [r["M"] for r in shape["rows"]] == [1, 2, 4, 8, 16, 32]
        for r in shape["rows"]:
            assert not [k for k in r if k.endswith("_error")], r
            assert r["act_quant_us"] > 0
            assert ("fused_us" in r) == ("int8_rows_us" in r) == (r["M"] <= 16)      # the decode entries take 16 rows
            assert ("tensor_core_us" in r) == (r["M"] >= 4)
            assert r["fastest_from_float_rows"] in ("fused", "int8_rows", "tensor_core")
            assert r["fastest_from_int8_rows"] in ("int8_rows", "tensor_core")
    t = d["tokens_per_s"]
    assert t["config2"]["decode_tokens_per_s"] > 0
    assert [r["batch"] for r in t["config4"]["rows"]] == [1, 3]
    assert all(r["prefill_tokens_per_s"] > 0 and r["decode_tokens_per_s"] > 0 for r in t["config4"]["rows"])
    b = d["cpu_baseline"]
    assert b["kind"] == "port" and b["cores"] >= 1 and b["value"] > 0 and "straight-through" in b["sample"]


def test_two_rank_line_is_the_same_job_sharded_with_gathers():
    d = _line([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", "29531", RUNNER, "--gpus", "2", "--steps", "3", "--warmup", "3"])
    assert d["n_gpus"] == 2 and d["scaling"] == "strong" and "column-parallel x2" in d["config"]["parallelism"]
    assert d["gpu_launches"] == 8 * 3 * d["timed_blocks"] * 2
    assert d["e2e"]["api"] == "ColumnParallelTernaryLinear chain"
    rows = d["sharded"]["rows"]
    assert [r["M"] for r in rows] == [1, 5, 16]
    for r in rows:
        assert "error" not in r, r
        assert r["matches_single_gpu"] is True                 # gathered shards == unsharded chain, bit for bit
        assert r["us_per_block_sharded"] > 0 and r["us_per_block_kernels_only"] > 0 and r["us_per_block_single_gpu"] > 0
    # the headline is the M = 1 sharded chain with its gathers
    assert abs(rows[0]["us_per_block_sharded"] * 2 / 1e3 - d["ms_per_step"]) < 1e-9
    assert d["roofline"]["algorithmic_bytes_per_launch"] < 40576             # a rank streams its shard only


def test_the_profiling_cases_run():
    """`bench.py --case ...` is the program the profiler captures: each case runs its few launches and reports."""
    for case in ("gemv", "gemm", "quantize", "actquant"):
        d = _line([sys.executable, RUNNER, "--case", case, "--case-m", "4", "--case-k", "256", "--case-n", "512"], timeout=300)
        assert d == {"case": case, "m": 4, "k": 256, "n": 512, "device_status": 0}
