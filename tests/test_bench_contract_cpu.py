"""CPU checks of bench.py's bookkeeping: the algorithmic byte counts the roofline fractions rest on, the peak
lookup, and the JSON line of the reference arm (the only arm that runs without a GPU)."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_algorithmic_bytes_of_the_config3_cells():
    import bench

    # ceil(K/4)*N packed weights + 4N scale + 2MK bf16 activations + 2MN bf16 outputs
    assert bench.algorithmic_bytes(1, 4096, 4096) == 4_227_072
    assert bench.algorithmic_bytes(4, 4096, 4096) == 4_276_224
    assert bench.algorithmic_bytes(16, 4096, 4096) == 4_472_832
    assert bench.algorithmic_bytes(1, 4096, 11008) == 11_346_432
    assert bench.algorithmic_bytes(4, 4096, 11008) == 11_437_056
    assert bench.algorithmic_bytes(16, 4096, 11008) == 11_799_552
    assert bench.algorithmic_bytes(1, 5, 3, bias=True) == 2 * 3 + 4 * 3 + 4 * 3 + 2 * 5 + 2 * 3     # ragged K rounds up


def test_peaks_come_from_the_measured_file_or_the_stated_fallback(tmp_path, monkeypatch):
    import bench

    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.load_peaks() == {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6540.2, "bf16_tflops": 1627.0}))
    peaks = bench.load_peaks()
    assert peaks["source"] == "measured" and peaks["hbm_gbs"] == 6540.2


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "packed_ternary_gemv_hbm_gbs" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["scaling"] == "strong" and "config5-decode-chain" in line["config"]["workload"]
    assert "straight-through" in line["cpu_baseline"]["sample"]


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_chain_bytes_are_the_four_projections_times_the_blocks():
    import bench

    shapes = bench.c5_projections()
    assert [(k, n) for _, k, n in shapes] == [(8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)]
    per_block = sum(bench.algorithmic_bytes(1, k, n) for _, k, n in shapes)
    assert bench.chain_bytes(1) == 8 * per_block and 213e6 < per_block < 216e6          # ~214 MB per block
    for _, _, n in shapes:                                      # every shard is whole 16-column blocks at 2, 4, 8 GPUs
        assert all(n % (16 * p) == 0 for p in (2, 4, 8))


def test_clock_sampler_reads_a_sampler_process_and_keeps_the_timed_window(tmp_path):
    """The sampler with a stand-in for nvidia-smi: a process that prints stamped csv lines every 20 ms.  Samples
    outside [mark_begin, mark_end] are dropped; throttle reasons are collected; a process that prints nothing gives
    an explicit reason instead of a clock record."""
    import time

    import bench

    script = (
        "import datetime, sys, time\n"
        "for i in range(400):\n"
        "    t = datetime.datetime.now().strftime('%Y/%m/%d %H:%M:%S.%f')[:-3]\n"
        "    print(f'{t}, {1900 + (i % 2) * 30}, 1965, Not Active, Not Active, Not Active, ' + ('Active' if i % 7 == 0 else 'Not Active'), flush=True)\n"
        "    time.sleep(0.02)\n")
    s = bench.ClockSampler(0, command=[sys.executable, "-c", script]).start()
    time.sleep(0.5)
    s.mark_begin()
    time.sleep(0.6)
    s.mark_end()
    time.sleep(0.3)
    clocks, reason = s.stop()
    assert reason is None and clocks["window"] == "timed region"
    assert 10 <= clocks["samples"] < clocks["samples_total"]
    assert clocks["sm_mhz"] in (1900.0, 1915.0, 1930.0) and clocks["sm_max_mhz"] == 1965.0
    assert clocks["reasons"] == ["sw_power_cap"]

    silent = bench.ClockSampler(0, command=[sys.executable, "-c", "import time; time.sleep(30)"]).start()
    assert silent.stop() == (None, "nvidia-smi printed no samples")
    missing = bench.ClockSampler(0, command=["/nonexistent/nvidia-smi"]).start()
    clocks, reason = missing.stop()
    assert clocks is None and "cannot start" in reason


def test_clock_lines_of_nvidia_smi_parse():
    import bench

    text = ("2026/11/25 09:02:11.123, 1965, 1965, Not Active, Not Active, Not Active, Active\n"
            "garbage\n"
            "2026/11/25 09:02:11.223, [N/A], 1965, Not Active, Not Active, Not Active, Not Active\n"
            "2026/11/25 09:02:11.323, 1350, 1965, Active, Not Active, Active, Not Active\n")
    rows = bench.ClockSampler.parse(text)
    assert len(rows) == 2 and rows[0][1:] == (1965.0, 1965.0, ["sw_power_cap"])
    assert rows[1][3] == ["hw_slowdown", "sw_thermal_slowdown"] and rows[1][0].microsecond == 323000
