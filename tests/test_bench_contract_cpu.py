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


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""
