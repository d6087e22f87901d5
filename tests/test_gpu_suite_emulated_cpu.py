"""The GPU-marked test files, run on the CPU against the host emulation of the C ABI (tests/emu/).  This does not
test the kernels; it tests the TESTS and the host code they drive: every oracle comparison, shape, hook and
bookkeeping step of the `-m gpu` suite executes here against an independent implementation of the same entry points
(the emulation decodes the real tiled layout with its own code), so a GPU run cannot fail on a mistake of the test
code, and the emulation and the oracle are checked against each other on every case."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_gpu_marked_files_pass_against_the_emulated_library():
    files = ["tests/test_act_quant_gpu.py", "tests/test_quantize_pack_gpu.py", "tests/test_modules_gpu.py",
             "tests/test_gemv_gemm_gpu.py", "tests/test_serving_decoder_gpu.py",
             "tests/test_tensor_core_full_rows_gpu.py", "tests/test_tiled_gemv_variants_gpu.py",
             "tests/test_weight_caches_and_new_entries_gpu.py"]
    runner = os.path.join(ROOT, "tests", "emu", "run_pytest.py")
    subprocess.run([sys.executable, "-c", "from tests.emu import runtime; runtime.build()"], check=True, cwd=ROOT)
    env = dict(os.environ, OMP_NUM_THREADS="2", MKL_NUM_THREADS="2")          # five processes share the host cores
    procs = [(f, subprocess.Popen([sys.executable, runner, f, "-m", "gpu", "-q", "-x", "-p", "no:cacheprovider"],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=ROOT, env=env))
             for f in files]
    passed = 0
    for f, proc in procs:                                      # one process per file, side by side
        out, _ = proc.communicate(timeout=1500)
        assert proc.returncode == 0, f + "\n" + out[-3000:]
        summary = out.strip().splitlines()[-1]
        assert " passed" in summary and "failed" not in summary and "error" not in summary, f + "\n" + out[-3000:]
        passed += int(summary.split(" passed")[0].split()[-1])
    assert passed >= 220, passed                               # the suite minus the few tests that need a real device
