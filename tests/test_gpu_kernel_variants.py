"""The kernels that an environment switch selects instead of the default one pass the same
teacher-forced parity cases.

The switches are read once per process (they exist for A/B timing runs), so every variant runs
the selected cases of test_gpu_kernels.py in a child interpreter with the switch set.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# shapes of test_lloyd_step_teacher_forced that reach the short-row tensor-core kernels
SHORT_ROWS = ("n2000_d14_k256 or n40000_d8_k128 or n60000_d20_k700 or n2000_d20_k130 or "
              "n50000_d14_k127 or n30000_d4_k200 or n30000_d12_k384 or n60000_d28_k300 or "
              "n129_d14_k9 or n30000_d13_k200 or n40000_d30_k150 or n40000_d29_k140")
FP64_SHAPES = ("n1000_d17_k127 or n2000_d14_k256 or n3000_d64_k300 or n60000_d20_k700 or "
               "n513_d130_k5 or n7_d3_k2")

VARIANTS = [
    # (environment, dtype the switch concerns, -k selection)
    ({"KMB_TC_SMALL": "0"}, "float32", SHORT_ROWS),       # general kernel with folded half norms
    ({"KMB_TC_SMALL": "1"}, "float32", SHORT_ROWS),       # sixteen workers on every tile
    ({"KMB_TQ_SS": "1"}, "float32", SHORT_ROWS),          # rows of <= 16 features: sample operand from shared memory
    ({"KMB_TQ_FIDX": "0"}, "float32", SHORT_ROWS),        # quads: index search on the integer pipe
    ({"KMB_TQ_ACC": "2"}, "float32", SHORT_ROWS),         # quads: two accumulators even when three fit
    ({"KMB_TQ_MMA": "1"}, "float32", SHORT_ROWS),         # quads: one MMA-issuing warp instead of two
    ({"KMB_TC_ROUND_LO": "0"}, "float32", "n60000_d64_k300 or n60000_d128_k130"),
    ({"KMB_F64_WM": "4"}, "float64", FP64_SHAPES),        # float64 MMA step, 128-sample CTAs
    ({"KMB_F64_WM": "2"}, "float64", FP64_SHAPES),        # float64 MMA step, 64-sample CTAs
    ({"KMB_F64_MMA": "0"}, "float64", FP64_SHAPES),       # float64 step on the CUDA cores
]


@pytest.mark.parametrize("env,dtype,shapes", VARIANTS,
                         ids=["-".join(f"{k}={v}" for k, v in e.items()) for e, _, _ in VARIANTS])
def test_switched_kernel_passes_the_parity_cases(env, dtype, shapes):
    child_env = dict(os.environ)
    child_env.update(env)
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_kernels.py"), "-q", "-x",
           "-p", "no:cacheprovider", "-m", "gpu",
           "-k", f"test_lloyd_step_teacher_forced and {dtype} and ({shapes})"]
    proc = subprocess.run(cmd, cwd=ROOT, env=child_env, capture_output=True, text=True, timeout=1200)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert " passed" in proc.stdout and "no tests ran" not in proc.stdout, tail
