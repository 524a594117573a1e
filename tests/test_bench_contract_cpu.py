"""CPU-only checks of the benchmark's contract and of host-side decisions of the library:
the reference arm prints one JSON line with the required keys, the synthetic-row generator
is reproducible and independent of how the rows are sharded, and the kernel-selection policy
answers as documented.  No kernel is launched here."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
         "--warmup", "0", "--cpu-sample-rows", "20000", "--config", "c2"],
        capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config",
                "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "Lloyd iterations/s" and line["higher_is_better"] is True
    assert line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] in ("port", "reference")
    assert line["cpu_baseline"]["cores"] >= 1 and "sample" in line["cpu_baseline"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"] > 0
    assert line["config"]["n"] == bench.CONFIGS["c2"]["n"]


def test_configs_are_the_documented_ones():
    shapes = {name: (c["n"], c["d"], c["k"], c["dtype"]) for name, c in bench.CONFIGS.items()}
    assert shapes["c1"] == (50_000, 14, 127, "f32")
    assert shapes["c2"] == (5_000_000, 14, 256, "f32")
    assert shapes["c3"] == (10_000_000, 128, 1024, "f32")
    assert shapes["c4"] == (2_000_000, 32, 64, "f64")
    assert shapes["c5"] == (20_000_000, 64, 4096, "f32")


@pytest.mark.parametrize("name", ["c1", "c3", "c5"])
def test_generated_rows_do_not_depend_on_the_sharding(name):
    cfg = dict(bench.CONFIGS[name])
    cfg["n"] = 3_000_000          # three generator chunks; only slices of it are produced here
    dev = torch.device("cpu")
    whole = bench.generate_rows(cfg, 999_000, 1_001_500, torch, dev, torch.float32)
    left = bench.generate_rows(cfg, 999_000, 1_000_000, torch, dev, torch.float32)
    right = bench.generate_rows(cfg, 1_000_000, 1_001_500, torch, dev, torch.float32)
    assert whole.shape == (2_500, cfg["d"])
    assert torch.equal(whole, torch.cat([left, right], dim=0))
    again = bench.generate_rows(cfg, 999_000, 1_001_500, torch, dev, torch.float32)
    assert torch.equal(whole, again)
    assert torch.isfinite(whole).all()


def test_kernel_selection_policy():
    from sklearn_numba_dpex_b200 import _cabi

    lib, f32, f64 = _cabi.lib, _cabi.KMB_F32, _cabi.KMB_F64
    auto, cc, tc = _cabi.ALGO_AUTO, _cabi.ALGO_CUDA_CORE, _cabi.ALGO_TF32X3
    # automatic choice: tensor cores for GEMM-sized fp32 problems only
    assert lib.kmb_lloyd_resolve_algo(f32, auto, 10_000_000, 128, 1024) == tc
    assert lib.kmb_lloyd_resolve_algo(f32, auto, 5_000_000, 16, 256) == tc
    assert lib.kmb_lloyd_resolve_algo(f32, auto, 50_000, 14, 127) == cc      # d not a multiple of 4
    assert lib.kmb_lloyd_resolve_algo(f32, auto, 1_000, 128, 1024) == cc     # too few rows
    assert lib.kmb_lloyd_resolve_algo(f32, auto, 1_000_000, 128, 16) == cc   # too few clusters
    assert lib.kmb_lloyd_resolve_algo(f32, auto, 1_000_000, 256, 1024) == cc  # d > 128
    assert lib.kmb_lloyd_resolve_algo(f64, auto, 2_000_000, 32, 64) == cc
    # an explicit request is honoured when the shape is supported, refused otherwise
    assert lib.kmb_lloyd_resolve_algo(f32, tc, 1_000, 8, 4) == tc
    assert lib.kmb_lloyd_resolve_algo(f32, cc, 10_000_000, 128, 1024) == cc
    with pytest.raises(NotImplementedError):
        _cabi.check(lib.kmb_lloyd_resolve_algo(f32, tc, 1_000, 14, 4))
    with pytest.raises(NotImplementedError):
        _cabi.check(lib.kmb_lloyd_resolve_algo(f32, tc, 1_000, 256, 4))
    # accumulator copies: one when the CUDA-core kernel keeps the sums in shared memory
    assert lib.kmb_lloyd_acc_copies(f32, cc, 50_000, 14, 127) == 1
    assert lib.kmb_lloyd_acc_copies(f32, cc, 1_000_000, 256, 1024) == 8
    assert lib.kmb_lloyd_acc_copies(f32, tc, 10_000_000, 128, 1024) == 16
    # workspace grows with k*d (split centroids) and is 256-byte granular
    small = lib.kmb_workspace_bytes(1_000_000, 16, 256)
    large = lib.kmb_workspace_bytes(1_000_000, 128, 65536)
    assert 0 < small < large


def test_null_and_size_arguments_are_rejected_before_any_launch():
    import ctypes

    from sklearn_numba_dpex_b200 import _cabi

    lib = _cabi.lib
    p = ctypes.c_void_p(256)   # never dereferenced: every call below must fail validation first
    with pytest.raises(ValueError):
        _cabi.check(lib.kmb_lloyd_step(0, 0, None, None, p, p, None, p, p, 1, 10, 4, 2, 0, None, 0, None))
    with pytest.raises(ValueError):
        _cabi.check(lib.kmb_assign_labels(0, 0, p, p, p, None, 10, 4, 2, 0, None, 0, None))
    with pytest.raises(ValueError):                                     # unknown flag bits
        _cabi.check(lib.kmb_lloyd_step(0, 0, p, None, p, p, None, p, p, 1, 10, 4, 2, 64, p, 1 << 20, None))
    with pytest.raises(ValueError):                                     # merge without the copies
        _cabi.check(lib.kmb_lloyd_finalize(0, None, 1, p, _cabi.FIN_MERGE, p, p, p, p, p, p, 2, 4, p,
                                           1 << 20, None))
    with pytest.raises(ValueError):                                     # tensor-core operands are fp32
        _cabi.check(lib.kmb_lloyd_finalize(1, p, 1, p, _cabi.FIN_PREPARE_TF32X3, p, p, p, p, p, p, 2, 4,
                                           p, 1 << 20, None))
    with pytest.raises(_cabi.KmbError):                                 # workspace too small
        _cabi.check(lib.kmb_lloyd_finalize(0, None, 1, p, 0, p, p, p, p, p, p, 2, 4, p, 16, None))
    with pytest.raises(ValueError):
        _cabi.check(lib.kmb_inertia(0, None, None, p, p, p, p, 10, 4, 2, None, 0, None))
    with pytest.raises(ValueError):
        _cabi.check(lib.kmb_kpp_step(0, p, None, p, p, None, p, p, 10, 4, 99, None))   # t > 16
    with pytest.raises(ValueError):
        _cabi.check(lib.kmb_kpp_sample(0, p, p, None, p, p, None, 0, p, 10, None))     # t = 0
    with pytest.raises(ValueError):
        _cabi.check(lib.kmb_gather_rows(0, p, None, 1, 4, p, None))
    assert _cabi.last_error() != ""


def test_reference_arm_uses_all_host_threads_under_a_launcher_that_exports_one():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm must set its
    own thread count from the affinity mask and say how many threads it used."""
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps",
         "1", "--warmup", "0", "--cpu-sample-rows", "20000", "--config", "c2"],
        capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][0])
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert line["cpu_baseline"]["extrapolated"] is True
    # the other ranks of the launch print nothing and exit 0
    env["RANK"] = "1"
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps",
         "1", "--warmup", "0", "--cpu-sample-rows", "20000", "--config", "c2"],
        capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_cpu_sample_is_deterministic_and_drawn_by_the_benchmark_generator():
    cfg = dict(bench.CONFIGS["c2"])
    X1, C1 = bench.cpu_sample(cfg, 5000)
    bench._CPU_SAMPLES.clear()
    X2, C2 = bench.cpu_sample(cfg, 5000)
    assert X1.shape == (5000, cfg["d"]) and C1.shape == (cfg["k"], cfg["d"])
    assert np.array_equal(X1, X2) and np.array_equal(C1, C2)
