"""The C/OpenMP restatement of the Lloyd iteration (oracle/lloyd_oracle.c) against the numpy
oracle, which is itself pinned to the reference's golden values (tests/test_oracle_golden.py).
The C port is what the benchmark times as the CPU baseline and what the mid-size GPU tests
use as their checker, so it has to be a checked program itself."""
import numpy as np
import pytest
from numpy.testing import assert_allclose, assert_array_equal

from oracle import c_oracle
from oracle import reference_cpu as ref

SHAPES = [(3000, 14, 127), (2000, 32, 64), (1001, 130, 37), (257, 3, 5)]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "n%d_d%d_k%d" % s)
@pytest.mark.parametrize("weighted", [False, True])
def test_c_port_iteration_equals_numpy_oracle(dtype, shape, weighted):
    n, d, k = shape
    rng = np.random.default_rng(n + 7 * d + 31 * k)
    centres = rng.uniform(-10, 10, size=(k, d))
    X = (centres[rng.integers(0, k, n)] + rng.standard_normal((n, d))).astype(dtype)
    C = X[rng.choice(n, size=k, replace=False)].copy()
    w = rng.uniform(0.5, 2.0, n).astype(dtype) if weighted else None
    labels, sums, counts, threads = c_oracle.lloyd_iteration(X, w, C)
    assert threads >= 1
    w_np = np.ones(n, dtype=dtype) if w is None else w
    step = ref.lloyd_iteration(X, w_np, C)
    # same arithmetic (multiply then add, features ascending, strict '<' upward): same labels
    assert_array_equal(labels, step["labels"])
    # private copies merged in thread order against a float64 accumulation rounded once
    rtol = 1e-6 if dtype == np.float32 else 1e-13
    scale = np.abs(X).max() * w_np.max() * max(n / k, 1.0)
    assert_allclose(sums, step["sums"], rtol=rtol, atol=rtol * scale)
    assert_allclose(counts, step["sizes"], rtol=rtol)
    # label-only mode gives the same labels and leaves the outputs alone
    labels2, _, _, _ = c_oracle.lloyd_iteration(X, w, C, update=False)
    assert_array_equal(labels2, labels)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_c_port_loop_equals_numpy_oracle_loop(dtype):
    rng = np.random.default_rng(5)
    centres = rng.uniform(-20, 20, size=(6, 4))
    X = (centres[np.arange(3000) % 6] + 2.5 * rng.standard_normal((3000, 4))).astype(dtype)
    w = np.ones(3000, dtype=dtype)
    init = X[[0, 1, 2, 3, 4, 5]].copy()
    for tol in (0.0, 1e-3):
        o_labels, _, o_C, o_iter = ref.lloyd(X, w, init, True, 60, False, tol)
        labels, C, n_iter, _ = c_oracle.lloyd(X, None, init, 60, tol)
        assert n_iter == o_iter
        assert_array_equal(labels, o_labels)
        assert_allclose(C, o_C, rtol=1e-5 if dtype == np.float32 else 1e-12)


def test_thread_count_can_be_fixed():
    assert c_oracle.set_num_threads(2) == 2
    assert c_oracle.lloyd_iteration(np.zeros((64, 2), dtype=np.float32), None,
                                    np.zeros((2, 2), dtype=np.float32))[3] == 2
    import os

    c_oracle.set_num_threads(len(os.sched_getaffinity(0)))
