"""Committed golden vectors (tests/golden/kmeans_small.npz, made by tests/golden/make_golden.py
from the pinned oracle): the oracle must still reproduce them, and the CUDA path must match
them through the drivers."""
import os

import numpy as np
import pytest
from numpy.testing import assert_allclose, assert_array_equal

from oracle import reference_cpu as ref

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kmeans_small.npz")
CASES = [("f32", np.float32, 1e-5), ("f64", np.float64, 1e-11)]


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.mark.parametrize("tag,dtype,rtol", CASES)
def test_oracle_reproduces_golden(golden, tag, dtype, rtol):
    X, w, init = golden[f"{tag}_X"], golden[f"{tag}_w"], golden[f"{tag}_init"]
    assert X.dtype == dtype
    labels, inertia, C, n_iter = ref.lloyd(X, w, init, False, 12, False, 0.0)
    assert_array_equal(labels, golden[f"{tag}_labels"])
    assert n_iter == int(golden[f"{tag}_n_iter"])
    assert_allclose(C, golden[f"{tag}_C"], rtol=1e-6 if dtype == np.float32 else 1e-13)
    assert_allclose(inertia, golden[f"{tag}_inertia"], rtol=1e-6 if dtype == np.float32 else 1e-13)
    _, idx = ref.kmeans_plusplus(X, w, 11, np.random.RandomState(7), scan="float64")
    assert_array_equal(idx, golden[f"{tag}_kpp_idx"])


@pytest.mark.gpu
@pytest.mark.parametrize("tag,dtype,rtol", CASES)
def test_cuda_path_matches_golden(golden, tag, dtype, rtol):
    import torch

    from sklearn_numba_dpex_b200.common import topk_idx
    from sklearn_numba_dpex_b200.kmeans.drivers import (get_euclidean_distances, kmeans_plusplus,
                                                        lloyd)
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState  # noqa: F401

    X, w, init = golden[f"{tag}_X"], golden[f"{tag}_w"], golden[f"{tag}_init"]
    Xd, wd, Cd = (torch.as_tensor(a).cuda() for a in (X, w, init))
    labels, inertia, C_t, n_iter = lloyd(Xd.T, wd, Cd.T, False, 12, False, 0.0)
    assert n_iter == int(golden[f"{tag}_n_iter"])
    ok, n_bad, n_unexplained = ref.labels_agree(labels.cpu().numpy(), golden[f"{tag}_labels"], X,
                                                golden[f"{tag}_C"])
    assert ok, (n_bad, n_unexplained)
    if n_bad == 0:
        assert_allclose(C_t.T.cpu().numpy(), golden[f"{tag}_C"], rtol=rtol, atol=rtol * 10)
        assert_allclose(float(inertia), float(golden[f"{tag}_inertia"]), rtol=rtol)
    _, idx = kmeans_plusplus(Xd.T, wd, 11, np.random.RandomState(7))
    assert_array_equal(idx.cpu().numpy(), golden[f"{tag}_kpp_idx"])
    Cg = torch.as_tensor(golden[f"{tag}_C"]).cuda()
    D = get_euclidean_distances(Xd[:50].T, Cg.T).cpu().numpy()
    assert_allclose(D, golden[f"{tag}_dist"], rtol=1e-4 if dtype == np.float32 else 1e-9)
    sq = ref.compute_inertia_per_sample(X, np.ones_like(w), golden[f"{tag}_C"], golden[f"{tag}_labels"])
    assert_array_equal(topk_idx(torch.as_tensor(sq).cuda(), 5).cpu().numpy(), golden[f"{tag}_top5"])
