"""Pins the CPU oracle to the known answers held by the reference's own tests.

Each case cites the reference test that holds the constants
(paths relative to the reference project root).
"""
import numpy as np
import pytest
from numpy.testing import assert_allclose, assert_array_equal
from sklearn.cluster import KMeans
from sklearn.datasets import make_blobs
from sklearn.utils import check_random_state

from oracle import reference_cpu as ref
from oracle.rng import Xoroshiro128ppStates

DTYPES = [np.float32, np.float64]


def test_xoroshiro128pp_raw():
    # sklearn_numba_dpex/common/tests/test_random.py:18-76
    expected_1 = [
        16756476715040848931, 6098722386207918385, 17541662578032534341,
        3771828211556203317, 6324094075403496319, 1696280121849217124,
        9039151786603216578, 1834868434787995627, 4294676528364711596,
        5649342080498856832,
    ]
    rng = Xoroshiro128ppStates(1, seed=42)
    assert [rng.next(0) for _ in expected_1] == expected_1

    expected_2 = [
        16052925335932940643, 13241858892588731496, 8234838429006980292,
        1690280486132429899, 6807031509475728656, 9789629428737685881,
        8662181912786361632, 11992761958092131212, 7748117140003924005,
        5731413122647051604,
    ]
    rng = Xoroshiro128ppStates(1, seed=42, subsequence_start=1)
    assert [rng.next(0) for _ in expected_2] == expected_2
    # state i+1 of a multi-state array is state i jumped once
    rng = Xoroshiro128ppStates(2, seed=42)
    assert [rng.next(1) for _ in expected_2] == expected_2


def test_xoroshiro128pp_floats():
    # sklearn_numba_dpex/common/tests/test_random.py:79-123
    expected = np.array(
        [0.9083704, 0.33061236, 0.9509354, 0.20447117, 0.34282982, 0.09195548,
         0.49001336, 0.09946841, 0.23281485, 0.3062514], dtype=np.float32)
    rng = Xoroshiro128ppStates(1, seed=42)
    got32 = [rng.uniform(0, np.float32) for _ in expected]
    assert_allclose(expected, got32)
    rng = Xoroshiro128ppStates(1, seed=42)
    got64 = [rng.uniform(0, np.float64) for _ in expected]
    # the reference compares with scikit-learn's assert_allclose, whose default
    # tolerance for float32 operands is 1e-4
    assert_allclose(got64, expected, rtol=1e-6)


def test_rng_quality():
    # sklearn_numba_dpex/common/tests/test_random.py:126-134 (smaller draw count)
    rng = Xoroshiro128ppStates(1, seed=42)
    vals = np.array([rng.uniform(0, np.float64) for _ in range(100000)])
    hist, _ = np.histogram(vals, bins=np.linspace(0, 1, 6))
    assert (np.abs(hist - 2e4) < 6e2).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_predict_centers(dtype):
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:113-122
    centers = np.arange(100, dtype=dtype).reshape(10, 10)
    labels, _ = ref.get_labels_inertia(centers, centers, np.ones(10, dtype=dtype), False)
    assert_array_equal(labels, np.arange(10))


def _oracle_fit(X, init, n_clusters, max_iter=300, tol=1e-4, sample_weight=None,
                random_state=None, n_init=1):
    """prepare_fit -> init -> lloyd -> unshift, the order the engine methods are called
    in (sklearn_numba_dpex/kmeans/engine.py:133-232)."""
    X = np.asarray(X)
    w = np.ones(X.shape[0], dtype=X.dtype) if sample_weight is None else sample_weight
    init_arr = np.array(init, dtype=X.dtype) if not isinstance(init, str) else init
    Xc, X_mean, init_c, tol_, uniform = ref.prepare_data_for_lloyd(X, init_arr, tol, w, True)
    rs = check_random_state(random_state)
    best = None
    for _ in range(n_init):
        if isinstance(init_c, str) and init_c == "k-means++":
            centers, _ = ref.kmeans_plusplus(Xc, w, n_clusters, rs)
        elif isinstance(init_c, str):
            idx = rs.choice(Xc.shape[0], size=n_clusters, replace=False, p=w / w.sum())
            centers = Xc[idx]
        else:
            centers = init_c
        labels, inertia, C, n_iter = ref.lloyd(Xc, w, centers, uniform, max_iter, False, tol_)
        if best is None or inertia < best[1]:
            best = (labels, inertia, C.copy(), n_iter)
    labels, inertia, C, n_iter = best
    ref.restore_data_after_lloyd(Xc, C, X_mean, True)
    return labels, inertia, C, n_iter


@pytest.mark.parametrize("dtype", DTYPES)
def test_relocated_clusters(dtype):
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:125-158
    X = np.array([[0, 0], [0.5, 0], [0.5, 1], [1, 1]], dtype=dtype)
    init = np.array([[0.5, 0.5], [3, 3]], dtype=dtype)
    labels, inertia, C, n_iter = _oracle_fit(X, init, 2)
    assert_allclose(inertia, 0.25)
    assert n_iter == 3
    if labels[0] == 0:
        assert_array_equal(labels, [0, 0, 1, 1])
        assert_allclose(C, [[0.25, 0], [0.75, 1]], atol=1e-6)
    else:
        assert_array_equal(labels, [1, 1, 0, 0])
        assert_allclose(C, [[0.75, 1.0], [0.25, 0.0]], atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_relocate_empty_clusters(dtype):
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:208-248
    X = np.array([-10.0, -9.5, -9.0, -8.5, -8.0, -1.0, 1.0, 9.0, 9.5, 10.0],
                 dtype=dtype).reshape(-1, 1)
    init = np.array([-10.0, -10.0, -10.0]).reshape(-1, 1)
    truth = KMeans(n_clusters=3, n_init=1, max_iter=1, init=init, algorithm="lloyd").fit(X)
    labels, inertia, C, n_iter = _oracle_fit(X, init, 3, max_iter=1)
    assert n_iter == 1 and truth.n_iter_ == 1
    expected = np.array([0, 0, 0, 0, 0, 0, 0, 2, 2, 1])
    assert ref.is_same_clustering(truth.labels_, labels, 3)
    assert ref.is_same_clustering(expected, labels, 3)
    assert_allclose(truth.cluster_centers_[truth.labels_], C[labels.astype(int)], rtol=1e-6)
    assert_allclose(truth.inertia_, inertia, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_same_results_as_sklearn_lloyd(dtype):
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:28-110
    X, _ = make_blobs(random_state=42)
    X = X.astype(dtype)
    truth = KMeans(random_state=42, algorithm="lloyd", max_iter=2, n_init=2, init="random",
                   n_clusters=8).fit(X)
    labels, inertia, C, _ = _oracle_fit(X, "random", 8, max_iter=2, random_state=42, n_init=2)
    assert_array_equal(truth.labels_, labels)
    rtol = 1e-5 if dtype == np.float32 else 1e-7
    assert_allclose(truth.cluster_centers_, C, rtol=rtol)
    assert_allclose(truth.inertia_, inertia, rtol=rtol)
    # transform / score back-ends
    assert_allclose(truth.transform(X), ref.euclidean_distances(X, C), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kmeans_plusplus_golden(dtype):
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:251-325: mean score over seeds 0..9
    # of the engine's k-means++ on scikit-learn's own test fixture.
    from sklearn.cluster.tests.test_k_means import X as X_fix
    from sklearn.cluster.tests.test_k_means import n_clusters

    X = X_fix.astype(dtype)
    kmeans = KMeans(n_clusters=n_clusters, init="k-means++")
    kmeans._n_threads = 1
    scores = []
    for seed in range(10):
        w = np.ones(X.shape[0], dtype=dtype)
        Xc, X_mean, _, _, _ = ref.prepare_data_for_lloyd(X, "k-means++", 1e-4, w, True)
        rs = check_random_state(seed)
        centers, idx = ref.kmeans_plusplus(Xc, w, n_clusters, rs)
        ref.restore_data_after_lloyd(Xc, centers, X_mean, True)
        kmeans.cluster_centers_ = np.ascontiguousarray(centers)
        scores.append(kmeans.score(X))
        assert_allclose(X[idx], centers, rtol=1e-5, atol=1e-5)
    assert_allclose(np.mean(scores), -865.257501, rtol=1e-7)


TOPK_CASES = [
    # sklearn_numba_dpex/common/tests/test_topk.py:9-26
    [0, 1, -2, -3, 4, -5, 6, 7, 8, -9, 10],
    [0, 8, -2, -3, 4, -5, 6, 7, 8, -9, 10],
    [0, 8, -2, -3, 4, -5, 6, 7, 8, -9, 8],
    [0, 8, 8, -3, 4, -5, 6, 7, 8, -9, 10],
    [0, 8, 8, -3, 4, -5, 6, 7, 8, -9, 8],
    [8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8],
]


@pytest.mark.parametrize("k", [1, 3])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", TOPK_CASES)
def test_topk(case, dtype, k):
    arr = np.array(case, dtype=dtype)
    vals = np.sort(ref.topk(arr, k))
    idx = ref.topk_idx(arr, k)
    assert_array_equal(vals, np.sort(arr)[-k:])
    assert len(set(idx.tolist())) == k
    assert set(arr[idx].tolist()) == set(np.sort(arr)[-k:].tolist())


def test_argmin_cases():
    # sklearn_numba_dpex/common/tests/test_reductions.py:109-133
    for values, expected in [([3.0, 1.0, 0.0, 2.0], 2), ([0.0, 1.0, 3.0, 2.0], 0),
                             ([3.0, 1.0, 2.0, -1.0, -2.0], 4), ([0.0, 1.0, 0.0], 0)]:
        assert ref.argmin_lowest_index(np.array(values, dtype=np.float32)) == expected


def test_distinct_clusters():
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:448-457
    assert ref.get_nb_distinct_clusters([0, 1, 0, 2, 2, 7, 6, 5, 3, 3], 8) == 7
