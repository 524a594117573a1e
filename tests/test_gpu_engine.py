"""Engine-level parity, mirroring the reference's own test file
sklearn_numba_dpex/kmeans/tests/test_kmeans.py case by case (line ranges cited per test),
plus end-to-end runs against the CPU oracle on the benchmark's small configuration."""
import numpy as np
import pytest
import torch
from numpy.testing import assert_allclose, assert_array_equal
from sklearn.cluster import KMeans as SkKMeans
from sklearn.cluster import kmeans_plusplus as sk_kmeans_plusplus
from sklearn.datasets import make_blobs

from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu

DTYPES = [np.float32, np.float64]


def _np(t):
    return t.cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)


def _rtol(dtype):
    return 1e-5 if dtype == np.float32 else 1e-7


@pytest.mark.parametrize("array_constr", ["numpy", "torch_cuda", "torch_cpu", "convert"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_kmeans_same_results(dtype, array_constr):
    # test_kmeans.py:28-110
    from sklearn_numba_dpex_b200.kmeans import KMeans

    X, _ = make_blobs(random_state=42)
    X = X.astype(dtype)
    X_array = {"numpy": X, "torch_cuda": torch.as_tensor(X).cuda(), "torch_cpu": torch.as_tensor(X),
               "convert": torch.as_tensor(X).cuda()}[array_constr]
    truth = SkKMeans(random_state=42, algorithm="lloyd", max_iter=2, n_init=2, init="random")
    engine = KMeans(random_state=42, algorithm="lloyd", max_iter=2, n_init=2, init="random",
                    engine_attributes="sklearn_types" if array_constr == "convert" else None)
    truth.fit(X)
    engine.fit(X_array)
    if array_constr == "convert":
        assert isinstance(engine.labels_, np.ndarray) and isinstance(engine.cluster_centers_, np.ndarray)
    rt = _rtol(dtype)
    assert_array_equal(truth.labels_, _np(engine.labels_))
    assert_allclose(truth.cluster_centers_, _np(engine.cluster_centers_), rtol=rt)
    assert_allclose(truth.inertia_, engine.inertia_, rtol=rt)

    assert_array_equal(truth.fit_predict(X), _np(engine.fit_predict(X_array)))
    assert_allclose(truth.fit_transform(X), _np(engine.fit_transform(X_array)), rtol=1e-4, atol=1e-5)
    assert_array_equal(truth.labels_, _np(engine.labels_))
    assert_array_equal(truth.predict(X), _np(engine.predict(X_array)))
    assert_allclose(truth.score(X), engine.score(X_array), rtol=rt)
    assert_allclose(truth.transform(X), _np(engine.transform(X_array)), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kmeans_predict_centers(dtype):
    # test_kmeans.py:113-122
    from sklearn_numba_dpex_b200.kmeans import KMeans

    kmeans = KMeans(n_clusters=10)
    centers = torch.arange(0, 100, dtype=torch.float32 if dtype == np.float32 else torch.float64,
                           device="cuda").reshape(10, 10).clone()
    kmeans.cluster_centers_ = centers
    assert_array_equal(_np(kmeans.predict(centers)), np.arange(10))


@pytest.mark.parametrize("dtype", DTYPES)
def test_kmeans_relocated_clusters(dtype):
    # test_kmeans.py:125-158
    from sklearn_numba_dpex_b200.kmeans import KMeans

    X = np.array([[0, 0], [0.5, 0], [0.5, 1], [1, 1]], dtype=dtype)
    init = np.array([[0.5, 0.5], [3, 3]], dtype=dtype)
    kmeans = KMeans(n_clusters=2, n_init=1, init=init).fit(X)
    assert_allclose(kmeans.inertia_, 0.25)
    assert kmeans.n_iter_ == 3
    labels, centers = _np(kmeans.labels_), _np(kmeans.cluster_centers_)
    if labels[0] == 0:
        assert_array_equal(labels, [0, 0, 1, 1])
        assert_allclose(centers, [[0.25, 0], [0.75, 1]], atol=1e-6)
    else:
        assert_array_equal(labels, [1, 1, 0, 0])
        assert_allclose(centers, [[0.75, 1.0], [0.25, 0.0]], atol=1e-6)
    # and the CPU oracle agrees with whichever outcome this build's fixed pairing rule gives
    o_labels, o_inertia, o_C, o_iter = ref.lloyd(*_oracle_prepared(X, init))
    assert o_iter == 3 and ref.is_same_clustering(o_labels, labels, 2)


def _oracle_prepared(X, init, tol=1e-4):
    w = np.ones(X.shape[0], dtype=X.dtype)
    Xc, _, init_c, tol_, uni = ref.prepare_data_for_lloyd(X, np.array(init, dtype=X.dtype), tol, w, True)
    return Xc, w, init_c, uni, 300, False, tol_


@pytest.mark.parametrize("dtype", DTYPES)
def test_euclidean_distance(dtype):
    # test_kmeans.py:161-181
    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

    rng = np.random.default_rng(42)
    a = rng.random(size=(1, 100), dtype=dtype)
    b = rng.standard_normal((1, 100), dtype=dtype)
    expected = np.sqrt(((a - b) ** 2).sum())
    estimator = KMeans(n_clusters=len(b))
    estimator.cluster_centers_ = b
    result = KMeansEngine(estimator).get_euclidean_distances(a)
    assert_allclose(_np(result), [[expected]], rtol=1e-4 if dtype == np.float32 else 1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
def test_inertia(dtype):
    # test_kmeans.py:184-205
    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

    rng = np.random.default_rng(42)
    X = rng.random((100, 10), dtype=dtype)
    sample_weight = rng.standard_normal(100, dtype=dtype)
    centers = rng.standard_normal((5, 10), dtype=dtype)
    estimator = KMeans(n_clusters=len(centers))
    estimator.cluster_centers_ = torch.as_tensor(centers).cuda()
    engine = KMeansEngine(estimator)
    Xp, swp = engine.prepare_prediction(X, sample_weight)
    labels = _np(engine.get_labels(Xp, swp))
    distances = ((X - centers[labels, :]) ** 2).sum(axis=1)
    expected = float(np.sum(distances * sample_weight))
    inertia = engine.get_score(Xp, swp)
    assert_allclose(float(inertia), expected, rtol=1e-4 if dtype == np.float32 else 1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_relocate_empty_clusters(dtype):
    # test_kmeans.py:208-248
    from sklearn.cluster._kmeans import _is_same_clustering

    from sklearn_numba_dpex_b200.kmeans import KMeans

    X = np.array([-10.0, -9.5, -9.0, -8.5, -8.0, -1.0, 1.0, 9.0, 9.5, 10.0], dtype=dtype).reshape(-1, 1)
    init = np.array([-10.0, -10.0, -10.0]).reshape(-1, 1)
    truth = SkKMeans(n_clusters=3, n_init=1, max_iter=1, init=init, algorithm="lloyd").fit(X)
    engine = KMeans(n_clusters=3, n_init=1, max_iter=1, init=init, algorithm="lloyd").fit(X)
    expected_labels = np.asarray([0, 0, 0, 0, 0, 0, 0, 2, 2, 1], dtype=np.int32)
    e_labels = _np(engine.labels_).astype(np.int32)
    assert truth.n_iter_ == 1 and engine.n_iter_ == 1
    assert _is_same_clustering(truth.labels_, e_labels, n_clusters=3)
    assert _is_same_clustering(truth.labels_, expected_labels, n_clusters=3)
    assert_allclose(truth.cluster_centers_[truth.labels_], _np(engine.cluster_centers_)[e_labels],
                    rtol=1e-6)
    assert_allclose(truth.inertia_, engine.inertia_, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kmeans_plusplus_same_quality(dtype):
    # test_kmeans.py:251-325: the third constant is the engine's own golden number
    from sklearn.cluster.tests.test_k_means import X as X_fix
    from sklearn.cluster.tests.test_k_means import n_clusters

    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

    X = X_fix.astype(dtype)
    scorer = SkKMeans(n_clusters=n_clusters, init="k-means++")
    scorer._n_threads = 1

    def score_with(centers):
        scorer.cluster_centers_ = np.ascontiguousarray(centers)
        return scorer.score(X)

    s_random, s_vanilla, s_engine = [], [], []
    for seed in range(10):
        s_random.append(score_with(np.random.default_rng(seed).choice(X, size=n_clusters, replace=False)))
        s_vanilla.append(score_with(sk_kmeans_plusplus(X, n_clusters, random_state=seed)[0]))
        kmeans = KMeans(n_clusters=n_clusters, init="k-means++", random_state=seed)
        engine = KMeansEngine(kmeans)
        Xp, _, sw = engine.prepare_fit(X)
        centers = engine.init_centroids(Xp, sw).T
        engine.unshift_centers(Xp, centers)
        s_engine.append(score_with(_np(centers).astype(dtype)))
    assert_allclose([np.mean(s_random), np.mean(s_vanilla), np.mean(s_engine)],
                    [-1827.22702, -892.39115, -865.257501], rtol=1e-7 if dtype == np.float64 else 2e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("array_constr", ["numpy", "torch_cuda"])
def test_kmeans_plusplus_output(array_constr, dtype):
    # test_kmeans.py:328-370
    from sklearn.cluster.tests.test_k_means import X as X_fix
    from sklearn.cluster.tests.test_k_means import n_clusters

    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

    Xn = X_fix.astype(dtype)
    X = Xn if array_constr == "numpy" else torch.as_tensor(Xn).cuda()
    sample_weight = np.random.default_rng(42).random(Xn.shape[0], dtype=dtype)
    engine = KMeansEngine(KMeans(init="k-means++", n_clusters=n_clusters, random_state=42))
    Xp, _, sw = engine.prepare_fit(X, sample_weight=sample_weight)
    centers_t, indices = engine._kmeans_plusplus(Xp, sw)
    centers = centers_t.T
    engine.unshift_centers(Xp, centers)
    centers, indices = _np(centers), _np(indices)
    assert indices.shape[0] == n_clusters
    assert (indices >= 0).all() and (indices <= Xn.shape[0]).all()
    assert centers.shape[0] == n_clusters
    assert (centers.max(axis=0) <= Xn.max(axis=0) + 1e-5).all()
    assert (centers.min(axis=0) >= Xn.min(axis=0) - 1e-5).all()
    assert centers.dtype.type == dtype
    assert_allclose(Xn[indices], centers, rtol=1e-5, atol=1e-5)


def test_kmeans_plusplus_dataorder():
    # test_kmeans.py:373-392
    from sklearn.cluster.tests.test_k_means import X as X_fix
    from sklearn.cluster.tests.test_k_means import n_clusters

    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

    est = KMeans(init="k-means++", n_clusters=n_clusters, random_state=42)
    engine = KMeansEngine(est)
    Xp, _, sw = engine.prepare_fit(X_fix)
    centers_c = _np(engine.init_centroids(Xp, sw).T)
    engine = KMeansEngine(est)
    Xp, _, sw = engine.prepare_fit(np.asfortranarray(X_fix))
    centers_f = _np(engine.init_centroids(Xp, sw).T)
    assert_allclose(centers_c, centers_f)


def test_engine_config_errors():
    # test_kmeans.py:395-445 pins argument errors of kernel factories; the analogous
    # configuration errors of this engine
    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine
    from sklearn_numba_dpex_b200.kmeans.drivers import lloyd

    try:
        KMeansEngine._CONFIG["order"] = "F"
        with pytest.raises(ValueError, match="only order='C' is supported"):
            KMeansEngine(KMeans())
    finally:
        KMeansEngine._CONFIG.clear()
    X = torch.zeros((10, 3), device="cuda")
    C = torch.zeros((2, 3), device="cuda")
    with pytest.raises(ValueError, match="algo must be one of"):
        lloyd(X.T, torch.ones(10, device="cuda"), C.T, True, algo="fast")
    with pytest.raises(NotImplementedError):
        lloyd(X.double().T, torch.ones(10, device="cuda").double(), C.double().T, True, algo="tf32x3")
    with pytest.raises(ValueError, match="n_samples=1 should be >= n_clusters"):
        KMeans(n_clusters=2, n_init=1).fit(np.zeros((1, 2), dtype=np.float32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [0, 7])
def test_kmeans_plusplus_matches_oracle(dtype, seed):
    """Same random stream, same candidates, same centres as the CPU restatement (float64
    prefix scan on both sides; the sequential compute-dtype scan of the reference can differ
    only when a threshold lands within rounding of a partial sum)."""
    from sklearn_numba_dpex_b200.kmeans.drivers import kmeans_plusplus

    rng = np.random.default_rng(seed)
    n, d, k = 5000, 9, 40
    X = (rng.standard_normal((n, d)) * 3).astype(dtype)
    w = rng.uniform(0.5, 1.5, n).astype(dtype)
    centers_t, indices = kmeans_plusplus(torch.as_tensor(X).cuda().T, torch.as_tensor(w).cuda(), k,
                                         np.random.RandomState(seed))
    exp_centers, exp_idx = ref.kmeans_plusplus(X, w, k, np.random.RandomState(seed), scan="float64")
    seq_centers, seq_idx = ref.kmeans_plusplus(X, w, k, np.random.RandomState(seed))
    got_idx = _np(indices)
    assert_array_equal(got_idx, exp_idx)
    assert_allclose(_np(centers_t.T), exp_centers)
    if dtype == np.float64:
        assert_array_equal(got_idx, seq_idx)


@pytest.mark.parametrize("dtype", DTYPES)
def test_full_fit_matches_oracle_c1_shape(dtype):
    """The n=50 000, d=14, k=127 blob configuration (k-means++ from seed 0, tol=0) at a
    bounded iteration count: the CUDA path and the oracle are started from the same initial
    centres and compared after every iteration is forced to the same labels (teacher
    forcing is implicit: the data are well separated, so labels agree exactly)."""
    from sklearn_numba_dpex_b200.kmeans.drivers import lloyd

    rng = np.random.default_rng(0)
    k, d, n = 127, 14, 50_000
    centers = rng.uniform(-10, 10, size=(k, d))
    X = (centers[np.arange(n) % k] + rng.standard_normal((n, d))).astype(dtype)
    w = np.ones(n, dtype=dtype)
    Xc, _, _, _, uni = ref.prepare_data_for_lloyd(X, "k-means++", 0.0, w, True)
    init, _ = ref.kmeans_plusplus(Xc, w, k, np.random.RandomState(0), scan="float64")
    max_iter = 8
    o_labels, o_inertia, o_C, o_iter = ref.lloyd(Xc, w, init, uni, max_iter, False, 0.0)
    labels, inertia, C_t, n_iter = lloyd(torch.as_tensor(Xc).cuda().T, torch.as_tensor(w).cuda(),
                                         torch.as_tensor(init).cuda().T, uni, max_iter, False, 0.0)
    assert n_iter == o_iter
    ok, n_bad, n_unexplained = ref.labels_agree(_np(labels), o_labels, Xc, o_C)
    assert ok, (n_bad, n_unexplained)
    rt = 1e-5 if dtype == np.float32 else 1e-12
    if n_bad == 0:
        assert_allclose(_np(C_t.T), o_C, rtol=rt * 10, atol=rt * 10 * np.abs(Xc).max())
    assert_allclose(float(inertia), float(o_inertia), rtol=1e-5 if dtype == np.float32 else 1e-10)


def test_full_fit_on_the_tensor_core_path_matches_oracle():
    """A shape that the automatic choice sends to the tensor-core step (fp32, n >= 32 768,
    k >= 128, d a multiple of 4), through the public estimator: fit from given centres,
    predict and score, against the oracle's Lloyd on the same centred data.  Two iterations
    only: the blobs overlap, and from the third iteration on a free-running loop drifts by a
    few dozen boundary samples from the oracle on BOTH kernels (CUDA cores: 1, 3, 11 labels
    after 3, 4, 6 iterations; tensor cores: 4, 18, 25), each flip moving two small clusters'
    centres; step-by-step agreement is what the teacher-forced kernel tests check."""
    from sklearn_numba_dpex_b200 import _cabi
    from sklearn_numba_dpex_b200.kmeans import KMeans

    rng = np.random.default_rng(3)
    k, d, n = 160, 24, 40_000
    assert _cabi.lib.kmb_lloyd_resolve_algo(_cabi.KMB_F32, _cabi.ALGO_AUTO, n, d, k) == _cabi.ALGO_TF32X3
    centers = rng.uniform(-10, 10, size=(k, d))
    X = (centers[np.arange(n) % k] + 0.7 * rng.standard_normal((n, d))).astype(np.float32)
    init = X[rng.choice(n, size=k, replace=False)].copy()
    w = np.ones(n, dtype=np.float32)
    max_iter = 2
    Xc, mean, init_c, _, uni = ref.prepare_data_for_lloyd(X, init, 0.0, w, True)
    o_labels, o_inertia, o_C, o_iter = ref.lloyd(Xc, w, init_c, uni, max_iter, False, 0.0)

    km = KMeans(n_clusters=k, init=init, n_init=1, max_iter=max_iter, tol=0.0, algorithm="lloyd")
    km.fit(torch.as_tensor(X).cuda())
    assert km.n_iter_ == o_iter
    ok, n_bad, n_unexplained = ref.labels_agree(_np(km.labels_), o_labels, Xc, o_C)
    assert ok, (n_bad, n_unexplained)
    assert_allclose(float(km.inertia_), float(o_inertia), rtol=1e-5)
    if n_bad == 0:
        o_centres = o_C + (mean if mean is not None else 0.0)
        assert_allclose(_np(km.cluster_centers_), o_centres, rtol=1e-4, atol=1e-4)
    # predict and score run the label-only form of the same kernel on the raw data
    pred = _np(km.predict(torch.as_tensor(X).cuda()))
    assert (pred != _np(km.labels_)).mean() < 1e-4
    assert_allclose(float(km.score(torch.as_tensor(X).cuda())), -float(o_inertia), rtol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_strict_convergence_and_tolerance_stop(dtype):
    """The loop must stop at the same iteration as the oracle, by strict convergence
    (tol=0, labels unchanged) and by the centre-shift tolerance.  The data overlap and the
    initial centres sit in two of the five blobs, so convergence takes several iterations
    (when labels already repeat at iteration 2, before the strict-convergence flag is armed,
    the stop depends on the shift being exactly zero, which float atomics do not guarantee
    in the reference either)."""
    from sklearn_numba_dpex_b200.kmeans.drivers import lloyd

    rng = np.random.default_rng(11)
    centers = rng.uniform(-20, 20, size=(5, 3))
    X = (centers[np.arange(2000) % 5] + 2.5 * rng.standard_normal((2000, 3))).astype(dtype)
    w = np.ones(2000, dtype=dtype)
    init = X[[0, 5, 10, 1, 6]].copy()
    for tol in (0.0, 1e-3, 1e-1):
        o = ref.lloyd(X, w, init, True, 50, False, tol)
        g = lloyd(torch.as_tensor(X).cuda().T, torch.as_tensor(w).cuda(), torch.as_tensor(init).cuda().T,
                  True, 50, False, tol)
        assert o[3] >= 4
        assert g[3] == o[3]
        ok, n_bad, n_unexplained = ref.labels_agree(_np(g[0]), o[0], X, o[2])
        assert ok, (n_bad, n_unexplained)
        if n_bad == 0:
            assert_allclose(_np(g[2].T), o[2], rtol=1e-5 if dtype == np.float32 else 1e-11, atol=1e-5)


# ------------------------------------------------------------------ testing mode
@pytest.mark.parametrize("dtype", DTYPES)
def test_testing_mode_conversions(dtype, monkeypatch):
    """With the testing-mode variable set the engine hands scikit-learn's own types around, as
    the reference does for scikit-learn's test-suite (engine.py:108-115, 156-170, 219-225,
    253-255, 287-290 there): numpy int32 labels, centres in the estimator's output dtype,
    numpy distances, and label utilities that accept numpy labels."""
    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine
    from sklearn_numba_dpex_b200.kmeans.engine import TESTING_MODE_ENV, NotSupportedByEngineError

    monkeypatch.setenv(TESTING_MODE_ENV, "1")
    X, _ = make_blobs(n_samples=300, centers=4, n_features=5, random_state=3)
    X = X.astype(dtype)
    init = X[:4].copy()
    est = KMeans(n_clusters=4, init=init, n_init=1, max_iter=5, tol=0.0, copy_x=False)
    engine = KMeansEngine(est)
    assert engine._is_in_testing_mode
    X_before = X.copy()
    Xp, _, sw = engine.prepare_fit(X)
    assert est._output_dtype == dtype
    centers_init_t = engine.init_centroids(Xp, sw)
    labels, inertia, centers, n_iter = engine.kmeans_single(Xp, sw, centers_init_t)
    assert isinstance(labels, np.ndarray) and labels.dtype == np.int32 and labels.shape == (300,)
    assert isinstance(centers, np.ndarray) and centers.dtype == dtype and centers.shape == (4, 5)
    assert centers.flags["C_CONTIGUOUS"]           # the transpose of the F-ordered (d, k) array
    engine.unshift_centers(Xp, centers)            # numpy centres, in place; X restored (copy_x=False)
    o = ref.lloyd(*_oracle_prepared(X_before, init, tol=0.0)[:4], 5, False, 0.0)
    mean = X_before.mean(axis=0, dtype=dtype)
    assert_array_equal(labels, o[0].astype(np.int32))
    assert_allclose(centers, o[2] + mean, rtol=_rtol(dtype) * 10, atol=1e-5)
    assert_allclose(_np(Xp), X_before, rtol=1e-6, atol=1e-6)

    # label utilities on numpy labels
    perm = np.array([2, 0, 3, 1], dtype=np.int32)
    assert engine.is_same_clustering(labels, perm[labels], 4) is True
    other = labels.copy()
    other[0] = (other[0] + 1) % 4
    assert engine.is_same_clustering(labels, other, 4) is False
    assert int(engine.count_distinct_clusters(labels)) == 4

    # prediction side
    est.cluster_centers_ = centers
    Xq, swq = engine.prepare_prediction(X_before, None)
    pred = engine.get_labels(Xq, swq)
    assert isinstance(pred, np.ndarray) and pred.dtype == np.int32
    assert_array_equal(pred, labels)
    dist = engine.get_euclidean_distances(X_before)
    assert isinstance(dist, np.ndarray) and dist.dtype == dtype and dist.shape == (300, 4)
    assert_allclose(dist, ref.euclidean_distances(X_before, centers), rtol=1e-4, atol=1e-5)
    assert np.isscalar(engine.get_score(Xq, swq)) or np.ndim(engine.get_score(Xq, swq)) == 0

    # unsupported requests raise instead of declining
    est2 = KMeans(n_clusters=2, algorithm="elkan")
    with pytest.raises(NotSupportedByEngineError):
        KMeansEngine(est2).accepts(X, None, None)
    monkeypatch.setenv(TESTING_MODE_ENV, "0")
    assert KMeansEngine(est2).accepts(X, None, None) is False
    monkeypatch.setenv(TESTING_MODE_ENV, "yes")
    with pytest.raises(ValueError, match="expected to take"):
        KMeansEngine(est2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_non_finite_inputs_are_rejected_for_every_array_type(dtype):
    # engine.py:319-331 of the reference validates every array type with force_all_finite=True
    from sklearn_numba_dpex_b200.kmeans import KMeans

    X = np.random.default_rng(0).standard_normal((50, 3)).astype(dtype)
    for bad in (np.nan, np.inf, -np.inf):
        Xb = X.copy()
        Xb[17, 1] = bad
        for arr in (Xb, torch.as_tensor(Xb), torch.as_tensor(Xb).cuda()):
            with pytest.raises(ValueError, match="NaN|infinity|inf"):
                KMeans(n_clusters=2, n_init=1).fit(arr)
    w = np.ones(50, dtype=dtype)
    w[3] = np.nan
    with pytest.raises(ValueError, match="NaN|infinity|inf"):
        KMeans(n_clusters=2, n_init=1).fit(torch.as_tensor(X).cuda(), sample_weight=torch.as_tensor(w).cuda())
    init = X[:2].copy()
    init[0, 0] = np.inf
    with pytest.raises(ValueError, match="NaN|infinity|inf"):
        KMeans(n_clusters=2, n_init=1, init=torch.as_tensor(init).cuda()).fit(torch.as_tensor(X).cuda())
    # finite data still pass
    KMeans(n_clusters=2, n_init=1, max_iter=2).fit(torch.as_tensor(X).cuda())


@pytest.mark.parametrize("weights", ["none", "uniform", "random"])
def test_random_init_keeps_numpys_index_stream(weights):
    """init="random" draws with numpy's RandomState.choice(n, k, replace=False, p=w/sum(w)) as the
    reference does (engine.py:188-196); with uniform weights the probabilities are rebuilt on the
    host instead of copying the weights back, and must give the very same rows."""
    from sklearn.utils import check_random_state

    from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

    rng = np.random.default_rng(9)
    n, d, k = 5000, 6, 17
    X = rng.standard_normal((n, d)).astype(np.float32) + 3.0
    sw = {"none": None, "uniform": np.full(n, 2.5, dtype=np.float32),
          "random": rng.uniform(0.1, 3.0, n).astype(np.float32)}[weights]
    est = KMeans(n_clusters=k, init="random", n_init=1, random_state=11)
    engine = KMeansEngine(est)
    Xp, _, swp = engine.prepare_fit(X, sample_weight=sw)
    assert engine.sample_weight_is_uniform == (weights != "random")
    centers = _np(engine.init_centroids(Xp, swp).T)
    w_np = np.ones(n, dtype=np.float32) if sw is None else sw
    idx = check_random_state(11).choice(n, size=k, replace=False, p=w_np / w_np.sum())
    assert_allclose(centers, _np(Xp)[idx])
