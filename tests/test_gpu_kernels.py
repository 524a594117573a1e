"""Kernel-level parity: each C-ABI entry point against the CPU oracle on seeded inputs.

Tolerances (stated by the task for this path): labels bit-exact except where the exact
squared distances of the two candidates tie within 1e-6 relative; centroid sums, centroids and
inertia within rtol 1e-5 (fp32) / 1e-12 (fp64), with an absolute floor tied to the magnitude
of the data for quantities that cancel to ~0.
"""
import os

import numpy as np
import pytest
import torch
from numpy.testing import assert_allclose, assert_array_equal

from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu

DTYPES = [np.float32, np.float64]
RTOL = {np.float32: 1e-5, np.float64: 1e-12}


def _dev(a):
    return torch.as_tensor(np.ascontiguousarray(a)).cuda()


def _blobs(rng, n, d, k, dtype, std=1.0):
    centers = rng.uniform(-10, 10, size=(k, d))
    X = centers[rng.integers(0, k, size=n)] + std * rng.standard_normal((n, d))
    return X.astype(dtype), centers.astype(dtype)


def _algos(dtype, n, d, k):
    from sklearn_numba_dpex_b200 import _cabi

    out = ["cuda_core"]
    code = _cabi.KMB_F32 if dtype == np.float32 else _cabi.KMB_F64
    if os.environ.get("KMB_TEST_NO_TC") == "1":
        return out
    # d that is not a multiple of 4 reaches the tensor-core step through a padded working copy
    d4 = (d + 3) // 4 * 4
    if _cabi.lib.kmb_lloyd_resolve_algo(code, _cabi.ALGO_TF32X3, n, d4, k) == _cabi.ALGO_TF32X3:
        out.append("tf32x3")
    return out


STEP_SHAPES = [
    # (n, d, k): edge tiles on purpose (n, d, k not multiples of the kernel tiles)
    (1, 1, 1), (7, 3, 2), (129, 14, 9), (1000, 17, 127), (513, 130, 5), (2000, 14, 256),
    (4096, 128, 1025), (3000, 64, 300), (50_000, 14, 127), (777, 32, 64), (2000, 20, 130),
    (1500, 100, 260), (40_000, 8, 128),
    # several sample tiles per CTA on the tensor-core step (buffer reuse and barrier phases across
    # tiles): odd and even numbers of centroid tiles, 1 to 4 feature chunks, resident and streamed
    # centroid stages, one and two sample tiles in flight
    (60_000, 64, 300), (60_000, 96, 200), (60_000, 128, 130), (70_000, 32, 600), (60_000, 20, 700),
    # short rows with one, two and four 8-feature slices (two or three accumulators in tensor memory)
    (30_000, 4, 200), (30_000, 12, 384), (60_000, 28, 300),
    # d padded to a multiple of 4 by the driver: the fold features go into the padding (two or
    # three spare features), also when the padded d fills its last 32-feature chunk (30 -> 32, 62 -> 64)
    (30_000, 13, 200), (40_000, 30, 150), (60_000, 62, 300), (40_000, 29, 140),
    # many clusters: labels above 32 767 and 65 535 / 128 centroid tiles per sample tile
    (2048, 8, 40_000),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", STEP_SHAPES, ids=lambda s: "n%d_d%d_k%d" % s)
@pytest.mark.parametrize("weighted", [False, True])
def test_lloyd_step_teacher_forced(dtype, shape, weighted):
    """One fused step from the oracle's state: labels, sums, counts, changed flag, new
    centroids, shift, empty list."""
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    n, d, k = shape
    rng = np.random.default_rng(n * 31 + d * 7 + k)
    X, _ = _blobs(rng, n, d, max(k, 1), dtype)
    C = X[rng.choice(n, size=k, replace=n < k)] + dtype(0.01) * rng.standard_normal((k, d)).astype(dtype)
    w = (rng.uniform(0.5, 2.0, size=n).astype(dtype) if weighted else np.ones(n, dtype=dtype))
    prev = rng.integers(0, k, size=n).astype(np.int32)
    ref_labels = ref.assign_labels(X, C)

    for algo in _algos(dtype, n, d, k):
        st = LloydState(_dev(X), _dev(w) if weighted else None, _dev(C), algo)
        st.labels.copy_(_dev(prev))
        st.have_prev = True
        st.launch_step()
        torch.cuda.synchronize()
        labels = st.labels_new.cpu().numpy().astype(np.int64)
        ok, n_bad, n_unexplained = ref.labels_agree(labels, ref_labels, X, C, rtol=1e-6)
        assert ok, f"{algo}: {n_unexplained} of {n_bad} label mismatches are not near-ties"

        # accumulators are checked against the oracle fed with the GPU's own labels, so a
        # legitimate near-tie does not blur the comparison
        sums, sizes = ref.accumulate_centroids(X.astype(np.float64), w.astype(np.float64), labels, k)
        packed = st.packed.cpu().numpy()
        dp = st.d  # feature count of the working copy (d rounded up to 4 on the padded path)
        scale = np.abs(X).max() * max(w.max(), 1.0) * max(n / k, 1.0)
        atol = RTOL[dtype] * scale
        got_sums = packed[: k * dp].reshape(k, dp)
        assert_allclose(got_sums[:, :d], sums, rtol=RTOL[dtype], atol=atol, err_msg=algo)
        assert not got_sums[:, d:].any()
        assert_allclose(packed[k * dp: k * dp + k], sizes, rtol=RTOL[dtype], err_msg=algo)
        assert packed[k * dp + k] == float((labels != prev).sum())

        rec = st.status_host  # not read yet: use the device record
        status = st.status_dev.cpu().numpy().view(_status_dtype())[0]
        empty = np.nonzero(sizes == 0)[0]
        assert status["n_empty"] == empty.size
        assert_array_equal(st.empty_list.cpu().numpy()[: empty.size], empty)
        assert status["changed"] == int((labels != prev).any())
        nz = sizes > 0
        with np.errstate(divide="ignore", invalid="ignore"):
            C_new = sums / sizes[:, None]
        got_C = st.C_new.cpu().numpy()[:, :d]
        catol = RTOL[dtype] * np.abs(X).max()
        assert_allclose(got_C[nz], C_new[nz], rtol=RTOL[dtype], atol=catol, err_msg=algo)
        if nz.all():
            shift = ((C.astype(np.float64) - C_new) ** 2).sum()
            assert_allclose(status["shift_total"], shift, rtol=1e-4 if dtype == np.float32 else 1e-9)
            h = 0.5 * (got_C.astype(np.float64) ** 2).sum(axis=1)
            assert_allclose(st.h_new.cpu().numpy(), h, rtol=1e-6 if dtype == np.float32 else 1e-13)


def _status_dtype():
    from sklearn_numba_dpex_b200._cabi import STATUS_DTYPE

    return STATUS_DTYPE


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_first_iteration_counts_all_as_changed(dtype):
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    rng = np.random.default_rng(5)
    X, C = _blobs(rng, 300, 5, 4, dtype)
    st = LloydState(_dev(X), None, _dev(C), "cuda_core")
    n_empty, changed, _ = st.step()
    assert changed == 1 and n_empty == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_labels_ties_pick_lowest_index_and_nan_never_wins(dtype):
    from sklearn_numba_dpex_b200.kmeans.drivers import get_labels_inertia

    # duplicated centroids: the lower index must win
    X = np.array([[0.0, 0.0], [1.0, 1.0], [5.0, 5.0]], dtype=dtype)
    C = np.array([[1.0, 1.0], [0.0, 0.0], [0.0, 0.0], [1.0, 1.0], [5.0, 5.0], [5.0, 5.0]], dtype=dtype)
    labels, _ = get_labels_inertia(_dev(X).T, _dev(C).T, _dev(np.ones(3, dtype=dtype)), False)
    assert_array_equal(labels.cpu().numpy(), [1, 0, 4])
    # a NaN centroid never wins; all-NaN gives label 0
    C2 = np.array([[np.nan, 0.0], [3.0, 3.0]], dtype=dtype)
    labels, _ = get_labels_inertia(_dev(X).T, _dev(C2).T, _dev(np.ones(3, dtype=dtype)), False)
    assert_array_equal(labels.cpu().numpy(), [1, 1, 1])
    C3 = np.full((2, 2), np.nan, dtype=dtype)
    labels, _ = get_labels_inertia(_dev(X).T, _dev(C3).T, _dev(np.ones(3, dtype=dtype)), False)
    assert_array_equal(labels.cpu().numpy(), [0, 0, 0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(100, 10, 5), (5000, 14, 127), (3001, 129, 33), (64, 1, 3)])
def test_inertia_and_distances(dtype, shape):
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:161-205 (negative weights are legal)
    from sklearn_numba_dpex_b200.kmeans.drivers import (get_euclidean_distances,
                                                        get_labels_inertia)

    n, d, k = shape
    rng = np.random.default_rng(42)
    X = rng.random((n, d)).astype(dtype)
    w = rng.standard_normal(n).astype(dtype)
    C = rng.standard_normal((k, d)).astype(dtype)
    labels, inertia = get_labels_inertia(_dev(X).T, _dev(C).T, _dev(w), True)
    labels = labels.cpu().numpy()
    ok, _, _ = ref.labels_agree(labels, ref.assign_labels(X, C), X, C)
    assert ok
    expected = ref.compute_inertia_per_sample(X, w, C, labels, exact=True)
    rtol = 1e-4 if dtype == np.float32 else 1e-9
    assert_allclose(float(inertia[0]), expected.sum(), rtol=rtol, atol=rtol * np.abs(expected).sum())
    D = get_euclidean_distances(_dev(X).T, _dev(C).T).cpu().numpy()
    assert D.shape == (n, k)
    assert_allclose(D, ref.euclidean_distances(X.astype(np.float64), C.astype(np.float64)),
                    rtol=1e-4 if dtype == np.float32 else 1e-7)


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
def test_topk_tie_cases(dtype, k):
    from sklearn_numba_dpex_b200.common import topk, topk_idx

    for case in TOPK_CASES:
        arr = np.array(case, dtype=dtype)
        vals = topk(_dev(arr), k).cpu().numpy()
        idx = topk_idx(_dev(arr), k).cpu().numpy()
        assert idx.dtype == np.int64
        assert_array_equal(np.sort(vals), np.sort(arr)[-k:])
        # deterministic rule of this build: descending value, ascending index
        assert_array_equal(idx, ref.topk_idx(arr, k))
        assert_array_equal(vals, ref.topk(arr, k))
    multi = np.array(TOPK_CASES, dtype=dtype)
    assert_array_equal(topk_idx(_dev(multi), k).cpu().numpy(), ref.topk_idx(multi, k))
    assert_array_equal(topk(_dev(multi), k).cpu().numpy(), ref.topk(multi, k))


@pytest.mark.parametrize("dtype", DTYPES)
def test_topk_random_and_errors(dtype):
    from sklearn_numba_dpex_b200.common import topk, topk_idx

    rng = np.random.default_rng(123)
    arr = rng.normal(size=(200, 1000)).astype(dtype)
    for k in (1, 3, 50):
        assert_array_equal(topk(_dev(arr), k).cpu().numpy(), -np.sort(-arr)[:, :k])
    big = rng.normal(size=1_000_003).astype(dtype)
    big[rng.integers(0, big.size, 1000)] = big.max()  # many ties at the top
    for k in (1, 7, 1500):
        assert_array_equal(topk_idx(_dev(big), k).cpu().numpy(), ref.topk_idx(big, k))
    with pytest.raises(ValueError, match="Expected k to be greater than or equal"):
        topk(_dev(arr[0, :5]), 6)
    with pytest.raises(ValueError, match="only supports dtypes"):
        topk(torch.arange(10, device="cuda"), 2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_relocation_kernel(dtype):
    from sklearn_numba_dpex_b200 import _cabi
    from sklearn_numba_dpex_b200._cabi import check, lib, ptr, stream_ptr

    rng = np.random.default_rng(9)
    n, d, k = 500, 6, 12
    X = rng.standard_normal((n, d)).astype(dtype)
    w = rng.uniform(0.5, 2, n).astype(dtype)
    labels = rng.integers(0, 9, size=n)  # clusters 9, 10, 11 stay empty
    sums, sizes = ref.accumulate_centroids(X, w, labels, k)
    empty = np.array([9, 10, 11], dtype=np.uint32)
    far = np.array([17, 3, 255], dtype=np.int64)
    exp_s, exp_c = sums.copy(), sizes.copy()
    ref.relocate_empty_clusters(X, w, exp_s, exp_c, labels, empty, far)
    acc_len = lib.kmb_lloyd_acc_len(d, k)
    acc = np.zeros(acc_len, dtype=dtype)
    acc[: k * d] = sums.ravel()
    acc[k * d: k * d + k] = sizes
    acc_d = _dev(acc)
    code = _cabi.dtype_code(acc_d.dtype)
    # keep every device buffer alive until the kernel has run
    Xd, wd, lab_d = _dev(X), _dev(w), _dev(labels.astype(np.int32))
    far_d, empty_d = _dev(far), _dev(empty.astype(np.int32))
    check(lib.kmb_relocate_empty_clusters(code, ptr(Xd), ptr(wd), ptr(lab_d), n, ptr(far_d),
                                          ptr(empty_d), 3, None, ptr(acc_d), d, k, stream_ptr()))
    torch.cuda.synchronize()
    got = acc_d.cpu().numpy()
    assert_allclose(got[: k * d].reshape(k, d), exp_s, rtol=1e-5, atol=1e-5)
    assert_allclose(got[k * d: k * d + k], exp_c, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1000, 5), (4099, 14), (513, 40), (3000, 128)])
def test_prepare_and_restore(dtype, shape):
    from sklearn_numba_dpex_b200.kmeans.drivers import (prepare_data_for_lloyd,
                                                        restore_data_after_lloyd)

    n, d = shape
    rng = np.random.default_rng(1)
    X = (rng.standard_normal((n, d)) + 3.0).astype(dtype)
    init = X[:4].copy()
    w = np.ones(n, dtype=dtype)
    Xd = _dev(X)
    X_t, X_mean, init_t, tol, uniform = prepare_data_for_lloyd(Xd.T, _dev(init).T, 1e-4, _dev(w), True)
    eX, eMean, eInit, eTol, eUni = ref.prepare_data_for_lloyd(X, init, 1e-4, w, True)
    rt = 1e-5 if dtype == np.float32 else 1e-11
    assert_allclose(X_mean.cpu().numpy(), eMean, rtol=rt)
    assert_allclose(X_t.T.cpu().numpy(), eX, rtol=rt, atol=rt * 10)
    assert_allclose(init_t.T.cpu().numpy(), eInit, rtol=rt, atol=rt * 10)
    assert_allclose(tol, eTol, rtol=1e-4 if dtype == np.float32 else 1e-10)
    assert uniform == eUni and uniform
    assert_array_equal(Xd.cpu().numpy(), X)  # copy_x=True leaves the input alone
    # in place + restore
    X_t2, X_mean2, _, _, uni2 = prepare_data_for_lloyd(Xd.T, "random", 1e-4,
                                                       _dev(rng.uniform(1, 2, n).astype(dtype)), False)
    assert X_t2.T.data_ptr() == Xd.data_ptr() and not uni2
    C = torch.zeros((d, 3), dtype=Xd.dtype, device="cuda").T.contiguous().T
    restore_data_after_lloyd(X_t2, C, X_mean2, False)
    assert_allclose(Xd.cpu().numpy(), X, rtol=rt, atol=rt * 10)
    assert_allclose(C.T.cpu().numpy(), np.tile(eMean, (3, 1)), rtol=rt)
    # already centred data: no shift recorded
    Z = np.array([[1.0, -1.0], [-1.0, 1.0]], dtype=dtype)
    _, zmean, _, _, _ = prepare_data_for_lloyd(_dev(Z).T, "random", 1e-4, _dev(np.ones(2, dtype=dtype)), True)
    assert zmean is None


@pytest.mark.parametrize("dtype", DTYPES)
def test_sum_reductions_reference_cases(dtype):
    """The cases of the reference's common/tests/test_reductions.py:16-70 that lie on the KMeans
    path: sums over the samples of every feature (its axis-1 sum of the (d, n) layout) on the
    small shapes listed there, and the two 1-D sums (0+1+2+3 = 6, 0+..+4 = 10), plus a size
    that spans many blocks."""
    from sklearn_numba_dpex_b200._cabi import check, dtype_code, lib, ptr, stream_ptr, workspace_for

    for shape in [(1, 1), (1, 3), (3, 1), (3, 5), (5, 3), (3, 4), (4, 3), (3, 9), (70_001, 5)]:
        a = np.arange(shape[0] * shape[1], dtype=dtype).reshape(shape) % 1000
        X = _dev(a)
        out = torch.empty(shape[1], dtype=torch.float64, device=X.device)
        ws, ws_bytes = workspace_for(X.device, shape[0], shape[1], 1)
        check(lib.kmb_col_sums(dtype_code(X.dtype), ptr(X), shape[0], shape[1], ptr(out), ptr(ws),
                               ws_bytes, stream_ptr(X.device)))
        assert_allclose(out.cpu().numpy(), a.astype(np.float64).sum(axis=0), rtol=1e-12)
    for length, expected in [(4, 6.0), (5, 10.0), (100_003, None)]:
        v = np.arange(length, dtype=dtype) % 100
        x = _dev(v)
        ws, ws_bytes = workspace_for(x.device, length, 1, 1)
        for square in (0, 1):
            out = torch.empty(1, dtype=torch.float64, device=x.device)
            check(lib.kmb_sum(dtype_code(x.dtype), ptr(x), length, square, ptr(out), ptr(ws), ws_bytes,
                              stream_ptr(x.device)))
            want = float((v.astype(np.float64) ** (2 if square else 1)).sum())
            assert float(out[0]) == pytest.approx(want, rel=1e-12)
            if expected is not None and not square:
                assert float(out[0]) == expected


def test_label_utilities():
    # sklearn_numba_dpex/kmeans/tests/test_kmeans.py:448-457
    from sklearn_numba_dpex_b200.kmeans.drivers import (get_nb_distinct_clusters,
                                                        is_same_clustering)

    labels = torch.tensor([0, 1, 0, 2, 2, 7, 6, 5, 3, 3], dtype=torch.int32, device="cuda")
    assert int(get_nb_distinct_clusters(labels, 8)) == 7
    a = torch.tensor([0, 0, 1, 2, 2], dtype=torch.int32, device="cuda")
    b = torch.tensor([2, 2, 0, 1, 1], dtype=torch.int32, device="cuda")
    c = torch.tensor([2, 1, 0, 1, 1], dtype=torch.int32, device="cuda")
    assert is_same_clustering(a, b, 3)
    assert not is_same_clustering(a, c, 3)
    rng = np.random.default_rng(0)
    big = rng.integers(0, 50, size=200_000)
    perm = rng.permutation(50)
    assert is_same_clustering(_dev(big.astype(np.int32)), _dev(perm[big].astype(np.int32)), 50)
    assert ref.is_same_clustering(big, perm[big], 50)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("algo", ["cuda_core", "tf32x3"])
def test_matmul_hook(dtype, algo):
    # sklearn_numba_dpex/common/tests/test_matmul.py:71-164 (prime-sized case included)
    from sklearn_numba_dpex_b200 import _cabi
    from sklearn_numba_dpex_b200._cabi import check, check_wait_error, lib, lloyd_workspace, ptr, stream_ptr

    code = _cabi.KMB_F32 if dtype == np.float32 else _cabi.KMB_F64
    rng = np.random.default_rng(3)
    if algo == "tf32x3" and os.environ.get("KMB_TEST_NO_TC") == "1":
        pytest.skip("tensor-core path disabled for this run")
    for m, n, kd in [(5, 3, 2), (100, 37, 64), (1999, 661, 563), (257, 129, 130), (1999, 661, 128),
                     (300, 1025, 96), (128, 128, 32)]:
        if algo == "tf32x3" and lib.kmb_lloyd_resolve_algo(code, _cabi.ALGO_TF32X3, m, kd, n) != _cabi.ALGO_TF32X3:
            continue
        A = rng.standard_normal((m, kd)).astype(dtype)
        B = rng.standard_normal((n, kd)).astype(dtype)
        Ad, Bd = _dev(A), _dev(B)
        out = torch.empty((m, n), dtype=Ad.dtype, device="cuda")
        ws, wsb = lloyd_workspace(out.device, m, kd, n)
        check(lib.kmb_matmul_nt(code, _cabi.ALGO_NAMES[algo], ptr(Ad), ptr(Bd), ptr(out),
                                m, n, kd, ptr(ws), wsb, stream_ptr()))
        torch.cuda.synchronize()
        check_wait_error(ws, out.device)
        expect = A.astype(np.float64) @ B.astype(np.float64).T
        tol = 2e-6 if dtype == np.float32 else 1e-13
        assert_allclose(out.cpu().numpy(), expect, rtol=0, atol=tol * np.sqrt(kd) * 4)


def test_wait_error_flag_is_sticky_and_reaches_the_status_record():
    """The time-out flag of the tensor-core kernel, exercised from the host only (no kernel is
    made to wait): a flag raised in the workspace's control block is reported by
    kmb_lloyd_wait_error, survives further steps (no launch clears it), travels in the status
    record of the next finalize, and is cleared by kmb_lloyd_workspace_init."""
    from sklearn_numba_dpex_b200._cabi import (KmbError, check, check_wait_error, lib, ptr, stream_ptr)
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    rng = np.random.default_rng(0)
    n, d, k = 40_000, 16, 128
    X, _ = _blobs(rng, n, d, k, np.float32)
    C = X[rng.choice(n, size=k, replace=False)].copy()
    st = LloydState(_dev(X), None, _dev(C), "auto")
    assert st.is_tc
    st.step()
    st.check_device_waits()                       # clean so far
    flag = torch.tensor([1], dtype=torch.int32, device="cuda").view(torch.uint8)
    base = (st.ws.data_ptr() + 255) // 256 * 256 - st.ws.data_ptr()
    st.ws[base: base + 4] = flag                  # what a timed-out wait would have stored
    with pytest.raises(KmbError, match="bounded wait"):
        st.check_device_waits()
    with pytest.raises(KmbError, match="bounded wait"):
        st.step()                                 # the flag rides on the status record
    with pytest.raises(KmbError, match="bounded wait"):
        st.check_device_waits()                   # and nothing has cleared it
    check(lib.kmb_lloyd_workspace_init(ptr(st.ws), st.ws_bytes, stream_ptr(st.X.device)))
    st.operands_ready = False
    st.check_device_waits()
    st.step()                                     # usable again
    check_wait_error(st.ws, st.X.device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3000, 5, 12), (40_000, 16, 130)], ids=lambda s: "n%d_d%d_k%d" % s)
def test_pipelined_loop_equals_step_by_step(dtype, shape):
    """`LloydState.run` enqueues iteration i + 1 before it has read the status of iteration i.
    On data whose first iterations relocate empty clusters (duplicated initial centres) and
    that then converges strictly, the pipelined loop must take the same decisions and end in
    the same state as the loop that reads every status first, and as the CPU oracle."""
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    n, d, k = shape
    rng = np.random.default_rng(n + k)
    X, _ = _blobs(rng, n, d, k, dtype, std=0.3)
    C = X[rng.choice(n, size=k, replace=False)].copy()
    C[1] = C[0]
    C[k - 1] = C[2]                       # two clusters start empty -> relocation in iteration 1
    w = np.ones(n, dtype=dtype)
    results = []
    for pipelined in (True, False):
        st = LloydState(_dev(X), None, _dev(C), "auto")
        out = st.run(40, 0.0, pipelined=pipelined)
        labels, total = st.final_labels_inertia()
        results.append((out, labels.cpu().numpy(), st.centers().cpu().numpy(), float(total[0]), st.it))
    (o1, l1, c1, i1, it1), (o2, l2, c2, i2, it2) = results
    assert o1["n_relocation_events"] >= 1 and o1["n_empty_max"] >= 2
    assert (o1["strict"], o1["n_relocation_events"]) == (o2["strict"], o2["n_relocation_events"])
    assert it1 == o1["n_iter"] and it2 == o2["n_iter"]
    assert o1["strict"] and 3 <= o1["n_iter"] < 40
    if dtype == np.float64:
        assert o1["n_iter"] == o2["n_iter"]
        assert_array_equal(l1, l2)
        assert_allclose(c1, c2, rtol=1e-11, atol=1e-11)
        assert_allclose(i1, i2, rtol=1e-11)
    else:
        # float32 sums are accumulated with unordered atomics: two runs of the SAME loop can flip
        # a boundary sample and then need a different number of iterations until no label
        # changes any more (usually one or two apart, seven have been seen), pipelined or not;
        # the float64 case above is the exact check of the loop's decisions
        assert abs(o1["n_iter"] - o2["n_iter"]) <= 12
        assert (l1 != l2).mean() < 1e-2
        assert_allclose(i1, i2, rtol=1e-3)
    # against the oracle's own free-running loop: a float32 run of ~25 iterations may flip a
    # boundary sample on the way and then converge an iteration apart, so only the end state
    # is compared, loosely; step-by-step agreement is what the teacher-forced tests check
    o_labels, o_inertia, o_C, o_iter = ref.lloyd(X, w, C, True, 40, False, 0.0)
    assert abs(o_iter - o1["n_iter"]) <= (0 if dtype == np.float64 else 12)
    assert (l1 != o_labels).mean() < 1e-2
    assert_allclose(i1, float(o_inertia), rtol=1e-4 if dtype == np.float32 else 1e-9)


def test_run_can_ignore_strict_convergence_and_counts_steps():
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    rng = np.random.default_rng(2)
    X, _ = _blobs(rng, 2000, 4, 5, np.float32, std=0.2)
    st = LloydState(_dev(X), None, _dev(X[:5].copy()), "auto")
    out = st.run(25, -1.0, stop_on_strict=False)
    assert out["n_iter"] == 25 and st.it == 25 and not out["strict"]
    seen = []
    st.event_hook = lambda kind, it: seen.append((kind, it))
    st.run(3, -1.0, stop_on_strict=False)
    st.event_hook = None
    assert seen == [("pre", 25), ("post", 25), ("pre", 26), ("post", 26), ("pre", 27), ("post", 27)]


@pytest.mark.parametrize("dtype", DTYPES)
def test_sharded_seeding_glue_kernels(dtype):
    """kmb_kpp_pick_owned and kmb_kpp_select_shards (the two glue kernels of a row-sharded
    k-means++ round) on gathered buffers made up here for four shards, against numpy."""
    from sklearn_numba_dpex_b200._cabi import check, dtype_code, lib, ptr, stream_ptr

    rng = np.random.default_rng(11)
    world, t, d, c = 4, 6, 10, 3
    tdt = torch.float32 if dtype == np.float32 else torch.float64
    code = dtype_code(tdt)
    dev = torch.device("cuda", torch.cuda.current_device())
    s = stream_ptr(dev)

    # ---- pick_owned: shares -> ends; thresholds on, before and after shard boundaries
    shares = rng.uniform(1.0, 3.0, size=world)
    ends = np.cumsum(shares)
    total = dtype(ends[-1])
    u = np.array([0.0, shares[0] / ends[-1], 0.3, 0.55, 0.999, 1.5], dtype=dtype)   # last one beyond every prefix
    rows = rng.standard_normal((world, t, d)).astype(dtype)
    ids = rng.integers(0, 1000, size=(world, t)).astype(np.int32)
    rows_off = np.array([0, 1000, 2000, 3000], dtype=np.int64)
    id_col = ids.view(np.float32) if dtype == np.float32 else ids.astype(dtype)
    gathered = np.concatenate([rows, id_col[:, :, None]], axis=2)
    r = (u * total).astype(np.float64)
    owner = np.minimum((ends[None, :] < r[:, None]).sum(axis=1), world - 1)
    want_ids = ids[owner, np.arange(t)].astype(np.int64) + rows_off[owner]
    want_rows = rows[owner, np.arange(t)]
    cand = torch.empty(t, dtype=torch.int32, device=dev)
    out_rows = torch.empty((t, d), dtype=tdt, device=dev)
    g_d, e_d, u_d = _dev(gathered), _dev(ends), _dev(u)          # kept alive until the results are read
    t_d, o_d = _dev(np.array([total], dtype=dtype)), _dev(rows_off)
    check(lib.kmb_kpp_pick_owned(code, ptr(g_d), world, t, d, ptr(e_d), ptr(u_d), ptr(t_d), ptr(o_d),
                                 ptr(cand), ptr(out_rows), s), "kmb_kpp_pick_owned")
    assert_array_equal(cand.cpu().numpy(), want_ids)
    assert_array_equal(out_rows.cpu().numpy(), want_rows)

    # ---- select_shards: potentials summed over the shards, lowest trial on ties
    shard_pots = rng.uniform(1.0, 2.0, size=(world, t))
    shard_pots[:, 4] = shard_pots[:, 1]                  # a tie between trials 1 and 4 ...
    shard_pots[:, 1] *= 0.25                             # ... made the minimum
    shard_pots[:, 4] *= 0.25
    pots_want = shard_pots.sum(axis=0).astype(dtype)
    best_want = int(np.argmin(pots_want))
    assert best_want == 1
    pots = torch.empty(t, dtype=tdt, device=dev)
    best = torch.zeros(1, dtype=torch.int32, device=dev)
    tot = torch.empty(1, dtype=tdt, device=dev)
    centers = torch.zeros((5, d), dtype=tdt, device=dev)
    indices = torch.full((5,), -1, dtype=torch.int32, device=dev)
    ends_out = torch.empty(world, dtype=torch.float64, device=dev)
    off_out = torch.empty(1, dtype=torch.float64, device=dev)
    sp_d = _dev(shard_pots)
    for shard in (0, 2):
        check(lib.kmb_kpp_select_shards(code, ptr(sp_d), world, shard, t, ptr(pots), ptr(best),
                                        ptr(tot), ptr(out_rows), ptr(cand), ptr(centers), ptr(indices), c, d,
                                        ptr(ends_out), ptr(off_out), s), "kmb_kpp_select_shards")
        assert_allclose(pots.cpu().numpy(), pots_want, rtol=1e-6 if dtype == np.float32 else 1e-15)
        assert int(best.cpu()) == best_want
        assert_allclose(float(tot.cpu()), pots_want[best_want], rtol=1e-6 if dtype == np.float32 else 1e-15)
        assert_array_equal(centers.cpu().numpy()[c], want_rows[best_want])
        assert int(indices.cpu()[c]) == int(want_ids[best_want])
        col = shard_pots[:, best_want]
        assert_allclose(ends_out.cpu().numpy(), np.cumsum(col), rtol=1e-15)
        assert_allclose(float(off_out.cpu()), np.cumsum(col)[shard] - col[shard], rtol=1e-14, atol=1e-15)
