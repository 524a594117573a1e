"""numpy restatement of the reference's KMeans drivers (test infrastructure only).

Arrays here are sample-major: ``X`` is ``(n_samples, n_features)`` and ``C`` is
``(n_clusters, n_features)``; the reference holds the transposes ``X_t (d, n)`` and
``centroids_t (d, k)``.  Each function names the reference lines it follows
(paths are relative to the reference project root).

Two arithmetic modes:
  * faithful  accumulates in the compute dtype, features in ascending order, the
              way one reference work-item does;
  * exact     accumulates in float64 (used to classify near-ties).
Where the reference's evaluation order is undefined (float atomics) the sum is
taken in float64 and rounded once to the compute dtype.
"""
import math

import numpy as np

from .rng import Xoroshiro128ppStates


# --------------------------------------------------------------------------- helpers
def _chunks(n, size):
    for start in range(0, n, size):
        yield start, min(n, start + size)


def half_l2_norm(C):
    """sklearn_numba_dpex/common/kernels.py:117-145  (sum over features, then / 2)."""
    C = np.asarray(C)
    T = C.dtype.type
    acc = np.zeros(C.shape[0], dtype=C.dtype)
    for f in range(C.shape[1]):
        acc += C[:, f] * C[:, f]
    return (acc / T(2.0)).astype(C.dtype)


def pseudo_inertia(X, C, h=None, exact=False, chunk=8192):
    """q[i, j] = h[j] - sum_f X[i, f] * C[j, f].

    kmeans/kernels/_base_kmeans_kernel_funcs.py:266-301 (multiply then add, feature
    by feature) and :351-366 (h - dot).
    """
    X = np.asarray(X)
    C = np.asarray(C)
    if exact:
        X64 = X.astype(np.float64)
        C64 = C.astype(np.float64)
        h64 = 0.5 * (C64 * C64).sum(axis=1)
        return h64[None, :] - X64 @ C64.T
    if h is None:
        h = half_l2_norm(C)
    n, d = X.shape
    out = np.empty((n, C.shape[0]), dtype=X.dtype)
    Ct = np.ascontiguousarray(C.T)
    for a, b in _chunks(n, chunk):
        dot = np.zeros((b - a, C.shape[0]), dtype=X.dtype)
        for f in range(d):
            dot += X[a:b, f : f + 1] * Ct[f : f + 1, :]
        out[a:b] = h[None, :] - dot
    return out


def assign_labels(X, C, h=None, exact=False, chunk=8192):
    """argmin_j q[i, j], strict '<' from +inf scanning j upward, so the lowest index
    wins ties and NaN never wins (_base_kmeans_kernel_funcs.py:351-366;
    kmeans/kernels/compute_labels.py:75-168)."""
    X = np.asarray(X)
    n = X.shape[0]
    labels = np.zeros(n, dtype=np.uint32)
    for a, b in _chunks(n, chunk):
        q = pseudo_inertia(X[a:b], C, h, exact=exact, chunk=chunk)
        q = np.where(np.isnan(q), np.inf, q)
        lab = np.argmin(q, axis=1)  # first occurrence of the minimum
        allinf = np.isinf(q[np.arange(b - a), lab]) & (q[np.arange(b - a), lab] > 0)
        lab[allinf] = 0
        labels[a:b] = lab
    return labels


def near_tie_mask(X, C, rtol=1e-6, chunk=8192):
    """True where the two smallest exact squared distances differ by <= rtol relative
    to the larger of them: on those samples two implementations may disagree."""
    X64 = np.asarray(X, dtype=np.float64)
    C64 = np.asarray(C, dtype=np.float64)
    n = X64.shape[0]
    mask = np.zeros(n, dtype=bool)
    if C64.shape[0] < 2:
        return mask
    cc = (C64 * C64).sum(axis=1)
    for a, b in _chunks(n, chunk):
        xx = (X64[a:b] * X64[a:b]).sum(axis=1)
        d2 = xx[:, None] - 2.0 * (X64[a:b] @ C64.T) + cc[None, :]
        part = np.partition(d2, 1, axis=1)[:, :2]
        scale = np.maximum(np.abs(part[:, 1]), xx + 1e-300)
        mask[a:b] = (part[:, 1] - part[:, 0]) <= rtol * scale
    return mask


def labels_agree(labels_a, labels_b, X, C, rtol=1e-6):
    """Labels must be equal except where the candidates' exact distances tie within
    `rtol` (relative).  Returns (ok, n_mismatch, n_unexplained)."""
    labels_a = np.asarray(labels_a).astype(np.int64)
    labels_b = np.asarray(labels_b).astype(np.int64)
    bad = np.nonzero(labels_a != labels_b)[0]
    if bad.size == 0:
        return True, 0, 0
    X64 = np.asarray(X, dtype=np.float64)[bad]
    C64 = np.asarray(C, dtype=np.float64)
    da = ((X64 - C64[labels_a[bad]]) ** 2).sum(axis=1)
    db = ((X64 - C64[labels_b[bad]]) ** 2).sum(axis=1)
    xx = (X64 * X64).sum(axis=1)
    scale = np.maximum(np.maximum(da, db), xx)
    unexplained = np.abs(da - db) > rtol * scale
    return not unexplained.any(), int(bad.size), int(unexplained.sum())


def accumulate_centroids(X, w, labels, k):
    """sums[j, :] = sum_{i: label_i = j} w_i * X[i, :],  sizes[j] = sum w_i
    (kmeans/kernels/lloyd_single_step.py:394-414).  The product w*x is rounded to the
    compute dtype as in the kernel; the order of the float atomics is undefined, so the
    accumulation itself is done in float64 and rounded once."""
    X = np.asarray(X)
    T = X.dtype
    labels = np.asarray(labels).astype(np.int64)
    sums = np.zeros((k, X.shape[1]), dtype=np.float64)
    for f in range(X.shape[1]):
        prod = (X[:, f] * w).astype(T)
        sums[:, f] = np.bincount(labels, weights=prod.astype(np.float64), minlength=k)
    sizes = np.bincount(labels, weights=np.asarray(w, dtype=np.float64), minlength=k)
    return sums.astype(T), sizes.astype(T)


def compute_inertia_per_sample(X, w, C, labels, exact=False):
    """w_i * sum_f (X[i,f] - C[label_i,f])**2, features ascending
    (kmeans/kernels/compute_inertia.py:14-39)."""
    X = np.asarray(X)
    C = np.asarray(C)
    labels = np.asarray(labels).astype(np.int64)
    if exact:
        diff = X.astype(np.float64) - C.astype(np.float64)[labels]
        return (diff * diff).sum(axis=1) * np.asarray(w, dtype=np.float64)
    acc = np.zeros(X.shape[0], dtype=X.dtype)
    for f in range(X.shape[1]):
        diff = X[:, f] - C[labels, f]
        acc += diff * diff
    return (acc * w).astype(X.dtype)


def tree_sum(values, dtype=None):
    """The reference sums with a multi-launch pairwise tree (common/reductions.py:
    214-393); numpy's pairwise float sum in the same dtype stands for it."""
    values = np.asarray(values)
    dtype = values.dtype if dtype is None else dtype
    return values.astype(dtype).sum(dtype=dtype)


def euclidean_distances(X, Y):
    """D[i, j] = sqrt(sum_f (Y[j,f] - X[i,f])**2)
    (kmeans/kernels/compute_euclidean_distances.py:63-152)."""
    X = np.asarray(X)
    Y = np.asarray(Y)
    out = np.zeros((X.shape[0], Y.shape[0]), dtype=X.dtype)
    for f in range(X.shape[1]):
        diff = Y[None, :, f] - X[:, f : f + 1]
        out += diff * diff
    return np.sqrt(out)


# ------------------------------------------------------------------- top-k / argmin
def topk_idx(values, k):
    """Indices of the k largest values (common/topk.py:194-270).  The reference leaves
    the output order and the choice among tied threshold values undefined; this
    restatement returns them by descending value, then ascending index."""
    values = np.asarray(values)
    if values.dtype not in (np.float32, np.float64):
        raise ValueError(f"topk currently only supports float32/float64, got {values.dtype}")
    if values.ndim == 2:
        return np.stack([topk_idx(row, k) for row in values])
    if values.shape[0] < k:
        raise ValueError(
            "Expected k to be greater than or equal to the number of items in the "
            f"search space, but got k={k} and {values.shape[0]} items in the search space."
        )
    order = np.lexsort((np.arange(values.shape[0]), -values.astype(np.float64)))
    return order[:k].astype(np.int64)


def topk(values, k):
    """The k largest values (common/topk.py:112-191), descending."""
    values = np.asarray(values)
    if values.ndim == 2:
        return np.stack([topk(row, k) for row in values])
    return values[topk_idx(values, k)]


def argmin_lowest_index(values):
    """1-D argmin, ties to the lowest index, int32 result
    (common/reductions.py:105-144, 165-169, 194-198)."""
    return np.int32(np.argmin(np.asarray(values)))


# --------------------------------------------------------------------- label helpers
def is_same_clustering(labels1, labels2, n_clusters):
    """kmeans/kernels/utils.py:199-253: mapping[l1] = l2 (last writer wins), then
    every sample must satisfy mapping[l1_i] == l2_i."""
    l1 = np.asarray(labels1).astype(np.int64)
    l2 = np.asarray(labels2).astype(np.int64)
    mapping = np.full(n_clusters, -1, dtype=np.int64)
    mapping[l1] = l2
    return bool((mapping[l1] == l2).all())


def get_nb_distinct_clusters(labels, n_clusters):
    """kmeans/kernels/utils.py:257-279."""
    return int(np.unique(np.asarray(labels)).shape[0])


# ------------------------------------------------------------------ data preparation
def prepare_data_for_lloyd(X, init, tol, sample_weight, copy_x=True):
    """kmeans/drivers.py:436-545.  Returns (X, X_mean | None, init, tol, uniform)."""
    X = np.asarray(X)
    T = X.dtype.type
    n, d = X.shape
    X_mean = (X.sum(axis=0, dtype=X.dtype) / T(n)).astype(X.dtype)
    if float((X_mean * X_mean).sum(dtype=X.dtype)) == 0.0:
        X_mean = None
    else:
        X = X.copy() if copy_x else X
        X -= X_mean[None, :]
        if isinstance(init, np.ndarray):
            init = init - X_mean[None, :].astype(init.dtype)
    variance = (X * X).sum(dtype=X.dtype)
    tol = (variance / (d * n)) * tol
    w = np.asarray(sample_weight)
    uniform = bool(w.sum(dtype=X.dtype) == T(w[0]) * n)
    return X, X_mean, init, tol, uniform


def restore_data_after_lloyd(X, best_centers, X_mean, copy_x):
    """kmeans/drivers.py:548-589 (in place)."""
    if X_mean is None:
        return
    best_centers += X_mean[None, :]
    if not copy_x:
        X += X_mean[None, :]


# ------------------------------------------------------------------------- relocation
def relocate_empty_clusters(X, w, sums, sizes, labels, empty_clusters, far_samples,
                            per_sample_inertia=None):
    """kmeans/kernels/utils.py:21-76.  `sums`/`sizes` are modified in place.  Pairs
    empty_clusters[i] with far_samples[i]."""
    T = X.dtype.type
    for j, q in zip(empty_clusters, far_samples):
        j = int(j)
        q = int(q)
        donor = int(labels[q])
        addend = (X[q, :] * T(w[q])).astype(X.dtype)
        sums[donor, :] -= addend
        sums[j, :] = addend
        sizes[donor] -= T(w[q])
        sizes[j] = T(w[q])
        if per_sample_inertia is not None:
            per_sample_inertia[q] = 0


# ------------------------------------------------------------------------------ lloyd
def lloyd_iteration(X, w, C, prev_labels=None, exact_labels=False,
                    relocation="reference"):
    """One pass of the loop body of kmeans/drivers.py:188-296: E-step, un-normalised
    sums and sizes, empty-cluster relocation, division.

    relocation = "reference": distances for the relocation are taken against the
      un-normalised sums (drivers.py:252-259 run before the division at :275);
    relocation = "sklearn": distances against the centres used by the E-step.

    Returns dict(labels, sums, sizes, empty, C_new, changed, far).
    """
    X = np.asarray(X)
    C = np.asarray(C)
    k = C.shape[0]
    h = half_l2_norm(C)
    labels = assign_labels(X, C, h, exact=exact_labels)
    changed = None if prev_labels is None else int((labels != np.asarray(prev_labels)).sum())
    sums, sizes = accumulate_centroids(X, w, labels, k)
    empty = np.nonzero(sizes == 0)[0].astype(np.uint32)
    far = None
    if empty.size:
        ref_c = sums if relocation == "reference" else C
        sq = compute_inertia_per_sample(X, np.ones_like(w), ref_c, labels)
        far = topk_idx(sq, int(empty.size))
        relocate_empty_clusters(X, w, sums, sizes, labels, empty, far)
    with np.errstate(divide="ignore", invalid="ignore"):
        C_new = (sums / sizes[:, None]).astype(X.dtype)
    return dict(labels=labels, sums=sums, sizes=sizes, empty=empty, C_new=C_new,
                changed=changed, far=far)


def centroid_shift_total(C_old, C_new):
    """kmeans/kernels/utils.py:86-110 then the tree sum (drivers.py:334-343)."""
    acc = np.zeros(C_old.shape[0], dtype=C_old.dtype)
    for f in range(C_old.shape[1]):
        diff = C_old[:, f] - C_new[:, f]
        acc += diff * diff
    return tree_sum(acc)


def lloyd(X, sample_weight, centers_init, use_uniform_weights=True, max_iter=300,
          verbose=False, tol=1e-4, exact_labels=False, relocation="reference",
          return_history=False):
    """kmeans/drivers.py:43-393.

    The strict-convergence flag lives in uninitialised memory and is first armed after
    the second iteration (drivers.py:176, 328-332); this restatement holds it at 0
    through iterations 1 and 2, so strict convergence can stop the loop at the end of
    iteration 3 at the earliest.
    """
    X = np.asarray(X)
    T = X.dtype.type
    w = np.asarray(sample_weight, dtype=X.dtype)
    C = np.array(centers_init, dtype=X.dtype, copy=True)
    n_iteration = 0
    shift = np.inf
    prev_labels = None
    armed = False
    history = []
    while n_iteration < max_iter and shift > tol:
        step = lloyd_iteration(X, w, C, prev_labels, exact_labels, relocation)
        C_old, C = C, step["C_new"]
        flag_set = armed and step["changed"] == 0
        prev_labels = step["labels"]
        n_iteration += 1
        if return_history:
            history.append(step)
        if n_iteration > 1:
            if flag_set:
                break
            armed = True
        shift = T(centroid_shift_total(C_old, C))
    h = half_l2_norm(C)
    labels = assign_labels(X, C, h, exact=exact_labels)
    inertia = tree_sum(compute_inertia_per_sample(X, w, C, labels))
    if return_history:
        return labels, inertia, C, n_iteration, history
    return labels, inertia, C, n_iteration


def get_labels_inertia(X, C, sample_weight, with_inertia=True):
    """kmeans/drivers.py:630-699."""
    labels = assign_labels(X, C)
    if not with_inertia:
        return labels, None
    inertia = tree_sum(compute_inertia_per_sample(X, sample_weight, C, labels))
    return labels, np.array([inertia])


# ---------------------------------------------------------------------------- kmeans++
def sample_center_candidate(closest, r):
    """kmeans/kernels/kmeans_plusplus.py:77-103: advance while r > running sum and the
    index is below n-1.  Sequential sum in the compute dtype.  r <= 0 yields -1 in the
    reference (the loop body never runs); clamped to 0 here."""
    T = closest.dtype.type
    cum = T(0)
    cand = -1
    last = closest.shape[0] - 1
    while r > cum and cand < last:
        cand += 1
        cum = T(cum + closest[cand])
    return max(cand, 0)


def sample_center_candidate_interval(closest, r, rel_eps):
    """The candidates a correctly rounded scan could return for threshold `r` when
    partial sums carry a relative error of `rel_eps`: all i whose float64 inclusive
    prefix interval touches r within the slack."""
    cum = np.cumsum(closest.astype(np.float64))
    slack = rel_eps * max(cum[-1], abs(float(r)))
    lo = int(np.searchsorted(cum, float(r) - slack, side="left"))
    hi = int(np.searchsorted(cum, float(r) + slack, side="left"))
    last = closest.shape[0] - 1
    return max(min(lo, last), 0), max(min(hi, last), 0)


def kmeans_plusplus(X, sample_weight, n_clusters, random_state, return_trace=False,
                    scan="sequential"):
    """kmeans/drivers.py:735-910.  `random_state` is an int seed or a numpy RandomState
    (the seed is then drawn as in common/random.py:156-157).

    scan = "sequential": compute-dtype running sum, as the reference's sampler;
    scan = "float64": first index whose float64 inclusive prefix reaches r.
    """
    X = np.asarray(X)
    T = X.dtype.type
    w = np.asarray(sample_weight, dtype=X.dtype)
    n, d = X.shape
    t = 2 + int(math.log(n_clusters))
    rng = Xoroshiro128ppStates(t, random_state)
    centers = np.empty((n_clusters, d), dtype=X.dtype)
    indices = np.full(n_clusters, -1, dtype=np.int32)

    first = int(rng.next(0) % n)
    indices[0] = first
    centers[0] = X[first]
    closest = np.zeros(n, dtype=X.dtype)
    for f in range(d):
        diff = X[:, f] - X[first, f]
        closest += diff * diff
    closest = (closest * w).astype(X.dtype)
    total = tree_sum(closest)
    trace = []
    for c in range(1, n_clusters):
        cands = np.empty(t, dtype=np.int64)
        thresholds = []
        for tau in range(t):
            u = rng.uniform(tau, X.dtype)
            r = T(u * total)
            thresholds.append(r)
            if scan == "sequential":
                cands[tau] = sample_center_candidate(closest, r)
            else:
                cum = np.cumsum(closest.astype(np.float64))
                cands[tau] = max(min(int(np.searchsorted(cum, float(r), side="left")), n - 1), 0)
        M = np.empty((t, n), dtype=X.dtype)
        for tau in range(t):
            acc = np.zeros(n, dtype=X.dtype)
            for f in range(d):
                diff = X[cands[tau], f] - X[:, f]
                acc += diff * diff
            M[tau] = np.minimum((acc * w).astype(X.dtype), closest)
        pots = np.array([tree_sum(M[tau]) for tau in range(t)], dtype=X.dtype)
        best = int(argmin_lowest_index(pots))
        if return_trace:
            trace.append(dict(closest=closest.copy(), total=total, thresholds=thresholds,
                              cands=cands.copy(), pots=pots.copy(), best=best))
        total = pots[best]
        closest = M[best]
        centers[c] = X[cands[best]]
        indices[c] = cands[best]
    if return_trace:
        return centers, indices, trace
    return centers, indices
