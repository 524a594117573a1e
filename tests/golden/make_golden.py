"""Generates tests/golden/kmeans_small.npz from the pinned CPU oracle.

    python tests/golden/make_golden.py

The reference itself cannot run without the numba_dpex / dpctl stack, so these vectors come
from the CPU restatement after it has been pinned to the reference's own known answers
(tests/test_oracle_golden.py).  They freeze seeded inputs and the oracle's outputs, so that a
drift of either the oracle or the CUDA path shows up as a diff against a committed file.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import reference_cpu as ref  # noqa: E402


def build():
    out = {}
    for tag, dtype in (("f32", np.float32), ("f64", np.float64)):
        rng = np.random.default_rng(2024)
        n, d, k = 600, 7, 11
        centers = rng.uniform(-8, 8, size=(k, d))
        X = (centers[rng.integers(0, k, n)] + 0.8 * rng.standard_normal((n, d))).astype(dtype)
        w = rng.uniform(0.5, 2.0, n).astype(dtype)
        init = X[rng.choice(n, k, replace=False)].copy()
        init[4] = 60.0  # starts empty: one relocation in the first iteration
        labels, inertia, C, n_iter = ref.lloyd(X, w, init, False, 12, False, 0.0)
        kpp_centers, kpp_idx = ref.kmeans_plusplus(X, w, k, np.random.RandomState(7), scan="float64")
        sq = ref.compute_inertia_per_sample(X, np.ones(n, dtype=dtype), C, labels)
        out.update({
            f"{tag}_X": X, f"{tag}_w": w, f"{tag}_init": init,
            f"{tag}_labels": labels.astype(np.int32), f"{tag}_inertia": np.asarray(inertia),
            f"{tag}_C": C, f"{tag}_n_iter": np.asarray(n_iter),
            f"{tag}_kpp_idx": kpp_idx, f"{tag}_kpp_centers": kpp_centers,
            f"{tag}_top5": ref.topk_idx(sq, 5),
            f"{tag}_dist": ref.euclidean_distances(X[:50], C),
        })
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kmeans_small.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
