"""KMeans engine for scikit-learn's engine API, computing on a B200 through libkmb200.

Same method set, argument meaning and return values as `KMeansEngine` of the reference
(sklearn_numba_dpex/kmeans/engine.py:36-392).  Arrays are torch CUDA tensors where the
reference uses dpctl tensors; numpy inputs are copied to the device.  The base class and the
exception type of scikit-learn's `feature/engine-api` branch are used when that branch is
installed; otherwise small stand-ins defined here take their place.
"""
import numbers
import os
from typing import Any, Dict

import numpy as np
import scipy.sparse as sp
import torch
from sklearn.utils import check_array, check_random_state
from sklearn.utils.validation import _is_arraylike_not_scalar

from .drivers import (all_finite, gather_rows, get_euclidean_distances, get_labels_inertia,
                      get_nb_distinct_clusters, is_same_clustering, kmeans_plusplus, lloyd,
                      prepare_data_for_lloyd, restore_data_after_lloyd)

try:  # scikit-learn feature/engine-api branch
    from sklearn.cluster._kmeans import KMeansCythonEngine as _BaseEngine
    from sklearn.exceptions import NotSupportedByEngineError
except ImportError:  # released scikit-learn: no engine API

    class NotSupportedByEngineError(NotImplementedError):
        """Raised, in testing mode, when the engine is asked for something it cannot do."""

    class _BaseEngine:
        def __init__(self, estimator):
            self.estimator = estimator


TESTING_MODE_ENV = "SKLEARN_NUMBA_DPEX_B200_TESTING_MODE"


def _check_array_no_finite_pass(array, **kwargs):
    """sklearn's check_array without its host-side finiteness scan (the keyword changed name in
    scikit-learn 1.6)."""
    try:
        return check_array(array, ensure_all_finite=False, **kwargs)
    except TypeError:
        return check_array(array, force_all_finite=False, **kwargs)


def _upload(host_array, device):
    """Host numpy array -> device tensor; asynchronous when the memory is page-locked."""
    t = torch.as_tensor(host_array)
    return t.to(device, non_blocking=t.is_pinned())


class _DeviceUnset:
    pass


class KMeansEngine(_BaseEngine):
    """Lloyd's k-means on one B200 (or on this rank's row shard of several).

    One fused kernel per iteration assigns every sample to its nearest centroid and
    accumulates the weighted sums and counts of the new centroids; the distance contraction
    runs on the tensor cores (3xTF32) when the shape makes it a dense GEMM and on the CUDA
    cores otherwise.
    """

    # Class-level overrides of `device` (cuda index or torch.device), `order` and `algo`
    # ("auto" | "cuda_core" | "tf32x3"), for tests and the benchmark
    # (reference: engine.py:70-75).
    _CONFIG: Dict[str, Any] = dict()

    engine_name = "kmeans"

    @staticmethod
    def convert_to_sklearn_types(name, value):
        if name in ["cluster_centers_", "labels_"] and isinstance(value, torch.Tensor):
            return value.cpu().numpy()
        return value

    def __init__(self, estimator):
        self.device = self._CONFIG.get("device", _DeviceUnset)
        # The kernels read samples as contiguous rows; "C" is the only supported order (the
        # reference, for its own layout reasons, supports only "F": engine.py:98-105).
        order = self._CONFIG.get("order", "C")
        if order != "C":
            raise ValueError("The kmb200 kernels read samples as contiguous rows: only "
                             f"order='C' is supported, got {order!r}")
        self.order = order
        self.algo = self._CONFIG.get("algo", "auto")
        self.estimator = estimator

        mode = os.getenv(TESTING_MODE_ENV, "0")
        if mode not in {"0", "1"}:
            raise ValueError(
                f"If the environment variable {TESTING_MODE_ENV} is set, it is expected to take "
                f'values in {{"0", "1"}}, but got {mode} instead.')
        self._is_in_testing_mode = mode == "1"

    # ------------------------------------------------------------------ engine protocol
    def accepts(self, X, y, sample_weight):
        if (algorithm := self.estimator.algorithm) not in ("lloyd", "auto", "full"):
            if self._is_in_testing_mode:
                raise NotSupportedByEngineError(
                    "The sklearn_numba_dpex_b200 engine for KMeans only support the Lloyd "
                    f"algorithm, {algorithm} is not supported.")
            return False
        if sp.issparse(X):
            return self._is_in_testing_mode
        return True

    def prepare_fit(self, X, y=None, sample_weight=None):
        estimator = self.estimator
        X = self._validate_data(X)
        estimator._check_params_vs_input(X)
        sample_weight = self._check_sample_weight(sample_weight, X)

        init = self.estimator.init
        if _is_arraylike_not_scalar(init):
            init = self._check_init(init, X)

        (X_t, X_mean, self.init, self.tol,
         self.sample_weight_is_uniform) = prepare_data_for_lloyd(
            X.T, init, estimator.tol, sample_weight, estimator.copy_x)

        self.X_mean = X_mean
        self.random_state = check_random_state(estimator.random_state)
        return X_t.T, y, sample_weight

    def unshift_centers(self, X, best_centers):
        if (X_mean := self.X_mean) is None:
            return
        if isinstance(best_centers, np.ndarray):
            # testing mode hands numpy centres around (see kmeans_single)
            best_centers += X_mean.cpu().numpy()
            if not self.estimator.copy_x:
                restore_data_after_lloyd(X.T, torch.zeros((X.shape[1], 1), dtype=X.dtype,
                                                          device=X.device), X_mean, False)
            return
        restore_data_after_lloyd(X.T, best_centers.T, X_mean, self.estimator.copy_x)

    def init_centroids(self, X, sample_weight):
        init = self.init
        n_clusters = self.estimator.n_clusters
        if isinstance(init, torch.Tensor):
            centers_t = init
        elif isinstance(init, str) and init == "k-means++":
            centers_t, _ = self._kmeans_plusplus(X, sample_weight)
        elif callable(init):
            centers = init(X, self.estimator.n_clusters, random_state=self.random_state)
            centers_t = self._check_init(centers, X)
        else:
            # Sampling without replacement is sequential: host numpy, as the reference
            # (engine.py:188-196), and the same index stream.  Uniform weights (known from
            # prepare_fit) are rebuilt on the host from their first element instead of being
            # copied back, which gives numpy the very same probabilities; the chosen rows are
            # gathered on the device.
            n_samples = X.shape[0]
            if getattr(self, "sample_weight_is_uniform", False):
                w0 = sample_weight[:1].cpu().numpy()[0]
                sample_weight_numpy = np.full(n_samples, w0, dtype=w0.dtype)
            else:
                sample_weight_numpy = sample_weight.cpu().numpy()
            p = sample_weight_numpy / sample_weight_numpy.sum()
            centers_idx = self.random_state.choice(n_samples, size=n_clusters, replace=False, p=p)
            centers_t = gather_rows(X, centers_idx).T
        return centers_t

    def _kmeans_plusplus(self, X, sample_weight):
        return kmeans_plusplus(X.T, sample_weight, self.estimator.n_clusters, self.random_state)

    def kmeans_single(self, X, sample_weight, centers_init_t):
        assignments_idx, inertia, best_centroids_t, n_iteration = lloyd(
            X.T, sample_weight, centers_init_t, self.sample_weight_is_uniform,
            self.estimator.max_iter, self.estimator.verbose, self.tol, algo=self.algo)
        if self._is_in_testing_mode:
            assignments_idx = assignments_idx.cpu().numpy().astype(np.int32)
            best_centroids_t = np.asfortranarray(best_centroids_t.cpu().numpy()).astype(
                self.estimator._output_dtype)
        return assignments_idx, inertia, best_centroids_t.T, n_iteration

    def is_same_clustering(self, labels, best_labels, n_clusters):
        if self._is_in_testing_mode:
            labels = torch.as_tensor(np.asarray(labels), device=self._device_or_default())
            best_labels = torch.as_tensor(np.asarray(best_labels), device=labels.device)
        return is_same_clustering(labels, best_labels, n_clusters)

    def count_distinct_clusters(self, best_labels):
        if self._is_in_testing_mode:
            best_labels = torch.as_tensor(np.asarray(best_labels), device=self._device_or_default())
        return get_nb_distinct_clusters(best_labels, self.estimator.n_clusters)

    def prepare_prediction(self, X, sample_weight):
        X = self._validate_data(X, reset=False)
        sample_weight = self._check_sample_weight(sample_weight, X)
        return X, sample_weight

    def get_labels(self, X, sample_weight):
        labels, _ = self._get_labels_inertia(X, sample_weight, with_inertia=False)
        if self._is_in_testing_mode:
            labels = labels.cpu().numpy().astype(np.int32)
        return labels

    def get_score(self, X, sample_weight):
        _, inertia = self._get_labels_inertia(X, sample_weight, with_inertia=True)
        return inertia

    def _get_labels_inertia(self, X, sample_weight, with_inertia=True):
        cluster_centers = self._check_init(self.estimator.cluster_centers_, X, copy=False)
        assignments_idx, inertia = get_labels_inertia(X.T, cluster_centers, sample_weight,
                                                      with_inertia, algo=self.algo)
        if with_inertia:
            inertia = inertia[0]
        return assignments_idx, inertia

    def prepare_transform(self, X):
        return X

    def get_euclidean_distances(self, X):
        X = self._validate_data(X, reset=False)
        cluster_centers = self._check_init(self.estimator.cluster_centers_, X, copy=False)
        euclidean_distances = get_euclidean_distances(X.T, cluster_centers)
        if self._is_in_testing_mode:
            euclidean_distances = euclidean_distances.cpu().numpy().astype(
                self.estimator._output_dtype)
        return euclidean_distances

    # ------------------------------------------------------------------------ validation
    def _device_or_default(self, X=None):
        if self.device is not _DeviceUnset:
            dev = self.device
            return torch.device("cuda", dev) if isinstance(dev, int) else torch.device(dev)
        if isinstance(X, torch.Tensor) and X.is_cuda:
            return X.device
        if not torch.cuda.is_available():
            raise RuntimeError("the sklearn_numba_dpex_b200 engine needs a CUDA device; there is "
                               "no CPU path")
        return torch.device("cuda", torch.cuda.current_device())

    def _validate_data(self, X, reset=True):
        """dtype float64 or float32 (anything else becomes float64, as scikit-learn does),
        2-D, dense, finite, row-major, on the device (reference: engine.py:293-336)."""
        device = self._device_or_default(X)
        accepted = (torch.float64, torch.float32)
        if sp.issparse(X):
            raise NotSupportedByEngineError("A sparse matrix was passed, but dense data is required")
        estimator = self.estimator
        if isinstance(X, torch.Tensor):
            if X.dim() != 2:
                raise ValueError(f"Expected 2D array, got {X.dim()}D array instead")
            if self._is_in_testing_mode and reset:
                estimator._output_dtype = (np.float32 if X.dtype == torch.float32 else np.float64)
            Xd = X.to(device=device, dtype=X.dtype if X.dtype in accepted else torch.float64)
            if not Xd.is_contiguous():
                Xd = Xd.contiguous()
            if Xd.shape[0] < 1:
                raise ValueError("Found array with 0 sample(s) while a minimum of 1 is required.")
            if not all_finite(Xd):
                raise ValueError("Input X contains NaN or infinity.")
        else:
            # shape / dtype / layout are validated on the host; the finiteness pass over the
            # n x d values runs on the device after the upload (one kernel at HBM speed, where
            # check_array would walk the array with the host cores first)
            Xn = _check_array_no_finite_pass(X, accept_sparse=False, dtype=[np.float64, np.float32],
                                             order="C", copy=False, estimator=estimator)
            if self._is_in_testing_mode and reset:
                estimator._output_dtype = Xn.dtype.type
            Xd = _upload(Xn, device)
            if not all_finite(Xd):
                raise ValueError("Input X contains NaN or infinity.")
        n_features = Xd.shape[1]
        if reset:
            estimator.n_features_in_ = n_features
        elif hasattr(estimator, "n_features_in_") and estimator.n_features_in_ != n_features:
            raise ValueError(
                f"X has {n_features} features, but {estimator.__class__.__name__} is expecting "
                f"{estimator.n_features_in_} features as input.")
        return Xd

    def _check_sample_weight(self, sample_weight, X):
        """reference: engine.py:338-374."""
        n_samples = X.shape[0]
        if sample_weight is None:
            return torch.ones(n_samples, dtype=X.dtype, device=X.device)
        if isinstance(sample_weight, numbers.Number):
            return torch.full((n_samples,), float(sample_weight), dtype=X.dtype, device=X.device)
        if isinstance(sample_weight, torch.Tensor):
            sw = sample_weight.to(device=X.device, dtype=X.dtype).contiguous()
            if not all_finite(sw):
                raise ValueError("Input sample_weight contains NaN or infinity.")
        else:
            sw = check_array(sample_weight, accept_sparse=False, order="C",
                             dtype=np.float64 if X.dtype == torch.float64 else np.float32,
                             ensure_2d=False, allow_nd=False, estimator=self.estimator,
                             input_name="sample_weight")
            sw = torch.as_tensor(sw).to(X.device)
        if sw.dim() != 1:
            raise ValueError("Sample weights must be 1D array or scalar")
        if tuple(sw.shape) != (n_samples,):
            raise ValueError("sample_weight.shape == {}, expected {}!".format(
                tuple(sw.shape), (n_samples,)))
        return sw

    def _check_init(self, init, X, copy=False):
        """Validated initial centres as a (d, k) tensor (reference: engine.py:376-392)."""
        if isinstance(init, torch.Tensor):
            if init.dim() != 2:
                raise ValueError(f"Expected 2D array, got {init.dim()}D array instead")
            init_d = init.to(device=X.device, dtype=X.dtype).contiguous().clone()
            if not all_finite(init_d):
                raise ValueError("Input init contains NaN or infinity.")
        else:
            init_n = check_array(init, dtype=np.float64 if X.dtype == torch.float64 else np.float32,
                                 accept_sparse=False, copy=True, order="C", ensure_2d=True,
                                 estimator=self.estimator, input_name="init")
            init_d = torch.as_tensor(init_n).to(X.device)
        self.estimator._validate_center_shape(X, init_d)
        return init_d.T
