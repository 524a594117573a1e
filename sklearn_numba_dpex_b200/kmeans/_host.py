"""Minimal host for the engine protocol.

scikit-learn's `feature/engine-api` branch, which discovers engines through the
`sklearn_engines` entry-point group and drives them from `KMeans.fit / predict / ...`, is not
a released scikit-learn.  `KMeans` below is a scikit-learn `KMeans` whose public methods call
the engine's methods in the order the engine's contract implies (prepare_fit ->
init_centroids / kmeans_single per init -> unshift_centers -> count_distinct_clusters;
prepare_prediction -> get_labels / get_score; prepare_transform -> get_euclidean_distances),
so that the engine can be used and tested with a released scikit-learn.  Results
(`cluster_centers_`, `labels_`) stay on the device as torch tensors unless
`engine_attributes="sklearn_types"` is asked for.
"""
import warnings

import numpy as np
import sklearn.cluster
from sklearn.exceptions import ConvergenceWarning
from sklearn.utils.validation import _is_arraylike_not_scalar, check_is_fitted

from .engine import KMeansEngine


class KMeans(sklearn.cluster.KMeans):
    """`sklearn.cluster.KMeans` computed by `KMeansEngine`.

    Parameters are scikit-learn's.  `engine_attributes="sklearn_types"` converts the fitted
    attributes to numpy (the branch's `config_context(engine_attributes=...)`)."""

    _engine_class = KMeansEngine

    def __init__(self, n_clusters=8, *, init="k-means++", n_init="auto", max_iter=300, tol=1e-4,
                 verbose=0, random_state=None, copy_x=True, algorithm="lloyd",
                 engine_attributes=None):
        super().__init__(n_clusters=n_clusters, init=init, n_init=n_init, max_iter=max_iter,
                         tol=tol, verbose=verbose, random_state=random_state, copy_x=copy_x,
                         algorithm=algorithm)
        self.engine_attributes = engine_attributes

    # the engine computes its own tolerance on the device (prepare_data_for_lloyd)
    def _check_params_vs_input(self, X, default_n_init=10):
        if X.shape[0] < self.n_clusters:
            raise ValueError(f"n_samples={X.shape[0]} should be >= n_clusters={self.n_clusters}.")
        if self.n_init == "auto":
            if isinstance(self.init, str) and self.init == "k-means++":
                self._n_init = 1
            elif isinstance(self.init, str) and self.init == "random":
                self._n_init = default_n_init
            elif callable(self.init):
                self._n_init = default_n_init
            else:
                self._n_init = 1
        else:
            self._n_init = self.n_init
        if _is_arraylike_not_scalar(self.init) and self._n_init != 1:
            warnings.warn("Explicit initial center position passed: performing only one init in "
                          f"{self.__class__.__name__} instead of n_init={self._n_init}.",
                          RuntimeWarning, stacklevel=2)
            self._n_init = 1

    def _get_engine(self, X=None, y=None, sample_weight=None):
        engine = self._engine_class(self)
        if X is not None and not engine.accepts(X, y, sample_weight):
            raise NotImplementedError(
                f"{self._engine_class.__name__} does not accept this input / parameter set")
        return engine

    def _convert(self, name, value):
        if self.engine_attributes == "sklearn_types":
            return self._engine_class.convert_to_sklearn_types(name, value)
        return value

    def fit(self, X, y=None, sample_weight=None):
        self._validate_params()
        engine = self._get_engine(X, y, sample_weight)
        X, y, sample_weight = engine.prepare_fit(X, y=y, sample_weight=sample_weight)
        self._n_threads = 1
        best_inertia, best_labels = None, None
        for _ in range(self._n_init):
            centers_init = engine.init_centroids(X, sample_weight)
            if self.verbose:
                print("Initialization complete")
            labels, inertia, centers, n_iter_ = engine.kmeans_single(X, sample_weight, centers_init)
            if best_inertia is None or (
                    inertia < best_inertia
                    and not engine.is_same_clustering(labels, best_labels, self.n_clusters)):
                best_labels, best_centers = labels, centers
                best_inertia, best_n_iter = inertia, n_iter_
        engine.unshift_centers(X, best_centers)
        distinct_clusters = engine.count_distinct_clusters(best_labels)
        if distinct_clusters < self.n_clusters:
            warnings.warn(
                "Number of distinct clusters ({}) found smaller than n_clusters ({}). Possibly "
                "due to duplicate points in X.".format(distinct_clusters, self.n_clusters),
                ConvergenceWarning, stacklevel=2)
        self.cluster_centers_ = self._convert("cluster_centers_", best_centers)
        self._n_features_out = best_centers.shape[0]
        self.labels_ = self._convert("labels_", best_labels)
        self.inertia_ = best_inertia
        self.n_iter_ = best_n_iter
        return self

    def fit_predict(self, X, y=None, sample_weight=None):
        return self.fit(X, sample_weight=sample_weight).labels_

    def predict(self, X):
        check_is_fitted(self)
        engine = self._get_engine(X)
        X, sample_weight = engine.prepare_prediction(X, None)
        return self._convert("labels_", engine.get_labels(X, sample_weight))

    def fit_transform(self, X, y=None, sample_weight=None):
        return self.fit(X, sample_weight=sample_weight)._transform(X)

    def transform(self, X):
        check_is_fitted(self)
        return self._transform(X)

    def _transform(self, X):
        engine = self._get_engine(X)
        X = engine.prepare_transform(X)
        return self._convert("labels_", engine.get_euclidean_distances(X))

    def score(self, X, y=None, sample_weight=None):
        check_is_fitted(self)
        engine = self._get_engine(X)
        X, sample_weight = engine.prepare_prediction(X, sample_weight)
        return -engine.get_score(X, sample_weight)

    def __sklearn_is_fitted__(self):
        return hasattr(self, "cluster_centers_")
