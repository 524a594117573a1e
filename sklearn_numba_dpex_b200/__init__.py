"""sklearn_numba_dpex_b200 — a B200-native KMeans engine for scikit-learn's engine API.

Entry point (for scikit-learn's feature/engine-api branch):
    sklearn_engines: kmeans = sklearn_numba_dpex_b200.kmeans.engine:KMeansEngine
With a released scikit-learn use `sklearn_numba_dpex_b200.kmeans.KMeans`.
"""
__version__ = "0.1.0"
