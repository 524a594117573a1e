"""The plugin is discoverable: pyproject.toml registers the engine in the `sklearn_engines`
entry-point group under the name `kmeans`, as the reference does (pyproject.toml:55-56 there),
and the registered object is the engine class with the protocol scikit-learn's engine API
calls."""
import importlib.metadata
import os
import tomllib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROTOCOL = ["accepts", "prepare_fit", "unshift_centers", "init_centroids", "kmeans_single",
            "is_same_clustering", "count_distinct_clusters", "prepare_prediction", "get_labels",
            "get_score", "prepare_transform", "get_euclidean_distances", "convert_to_sklearn_types"]


def _declared():
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as fh:
        return tomllib.load(fh)


def test_entry_point_is_declared_and_resolves_to_the_engine():
    meta = _declared()
    group = meta["project"]["entry-points"]["sklearn_engines"]
    assert list(group) == ["kmeans"]
    ep = importlib.metadata.EntryPoint(name="kmeans", value=group["kmeans"], group="sklearn_engines")
    engine_class = ep.load()
    from sklearn_numba_dpex_b200.kmeans.engine import KMeansEngine

    assert engine_class is KMeansEngine
    assert engine_class.engine_name == "kmeans"
    for method in PROTOCOL:
        assert callable(getattr(engine_class, method)), method
    # the provider name scikit-learn derives from the entry point's module
    assert ep.module.split(".")[0] == "sklearn_numba_dpex_b200"


def test_installed_distribution_exposes_the_same_entry_point():
    """When the distribution is installed (pip install -e . --no-build-isolation), discovery
    through importlib.metadata gives the same class; in a source checkout that was never
    installed there is nothing to look up and the declaration test above is the check."""
    found = [ep for ep in importlib.metadata.entry_points(group="sklearn_engines")
             if ep.value.startswith("sklearn_numba_dpex_b200.")]
    for ep in found:
        from sklearn_numba_dpex_b200.kmeans.engine import KMeansEngine

        assert ep.name == "kmeans" and ep.load() is KMeansEngine


def test_package_data_names_the_library_and_the_build_hook_exists():
    meta = _declared()
    assert "libkmb200.so" in meta["tool"]["setuptools"]["package-data"]["sklearn_numba_dpex_b200"]
    assert os.path.exists(os.path.join(ROOT, "setup.py"))
    assert os.path.exists(os.path.join(ROOT, "sklearn_numba_dpex_b200", "build.py"))
