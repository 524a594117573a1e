"""Generic device helpers of the engine: top-k, RNG, reductions (mirrors the reference's
sklearn_numba_dpex/common package for the pieces the KMeans path uses)."""
from .random import create_xoroshiro128pp_states, get_random_raw  # noqa: F401
from .topk import topk, topk_idx  # noqa: F401
