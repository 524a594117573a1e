"""xoroshiro128++ streams, bit-exact with the reference's device RNG
(sklearn_numba_dpex/common/random.py:29-292).

The reference runs this purely sequential 64-bit integer code on a single work-item (it even
moves it to the host's CPU device when it can, random.py:171-182).  Here it is host code in
the C library: states are a numpy ``uint64 (n_states, 2)`` array.
"""
import ctypes
import random

import numpy as np

from .._cabi import check, lib

_U64P = ctypes.POINTER(ctypes.c_uint64)


def _states_ptr(states):
    if not (isinstance(states, np.ndarray) and states.dtype == np.uint64 and states.ndim == 2
            and states.shape[1] == 2 and states.flags.c_contiguous):
        raise ValueError("states must be a C-contiguous uint64 array of shape (n_states, 2)")
    return states.ctypes.data_as(_U64P)


def create_xoroshiro128pp_states(n_states, subsequence_start=0, seed=None, device=None):
    """`n_states` generator states, each 2**64 steps after its predecessor.  `seed` may be an
    int, None, or an object with ``randint`` (a numpy RandomState), exactly as in the
    reference (random.py:124-185).  `device` is accepted for signature compatibility."""
    if seed is None:
        seed = random.randint(0, np.iinfo(np.int64).max - 1)
    if hasattr(seed, "randint"):
        seed = int(seed.randint(0, np.iinfo(np.int64).max - 1))
    states = np.zeros((max(int(n_states), 0), 2), dtype=np.uint64)
    if n_states > 0:
        check(lib.kmb_xoroshiro_init(_states_ptr(states), int(n_states),
                                     ctypes.c_uint64(int(seed) & 0xFFFFFFFFFFFFFFFF),
                                     int(subsequence_start)), "kmb_xoroshiro_init")
    return states


def get_random_raw(states):
    """One raw uint64 from states[0], which advances (random.py:29-39)."""
    return np.array([lib.kmb_xoroshiro_next(_states_ptr(states), 0)], dtype=np.uint64)


def rand_uniform(states, state_idx, dtype):
    """One float in [0, 1) from states[state_idx] (random.py:56-121)."""
    x = lib.kmb_xoroshiro_next(_states_ptr(states), int(state_idx))
    if np.dtype(dtype) == np.float32:
        return np.float32(lib.kmb_u64_to_unit_f32(x))
    if np.dtype(dtype) == np.float64:
        return np.float64(lib.kmb_u64_to_unit_f64(x))
    raise ValueError(f"Expected dtype.name in {{float32, float64}} but got dtype.name == {np.dtype(dtype).name}")


def uniform_draws(states, n_rounds, dtype):
    """(n_rounds, n_states) uniforms: round r takes one value from every state, in state
    order, the way the k-means++ sampler consumes them (one per trial per round)."""
    n_states = states.shape[0]
    out = np.empty((n_rounds, n_states), dtype=dtype)
    for r in range(n_rounds):
        for s in range(n_states):
            out[r, s] = rand_uniform(states, s, dtype)
    return out
