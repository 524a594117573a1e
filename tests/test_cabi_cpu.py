"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header
declares, its host-only entry points (RNG, sizing) agree with the oracle, and argument
errors come back as the documented exceptions.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle.rng import Xoroshiro128ppStates

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kmb200.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kmb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sklearn_numba_dpex_b200 import _cabi

    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(_cabi.lib, name), f"{name} is declared in kmb200.h but not exported"
    # and the binding covers the whole header
    assert sorted(_cabi.EXPORTED_SYMBOLS) == declared


def test_sizing_entry_points():
    from sklearn_numba_dpex_b200._cabi import lib

    assert lib.kmb_version() >= 100
    assert lib.kmb_lloyd_acc_len(14, 256) == (256 * 14 + 256 + 1 + 63) // 64 * 64
    assert lib.kmb_lloyd_acc_len(128, 1024) % 64 == 0
    assert lib.kmb_workspace_bytes(10_000_000, 128, 1024) > 0
    assert lib.kmb_kpp_block_rows() > 0
    assert lib.kmb_topk_workspace_bytes(1, 1000, 3) > 0


def test_rng_matches_oracle_and_reference_constants():
    from sklearn_numba_dpex_b200.common.random import (create_xoroshiro128pp_states,
                                                       get_random_raw, rand_uniform)

    # sklearn_numba_dpex/common/tests/test_random.py:35-46 (first three values)
    states = create_xoroshiro128pp_states(1, seed=42)
    got = [int(get_random_raw(states)[0]) for _ in range(3)]
    assert got == [16756476715040848931, 6098722386207918385, 17541662578032534341]
    for seed in (0, 1, 42, 2**40 + 7):
        for n_states in (1, 3, 8):
            ours = create_xoroshiro128pp_states(n_states, seed=seed)
            theirs = Xoroshiro128ppStates(n_states, seed)
            np.testing.assert_array_equal(ours, theirs.as_array())
            for idx in range(n_states):
                for dtype in (np.float32, np.float64):
                    assert rand_uniform(ours, idx, dtype) == theirs.uniform(idx, dtype)
    ours = create_xoroshiro128pp_states(1, seed=42, subsequence_start=1)
    assert int(get_random_raw(ours)[0]) == 16052925335932940643
    # a numpy RandomState seeds like the reference (common/random.py:156-157)
    a = create_xoroshiro128pp_states(2, seed=np.random.RandomState(3))
    b = Xoroshiro128ppStates(2, np.random.RandomState(3)).as_array()
    np.testing.assert_array_equal(a, b)


def test_errors_map_to_exceptions():
    from sklearn_numba_dpex_b200 import _cabi

    with pytest.raises(ValueError):
        _cabi.check(_cabi.lib.kmb_lloyd_resolve_algo(7, 0, 10, 2, 2))
    assert "dtype" in _cabi.last_error()
    with pytest.raises(ValueError):
        _cabi.check(_cabi.lib.kmb_half_l2_norm(0, None, None, 3, 3, None))
    # tensor-core step is fp32 only
    with pytest.raises(NotImplementedError):
        _cabi.check(_cabi.lib.kmb_lloyd_resolve_algo(_cabi.KMB_F64, _cabi.ALGO_TF32X3, 1000, 64, 64))
    with pytest.raises(ValueError, match="Expected k to be greater than or equal"):
        _cabi.check(_cabi.lib.kmb_topk(0, ctypes.c_void_p(16), 1, 3, 5, ctypes.c_void_p(16), None,
                                       ctypes.c_void_p(16), 1 << 20, None))


def test_padding_features_flag_is_checked_before_any_launch():
    """KMB_LLOYD_PAD_FEATURES: bits 8-9 of the flags of the step, assign, finalize and plan calls.
    The argument checks run on the host, so they can be exercised without a GPU."""
    from sklearn_numba_dpex_b200 import _cabi

    assert [_cabi.pad_features_flag(n) for n in range(4)] == [0, 256, 512, 768]
    with pytest.raises(ValueError):
        _cabi.pad_features_flag(4)
    p = ctypes.c_void_p(256)
    lib = _cabi.lib
    # three padding features in rows of two: rejected by every entry point that takes the flag
    with pytest.raises(ValueError, match="padding features"):
        _cabi.check(lib.kmb_lloyd_step(0, _cabi.ALGO_CUDA_CORE, p, p, p, p, p, p, p, 1, 10, 2, 2,
                                       _cabi.pad_features_flag(3), p, 1 << 20, None))
    with pytest.raises(ValueError, match="padding features"):
        _cabi.check(lib.kmb_assign_labels(0, _cabi.ALGO_CUDA_CORE, p, p, p, p, 10, 2, 2,
                                          _cabi.pad_features_flag(2), p, 1 << 20, None))
    with pytest.raises(ValueError, match="padding features"):
        _cabi.check(lib.kmb_lloyd_finalize(0, p, 1, p, _cabi.FIN_MERGE | _cabi.pad_features_flag(3), p, p,
                                           p, p, p, p, 2, 2, p, 1 << 20, None))
    # unknown bits are still rejected
    with pytest.raises(ValueError, match="unknown flag bits"):
        _cabi.check(lib.kmb_lloyd_step(0, _cabi.ALGO_CUDA_CORE, p, p, p, p, p, p, p, 1, 10, 2, 2,
                                       1 << 12, p, 1 << 20, None))


def test_engine_rejects_cpu_only_process():
    import torch

    if torch.cuda.is_available():
        pytest.skip("process has a GPU")
    from sklearn_numba_dpex_b200.kmeans import KMeans

    with pytest.raises(RuntimeError, match="no CPU path"):
        KMeans(n_clusters=2, n_init=1).fit(np.zeros((4, 2), dtype=np.float32))
