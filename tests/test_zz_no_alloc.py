"""The allocation-free top-k entry point against the workspace-based one.

`kmb_topk_idx_static` serves hosts that cannot allocate device memory when they need a
top-k (their memory is fully handed to an arena of their own, or they sit in a loop where
the allocator's device-wide synchronisation is not acceptable): its scratch is an array
built into the library.  It must return exactly what `kmb_topk` returns, also on the second
of two back-to-back calls, when the scratch still holds the first call's histograms.
This file is collected last on purpose, so that a run stopping at the first failure has
already run every other test; it also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_topk_idx(values_dev, k):
    from sklearn_numba_dpex_b200._cabi import check, dtype_code, lib, ptr, stream_ptr

    n = values_dev.numel()
    nbytes = lib.kmb_topk_workspace_bytes(1, n, k)
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=values_dev.device)
    out = torch.empty(k, dtype=torch.int64, device=values_dev.device)
    check(lib.kmb_topk(dtype_code(values_dev.dtype), ptr(values_dev), 1, n, k, None, ptr(out),
                       ptr(ws), ws.numel(), stream_ptr()), "kmb_topk")
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _static_topk_idx(values_dev, k):
    from sklearn_numba_dpex_b200._cabi import check, dtype_code, lib, ptr, stream_ptr

    out = torch.full((k,), -1, dtype=torch.int64, device=values_dev.device)
    check(lib.kmb_topk_idx_static(dtype_code(values_dev.dtype), ptr(values_dev), values_dev.numel(),
                                  k, ptr(out), stream_ptr()), "kmb_topk_idx_static")
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_static_scratch_topk_matches_workspace_topk_twice_in_a_row(dtype):
    rng = np.random.default_rng(17)
    first = rng.standard_normal(300_007).astype(dtype)
    first[rng.integers(0, first.size, 500)] = first.max()       # ties at the threshold
    second = (rng.random(4_099) * 10 - 5).astype(dtype)          # different size, different k
    a_dev, b_dev = torch.as_tensor(first).cuda(), torch.as_tensor(second).cuda()

    got_a = _static_topk_idx(a_dev, 700)
    got_b = _static_topk_idx(b_dev, 4096)   # right after: the scratch holds call one's state
    np.testing.assert_array_equal(got_a, _reference_topk_idx(a_dev, 700))
    np.testing.assert_array_equal(got_b, _reference_topk_idx(b_dev, 4096))
    # and once more with the first input, after a larger-k call dirtied the whole scratch
    np.testing.assert_array_equal(_static_topk_idx(a_dev, 1), _reference_topk_idx(a_dev, 1))


def test_static_scratch_topk_rejects_sizes_beyond_its_scratch():
    from sklearn_numba_dpex_b200 import _cabi

    vals = torch.zeros(10_000, device="cuda")
    out = torch.empty(5000, dtype=torch.int64, device="cuda")
    rc = _cabi.lib.kmb_topk_idx_static(_cabi.KMB_F32, _cabi.ptr(vals), vals.numel(), 4097,
                                       _cabi.ptr(out), _cabi.stream_ptr())
    assert rc == _cabi.KMB_ERR_INVALID
    assert "4096" in _cabi.last_error()
    with pytest.raises(ValueError, match="Expected k to be greater than or equal"):
        _cabi.check(_cabi.lib.kmb_topk_idx_static(_cabi.KMB_F32, _cabi.ptr(vals), 5, 6,
                                                  _cabi.ptr(out), _cabi.stream_ptr()))
