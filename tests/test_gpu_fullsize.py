"""Full-size configurations of the benchmark through size-independent properties.

The CPU oracle cannot finish n = 10 M in seconds, so at full size the fused step is checked by
invariants of the algorithm plus an exact check on a random sample of rows:
  * the cluster counts add up to n and the cluster sums add up to the column sums of X;
  * the labels of the fused step equal those of the label-only kernel on the same centroids;
  * on 8 192 random rows the labels equal the oracle's (up to 1e-6 near-ties);
  * the "changed" flag agrees with a direct comparison of two label vectors;
  * per-sample inertia summed on the host equals the kernel's total.
Data come from the benchmark's own seeded generator."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@pytest.mark.parametrize("name", ["c3", "c2", "c4"])
def test_fused_step_invariants_at_full_size(name):
    import bench
    from sklearn_numba_dpex_b200 import dist as kdist
    from sklearn_numba_dpex_b200._cabi import check, lib, ptr, stream_ptr
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    free, _ = torch.cuda.mem_get_info()
    cfg = dict(bench.CONFIGS[name])
    tdt = torch.float32 if cfg["dtype"] == "f32" else torch.float64
    need = cfg["n"] * cfg["d"] * tdt.itemsize * 2.5
    if free < need:
        pytest.skip("not enough free device memory for the full-size case")
    dev = torch.device("cuda", torch.cuda.current_device())
    n, d, k = cfg["n"], cfg["d"], cfg["k"]
    X = bench.generate_rows(cfg, 0, n, torch, dev, tdt)
    C0 = bench.initial_centres(cfg, X, 0, n, torch, kdist)
    st = LloydState(X, None, C0, "auto")
    dp = st.d                      # padded feature count when the tensor-core step pads d
    st.step()                      # iteration 1 (may relocate), then a clean second iteration
    C_used = st.C.clone()
    st.launch_step()
    torch.cuda.synchronize()
    st.check_device_waits()
    labels = st.labels_new.clone()
    packed = st.packed.clone()

    # counts and sums
    counts = packed[k * dp: k * dp + k].double()
    assert float(counts.sum()) == float(n)
    col = torch.stack([st.X[i:i + 1_000_000].double().sum(dim=0)
                       for i in range(0, n, 1_000_000)]).sum(dim=0)
    sums_total = packed[: k * dp].reshape(k, dp).double().sum(dim=0)
    scale = float(st.X.abs().max()) * n
    if tdt == torch.float32:
        assert torch.allclose(sums_total, col, rtol=1e-4, atol=1e-7 * scale)
    else:   # fp64: the stated 1e-12 on sums of n / k ~ 31 000 terms each
        assert torch.allclose(sums_total, col, rtol=1e-12, atol=1e-16 * scale)

    # label-only kernel agrees with the fused step
    lab2 = torch.empty_like(labels)
    check(lib.kmb_assign_labels(st.dtype, st.algo, ptr(st.X), ptr(C_used), ptr(st.h), ptr(lab2), n, dp,
                                k, st._pad_flag, ptr(st.ws), st.ws_bytes, stream_ptr(dev)))
    torch.cuda.synchronize()
    st.check_device_waits()
    assert int((lab2 != labels).sum()) == 0

    # changed flag
    changed = packed[k * dp + k].item()
    assert (changed != 0.0) == bool((labels != st.labels).any())

    # exact check on a sample of rows
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(n, size=8192, replace=False))
    Xs = st.X[torch.as_tensor(rows, device=dev)].cpu().numpy()[:, :d]
    Cn = C_used.cpu().numpy()[:, :d]
    ok, n_bad, n_unexplained = ref.labels_agree(labels[torch.as_tensor(rows, device=dev)].cpu().numpy(),
                                                ref.assign_labels(Xs, Cn, exact=True), Xs, Cn)
    assert ok, (n_bad, n_unexplained)

    # inertia: kernel total against the host sum of the per-sample values
    per = torch.empty(n, dtype=tdt, device=dev)
    tot = torch.empty(1, dtype=tdt, device=dev)
    check(lib.kmb_inertia(st.dtype, ptr(st.X), None, ptr(C_used), ptr(labels), ptr(per), ptr(tot), n, dp,
                          k, ptr(st.scratch), st.scratch_bytes, stream_ptr(dev)))
    torch.cuda.synchronize()
    assert abs(float(tot[0]) - float(per.double().sum())) <= 1e-6 * float(per.double().sum())
    d2 = ((Xs.astype(np.float64) - Cn.astype(np.float64)[labels[torch.as_tensor(rows, device=dev)].cpu().numpy()]) ** 2).sum(axis=1)
    rt = 1e-4 if tdt == torch.float32 else 1e-12
    np.testing.assert_allclose(per[torch.as_tensor(rows, device=dev)].cpu().numpy(), d2, rtol=rt, atol=rt)
