"""Row-sharded Lloyd and k-means++ on 2 GPUs (NCCL) against the single-GPU run of the same data:
labels equal up to 1e-6 near-ties, centroids and inertia within fp32 tolerance, iteration by
iteration from shared centres, with an initialisation that forces an empty-cluster relocation
across shards; then a free-running comparison and the seeding.  Skipped with fewer
than two GPUs.  Ranks only leave between steps; NVLS is off so that a failing rank cannot
leave multicast state behind."""
import os
import socket
import traceback

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_data():
    rng = np.random.default_rng(21)
    n, d, k = 40_001, 32, 150
    centers = rng.uniform(-10, 10, size=(k, d))
    X = (centers[rng.integers(0, k, n)] + rng.standard_normal((n, d))).astype(np.float32)
    init = X[rng.choice(n, k, replace=False)].copy()
    init[7] = init[3]            # duplicate centre: cluster 7 starts empty -> relocation
    init[100] = 1e3              # far away: empty as well
    w = rng.uniform(0.5, 1.5, n).astype(np.float32)
    return X, init, w


def _rank_main(rank, world, port, queue):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as tdist

        from sklearn_numba_dpex_b200 import dist as kdist
        from oracle import reference_cpu as ref
        from sklearn_numba_dpex_b200.kmeans.drivers import (get_labels_inertia, kmeans_plusplus,
                                                            lloyd, prepare_data_for_lloyd,
                                                            restore_data_after_lloyd)

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        X, init, w = _make_data()
        # a short collective timeout: if the other rank fails, this one errors out instead of
        # waiting for it
        import datetime
        tdist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                 timeout=datetime.timedelta(seconds=90))
        start, stop = kdist.shard_bounds(X.shape[0], rank, world)
        Xs = torch.as_tensor(X[start:stop]).to(dev)
        ws = torch.as_tensor(w[start:stop]).to(dev)
        out = []

        # --- Lloyd, teacher-forced: every pass of the loop below starts both runs from the SAME centres and does
        # one iteration.  fp32 atomics make the cluster sums differ in the last bits from run to
        # run, and on this data a sample that sits on a boundary then sends a free-running loop
        # into one of two end states 24 labels apart (also between two single-GPU runs), so a
        # free-running comparison is only made loosely at the end.  The first pass relocates the two
        # empty clusters across shards.
        centres = torch.as_tensor(init).to(dev)
        for rnd in range(3):
            single = None
            if rank == 0:
                Xd, wd = torch.as_tensor(X).to(dev), torch.as_tensor(w).to(dev)
                X_t, mean, init_t, tol, uni = prepare_data_for_lloyd(Xd.T, centres.T, 1e-4, wd, True)
                labels, inertia, C_t, n_iter = lloyd(X_t, wd, init_t, uni, 1, False, 0.0,
                                                     algo="cuda_core")
                single = (labels.cpu().numpy(), float(inertia), C_t.T.cpu().numpy(),
                          mean.cpu().numpy(), float(tol), X_t.T.cpu().numpy())
            with kdist.sharded_rows():
                X_t, mean, init_t, tol, uni = prepare_data_for_lloyd(Xs.T, centres.T, 1e-4, ws, True)
                labels, inertia, C_t, n_iter = lloyd(X_t, ws, init_t, uni, 1, False, 0.0,
                                                     algo="cuda_core")
                all_labels = kdist.all_gather_cat(labels.to(torch.int64)).cpu().numpy()
                _, score = get_labels_inertia(X_t, C_t, ws, True)
            if rank == 0:
                s_labels, s_inertia, s_C, s_mean, s_tol, s_Xc = single
                np.testing.assert_allclose(mean.cpu().numpy(), s_mean, rtol=1e-5, atol=1e-6)
                np.testing.assert_allclose(float(tol), s_tol, rtol=1e-5)
                # same labels in the E-step => same sums up to rounding
                np.testing.assert_allclose(C_t.T.cpu().numpy(), s_C, rtol=1e-4, atol=1e-4)
                # returned labels belong to the returned centres, which differ in the last bits
                ok, n_bad, n_unexplained = ref.labels_agree(all_labels, s_labels, s_Xc, s_C, rtol=1e-6)
                assert ok, f"round {rnd}: {n_unexplained} of {n_bad} label mismatches are not near-ties"
                np.testing.assert_allclose(float(inertia), s_inertia, rtol=1e-5)
                np.testing.assert_allclose(float(score[0]), s_inertia, rtol=1e-5)
                out.append(int(n_bad))
            # both runs continue from the sharded result (feature means added back, in place)
            restore_data_after_lloyd(X_t, C_t, mean, True)
            centres = C_t.T.contiguous().clone()

        # --- Lloyd, free-running 6 iterations with the automatic kernel choice (tensor-core
        # step on the single GPU, CUDA-core step on the shards): same clustering quality
        if rank == 0:
            Xd, wd, Cd = (torch.as_tensor(a).to(dev) for a in (X, w, init))
            X_t, mean, init_t, tol, uni = prepare_data_for_lloyd(Xd.T, Cd.T, 1e-4, wd, True)
            s_labels, s_inertia, _, s_iter = lloyd(X_t, wd, init_t, uni, 6, False, 0.0)
            s_labels, s_inertia = s_labels.cpu().numpy(), float(s_inertia)
        with kdist.sharded_rows():
            Cd = torch.as_tensor(init).to(dev)
            X_t, mean, init_t, tol, uni = prepare_data_for_lloyd(Xs.T, Cd.T, 1e-4, ws, True)
            labels, inertia, C_t, n_iter = lloyd(X_t, ws, init_t, uni, 6, False, 0.0)
            all_labels = kdist.all_gather_cat(labels.to(torch.int64)).cpu().numpy()
        if rank == 0:
            assert n_iter == s_iter
            np.testing.assert_allclose(float(inertia), s_inertia, rtol=1e-3)
            assert (all_labels != s_labels).mean() < 2e-3

        # --- k-means++: same random stream, same candidates, same centres
        if rank == 0:
            Xd, wd = torch.as_tensor(X).to(dev), torch.as_tensor(w).to(dev)
            s_kpp_C, s_kpp_idx = kmeans_plusplus(Xd.T, wd, 40, np.random.RandomState(5))
        with kdist.sharded_rows():
            kpp_C, kpp_idx = kmeans_plusplus(Xs.T, ws, 40, np.random.RandomState(5))
        if rank == 0:
            np.testing.assert_array_equal(kpp_idx.cpu().numpy(), s_kpp_idx.cpu().numpy())
            np.testing.assert_allclose(kpp_C.T.cpu().numpy(), s_kpp_C.T.cpu().numpy())
        tdist.barrier()
        torch.cuda.synchronize()
        queue.put((rank, "ok", out))
        tdist.destroy_process_group()
    except Exception:  # pragma: no cover
        queue.put((rank, "error", traceback.format_exc()))


def test_two_gpu_lloyd_equals_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            results.append(queue.get(timeout=240))
            if results[-1][1] != "ok":
                break  # the other rank may be stuck in a collective: do not wait for it
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    results.sort()
    assert [r[1] for r in results] == ["ok", "ok"], results[-1][2] if results else "no result"
