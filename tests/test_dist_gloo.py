"""Host-side logic of the row-sharded path, on CPU with the gloo backend (world size 2):
shard bounds, the per-iteration packed all-reduce, the global top-m merge used by sharded
relocation, and the host-side guards (ranks that disagree, a rank that raises).  The
per-shard arithmetic is the CPU oracle's; no GPU is touched."""
import os
import socket
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as tdist
import torch.multiprocessing as mp

from oracle import reference_cpu as ref


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, queue):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        tdist.init_process_group("gloo", rank=rank, world_size=world)
        from sklearn_numba_dpex_b200 import dist as kdist

        kdist.enable()
        out = globals()[fn_name](rank, world, kdist)
        queue.put((rank, "ok", out))
    except Exception:  # pragma: no cover - reported to the parent
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if tdist.is_initialized():
            tdist.destroy_process_group()


def _run(fn_name, world=2):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    return sorted(results)


def _data():
    rng = np.random.default_rng(3)
    n, d, k = 1001, 6, 9
    X = rng.standard_normal((n, d)).astype(np.float64) * 3
    C = X[rng.choice(n, k, replace=False)].copy()
    w = rng.uniform(0.5, 2.0, n)
    return X, C, w


def _case_sharded_iteration(rank, world, kdist):
    X, C, w = _data()
    n, d = X.shape
    k = C.shape[0]
    start, stop = kdist.shard_bounds(n, rank, world)
    labels = ref.assign_labels(X[start:stop], C)
    sums, sizes = ref.accumulate_centroids(X[start:stop], w[start:stop], labels, k)
    packed = torch.zeros(k * d + k + 1, dtype=torch.float64)
    packed[: k * d] = torch.as_tensor(sums.ravel())
    packed[k * d: k * d + k] = torch.as_tensor(sizes)
    packed[k * d + k] = float(stop - start)
    kdist.all_reduce_sum_(packed)
    # every rank now derives the same centroids as the unsharded oracle
    full = ref.lloyd_iteration(X, w, C)
    got = packed[: k * d].reshape(k, d).numpy() / packed[k * d: k * d + k].numpy()[:, None]
    np.testing.assert_allclose(got, full["C_new"], rtol=1e-12)
    assert packed[k * d + k].item() == n
    gathered = kdist.all_gather_cat(torch.as_tensor(labels.astype(np.int64)))
    np.testing.assert_array_equal(gathered.numpy(), full["labels"])
    return (start, stop)


def _case_merge_topk(rank, world, kdist):
    X, C, w = _data()
    n = X.shape[0]
    m = 5
    start, stop = kdist.shard_bounds(n, rank, world)
    values = torch.as_tensor((X ** 2).sum(axis=1))
    values[10] = values[900] = values.max() + 1.0  # a tie across the two shards
    local = values[start:stop]
    top = torch.topk(local, m)
    winners, vals, gidx = kdist.merge_topk(top.values, top.indices + start, m)
    expect = ref.topk_idx(values.numpy(), m)
    np.testing.assert_array_equal(gidx[winners].numpy(), expect)
    return gidx[winners].tolist()


def _case_sharded_sampling(rank, world, kdist):
    """One sampling round of the row-sharded k-means++: every rank searches its own shard from
    its exclusive prefix, the owners' answers are picked, and the result equals the search over
    the unsharded potentials.  Potentials are small integers, so every partial sum is exact."""
    X, _, _ = _data()
    n, d = X.shape
    rng = np.random.default_rng(5)
    pot = rng.integers(0, 7, size=n).astype(np.float64)
    pot[:3] = 0.0                                   # leading zeros: index 0 must not win r > 0
    start, stop = kdist.shard_bounds(n, rank, world)
    local = torch.as_tensor(pot[start:stop])
    ends, offset = kdist.shard_prefix(local.sum().reshape(1))
    total = float(pot.sum())
    assert float(ends[-1]) == total
    first_shard_total = float(pot[: kdist.shard_bounds(n, 0, world)[1]].sum())
    # thresholds: inside each shard, exactly on the shard boundary, the very first and last unit
    r = torch.tensor([1.0, first_shard_total, first_shard_total + 1.0, total, 0.25 * total,
                      0.75 * total], dtype=torch.float64)
    t = r.numel()
    prefix = offset + torch.cumsum(local, 0)
    # local answer of every rank (what the sampling kernel returns): first local row whose
    # inclusive prefix reaches r, the last row when none does
    cand_local = torch.clamp((prefix.reshape(1, -1) < r.reshape(-1, 1)).sum(dim=1), max=local.numel() - 1)
    rows_local = torch.as_tensor(X[start:stop])[cand_local]
    rows_off = torch.tensor([kdist.shard_bounds(n, q, world)[0] for q in range(world)], dtype=torch.int64)
    cand, rows = kdist.pick_owned_candidates(r, ends, cand_local.to(torch.int32), rows_local, rows_off)
    expect = np.minimum(np.searchsorted(np.cumsum(pot), r.numpy(), side="left"), n - 1)
    np.testing.assert_array_equal(cand.numpy(), expect)
    np.testing.assert_array_equal(rows.numpy(), X[expect])
    assert cand.dtype == torch.int32 and rows.shape == (t, d)
    return cand.tolist()


def _case_guards(rank, world, kdist):
    kdist.check_same_across_ranks(d=4, k=7)
    with pytest.raises(ValueError, match="ranks disagree"):
        kdist.check_same_across_ranks(k=7 + rank)
    # a rank that fails before the collective tells the others on the host; nobody enters it
    failed = kdist.all_gather_object(rank == 1)
    assert failed == [False, True]
    return True


def test_shard_bounds_cover_rows_exactly():
    from sklearn_numba_dpex_b200.dist import shard_bounds

    for n in (0, 1, 7, 1000, 10_000_000):
        for world in (1, 2, 3, 8):
            edges = [shard_bounds(n, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1


def test_sharded_iteration_equals_single():
    results = _run("_case_sharded_iteration")
    assert [r[1] for r in results] == ["ok", "ok"], results
    assert results[0][2][1] == results[1][2][0]


def test_merge_topk_across_ranks():
    results = _run("_case_merge_topk")
    assert [r[1] for r in results] == ["ok", "ok"], results
    assert results[0][2] == results[1][2]


def test_sharded_sampling_round_picks_the_owners_candidates():
    results = _run("_case_sharded_sampling")
    assert [r[1] for r in results] == ["ok", "ok"], results
    assert results[0][2] == results[1][2]


def test_host_side_guards():
    results = _run("_case_guards")
    assert [r[1] for r in results] == ["ok", "ok"], results
