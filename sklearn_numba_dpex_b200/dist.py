"""Row sharding over the GPUs of one box: one process per GPU, torch.distributed plumbing.

The reference is single-device (it has no collective call sites); sharding is an addition
of this engine.  Samples are split into contiguous row blocks, centroids are replicated, and
per Lloyd iteration ONE all-reduce of the packed accumulator
``[sums k*d | counts k | changed 1]`` is issued on the compute stream.  Everything here works
on CPU tensors with the gloo backend as well, which is how the multi-rank logic is tested
without GPUs.
"""
import contextlib

import torch
import torch.distributed as tdist

_STATE = {"enabled": False, "group": None}


def enable(group=None):
    """Treat the X handed to the drivers as THIS rank's row shard from now on."""
    if not tdist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    _STATE["enabled"] = True
    _STATE["group"] = group


def disable():
    _STATE["enabled"] = False
    _STATE["group"] = None


@contextlib.contextmanager
def sharded_rows(group=None):
    enable(group)
    try:
        yield
    finally:
        disable()


def active():
    return _STATE["enabled"] and tdist.is_initialized() and world_size() > 1


def world_size():
    return tdist.get_world_size(_STATE["group"]) if tdist.is_initialized() else 1


def rank():
    return tdist.get_rank(_STATE["group"]) if tdist.is_initialized() else 0


def shard_bounds(n, r=None, world=None):
    """Contiguous block [start, stop) of rank r among `world` ranks: the first n % world
    ranks hold one extra row."""
    r = rank() if r is None else r
    world = world_size() if world is None else world
    base, extra = divmod(int(n), int(world))
    start = r * base + min(r, extra)
    return start, start + base + (1 if r < extra else 0)


def all_reduce_sum_(t):
    """In-place sum over ranks (no-op when sharding is off)."""
    if active():
        tdist.all_reduce(t, op=tdist.ReduceOp.SUM, group=_STATE["group"])
    return t


def all_gather_cat(t):
    """Concatenation over ranks along dim 0; the ranks' leading dimensions may differ
    (shorter pieces are padded for the collective and trimmed afterwards)."""
    if not active():
        return t
    lengths = all_gather_object(int(t.shape[0]))
    longest = max(lengths)
    padded = t.contiguous()
    if t.shape[0] < longest:
        pad = torch.zeros((longest - t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        padded = torch.cat([padded, pad], dim=0)
    out = [torch.empty_like(padded) for _ in range(world_size())]
    tdist.all_gather(out, padded, group=_STATE["group"])
    return torch.cat([piece[:length] for piece, length in zip(out, lengths)], dim=0)


def all_gather_same(t):
    """Concatenation over ranks along dim 0 of tensors that have the SAME shape on every rank:
    one collective, no host round trip (use all_gather_cat when lengths may differ)."""
    if not active():
        return t
    t = t.contiguous()
    if t.is_cuda:
        out = torch.empty((world_size() * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype,
                          device=t.device)
        tdist.all_gather_into_tensor(out, t, group=_STATE["group"])
        return out
    pieces = [torch.empty_like(t) for _ in range(world_size())]
    tdist.all_gather(pieces, t, group=_STATE["group"])
    return torch.cat(pieces, dim=0)


def all_gather_object(obj):
    if not active():
        return [obj]
    out = [None] * world_size()
    tdist.all_gather_object(out, obj, group=_STATE["group"])
    return out


def broadcast_(t, src):
    if active():
        tdist.broadcast(t, src=src, group=_STATE["group"])
    return t


def check_same_across_ranks(**named_values):
    """Host-side guard run before a sharded loop: every rank must agree on these values
    (shapes, dtypes, seeds).  Raises ValueError on every rank when they do not."""
    if not active():
        return
    gathered = all_gather_object(named_values)
    first = gathered[0]
    for r, other in enumerate(gathered):
        if other != first:
            raise ValueError(
                f"ranks disagree on {sorted(named_values)}: rank 0 has {first}, rank {r} has {other}"
            )


def merge_topk(values, global_idx, m):
    """Global top-m out of per-rank candidates.  `values` (c,) and `global_idx` (c,) are this
    rank's candidates; c is the same on every rank (pad with -inf / -1).  Returns the
    positions, in the gathered candidate list, of the m winners ordered by descending value
    then ascending global index, together with the gathered arrays."""
    vals = all_gather_same(values)
    idx = all_gather_same(global_idx)
    # descending value, ascending index: stable sort on index first, then on value
    order = torch.argsort(idx, stable=True)
    order = order[torch.argsort(vals[order], descending=True, stable=True)]
    return order[:m], vals, idx


def shard_prefix(local_total):
    """Row shards of a prefix-sum search.  `local_total` is a float64 tensor of one element, this
    rank's share of a global sum.  Returns (ends, offset): the inclusive prefix of the shares
    over the ranks (the same on every rank) and the exclusive prefix of THIS rank, i.e. the
    amount a local running sum has to start from."""
    shares = all_gather_same(local_total.reshape(1))
    ends = torch.cumsum(shares, 0)
    return ends, ends[rank()] - shares[rank()]


def pick_owned_candidates(thresholds, ends, cand_local, rows_local, rows_offset):
    """Every rank searched its own shard for each of the t thresholds; the valid answer for a
    threshold is the one of its OWNER, the first rank whose inclusive prefix `ends` reaches it
    (the last rank when rounding leaves none).  Gathers all ranks' local candidates
    (`cand_local` (t,) local row ids, `rows_local` (t, d) the rows themselves) and returns the
    owners' ones with GLOBAL row ids: (cand_global int32 (t,), rows_global (t, d)), identical
    on every rank.  `rows_offset` (world,) holds the first global row id of every rank."""
    world = world_size()
    t = int(cand_local.shape[0])
    d = int(rows_local.shape[1])
    owner = torch.clamp((ends.reshape(1, -1) < thresholds.reshape(-1, 1).to(ends.dtype)).sum(dim=1),
                        max=world - 1)
    # ONE collective for ids and rows: the ids travel as an extra column of the rows (bit pattern
    # of the int32 in a float32 column, exact value in a float64 one)
    dt = rows_local.dtype
    ids32 = cand_local.to(torch.int32).reshape(t, 1)
    id_col = ids32.view(torch.float32) if dt == torch.float32 else ids32.to(dt)
    packed = all_gather_same(torch.cat([rows_local, id_col], dim=1).reshape(1, t, d + 1))   # (world, t, d + 1)
    picked = torch.gather(packed, 0, owner.reshape(1, t, 1).expand(1, t, d + 1))[0]        # (t, d + 1)
    ids = picked[:, d].contiguous()
    ids = ids.view(torch.int32) if dt == torch.float32 else ids.to(torch.int32)
    cand_global = ids.to(torch.int64) + rows_offset[owner]
    return cand_global.to(torch.int32).contiguous(), picked[:, :d].contiguous()


def prefix_from_shares(shares):
    """(ends, offset) of `shard_prefix` from shares that every rank already holds: `shares` is a
    float64 tensor (world,), rank r's share of a global sum, identical on all ranks."""
    ends = torch.cumsum(shares, 0)
    return ends, ends[rank()] - shares[rank()]

