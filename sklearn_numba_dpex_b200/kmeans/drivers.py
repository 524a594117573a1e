"""Host-side drivers of the KMeans engine: same entry points, argument meaning and return
values as sklearn_numba_dpex/kmeans/drivers.py of the reference, on torch CUDA tensors.

Layout.  The reference's signatures take the transposes ``X_t (n_features, n_samples)`` and
``centroids_t (n_features, n_clusters)``.  They are kept, but the kernels want samples as
contiguous rows: a ``X_t`` that is the ``.T`` view of a row-major ``X`` (what the engine
passes) costs nothing; a C-contiguous ``X_t`` is transposed into a new buffer once.

Every O(n) operation is a kmb200 kernel called through the C ABI; torch is used for
memory, streams and the collectives.
"""
import ctypes
import math

import numpy as np
import torch

from .. import dist
from .._cabi import (ALGO_AUTO, ALGO_NAMES, FIN_CLEAR_ACC, FIN_MERGE, FIN_PREPARE_TF32X3, PLAN_HAVE_PREV,
                     PLAN_OPERANDS_READY, LloydPlan,
                     STATUS_DTYPE, STEP_ACC_CLEARED, STEP_OPERANDS_READY, KmbError, c_void_p, check,
                     pad_features_flag,
                     check_wait_error, dtype_code, host_device_pointer, lib, lloyd_workspace, ptr,
                     stream_ptr,
                     workspace_for)


# ----------------------------------------------------------------------------- helpers
def _rows(X_t, name="X_t"):
    """(n, d) contiguous row view/copy of a logical (d, n) tensor."""
    if not isinstance(X_t, torch.Tensor) or not X_t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if X_t.dim() != 2:
        raise ValueError(f"{name} must be 2-dimensional")
    X = X_t.T
    return X if X.is_contiguous() else X.contiguous()


def _np_dtype(t):
    return np.float32 if t.dtype == torch.float32 else np.float64


def _algo_code(algo):
    if isinstance(algo, str):
        if algo not in ALGO_NAMES:
            raise ValueError(f"algo must be one of {sorted(ALGO_NAMES)}, got {algo!r}")
        return ALGO_NAMES[algo]
    return int(algo)


def _weights_or_none(sample_weight, use_uniform_weights):
    """NULL weights mean all ones inside the kernels; use that when the weights are
    uniformly 1 (one scalar read)."""
    if sample_weight is None:
        return None
    if use_uniform_weights and sample_weight.numel() > 0 and float(sample_weight[0]) == 1.0:
        return None
    return sample_weight


class LloydState:
    """Buffers and iterations of the Lloyd loop (kmeans/drivers.py:146-343 of the reference
    allocates the same set once per call).

    Iteration `it` reads the centroids in slot it % 3 and the labels of iteration it - 1, and
    writes the labels, the merged sums, the empty list and the status record of slot it % 2 and
    the centroids of slot (it + 1) % 3.  The extra slots let `run()` enqueue iteration it + 1
    before the status of iteration `it` has been read: when that status asks for a relocation
    (or ends the loop) everything iteration `it` produced is still in place.  `C`, `labels`,
    `packed`, ... name the slots of the current iteration `self.it`."""

    def __init__(self, X, sample_weight, centers, algo=ALGO_AUTO):
        n, d = X.shape
        k = centers.shape[0]
        dev, dt = X.device, X.dtype
        self.dtype = dtype_code(dt)
        self.d_orig = d
        want = _algo_code(algo)
        # The tensor-core step moves sample tiles with TMA, whose row pitch must be a multiple
        # of 16 bytes: when it is wanted and d is not a multiple of 4, work on a copy of the
        # samples and centres padded with zero features (distances and sums are unchanged).
        # Over row shards the choice follows the TOTAL number of rows, so that every rank takes
        # the same kernel and the same padding whatever the size of its own shard.
        n_policy = int(sum(dist.all_gather_object(int(n)))) if dist.active() else n
        d4 = (d + 3) // 4 * 4
        if (dt == torch.float32 and d4 != d and want != ALGO_NAMES["cuda_core"]
                and lib.kmb_lloyd_resolve_algo(self.dtype, want, n_policy, d4, k)
                == ALGO_NAMES["tf32x3"]):
            Xp = torch.zeros((n, d4), dtype=dt, device=dev)
            Xp[:, :d] = X
            Cp = torch.zeros((k, d4), dtype=dt, device=dev)
            Cp[:, :d] = centers
            X, centers, d = Xp, Cp, d4
        self.X = X
        self.w = sample_weight
        self.n, self.d, self.k = n, d, k
        # zero features added above: the step keeps its two extra contraction features there
        self._pad_flag = pad_features_flag(d - self.d_orig)
        self.algo = check(lib.kmb_lloyd_resolve_algo(self.dtype, want, n_policy, d, k),
                          "kmb_lloyd_resolve_algo")
        self.is_tc = self.algo == ALGO_NAMES["tf32x3"]
        self.acc_len = lib.kmb_lloyd_acc_len(d, k)
        self.n_copies = check(lib.kmb_lloyd_acc_copies(self.dtype, self.algo, n, d, k))
        self.it = 0                              # iterations completed so far
        self._Cs = [centers.contiguous().clone()] + [torch.empty((k, d), dtype=dt, device=dev)
                                                     for _ in range(2)]
        self._hs = [torch.empty(k, dtype=dt, device=dev) for _ in range(3)]
        self._labs = [torch.empty(n, dtype=torch.int32, device=dev) for _ in range(2)]
        self._packs = [torch.empty(self.acc_len, dtype=dt, device=dev) for _ in range(2)]
        self._empties = [torch.empty(k, dtype=torch.int32, device=dev) for _ in range(2)]
        self.shifts = torch.empty(k, dtype=dt, device=dev)
        # The copies start at zero and every finalize (or merge) clears them again once read,
        # so no step has to clear them.
        self.acc = torch.zeros((self.n_copies, self.acc_len), dtype=dt, device=dev)
        # Status records: page-locked host memory that the finalize kernel writes directly (no
        # copy to enqueue), one record per slot, each followed on the stream by an event.
        self._status = torch.zeros((2, 32), dtype=torch.uint8).pin_memory()
        self._status_ptrs = [host_device_pointer(self._status[i]) for i in range(2)]
        self._events = [torch.cuda.Event() for _ in range(2)]
        for ev in self._events:
            ev.record(torch.cuda.current_stream(dev))       # creates the handle
        self._event_handles = [c_void_p(ev.cuda_event) for ev in self._events]
        # iterations -> (event before, event after) the fused kernel, for callers that time it
        self.step_events = {}
        # A workspace of this state's own: the tensor-core operands that a finalize writes for
        # the next step, and the sticky time-out flag, live there between calls.  The row-scan
        # calls of this state (inertia, top-k) use the shared scratch buffer instead.
        self.ws, self.ws_bytes = lloyd_workspace(dev, n, d, k, own=True)
        self.scratch, self.scratch_bytes = workspace_for(dev, n, d, k)
        self.sq_dist = None
        self.have_prev = False
        self._operands_slot = None               # centroid slot whose split operands sit in ws
        self.kernel_launches = 0
        self.event_hook = None                   # callable(kind, it) around the fused kernel
        self._calm = False                       # the last finished iteration had no empty cluster
        check(lib.kmb_half_l2_norm(self.dtype, ptr(self.C), ptr(self.h), k, d, stream_ptr(dev)),
              "kmb_half_l2_norm")
        self.kernel_launches += 1
        # The whole ring described once, so that a single-GPU iteration is ONE call into the
        # library (kmb_lloyd_plan_launch) instead of one per kernel.
        plan = LloydPlan()
        plan.dtype, plan.algo, plan.d, plan.k = self.dtype, self.algo, d, k
        plan.n_copies, plan.n = self.n_copies, n
        plan.X = X.data_ptr()
        plan.w = sample_weight.data_ptr() if sample_weight is not None else None
        for i in range(3):
            plan.C[i] = self._Cs[i].data_ptr()
            plan.h[i] = self._hs[i].data_ptr()
        for i in range(2):
            plan.labels[i] = self._labs[i].data_ptr()
            plan.merged[i] = self._packs[i].data_ptr()
            plan.empty_list[i] = self._empties[i].data_ptr()
            plan.status[i] = self._status_ptrs[i].value
        plan.acc, plan.shifts = self.acc.data_ptr(), self.shifts.data_ptr()
        plan.workspace, plan.workspace_bytes = self.ws.data_ptr(), self.ws_bytes
        self._plan = plan
        self._plan_ref = ctypes.byref(plan)

    # -- the slots of the current iteration -------------------------------------------
    C = property(lambda self: self._Cs[self.it % 3])
    C_new = property(lambda self: self._Cs[(self.it + 1) % 3])
    h = property(lambda self: self._hs[self.it % 3])
    h_new = property(lambda self: self._hs[(self.it + 1) % 3])
    labels = property(lambda self: self._labs[(self.it + 1) % 2])       # of iteration it - 1
    labels_new = property(lambda self: self._labs[self.it % 2])
    packed = property(lambda self: self._packs[self.it % 2])
    empty_list = property(lambda self: self._empties[self.it % 2])
    status_dev = property(lambda self: self._status[self.it % 2])
    status_host = property(lambda self: self._status[(self.it + 1) % 2])   # last finished iteration
    packed_last = property(lambda self: self._packs[(self.it + 1) % 2])    # last finished iteration

    @property
    def operands_ready(self):
        return self.is_tc and self._operands_slot == self.it % 3

    @operands_ready.setter
    def operands_ready(self, value):
        self._operands_slot = (self.it % 3) if value else None

    # -- pieces -----------------------------------------------------------------------
    def _finalize(self, it, merge, clear):
        """One kernel: (merge of the copies,) division, shifts, next half norms, operands of
        the next tensor-core step, empty list, status record of iteration `it`."""
        flags = self._pad_flag | (FIN_MERGE if merge else 0) | (FIN_CLEAR_ACC if clear else 0) | \
            (FIN_PREPARE_TF32X3 if self.is_tc else 0)
        dev = self.X.device
        check(lib.kmb_lloyd_finalize(self.dtype, ptr(self.acc), self.n_copies,
                                     ptr(self._packs[it % 2]), flags, ptr(self._Cs[it % 3]),
                                     ptr(self._Cs[(it + 1) % 3]), ptr(self._hs[(it + 1) % 3]),
                                     ptr(self.shifts), ptr(self._empties[it % 2]),
                                     self._status_ptrs[it % 2], self.k, self.d, ptr(self.ws),
                                     self.ws_bytes, stream_ptr(dev)), "kmb_lloyd_finalize")
        self._events[it % 2].record(torch.cuda.current_stream(dev))
        self.kernel_launches += 1
        self._operands_slot = (it + 1) % 3 if self.is_tc else None

    def _launch_fused(self, it):
        """The fused kernel of iteration `it`: its labels and the accumulator copies."""
        ready = self.is_tc and self._operands_slot == it % 3
        flags = self._pad_flag | STEP_ACC_CLEARED | (STEP_OPERANDS_READY if ready else 0)
        prev = self._labs[(it + 1) % 2] if (self.have_prev or it > 0) else None
        if self.event_hook is not None:
            self.event_hook("pre", it)
        ev = self.step_events.get(it)
        stream = torch.cuda.current_stream(self.X.device)
        if ev:
            ev[0].record(stream)
        check(lib.kmb_lloyd_step(self.dtype, self.algo, ptr(self.X), ptr(self.w),
                                 ptr(self._Cs[it % 3]), ptr(self._hs[it % 3]), ptr(prev),
                                 ptr(self._labs[it % 2]), ptr(self.acc), self.n_copies, self.n,
                                 self.d, self.k, flags, ptr(self.ws), self.ws_bytes,
                                 stream_ptr(self.X.device)), "kmb_lloyd_step")
        if ev:
            ev[1].record(stream)
        if self.event_hook is not None:
            self.event_hook("post", it)
        self.kernel_launches += 1 + (1 if self.is_tc and not ready else 0)

    def _launch_reduce_finalize(self, it):
        """Everything of iteration `it` after the fused kernel, enqueued without a host read:
        one kernel on one GPU; merge, all-reduce, finalize over row shards."""
        if dist.active():
            check(lib.kmb_lloyd_merge_copies(self.dtype, ptr(self.acc), self.n_copies,
                                             self.acc_len, ptr(self._packs[it % 2]), 1,
                                             stream_ptr(self.X.device)), "kmb_lloyd_merge_copies")
            self.kernel_launches += 1
            dist.all_reduce_sum_(self._packs[it % 2])
            self._finalize(it, merge=False, clear=False)
        else:
            self._finalize(it, merge=True, clear=True)

    def _launch(self, it):
        """Enqueues iteration `it`: fused kernel, reduction, finalize."""
        if dist.active() or self.event_hook is not None:
            self._launch_fused(it)
            self._launch_reduce_finalize(it)
            return
        ready = self.is_tc and self._operands_slot == it % 3
        flags = self._pad_flag | (PLAN_HAVE_PREV if (self.have_prev or it > 0) else 0) | \
            (PLAN_OPERANDS_READY if ready else 0)
        ev = self.step_events.get(it)
        stream = c_void_p(torch.cuda.current_stream(self.X.device).cuda_stream)
        check(lib.kmb_lloyd_plan_launch(self._plan_ref, it, flags,
                                        c_void_p(ev[0].cuda_event) if ev else None,
                                        c_void_p(ev[1].cuda_event) if ev else None,
                                        self._event_handles[it % 2], stream), "kmb_lloyd_plan_launch")
        self.kernel_launches += 2 + (1 if self.is_tc and not ready else 0)
        self._operands_slot = (it + 1) % 3 if self.is_tc else None

    def launch_fused_step(self):
        self._launch_fused(self.it)

    def launch_reduce_finalize(self):
        self._launch_reduce_finalize(self.it)

    def launch_step(self):
        """E-step + accumulation + reduction + finalize of the current iteration, all enqueued
        (no host read)."""
        self._launch(self.it)

    def _wait_status(self, it):
        """Waits for the status record of iteration `it`: (n_empty, changed, shift_total)."""
        self._events[it % 2].synchronize()
        rec = self._status[it % 2].numpy().view(STATUS_DTYPE)[0]
        if int(rec["wait_error"]) != 0:
            self._operands_slot = None
            raise KmbError("a bounded wait inside the tcgen05 Lloyd kernel ran out; the results "
                           "of this iteration are invalid")
        return int(rec["n_empty"]), int(rec["changed"]), float(rec["shift_total"])

    def _relocate(self, n_empty):
        """kmeans/drivers.py:238-272 and 396-433 of the reference.  The distances that rank
        the samples are taken against the un-normalised sums, exactly as there (the inertia
        kernel runs before the division by the cluster sizes)."""
        dev, dt = self.X.device, self.X.dtype
        if self.sq_dist is None:
            self.sq_dist = torch.empty(self.n, dtype=dt, device=dev)
        check(lib.kmb_inertia(self.dtype, ptr(self.X), None, ptr(self.packed),
                              ptr(self.labels_new), ptr(self.sq_dist), None, self.n, self.d,
                              self.k, ptr(self.scratch), self.scratch_bytes, stream_ptr(dev)),
              "kmb_inertia")
        m_local = min(n_empty, self.n)
        far = topk_idx_1d(self.sq_dist, m_local) if m_local > 0 else \
            torch.empty(0, dtype=torch.int64, device=dev)
        if dist.active():
            X_rows, w_rows, lab_rows, far = _gather_relocation_candidates(self, far, n_empty)
        else:
            X_rows, w_rows, lab_rows = self.X, self.w, self.labels_new
        check(lib.kmb_relocate_empty_clusters(self.dtype, ptr(X_rows), ptr(w_rows), ptr(lab_rows),
                                              X_rows.shape[0], ptr(far), ptr(self.empty_list),
                                              min(n_empty, int(far.numel())), None,
                                              ptr(self.packed), self.d, self.k, stream_ptr(dev)),
              "kmb_relocate_empty_clusters")
        self.kernel_launches += 2
        self._finalize(self.it, merge=False, clear=False)

    def inertia_against_sums(self):
        """What the reference prints per iteration when verbose: the weighted inertia of the
        NEW assignments against `new_centroids_t` as it stands at that point of the loop, i.e.
        the merged sums before relocation and before the division by the cluster sizes
        (kmeans/drivers.py:223-236 of the reference run ahead of :275)."""
        dev = self.X.device
        total = torch.empty(1, dtype=self.X.dtype, device=dev)
        check(lib.kmb_inertia(self.dtype, ptr(self.X), ptr(self.w), ptr(self.packed),
                              ptr(self.labels_new), None, ptr(total), self.n, self.d, self.k,
                              ptr(self.scratch), self.scratch_bytes, stream_ptr(dev)), "kmb_inertia")
        self.kernel_launches += 2
        dist.all_reduce_sum_(total)
        return float(total[0])

    def step(self, before_relocation=None):
        """One Lloyd iteration, start to finish.  Returns (n_empty_before_relocation, changed,
        shift_total).  `before_relocation`, when given, is called once the merged sums and the
        new labels exist and before empty clusters are relocated."""
        self._launch(self.it)
        n_empty, changed, shift = self._wait_status(self.it)
        if before_relocation is not None:
            before_relocation(self)
        if n_empty > 0:
            self._relocate(n_empty)
            _, _, shift = self._wait_status(self.it)
        self._calm = n_empty == 0
        self.it += 1
        return n_empty, changed, shift

    def run(self, max_iter, tol=0.0, before_relocation=None, pipelined=True, stop_on_strict=True):
        """The loop of `lloyd` (kmeans/drivers.py:188-343 of the reference) from the current
        state: iterates until max_iter, a total shift <= tol, or strict convergence (labels
        unchanged, armed after the second iteration as in the reference).  Returns a dict with
        n_iter, strict, shift, n_relocation_events, n_empty_max.

        Pipelined: iteration i + 1 is enqueued BEFORE the status of iteration i is read (once an
        iteration without empty clusters has been seen), so the GPU never idles while the host
        decides; it is run again only when iteration i had to relocate empty clusters, and simply
        ignored when iteration i ended the loop.  With a
        callback (verbose mode) the loop runs unpipelined.  `stop_on_strict=False` keeps iterating
        after the labels have stopped changing (the benchmark times a fixed number of steps)."""
        T = np.float32 if self.X.dtype == torch.float32 else np.float64
        pipelined = bool(pipelined) and before_relocation is None
        n_iter, shift, armed, strict = 0, np.inf, False, False
        events, n_empty_max = 0, 0
        launched = False                          # iteration self.it is already in flight
        while n_iter < max_iter and shift > tol:
            if not launched:
                self._launch(self.it)
            launched = False
            # speculate only when the last known iteration had no empty cluster: a relocation
            # throws the speculative iteration away, a whole pass over the samples (the first
            # iterations from a random-row init usually relocate)
            speculate = pipelined and n_iter + 1 < max_iter and self._calm
            if speculate:
                self._launch(self.it + 1)
            n_empty, changed, shift_total = self._wait_status(self.it)
            if before_relocation is not None:
                before_relocation(self)
            if n_empty > 0:
                # (the speculative iteration ran from centroids that are about to change)
                self._relocate(n_empty)
                _, _, shift_total = self._wait_status(self.it)
                speculate = False
            events += int(n_empty > 0)
            n_empty_max = max(n_empty_max, n_empty)
            self._calm = n_empty == 0
            self.it += 1
            launched = speculate
            n_iter += 1
            if n_iter > 1:
                if armed and changed == 0 and stop_on_strict:
                    strict = True
                    break
                armed = True
            shift = T(shift_total)
        if launched:
            # an iteration in flight that the loop did not need: let it finish (it wrote only
            # slots of its own and the operands of centroids nobody will use) and forget it
            self._events[self.it % 2].synchronize()
            self._operands_slot = None
        return dict(n_iter=n_iter, strict=strict, shift=shift, n_relocation_events=events,
                    n_empty_max=n_empty_max)

    def final_labels_inertia(self):
        dev = self.X.device
        labels = self._labs[self.it % 2]          # free: the next iteration would write it
        check(lib.kmb_assign_labels(self.dtype, self.algo, ptr(self.X), ptr(self.C), ptr(self.h),
                                    ptr(labels), self.n, self.d, self.k, self._pad_flag,
                                    ptr(self.ws), self.ws_bytes, stream_ptr(dev)), "kmb_assign_labels")
        self._operands_slot = (self.it % 3) if self.is_tc else None
        total = torch.empty(1, dtype=self.X.dtype, device=dev)
        check(lib.kmb_inertia(self.dtype, ptr(self.X), ptr(self.w), ptr(self.C), ptr(labels),
                              None, ptr(total), self.n, self.d, self.k, ptr(self.scratch),
                              self.scratch_bytes, stream_ptr(dev)), "kmb_inertia")
        self.kernel_launches += 3 + (1 if self.is_tc else 0)
        dist.all_reduce_sum_(total)
        self.check_device_waits()
        return labels, total

    def centers(self):
        """Current centroids (k, d) without the padding features, contiguous."""
        if self.d == self.d_orig:
            return self.C
        return self.C[:, : self.d_orig].contiguous()

    def check_device_waits(self):
        """Raises if a bounded wait inside the tensor-core kernel ran out on this state's
        workspace (the flag is sticky, so this covers every launch since the state was made)."""
        if self.is_tc:
            check_wait_error(self.ws, self.X.device)


def _gather_relocation_candidates(state, far_local, n_empty):
    """Sharded relocation: every rank offers its local top candidates; all ranks pick the
    same global winners and apply the relocation to their replicated sums."""
    dev, dt = state.X.device, state.X.dtype
    m = n_empty
    counts = dist.all_gather_object(int(state.n))
    offset = sum(counts[: dist.rank()])
    vals = torch.full((m,), -math.inf, dtype=dt, device=dev)
    gidx = torch.full((m,), -1, dtype=torch.int64, device=dev)
    rows = torch.zeros((m, state.d), dtype=dt, device=dev)
    wts = torch.zeros((m,), dtype=dt, device=dev)
    labs = torch.zeros((m,), dtype=torch.int32, device=dev)
    c = int(far_local.numel())
    if c:
        vals[:c] = state.sq_dist[far_local]
        gidx[:c] = far_local + offset
        rows[:c] = state.X[far_local]
        wts[:c] = state.w[far_local] if state.w is not None else 1.0
        labs[:c] = state.labels_new[far_local]
    winners, _, _ = dist.merge_topk(vals, gidx, m)
    rows_g = dist.all_gather_same(rows)
    wts_g = dist.all_gather_same(wts)
    labs_g = dist.all_gather_same(labs)
    valid = dist.all_gather_same(gidx)[winners] >= 0
    winners = winners[valid]
    return rows_g.contiguous(), wts_g.contiguous(), labs_g.contiguous(), winners.contiguous()


# -------------------------------------------------------------------------------- lloyd
def lloyd(X_t, sample_weight, centroids_t, use_uniform_weights, max_iter=300, verbose=False,
          tol=1e-4, algo="auto", stats=None):
    """Lloyd's algorithm.  Same contract as `lloyd` of the reference
    (sklearn_numba_dpex/kmeans/drivers.py:43-393): returns
    ``(labels (n,), inertia (host scalar of the compute dtype), centroids_t (d, k), n_iter)``.

    Labels are int32 holding the reference's uint32 values.  The strict-convergence test
    follows the reference: the flag is first armed after the second iteration, so the loop
    can stop on unchanged labels at the end of the third iteration at the earliest.

    `stats`, when a dict, receives `n_relocation_events` (iterations that had to relocate empty
    clusters), `n_empty_max` and `kernel_launches`.
    """
    X = _rows(X_t)
    C0 = _rows(centroids_t, "centroids_t")
    if X.dtype != C0.dtype:
        raise ValueError("X_t and centroids_t must share one dtype")
    if X.shape[1] != C0.shape[1]:
        raise ValueError("X_t and centroids_t disagree on n_features")
    T = _np_dtype(X)
    w = _weights_or_none(sample_weight, use_uniform_weights)
    state = LloydState(X, w, C0, algo)
    if dist.active():
        dist.check_same_across_ranks(d=state.d, k=state.k, dtype=str(X.dtype),
                                     max_iter=int(max_iter), tol=float(tol))

    verbose = bool(verbose)
    counter = {"it": 0}

    def report(st):
        print(f"Iteration {counter['it']}, inertia {st.inertia_against_sums():5.3e}")
        counter["it"] += 1

    out = state.run(int(max_iter), tol, before_relocation=report if verbose else None)
    n_iteration, strict, shift = out["n_iter"], out["strict"], out["shift"]
    n_reloc_events, n_empty_max = out["n_relocation_events"], out["n_empty_max"]

    if verbose:
        converged_at = n_iteration - 1
        if strict or shift == 0:
            print(f"Converged at iteration {converged_at}: strict convergence.")
        elif shift <= tol:
            print(f"Converged at iteration {converged_at}: center shift {shift} within "
                  f"tolerance {tol}.")

    labels, total = state.final_labels_inertia()
    inertia = total.cpu().numpy()[0]
    if isinstance(stats, dict):
        stats.update(n_relocation_events=n_reloc_events, n_empty_max=n_empty_max,
                     kernel_launches=state.kernel_launches)
    return labels, inertia, state.centers().T, n_iteration


# ---------------------------------------------------------------------------- top-k
def _topk_call(array_in, k, want_values, want_idx):
    if not isinstance(array_in, torch.Tensor) or not array_in.is_cuda:
        raise ValueError("array_in must be a CUDA tensor")
    if array_in.dtype not in (torch.float32, torch.float64):
        raise ValueError(
            f"topk currently only supports dtypes in (float32, float64), but got dtype="
            f"{array_in.dtype} .")
    is_1d = array_in.dim() == 1
    arr = array_in.reshape(1, -1) if is_1d else array_in
    arr = arr.contiguous()
    n_rows, n_cols = arr.shape
    if n_cols < k:
        raise ValueError(
            "Expected k to be greater than or equal to the number of items in the search "
            f"space, but got k={k} and {n_cols} items in the search space.")
    dev = arr.device
    nbytes = lib.kmb_topk_workspace_bytes(n_rows, n_cols, k)
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
    vals = torch.empty((n_rows, k), dtype=arr.dtype, device=dev) if want_values else None
    idx = torch.empty((n_rows, k), dtype=torch.int64, device=dev) if want_idx else None
    check(lib.kmb_topk(dtype_code(arr.dtype), ptr(arr), n_rows, n_cols, k, ptr(vals), ptr(idx),
                       ptr(ws), ws.numel(), stream_ptr(dev)), "kmb_topk")
    if is_1d:
        vals = vals.reshape(-1) if vals is not None else None
        idx = idx.reshape(-1) if idx is not None else None
    return vals, idx


def topk_idx_1d(values, k):
    return _topk_call(values, k, False, True)[1]


# ----------------------------------------------------------------- data preparation
def _device_sum(t, square):
    dev = t.device
    out = torch.empty(1, dtype=torch.float64, device=dev)
    flat = t.reshape(-1)
    ws, ws_bytes = workspace_for(dev, flat.numel(), 1, 1)
    check(lib.kmb_sum(dtype_code(t.dtype), ptr(flat), flat.numel(), int(square), ptr(out), ptr(ws),
                      ws_bytes, stream_ptr(dev)), "kmb_sum")
    return out


def all_finite(t):
    """True when no element of the tensor is NaN or infinite (one pass on the device)."""
    if t.numel() == 0:
        return True
    dev = t.device
    t = t if t.is_contiguous() else t.contiguous()
    out = torch.empty(1, dtype=torch.float64, device=dev)
    flat = t.reshape(-1)
    ws, ws_bytes = workspace_for(dev, flat.numel(), 1, 1)
    check(lib.kmb_sum(dtype_code(t.dtype), ptr(flat), flat.numel(), 2, ptr(out), ptr(ws), ws_bytes,
                      stream_ptr(dev)), "kmb_sum")
    return float(out[0]) == 0.0


def gather_rows(X, row_ids):
    """X[row_ids] for host or device integer ids, gathered by the library (k, d)."""
    dev = X.device
    ids = torch.as_tensor(np.asarray(row_ids), dtype=torch.int32).to(dev) \
        if not isinstance(row_ids, torch.Tensor) else row_ids.to(device=dev, dtype=torch.int32)
    ids = ids.contiguous()
    X = X if X.is_contiguous() else X.contiguous()
    out = torch.empty((ids.numel(), X.shape[1]), dtype=X.dtype, device=dev)
    check(lib.kmb_gather_rows(dtype_code(X.dtype), ptr(X), ptr(ids), ids.numel(), X.shape[1],
                              ptr(out), stream_ptr(dev)), "kmb_gather_rows")
    return out


def _add_row_vector_(X, vec, sign):
    check(lib.kmb_add_row_vector(dtype_code(X.dtype), ptr(X), X.shape[0], X.shape[1], ptr(vec),
                                 float(sign), stream_ptr(X.device)), "kmb_add_row_vector")


def prepare_data_for_lloyd(X_t, init, tol, sample_weight, copy_x):
    """Centre the data, rescale the tolerance, test the weights for uniformity.  Same contract
    as the reference's function (sklearn_numba_dpex/kmeans/drivers.py:436-545): returns
    ``(X_t, X_mean | None, init, tol, sample_weight_is_uniform)``; `init` is a (d, k) tensor or
    a non-array init spec passed through.  With ``copy_x=False`` X is centred in place (when
    its rows are contiguous) and put back by `restore_data_after_lloyd`."""
    X = _rows(X_t)
    n, d = X.shape
    T = _np_dtype(X)
    dev = X.device
    n_total = n
    col = torch.empty(d, dtype=torch.float64, device=dev)
    ws, ws_bytes = workspace_for(dev, n, d, 1)
    check(lib.kmb_col_sums(dtype_code(X.dtype), ptr(X), n, d, ptr(col), ptr(ws), ws_bytes,
                           stream_ptr(dev)), "kmb_col_sums")
    if dist.active():
        dist.all_reduce_sum_(col)
        n_total = int(sum(dist.all_gather_object(int(n))))
    X_mean = (col.to(X.dtype) / T(n_total)).contiguous()
    mean_sq = float(_device_sum(X_mean, True)[0])
    if mean_sq == 0.0:
        X_mean = None
    else:
        X = X.clone() if copy_x else X
        _add_row_vector_(X, X_mean, -1.0)
        if isinstance(init, torch.Tensor):
            init_rows = _rows(init, "init").clone()
            _add_row_vector_(init_rows, X_mean, -1.0)
            init = init_rows.T
    variance = _device_sum(X, True)
    dist.all_reduce_sum_(variance)
    tol = T(T(float(variance[0])) / T(d * n_total)) * tol
    wsum = _device_sum(sample_weight, False)
    w0 = sample_weight[:1].to(torch.float64)
    if dist.active():
        dist.all_reduce_sum_(wsum)
        dist.broadcast_(w0, 0)
    uniform = bool(T(float(wsum[0])) == T(float(w0[0])) * n_total)
    if dist.active():
        w_all_equal = bool(float(sample_weight[0]) == float(w0[0])) if n else True
        uniform = uniform and all(dist.all_gather_object(w_all_equal))
    return X.T, X_mean, init, tol, uniform


def restore_data_after_lloyd(X_t, best_centers_t, X_mean, copy_x):
    """Adds the feature means back, in place (sklearn_numba_dpex/kmeans/drivers.py:548-589)."""
    if X_mean is None:
        return
    C = best_centers_t.T
    if C.is_contiguous():
        _add_row_vector_(C, X_mean, 1.0)
    else:
        best_centers_t += X_mean.reshape(-1, 1)
    if not copy_x:
        X = X_t.T
        if X.is_contiguous():
            _add_row_vector_(X, X_mean, 1.0)
        else:
            X_t += X_mean.reshape(-1, 1)


# ------------------------------------------------------------------- label utilities
def _as_i32(labels):
    if labels.dtype == torch.int32:
        return labels.contiguous()
    return labels.to(torch.int32).contiguous()


def is_same_clustering(labels1, labels2, n_clusters):
    """Equal up to a permutation of the label values
    (sklearn_numba_dpex/kmeans/drivers.py:592-602)."""
    l1, l2 = _as_i32(labels1), _as_i32(labels2)
    dev = l1.device
    mapping = torch.empty(n_clusters, dtype=torch.int32, device=dev)
    result = torch.empty(1, dtype=torch.int32, device=dev)
    check(lib.kmb_same_clustering(ptr(l1), ptr(l2), l1.numel(), n_clusters, ptr(mapping),
                                  ptr(result), stream_ptr(dev)), "kmb_same_clustering")
    if dist.active():
        result = result.clone()
        torch.distributed.all_reduce(result, op=torch.distributed.ReduceOp.MIN)
    return bool(result.cpu()[0])


def get_nb_distinct_clusters(labels, n_clusters):
    """Number of distinct labels (sklearn_numba_dpex/kmeans/drivers.py:605-627)."""
    lab = _as_i32(labels)
    dev = lab.device
    seen = torch.empty(n_clusters, dtype=torch.int32, device=dev)
    out = torch.empty(1, dtype=torch.int32, device=dev)
    check(lib.kmb_count_distinct(ptr(lab), lab.numel(), n_clusters, ptr(seen), ptr(out),
                                 stream_ptr(dev)), "kmb_count_distinct")
    if dist.active():
        torch.distributed.all_reduce(seen, op=torch.distributed.ReduceOp.MAX)
        return np.int32(int((seen > 0).sum().cpu()))
    return out.cpu().numpy()[0]


# ------------------------------------------------------------ predict / score / transform
def get_labels_inertia(X_t, centroids_t, sample_weight, with_inertia, algo="auto"):
    """Labels and (optionally) inertia against given centroids.  Same contract as the
    reference (sklearn_numba_dpex/kmeans/drivers.py:630-699): inertia is a 1-element numpy
    array, or None."""
    X = _rows(X_t)
    C = _rows(centroids_t, "centroids_t")
    n, d = X.shape
    k = C.shape[0]
    dev = X.device
    code = dtype_code(X.dtype)
    h = torch.empty(k, dtype=X.dtype, device=dev)
    labels = torch.empty(n, dtype=torch.int32, device=dev)
    ws, ws_bytes = lloyd_workspace(dev, n, d, k)
    check(lib.kmb_half_l2_norm(code, ptr(C), ptr(h), k, d, stream_ptr(dev)), "kmb_half_l2_norm")
    check(lib.kmb_assign_labels(code, _algo_code(algo), ptr(X), ptr(C), ptr(h), ptr(labels), n, d,
                                k, 0, ptr(ws), ws_bytes, stream_ptr(dev)), "kmb_assign_labels")
    if lib.kmb_lloyd_resolve_algo(code, _algo_code(algo), n, d, k) == ALGO_NAMES["tf32x3"]:
        check_wait_error(ws, dev)      # before the inertia call reuses the shared buffer
    if not with_inertia:
        return labels, None
    total = torch.empty(1, dtype=X.dtype, device=dev)
    check(lib.kmb_inertia(code, ptr(X), ptr(sample_weight), ptr(C), ptr(labels), None, ptr(total),
                          n, d, k, ptr(ws), ws_bytes, stream_ptr(dev)), "kmb_inertia")
    dist.all_reduce_sum_(total)
    return labels, total.cpu().numpy()


# Rows per launch of the distance kernel: bounds the grid and lets callers that cannot hold the
# whole (n, k) result walk it block by block.
DISTANCE_ROWS_PER_LAUNCH = 1 << 22


def get_euclidean_distances(X_t, Y_t):
    """(n, k) euclidean distances, returned like the reference as the transposed view of a
    (k, n) array (sklearn_numba_dpex/kmeans/drivers.py:702-732).  The result holds n * k
    elements (41 GB for 10 M samples and 1 024 centres in float32): when it does not fit the
    free device memory a MemoryError says so and points at `iter_euclidean_distances`."""
    X = _rows(X_t)
    Y = _rows(Y_t, "Y_t")
    n, d = X.shape
    k = Y.shape[0]
    need = n * k * X.element_size()
    free, _ = torch.cuda.mem_get_info(X.device)
    if need > free:
        raise MemoryError(
            f"the ({n}, {k}) distance matrix needs {need / 1e9:.1f} GB and {free / 1e9:.1f} GB of "
            "device memory are free; walk it in row blocks with iter_euclidean_distances")
    out_t = torch.empty((k, n), dtype=X.dtype, device=X.device)
    for start in range(0, n, DISTANCE_ROWS_PER_LAUNCH):
        stop = min(n, start + DISTANCE_ROWS_PER_LAUNCH)
        check(lib.kmb_euclidean_distances(dtype_code(X.dtype), ptr(X[start:stop]), ptr(Y),
                                          ptr(out_t[:, start:]), stop - start, d, k, n,
                                          stream_ptr(X.device)), "kmb_euclidean_distances")
    return out_t.T


def iter_euclidean_distances(X_t, Y_t, rows_per_block=None):
    """Yields (start, stop, D) with D the (stop - start, k) distances of samples
    [start, stop), block after block, for results too large to hold at once.  The block buffer
    is reused: consume (or copy) D before asking for the next block."""
    X = _rows(X_t)
    Y = _rows(Y_t, "Y_t")
    n, d = X.shape
    k = Y.shape[0]
    if rows_per_block is None:
        budget = 1 << 30                           # about 1 GB of distances per block
        rows_per_block = max(128, min(n, budget // (k * X.element_size())))
    rows_per_block = int(rows_per_block)
    buf = torch.empty((k, min(n, rows_per_block)), dtype=X.dtype, device=X.device)
    for start in range(0, n, rows_per_block):
        stop = min(n, start + rows_per_block)
        check(lib.kmb_euclidean_distances(dtype_code(X.dtype), ptr(X[start:stop]), ptr(Y), ptr(buf),
                                          stop - start, d, k, buf.shape[1], stream_ptr(X.device)),
              "kmb_euclidean_distances")
        yield start, stop, buf[:, : stop - start].T


# ------------------------------------------------------------------------- k-means++
def kmeans_plusplus(X_t, sample_weight, n_clusters, random_state):
    """Greedy k-means++ seeding with ``2 + int(log(k))`` trials per round.  Same contract as
    the reference (sklearn_numba_dpex/kmeans/drivers.py:735-910): returns
    ``(centers_t (d, k), center_indices int32 (k,))``.

    The random stream is the reference's (xoroshiro128++, one state per trial, seeded from
    `random_state`), drawn on the host ahead of the loop since each round consumes exactly
    one value per trial.  Candidates are the first index whose inclusive prefix sum of the
    current potentials reaches ``u * total``; the prefix is evaluated in float64 by a
    two-level scan, where the reference runs a sequential sum in the compute dtype.
    """
    from ..common.random import create_xoroshiro128pp_states, get_random_raw, uniform_draws

    X = _rows(X_t)
    n, d = X.shape
    k = int(n_clusters)
    dev, dt = X.device, X.dtype
    code = dtype_code(dt)
    T = _np_dtype(X)
    t = 2 + int(math.log(k))
    sharded = dist.active()
    counts = dist.all_gather_object(int(n)) if sharded else [n]
    n_total = int(sum(counts))
    row0 = int(sum(counts[: dist.rank()])) if sharded else 0
    states = create_xoroshiro128pp_states(t, seed=random_state)
    first = int(get_random_raw(states)[0] % np.uint64(n_total))
    u_host = uniform_draws(states, k - 1, T)  # (k-1, t)
    if sharded:
        dist.check_same_across_ranks(first=first, k=k, d=d, u_sum=float(u_host.sum()))
    u = torch.from_numpy(u_host).to(dev) if k > 1 else torch.empty((0, t), dtype=dt, device=dev)

    block = lib.kmb_kpp_block_rows()
    nb = (n + block - 1) // block
    M = [torch.empty((t, n), dtype=dt, device=dev) for _ in range(2)]
    bsum = [torch.empty((t, nb), dtype=torch.float64, device=dev) for _ in range(2)]
    best = torch.zeros(1, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=dt, device=dev)
    cand = torch.empty(t, dtype=torch.int32, device=dev)
    cand_rows = torch.empty((t, d), dtype=dt, device=dev)
    pots = torch.empty(t, dtype=dt, device=dev)
    centers = torch.empty((k, d), dtype=dt, device=dev)
    indices = torch.full((k,), -1, dtype=torch.int32, device=dev)
    w = sample_weight
    s = stream_ptr(dev)

    if not sharded:
        pots64 = torch.empty(t, dtype=torch.float64, device=dev)
        check(lib.kmb_kpp_init(code, ptr(X), ptr(w), first, None, ptr(M[0]), ptr(bsum[0]),
                               ptr(centers), ptr(indices), n, d, s), "kmb_kpp_init")
        check(lib.kmb_kpp_select(code, ptr(bsum[0]), None, 1, nb, None, ptr(best), ptr(total), None,
                                 None, None, None, 0, d, s), "kmb_kpp_select")
        cur = 0
        for c in range(1, k):
            nxt = 1 - cur
            check(lib.kmb_kpp_sample(code, ptr(M[cur]), ptr(bsum[cur]), ptr(best), ptr(total),
                                     ptr(u[c - 1]), None, t, ptr(cand), n, s), "kmb_kpp_sample")
            check(lib.kmb_gather_rows(code, ptr(X), ptr(cand), t, d, ptr(cand_rows), s),
                  "kmb_gather_rows")
            check(lib.kmb_kpp_step(code, ptr(X), ptr(w), ptr(cand_rows), ptr(M[cur]), ptr(best),
                                   ptr(M[nxt]), ptr(bsum[nxt]), n, d, t, s), "kmb_kpp_step")
            # the t potentials by t CTAs, then the single-CTA choice (the select kernel alone
            # would walk all t x nb block sums with one CTA: 40 us of a 270 us round at n = 2.5 M)
            check(lib.kmb_kpp_potentials(ptr(bsum[nxt]), t, nb, ptr(pots64), s), "kmb_kpp_potentials")
            check(lib.kmb_kpp_select(code, None, ptr(pots64), t, nb, ptr(pots), ptr(best),
                                     ptr(total), ptr(cand_rows), ptr(cand), ptr(centers),
                                     ptr(indices), c, d, s), "kmb_kpp_select")
            cur = nxt
        return centers.T, indices

    # ---- row shards: every rank scans its own rows; per round one all-gather of the local
    # candidates (row + id) and one of the local potentials, two glue kernels, no host sync
    world, me = dist.world_size(), dist.rank()
    first_row = torch.zeros(d, dtype=dt, device=dev)
    if row0 <= first < row0 + n:
        first_row.copy_(X[first - row0])
    dist.all_reduce_sum_(first_row)
    check(lib.kmb_kpp_init(code, ptr(X), ptr(w), first, ptr(first_row), ptr(M[0]), ptr(bsum[0]),
                           ptr(centers), ptr(indices), n, d, s), "kmb_kpp_init")
    pots64 = torch.empty(t, dtype=torch.float64, device=dev)
    check(lib.kmb_kpp_potentials(ptr(bsum[0]), 1, nb, ptr(pots64), s), "kmb_kpp_potentials")
    local_tot = pots64[:1].clone()                       # this shard's share of the potential
    glob = dist.all_reduce_sum_(pots64[:1].clone())
    total.copy_(glob.to(dt))
    rows_off = torch.tensor([sum(counts[:r]) for r in range(world)], dtype=torch.int64, device=dev)
    cur = 0
    ends0, my_offset = dist.shard_prefix(local_tot)                  # float64
    ends = ends0.contiguous().clone()                                # (world,) inclusive prefix of the shares
    offset = my_offset.reshape(1).contiguous().clone()               # this shard's exclusive prefix
    cand_glob = torch.empty(t, dtype=torch.int32, device=dev)
    rows_glob = torch.empty((t, d), dtype=dt, device=dev)
    for c in range(1, k):
        nxt = 1 - cur
        check(lib.kmb_kpp_sample(code, ptr(M[cur]), ptr(bsum[cur]), ptr(best), ptr(total),
                                 ptr(u[c - 1]), ptr(offset), t, ptr(cand), n, s), "kmb_kpp_sample")
        check(lib.kmb_gather_rows(code, ptr(X), ptr(cand), t, d, ptr(cand_rows), s),
              "kmb_gather_rows")
        # ONE all-gather of (row, local id) per trial; the owner of trial tau (first shard whose
        # inclusive prefix reaches r = u * total) is picked out of it by one kernel
        id_col = cand.view(torch.float32) if dt == torch.float32 else cand.to(dt)
        gathered = dist.all_gather_same(torch.cat([cand_rows, id_col.reshape(t, 1)], dim=1)
                                        .reshape(1, t, d + 1))
        check(lib.kmb_kpp_pick_owned(code, ptr(gathered), world, t, d, ptr(ends), ptr(u[c - 1]),
                                     ptr(total), ptr(rows_off), ptr(cand_glob), ptr(rows_glob), s),
              "kmb_kpp_pick_owned")
        check(lib.kmb_kpp_step(code, ptr(X), ptr(w), ptr(rows_glob), ptr(M[cur]), ptr(best),
                               ptr(M[nxt]), ptr(bsum[nxt]), n, d, t, s), "kmb_kpp_step")
        check(lib.kmb_kpp_potentials(ptr(bsum[nxt]), t, nb, ptr(pots64), s), "kmb_kpp_potentials")
        # one all-gather of every shard's t potentials serves two purposes: their sum over the
        # shards (the same fixed order on every rank) is what the choice is made on, and the
        # chosen candidate's column holds the shares the next round's sampler needs
        shard_pots = dist.all_gather_same(pots64.reshape(1, t))      # (world, t)
        check(lib.kmb_kpp_select_shards(code, ptr(shard_pots), world, me, t, ptr(pots), ptr(best),
                                        ptr(total), ptr(rows_glob), ptr(cand_glob), ptr(centers),
                                        ptr(indices), c, d, ptr(ends), ptr(offset), s),
              "kmb_kpp_select_shards")
        cur = nxt
    return centers.T, indices
