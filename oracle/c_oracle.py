"""ctypes front end of the C restatement (test infrastructure only)."""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None


def _load():
    global _lib
    if _lib is None:
        path = _build.build()   # rebuilds only when the source is newer than the library
        _lib = ctypes.CDLL(path)
        for name in ("oracle_lloyd_iter_f32", "oracle_lloyd_iter_f64"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int, ctypes.c_int] + \
                [ctypes.c_void_p] * 3 + [ctypes.c_int]
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads():
    return _load().oracle_num_threads()


def lloyd_iteration(X, w, C, update=True):
    """One E-step (+ accumulation) on all host threads.  X (n, d), C (k, d) C-contiguous.
    Returns (labels uint32, sums (k, d), counts (k,), threads_used)."""
    lib = _load()
    X = np.ascontiguousarray(X)
    T = X.dtype
    n, d = X.shape
    k = C.shape[0]
    Ct = np.ascontiguousarray(np.asarray(C, dtype=T).T)
    acc = np.zeros(k, dtype=T)
    for f in range(d):  # half norms: features in ascending order, then / 2
        acc += Ct[f] * Ct[f]
    h = (acc / T.type(2)).astype(T)
    labels = np.empty(n, dtype=np.uint32)
    sums = np.zeros((k, d), dtype=T)
    counts = np.zeros(k, dtype=T)
    wp = None if w is None else np.ascontiguousarray(w, dtype=T)
    fn = lib.oracle_lloyd_iter_f32 if T == np.float32 else lib.oracle_lloyd_iter_f64
    used = fn(X.ctypes.data, None if wp is None else wp.ctypes.data, Ct.ctypes.data, h.ctypes.data,
              n, d, k, labels.ctypes.data, sums.ctypes.data, counts.ctypes.data, int(update))
    if used < 0:
        raise MemoryError("oracle_lloyd_iter: allocation failed")
    return labels, sums, counts, used


def set_num_threads(count):
    """Fixes the OpenMP thread count of the following calls (launchers such as torchrun export
    OMP_NUM_THREADS=1, which would otherwise silently make this a one-thread program)."""
    lib = _load()
    lib.oracle_set_num_threads.argtypes = [ctypes.c_int]
    lib.oracle_set_num_threads.restype = None
    lib.oracle_set_num_threads(int(count))
    return lib.oracle_num_threads()


def lloyd(X, w, centers_init, max_iter=300, tol=1e-4):
    """The reference's Lloyd loop (kmeans/drivers.py:188-343: same stopping rules as
    oracle.reference_cpu.lloyd) with the E-step and the accumulation done by the C
    restatement, for cases too large for the numpy one.  Empty clusters are not handled here
    (the relocation path is the numpy oracle's): raises if one appears.
    Returns (labels, C, n_iter, shifts) where shifts lists the total squared shift of every
    iteration."""
    X = np.ascontiguousarray(X)
    T = X.dtype.type
    C = np.array(centers_init, dtype=X.dtype, copy=True)
    n_iter, shift, prev, armed, shifts = 0, np.inf, None, False, []
    while n_iter < max_iter and shift > tol:
        labels, sums, counts, _ = lloyd_iteration(X, w, C)
        if (counts == 0).any():
            raise RuntimeError("empty cluster: use oracle.reference_cpu.lloyd for this case")
        C_new = (sums / counts[:, None]).astype(X.dtype)
        changed = None if prev is None else int((labels != prev).sum())
        flag_set = armed and changed == 0
        prev = labels
        n_iter += 1
        C_old, C = C, C_new
        if n_iter > 1:
            if flag_set:
                break
            armed = True
        acc = np.zeros(C.shape[0], dtype=X.dtype)
        for f in range(C.shape[1]):
            diff = C_old[:, f] - C[:, f]
            acc += diff * diff
        shift = T(acc.sum(dtype=X.dtype))
        shifts.append(float(shift))
    labels, _, _, _ = lloyd_iteration(X, w, C, update=False)
    return labels, C, n_iter, shifts
