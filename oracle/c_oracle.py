"""ctypes front end of the C restatement (test infrastructure only)."""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None


def _load():
    global _lib
    if _lib is None:
        path = _build.LIB if os.path.exists(_build.LIB) else _build.build()
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
