"""ctypes binding of libkmb200.so (declared in include/kmb200.h).

The library is the product; there is no other back end.  If it is missing the import
fails with the build command, it never falls back to another implementation.
"""
import ctypes
import os
from ctypes import (POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_uint32, c_uint64, c_void_p)

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkmb200.so")

KMB_F32, KMB_F64 = 0, 1
KMB_OK, KMB_ERR_INVALID, KMB_ERR_CUDA, KMB_ERR_UNSUPPORTED, KMB_ERR_WORKSPACE = 0, -1, -2, -3, -4
ALGO_AUTO, ALGO_CUDA_CORE, ALGO_TF32X3 = 0, 1, 2
ALGO_NAMES = {"auto": ALGO_AUTO, "cuda_core": ALGO_CUDA_CORE, "tf32x3": ALGO_TF32X3}
STEP_ACC_CLEARED, STEP_OPERANDS_READY = 1, 2
FIN_MERGE, FIN_CLEAR_ACC, FIN_PREPARE_TF32X3 = 1, 2, 4


class KmbError(RuntimeError):
    """A kmb200 call failed inside CUDA or on its workspace."""


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA kernels are not built. Run "
            "`python -m sklearn_numba_dpex_b200.build` (needs nvcc); there is no fallback."
        )
    return ctypes.CDLL(LIB_PATH)


lib = _load()

_P = c_void_p
_SIGNATURES = {
    "kmb_last_error": (c_char_p, []),
    "kmb_version": (c_int, []),
    "kmb_device_info": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "kmb_host_device_pointer": (c_int, [_P, POINTER(c_void_p)]),
    "kmb_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "kmb_lloyd_acc_len": (c_int64, [c_int, c_int]),
    "kmb_lloyd_acc_copies": (c_int, [c_int, c_int, c_int64, c_int, c_int]),
    "kmb_lloyd_resolve_algo": (c_int, [c_int, c_int, c_int64, c_int, c_int]),
    "kmb_half_l2_norm": (c_int, [c_int, _P, _P, c_int, c_int, _P]),
    "kmb_lloyd_workspace_init": (c_int, [_P, c_size_t, _P]),
    "kmb_lloyd_step": (c_int, [c_int, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, c_int64, c_int,
                               c_int, c_int, _P, c_size_t, _P]),
    "kmb_lloyd_wait_error": (c_int, [_P, POINTER(c_int), _P]),
    "kmb_lloyd_merge_copies": (c_int, [c_int, _P, c_int, c_int64, _P, c_int, _P]),
    "kmb_lloyd_finalize": (c_int, [c_int, _P, c_int, _P, c_int, _P, _P, _P, _P, _P, _P, c_int,
                                   c_int, _P, c_size_t, _P]),
    "kmb_assign_labels": (c_int, [c_int, c_int, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P,
                                  c_size_t, _P]),
    "kmb_inertia": (c_int, [c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, _P, c_size_t,
                            _P]),
    "kmb_euclidean_distances": (c_int, [c_int, _P, _P, _P, c_int64, c_int, c_int, c_int64, _P]),
    "kmb_relocate_empty_clusters": (c_int, [c_int, _P, _P, _P, c_int64, _P, _P, c_int, _P, _P, c_int,
                                            c_int, _P]),
    "kmb_topk": (c_int, [c_int, _P, c_int, c_int64, c_int, _P, _P, _P, c_size_t, _P]),
    "kmb_topk_workspace_bytes": (c_size_t, [c_int, c_int64, c_int]),
    "kmb_topk_idx_static": (c_int, [c_int, _P, c_int64, c_int, _P, _P]),
    "kmb_kpp_block_rows": (c_int, []),
    "kmb_kpp_init": (c_int, [c_int, _P, _P, c_int64, _P, _P, _P, _P, _P, c_int64, c_int, _P]),
    "kmb_kpp_sample": (c_int, [c_int, _P, _P, _P, _P, _P, _P, c_int, _P, c_int64, _P]),
    "kmb_gather_rows": (c_int, [c_int, _P, _P, c_int, c_int, _P, _P]),
    "kmb_kpp_step": (c_int, [c_int, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, _P]),
    "kmb_kpp_potentials": (c_int, [_P, c_int, c_int64, _P, _P]),
    "kmb_kpp_pick_owned": (c_int, [c_int, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P]),
    "kmb_kpp_select_shards": (c_int, [c_int, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, c_int,
                                      c_int, _P, _P, _P]),
    "kmb_kpp_select": (c_int, [c_int, _P, _P, c_int, c_int64, _P, _P, _P, _P, _P, _P, _P, c_int,
                               c_int, _P]),
    "kmb_col_sums": (c_int, [c_int, _P, c_int64, c_int, _P, _P, c_size_t, _P]),
    "kmb_sum": (c_int, [c_int, _P, c_int64, c_int, _P, _P, c_size_t, _P]),
    "kmb_add_row_vector": (c_int, [c_int, _P, c_int64, c_int, _P, c_double, _P]),
    "kmb_same_clustering": (c_int, [_P, _P, c_int64, c_int, _P, _P, _P]),
    "kmb_count_distinct": (c_int, [_P, c_int64, c_int, _P, _P, _P]),
    "kmb_xoroshiro_init": (c_int, [POINTER(c_uint64), c_int, c_uint64, c_int]),
    "kmb_xoroshiro_next": (c_uint64, [POINTER(c_uint64), c_int]),
    "kmb_u64_to_unit_f32": (c_float, [c_uint64]),
    "kmb_u64_to_unit_f64": (c_double, [c_uint64]),
    "kmb_measure_fma_peak": (c_int, [c_int, c_int, POINTER(c_double), _P, _P]),
    "kmb_matmul_nt": (c_int, [c_int, c_int, _P, _P, _P, c_int64, c_int, c_int, _P, c_size_t, _P]),
}

class LloydPlan(ctypes.Structure):
    """kmb_lloyd_plan of include/kmb200.h."""
    _fields_ = [("dtype", c_int32), ("algo", c_int32), ("d", c_int32), ("k", c_int32),
                ("n_copies", c_int32), ("reserved", c_int32), ("n", c_int64),
                ("X", c_void_p), ("w", c_void_p), ("C", c_void_p * 3), ("h", c_void_p * 3),
                ("labels", c_void_p * 2), ("acc", c_void_p), ("merged", c_void_p * 2),
                ("shifts", c_void_p), ("empty_list", c_void_p * 2), ("status", c_void_p * 2),
                ("workspace", c_void_p), ("workspace_bytes", c_size_t)]


_SIGNATURES["kmb_lloyd_plan_launch"] = (c_int, [POINTER(LloydPlan), c_int64, c_int, _P, _P, _P, _P])
PLAN_HAVE_PREV, PLAN_OPERANDS_READY = 1, 2


def pad_features_flag(n_pad):
    """KMB_LLOYD_PAD_FEATURES(n): bits 8-9 of the flags of the step, finalize and plan calls."""
    if not 0 <= int(n_pad) <= 3:
        raise ValueError("the number of padding features must be 0..3")
    return (int(n_pad) & 3) << 8

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error():
    msg = lib.kmb_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status, what=""):
    """Turns a negative kmb_status into the exception the reference would raise for the
    same mistake: ValueError for bad arguments, NotImplementedError for unsupported
    requests, KmbError for CUDA / workspace failures."""
    if status >= 0:
        return status
    msg = f"{what}: {last_error()}" if what else last_error()
    if status == KMB_ERR_INVALID:
        raise ValueError(msg)
    if status == KMB_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise KmbError(msg)


def dtype_code(torch_dtype):
    if torch_dtype == torch.float32:
        return KMB_F32
    if torch_dtype == torch.float64:
        return KMB_F64
    raise ValueError(f"Expected float32 or float64 data but got {torch_dtype}")


def ptr(t):
    """Device (or host) address of a tensor's first element; None -> NULL."""
    if t is None:
        return None
    return c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda_tensor(t, name, dtype=None, contiguous=True):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


class Workspace:
    """One scratch buffer per (device) reused by every call; grows on demand."""

    _cache = {}

    @classmethod
    def get(cls, device, nbytes):
        key = (device.type, device.index)
        buf = cls._cache.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(int(nbytes) + 256, dtype=torch.uint8, device=device)
            cls._cache[key] = buf
        return buf


def workspace_for(device, n, d, k):
    """The shared scratch buffer of `device`, large enough for any call on these sizes.  Its
    contents do not survive the next call that uses it."""
    nbytes = lib.kmb_workspace_bytes(int(n), int(d), int(k))
    buf = Workspace.get(device, nbytes)
    return buf, buf.numel()


def lloyd_workspace(device, n, d, k, own=False):
    """A workspace for the Lloyd entry points with its control block cleared: the shared
    buffer, or (own=True) a buffer of its own whose tensor-core operands and time-out flag
    persist between calls."""
    if own:
        nbytes = lib.kmb_workspace_bytes(int(n), int(d), int(k))
        buf = torch.empty(int(nbytes) + 256, dtype=torch.uint8, device=device)
    else:
        buf, _ = workspace_for(device, n, d, k)
    check(lib.kmb_lloyd_workspace_init(ptr(buf), buf.numel(), stream_ptr(device)),
          "kmb_lloyd_workspace_init")
    return buf, buf.numel()


def host_device_pointer(pinned_tensor):
    """Device address of a page-locked host tensor (for records a kernel writes directly)."""
    if pinned_tensor.is_cuda or not pinned_tensor.is_pinned():
        raise ValueError("host_device_pointer needs a page-locked host tensor")
    out = c_void_p()
    check(lib.kmb_host_device_pointer(ptr(pinned_tensor), ctypes.byref(out)),
          "kmb_host_device_pointer")
    return out


def check_wait_error(ws, device):
    """Raises KmbError if a bounded wait of the tensor-core kernel ran out on `ws`."""
    flag = c_int(0)
    check(lib.kmb_lloyd_wait_error(ptr(ws), ctypes.byref(flag), stream_ptr(device)),
          "kmb_lloyd_wait_error")


def device_info(index=0):
    sm, major, minor = c_int(), c_int(), c_int()
    check(lib.kmb_device_info(index, ctypes.byref(sm), ctypes.byref(major), ctypes.byref(minor)))
    return sm.value, major.value, minor.value


STATUS_DTYPE = np.dtype([("n_empty", np.int32), ("changed", np.int32), ("shift_total", np.float64),
                         ("inertia", np.float64), ("wait_error", np.int32), ("reserved", np.int32)])
assert STATUS_DTYPE.itemsize == 32
