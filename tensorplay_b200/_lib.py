"""ctypes binding of libtpb200.so (the C ABI declared in include/tpb200.h).

There is no fallback: if the shared library is missing or fails to load, importing an operator
raises.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# TPB200_CHECKED=1 in the environment selects the range-checking build of the same sources
# (libtpb200_checked.so: see "checked build" in include/tpb200.h); it must exist, nothing falls back.
CHECKED = os.environ.get("TPB200_CHECKED", "") not in ("", "0")
# TPB200_TRACE=1 selects the development build with phase stamps (tensorplay_b200/trace.py reads them)
TRACE = not CHECKED and os.environ.get("TPB200_TRACE", "") not in ("", "0")
LIB_PATH = os.path.join(_PKG, "libtpb200_checked.so" if CHECKED else ("libtpb200_trace.so" if TRACE else "libtpb200.so"))

# error codes of include/tpb200.h
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_DIM_RANGE, ERR_EMPTY, ERR_WORKSPACE, ERR_CUDA = range(7)
F32 = 0
OP = {"sum": 0, "mean": 1, "var": 2, "std": 3, "max": 4, "min": 5, "argmax": 6, "argmin": 7,
      "max_argmax": 8, "min_argmin": 9, "prod": 10, "norm1": 11, "norm2": 12, "norm_inf": 13,
      "norm_neg_inf": 14, "all": 15, "any": 16}
PARTIAL_BYTES = 40
MAX_DIMS = 8

# every symbol include/tpb200.h declares
SYMBOLS = [
    "tpb200_last_error", "tpb200_version", "tpb200_reduce", "tpb200_reduce_workspace_bytes",
    "tpb200_topk", "tpb200_topk_workspace_bytes", "tpb200_reduce_partial",
    "tpb200_reduce_partial_workspace_bytes", "tpb200_reduce_combine", "tpb200_topk_merge",
    "tpb200_device_status", "tpb200_check_report", "tpb200_check_trim_next", "tpb200_reduce_all_noalloc", "tpb200_exchange_buffer_bytes",
    "tpb200_reduce_fused_exchange", "tpb200_topk_plan_info", "tpb200_set_exchange_wait_polls",
    "tpb200_softmax", "tpb200_median", "tpb200_median_workspace_bytes",
    "tpb200_comm_create", "tpb200_comm_destroy", "tpb200_comm_size", "tpb200_comm_fused", "tpb200_comm_stream",
    "tpb200_comm_synchronize", "tpb200_comm_result_values", "tpb200_comm_result_indices",
    "tpb200_reduce_sharded", "tpb200_topk_sharded", "tpb200_strided_copy",
]

_I64P = ctypes.POINTER(ctypes.c_int64)
_lib = None


class Tpb200Error(RuntimeError):
    """A non-zero status from the C ABI; .code holds the TPB200_ERR_* value."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tensorplay_b200.build{' --checked' if CHECKED else (' --trace' if TRACE else '')}` "
            "(needs nvcc; there is no CPU or PyTorch fallback)")
    L = ctypes.CDLL(LIB_PATH)
    vp, i, i64, u64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t
    L.tpb200_last_error.restype = ctypes.c_char_p
    L.tpb200_last_error.argtypes = []
    L.tpb200_version.restype = i
    L.tpb200_version.argtypes = []
    L.tpb200_check_report.restype = i
    L.tpb200_check_report.argtypes = [_I64P, i]
    L.tpb200_check_trim_next.restype = i
    L.tpb200_check_trim_next.argtypes = [i64]
    L.tpb200_reduce.restype = i
    L.tpb200_reduce.argtypes = [i, vp, i, i, _I64P, _I64P, u64, i, i64, vp, vp, vp, sz, vp]
    L.tpb200_reduce_workspace_bytes.restype = sz
    L.tpb200_reduce_workspace_bytes.argtypes = [i, i, i, _I64P, _I64P, u64]
    L.tpb200_topk.restype = i
    L.tpb200_topk.argtypes = [vp, i, i, _I64P, _I64P, i, i64, i, i, vp, vp, vp, sz, vp]
    L.tpb200_topk_workspace_bytes.restype = sz
    L.tpb200_topk_workspace_bytes.argtypes = [i, i, _I64P, _I64P, i, i64]
    L.tpb200_reduce_partial.restype = i
    L.tpb200_reduce_partial.argtypes = [i, vp, i, i64, i64, vp, vp, sz, vp]
    L.tpb200_reduce_partial_workspace_bytes.restype = sz
    L.tpb200_reduce_partial_workspace_bytes.argtypes = [i, i, i64]
    L.tpb200_reduce_combine.restype = i
    L.tpb200_reduce_combine.argtypes = [i, vp, i, i64, i64, vp, vp, vp]
    L.tpb200_topk_merge.restype = i
    L.tpb200_topk_merge.argtypes = [vp, vp, i64, i64, i, vp, i64, vp, vp, vp]
    L.tpb200_reduce_all_noalloc.restype = i
    L.tpb200_reduce_all_noalloc.argtypes = [i, vp, i, i64, i64, vp, vp, vp]
    L.tpb200_exchange_buffer_bytes.restype = sz
    L.tpb200_exchange_buffer_bytes.argtypes = []
    L.tpb200_reduce_fused_exchange.restype = i
    L.tpb200_reduce_fused_exchange.argtypes = [i, vp, i, i64, i64, i64, i64, i, i, ctypes.POINTER(ctypes.c_void_p), vp, vp, vp, sz, vp]
    L.tpb200_softmax.restype = i
    L.tpb200_softmax.argtypes = [i, vp, i, i, _I64P, _I64P, i, vp, vp]
    L.tpb200_median.restype = i
    L.tpb200_median.argtypes = [vp, i, i, _I64P, _I64P, vp, vp, sz, vp]
    L.tpb200_median_workspace_bytes.restype = sz
    L.tpb200_median_workspace_bytes.argtypes = []
    vpp = ctypes.POINTER(vp)
    L.tpb200_comm_create.restype = i
    L.tpb200_comm_create.argtypes = [i, ctypes.POINTER(i), vpp]
    L.tpb200_comm_destroy.restype = i
    L.tpb200_comm_destroy.argtypes = [vp]
    L.tpb200_comm_size.restype = i
    L.tpb200_comm_size.argtypes = [vp]
    L.tpb200_comm_fused.restype = i
    L.tpb200_comm_fused.argtypes = [vp]
    L.tpb200_comm_stream.restype = vp
    L.tpb200_comm_stream.argtypes = [vp, i]
    L.tpb200_comm_synchronize.restype = i
    L.tpb200_comm_synchronize.argtypes = [vp]
    L.tpb200_comm_result_values.restype = vp
    L.tpb200_comm_result_values.argtypes = [vp, i]
    L.tpb200_comm_result_indices.restype = vp
    L.tpb200_comm_result_indices.argtypes = [vp, i]
    L.tpb200_reduce_sharded.restype = i
    L.tpb200_reduce_sharded.argtypes = [vp, i, vpp, _I64P, i, i64, vpp, vpp]
    L.tpb200_topk_sharded.restype = i
    L.tpb200_topk_sharded.argtypes = [vp, vpp, _I64P, i, i64, i, vpp, vpp]
    L.tpb200_strided_copy.restype = i
    L.tpb200_strided_copy.argtypes = [vp, _I64P, vp, _I64P, i, i, _I64P, vp]
    L.tpb200_set_exchange_wait_polls.restype = i
    L.tpb200_set_exchange_wait_polls.argtypes = [i]
    L.tpb200_topk_plan_info.restype = i
    L.tpb200_topk_plan_info.argtypes = [i, i, _I64P, _I64P, i, i64, _I64P, i]
    L.tpb200_device_status.restype = i
    L.tpb200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    _lib = L
    return L


def i64_array(values):
    n = max(1, len(values))
    return (ctypes.c_int64 * n)(*values)


def check(rc: int) -> None:
    """Map a C status to the exception the reference raises for the same condition
    (p10/include/Exception.h:20-43; messages at p10/src/backend/cpu/ReductionKernels.cpp:55-57,240)."""
    if rc == OK:
        return
    msg = lib().tpb200_last_error().decode()
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise Tpb200Error(rc, msg)


PLAN_FIELDS = ("scan_kernel", "scan_slices", "scan_warps", "select", "select_ctas_per_row", "select_warps",
               "select_rank", "select_cap", "select_sample_tiles", "launches", "workspace_bytes")


def topk_plan_info(sizes, strides, dim: int, k: int) -> dict:
    """The planner's choice for a top-k call on a float32 tensor of these sizes / strides."""
    info = (ctypes.c_int64 * len(PLAN_FIELDS))()
    check(lib().tpb200_topk_plan_info(F32, len(sizes), i64_array(list(sizes)), i64_array(list(strides)), dim, k,
                                      info, len(PLAN_FIELDS)))
    return dict(zip(PLAN_FIELDS, [int(v) for v in info]))


CHECK_INFO = ("checked_build", "violations", "file", "line", "address", "bytes")


def check_report() -> dict:
    """Synchronise and return (then clear) the checked build's record: how many accesses fell outside
    the ranges registered for their call, and where the first one was (file id, line, address, size).
    In the ordinary build "checked_build" is 0 and the rest is zero."""
    info = (ctypes.c_int64 * len(CHECK_INFO))()
    check(lib().tpb200_check_report(info, len(CHECK_INFO)))
    return dict(zip(CHECK_INFO, (int(v) for v in info)))


def check_trim_next(nbytes: int) -> None:
    """The checker's own test (checked build only): the next call registers every range `nbytes`
    shorter at its end."""
    check(lib().tpb200_check_trim_next(int(nbytes)))


def device_status() -> int:
    """Synchronise and return (then clear) the per-device status word; 0 = every kernel finished
    its waits."""
    v = ctypes.c_int(0)
    check(lib().tpb200_device_status(ctypes.byref(v)))
    return v.value
