"""TEST INFRASTRUCTURE ONLY -- ctypes front end of the CPU checkers.

Only tests/, the smoke test and the CPU-baseline leg of the benchmark may import this module;
the product package (tensorplay_b200) never does.

Three checkers live here:

* ``reduce`` / ``topk`` / ``topk_sort``: the plain-C restatement in tp_oracle.c
  (libtporacle.so), bit-identical to TensorPlay's CPU kernels
  (p10/src/backend/cpu/ReductionKernels.cpp:72-855); top-k: parity unpinned (the reference has
  no top-k; the contract is held by self-consistency only, see tp_oracle.c);
* ``ref_reduce``: the reference's own compiled CPU path (oracle/_ref/libtpref.so, built by
  build_ref.sh where a TensorPlay checkout exists), used to validate the restatement and as
  the timed CPU baseline;
* ``truth64``: a float64 numpy evaluation of the same reductions, the accuracy anchor for
  sum / mean / var / std.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

OPS = {"sum": 0, "mean": 1, "var": 2, "std": 3, "max": 4, "min": 5, "argmax": 6, "argmin": 7,
       "prod": 8, "norm": 9, "all": 10, "any": 11}
_MORE = ("prod", "norm", "all", "any")
_I64P = ctypes.POINTER(ctypes.c_int64)
_F32P = ctypes.POINTER(ctypes.c_float)

_lib = None
_ref = None


def reference_env() -> dict:
    """Environment for the build scripts: TP_REFERENCE_ROOT names the TensorPlay checkout; when it is
    not set, a checkout in a directory `reference` beside this repository is used if there is one."""
    env = dict(os.environ)
    if not env.get("TP_REFERENCE_ROOT"):
        sibling = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
        if os.path.isfile(os.path.join(sibling, "p10", "src", "backend", "cpu", "ReductionKernels.cpp")):
            env["TP_REFERENCE_ROOT"] = sibling
    return env


def build(force: bool = False) -> None:
    """Compile libtporacle.so (and the reference path when its sources are present)."""
    so = os.path.join(_HERE, "libtporacle.so")
    src = os.path.join(_HERE, "tp_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libtporacle.so"], stdout=subprocess.DEVNULL)
    subprocess.check_call(["bash", os.path.join(_HERE, "build_ref.sh")], stdout=subprocess.DEVNULL, env=reference_env())


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        so = os.path.join(_HERE, "libtporacle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        L.tpo_reduce.restype = ctypes.c_int
        L.tpo_reduce.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, _I64P, _I64P, ctypes.c_int,
                                 _I64P, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        L.tpo_reduce_more.restype = ctypes.c_int
        L.tpo_reduce_more.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, _I64P, _I64P, ctypes.c_int,
                                      _I64P, ctypes.c_double, ctypes.c_void_p]
        L.tpo_out_numel.restype = ctypes.c_int64
        L.tpo_out_numel.argtypes = [ctypes.c_int, _I64P, ctypes.c_int, _I64P]
        for f in (L.tpo_topk, L.tpo_topk_sort):
            f.restype = ctypes.c_int
            f.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                          ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.tpo_softmax.restype = ctypes.c_int
        L.tpo_softmax.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
        L.tpo_median.restype = ctypes.c_int
        L.tpo_median.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libtpref.so"))


def ref() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        L = ctypes.CDLL(os.path.join(_HERE, "_ref", "libtpref.so"))
        L.tpref_reduce.restype = ctypes.c_int
        L.tpref_reduce.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, _I64P, _I64P, ctypes.c_int,
                                   _I64P, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_int64]
        L.tpref_reduce_more.restype = ctypes.c_int
        L.tpref_reduce_more.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, _I64P, _I64P, ctypes.c_int,
                                        _I64P, ctypes.c_int, ctypes.c_double, ctypes.c_void_p, ctypes.c_int64]
        L.tpref_last_error.restype = ctypes.c_char_p
        L.tpref_softmax.restype = ctypes.c_int
        L.tpref_softmax.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, _I64P, _I64P, ctypes.c_int64,
                                    ctypes.c_void_p, ctypes.c_int64]
        L.tpref_median.restype = ctypes.c_int
        L.tpref_median.argtypes = [ctypes.c_void_p, ctypes.c_int, _I64P, _I64P, ctypes.c_void_p]
        _ref = L
    return _ref


def _arr(v):
    a = (ctypes.c_int64 * max(1, len(v)))(*v)
    return a


def _norm_dims(dims, ndim):
    if dims is None:
        return None
    if isinstance(dims, int):
        dims = [dims]
    return [int(d) for d in dims]


def out_shape(shape, dims, keepdim=False):
    nd = len(shape)
    if dims is None or len(dims) == 0:
        red = set(range(nd))
    else:
        red = {d % nd if nd else 0 for d in dims}
    o = []
    for i, s in enumerate(shape):
        if i in red:
            if keepdim:
                o.append(1)
        else:
            o.append(s)
    return tuple(o)


def _prep(x):
    assert x.dtype == np.float32
    sizes = list(x.shape)
    strides = [s // 4 for s in x.strides]
    return sizes, strides


def reduce(op: str, x: np.ndarray, dims=None, keepdim: bool = False, correction: int = 1, p: float = 2.0):
    """C restatement.  dims=None is the overload without a dim argument.  `p` is norm's exponent."""
    dims = _norm_dims(dims, x.ndim)
    sizes, strides = _prep(x)
    oshape = out_shape(x.shape, dims, keepdim)
    n_out = int(np.prod(oshape, dtype=np.int64)) if len(oshape) else 1
    if op in _MORE:
        out = np.empty(max(n_out, 1), dtype=np.uint8 if op in ("all", "any") else np.float32)
        rc = lib().tpo_reduce_more(OPS[op], x.ctypes.data, x.ndim, _arr(sizes), _arr(strides),
                                   -1 if dims is None else len(dims), _arr(dims or []), float(p), out.ctypes.data)
        if rc == -2:
            raise RuntimeError("Dimension out of range")
        if rc == -3:
            raise RuntimeError(("max" if p > 0 else "min") + "(): Expected reduction dim to be non-empty")
        if rc != 0:
            raise RuntimeError(f"tpo_reduce_more failed: {rc}")
        out = out[:n_out].reshape(oshape)
        return out.astype(bool) if op in ("all", "any") else out
    is_idx = op in ("argmax", "argmin")
    out = np.empty(max(n_out, 1), dtype=np.int64 if is_idx else np.float32)
    nd = -1 if dims is None else len(dims)
    rc = lib().tpo_reduce(OPS[op], x.ctypes.data, x.ndim, _arr(sizes), _arr(strides), nd,
                          _arr(dims or []), int(correction),
                          None if is_idx else out.ctypes.data, out.ctypes.data if is_idx else None)
    if rc == -2:
        raise RuntimeError("Dimension out of range")
    if rc == -3:
        raise RuntimeError(f"{op}(): Expected reduction dim to be non-empty")
    if rc != 0:
        raise RuntimeError(f"tpo_reduce failed: {rc}")
    return out[:n_out].reshape(oshape)


def ref_reduce(op: str, x: np.ndarray, dims=None, keepdim: bool = False, correction: int = 1, p: float = 2.0):
    """The reference's own compiled CPU code (requires oracle/_ref/libtpref.so)."""
    dims = _norm_dims(dims, x.ndim)
    sizes, strides = _prep(x)
    oshape = out_shape(x.shape, dims, keepdim)
    n_out = int(np.prod(oshape, dtype=np.int64)) if len(oshape) else 1
    if op in _MORE:
        out = np.empty(max(n_out, 1), dtype=np.uint8 if op in ("all", "any") else np.float32)
        L = ref()
        rc = L.tpref_reduce_more(OPS[op], x.ctypes.data, x.ndim, _arr(sizes), _arr(strides),
                                 -1 if dims is None else len(dims), _arr(dims or []), int(keepdim), float(p),
                                 out.ctypes.data, n_out)
        if rc != 0:
            raise RuntimeError(L.tpref_last_error().decode())
        out = out[:n_out].reshape(oshape)
        return out.astype(bool) if op in ("all", "any") else out
    is_idx = op in ("argmax", "argmin")
    out = np.empty(max(n_out, 1), dtype=np.int64 if is_idx else np.float32)
    nd = -1 if dims is None else len(dims)
    L = ref()
    rc = L.tpref_reduce(OPS[op], x.ctypes.data, x.ndim, _arr(sizes), _arr(strides), nd, _arr(dims or []),
                        int(keepdim), int(correction), None if is_idx else out.ctypes.data,
                        out.ctypes.data if is_idx else None, n_out)
    if rc != 0:
        raise RuntimeError(L.tpref_last_error().decode())
    return out[:n_out].reshape(oshape)


def _topk(fn, x: np.ndarray, k: int, dim: int, largest: bool):
    assert x.dtype == np.float32
    dim = dim % x.ndim
    xm = np.moveaxis(x, dim, -1)
    xm = np.ascontiguousarray(xm)
    L = xm.shape[-1]
    rows = xm.size // L if L else 0
    vals = np.empty((rows, k), dtype=np.float32)
    idx = np.empty((rows, k), dtype=np.int64)
    rc = fn(xm.ctypes.data, rows, L, L, 1, k, int(bool(largest)), vals.ctypes.data, idx.ctypes.data)
    if rc != 0:
        raise RuntimeError("selected index k out of range")
    oshape = xm.shape[:-1] + (k,)
    return (np.moveaxis(vals.reshape(oshape), -1, dim), np.moveaxis(idx.reshape(oshape), -1, dim))


def topk(x, k, dim=-1, largest=True):
    """Selection form (heap scan + sort of the survivors)."""
    return _topk(lib().tpo_topk, x, k, dim, largest)


def topk_sort(x, k, dim=-1, largest=True):
    """Definition form (stable sort of every row)."""
    return _topk(lib().tpo_topk_sort, x, k, dim, largest)


def truth64(op: str, x: np.ndarray, dims=None, keepdim: bool = False, correction: int = 1, p: float = 2.0):
    """float64 evaluation with numpy (pairwise summation in double): the accuracy anchor."""
    dims = _norm_dims(dims, x.ndim)
    ax = None if dims is None or len(dims) == 0 else tuple(d % x.ndim for d in dims)
    x64 = x.astype(np.float64)
    if op == "prod":
        return x64.prod(axis=ax, keepdims=keepdim)
    if op == "norm":
        a = np.abs(x64)
        if np.isinf(p):
            return a.max(axis=ax, keepdims=keepdim) if p > 0 else a.min(axis=ax, keepdims=keepdim)
        return (a ** p).sum(axis=ax, keepdims=keepdim) ** (1.0 / p)
    if op == "sum":
        return x64.sum(axis=ax, keepdims=keepdim)
    if op == "mean":
        return x64.mean(axis=ax, keepdims=keepdim)
    if op in ("var", "std"):
        n = x.size if ax is None else int(np.prod([x.shape[a] for a in ax]))
        m = x64.mean(axis=ax, keepdims=True)
        ssq = ((x64 - m) ** 2).sum(axis=ax, keepdims=keepdim)
        with np.errstate(divide="ignore", invalid="ignore"):
            v = ssq / max(0, n - correction)
        return np.sqrt(v) if op == "std" else v
    raise ValueError(op)


def softmax(x: np.ndarray, dim: int, log: bool = False) -> np.ndarray:
    """C restatement of softmax / log_softmax along `dim` (float32 chain of the reference)."""
    assert x.dtype == np.float32 and x.ndim >= 1
    d = dim % x.ndim
    xc = np.ascontiguousarray(x)
    outer = int(np.prod(x.shape[:d], dtype=np.int64))
    inner = int(np.prod(x.shape[d + 1:], dtype=np.int64))
    out = np.empty_like(xc)
    rc = lib().tpo_softmax(int(log), xc.ctypes.data, outer, x.shape[d], inner, out.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"tpo_softmax failed: {rc}")
    return out


def ref_softmax(x: np.ndarray, dim: int, log: bool = False) -> np.ndarray:
    """The reference's own compiled CPU softmax / log_softmax."""
    sizes, strides = _prep(x)
    out = np.empty(x.shape, dtype=np.float32)
    L = ref()
    rc = L.tpref_softmax(int(log), x.ctypes.data, x.ndim, _arr(sizes), _arr(strides), int(dim), out.ctypes.data, out.size)
    if rc != 0:
        raise RuntimeError(L.tpref_last_error().decode())
    return out


def median(x: np.ndarray) -> np.float32:
    """C restatement of the whole-tensor median (NaNs rank last)."""
    xc = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.empty(1, dtype=np.float32)
    rc = lib().tpo_median(xc.ctypes.data, xc.size, out.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"tpo_median failed: {rc}")
    return out[0]


def ref_median(x: np.ndarray) -> np.float32:
    sizes, strides = _prep(x)
    out = np.empty(1, dtype=np.float32)
    L = ref()
    rc = L.tpref_median(x.ctypes.data, x.ndim, _arr(sizes), _arr(strides), out.ctypes.data)
    if rc != 0:
        raise RuntimeError(L.tpref_last_error().decode())
    return out[0]


def truth64_softmax(x: np.ndarray, dim: int, log: bool = False) -> np.ndarray:
    x64 = x.astype(np.float64)
    m = x64.max(axis=dim, keepdims=True)
    e = np.exp(x64 - m)
    s = e.sum(axis=dim, keepdims=True)
    return (x64 - m) - np.log(s) if log else e / s
