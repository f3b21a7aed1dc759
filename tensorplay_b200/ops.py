"""Host-side mirror of TensorPlay's reduction operators on top of the tpb200 C ABI.

Names, argument meaning and error behaviour follow the reference's Tensor methods
(src/bindings/python/Tensor.cpp:1102-1225; schema config/native_functions.yaml:695-794):

    sum(x, dim=None, keepdim=False, *, dtype=None)      mean(...) likewise
    var(x, dim=None, correction=1, keepdim=False)       std(...) likewise
    max(x, dim=None, keepdim=False)  -> values only, as max.dim in the reference
    min(...)                            (native_functions.yaml:720-733)
    argmax(x, dim=None, keepdim=False)                  argmin(...) likewise
    prod(x, dim=None, keepdim=False, *, dtype=None)
    norm(x, p=2.0, dim=None, keepdim=False)             p in {1, 2, inf, -inf}
    all(x, dim=None, keepdim=False) / any(...)          -> bool tensor
    topk(x, k, dim=-1, largest=True, sorted=True) -> (values, indices)   [new operator]
    softmax(x, dim, dtype=None) / log_softmax(x, dim, dtype=None)
    median(x)                                            -> 0-dim tensor, whole tensor only
    copy_(dst, src)                                      strided float32 copy (Tensor.copy_ / contiguous())
    max_with_indices / min_with_indices(x, dim, keepdim=False) -> (values, indices), one pass

`dim` may be an int, a list of ints (sum/mean/var/std/max/min) or None.  Tensors are torch CUDA
tensors: torch is used for device memory and streams only; every number is produced by the
sm_100a kernels in libtpb200.so.  Strided views are consumed in place.
"""
from __future__ import annotations

import builtins as _py

import torch

from . import _lib

_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """Per (device, stream) scratch buffer, grown on demand and reused across calls."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(_py.max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check_input(x: torch.Tensor, what: str) -> None:
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"{what}: expected a tensor")
    if not x.is_cuda:
        raise RuntimeError(f"{what}: tpb200 kernels run on CUDA tensors only (got {x.device}); there is no CPU path")
    if x.dtype != torch.float32:
        raise NotImplementedError(f"{what} not implemented for this dtype ({x.dtype}); float32 only")
    if x.dim() > _lib.MAX_DIMS:
        raise NotImplementedError(f"{what}: tensors of rank {x.dim()} are not supported")


def _dims_mask(x: torch.Tensor, dim) -> tuple[int, list[int]]:
    """(reduce mask, normalised dims); mask 0 = whole tensor.  Out-of-range raises like
    compute_reduction_shape (p10/src/backend/cpu/ReductionKernels.cpp:48-58)."""
    if dim is None:
        return 0, list(range(x.dim()))
    dims = [dim] if isinstance(dim, int) else list(dim)
    if len(dims) == 0:
        return 0, list(range(x.dim()))
    nd = x.dim()
    out, mask = [], 0
    for d in dims:
        d = int(d)
        dd = d + nd if d < 0 else d
        if dd < 0 or dd >= nd:   # a 0-dim tensor has no valid dim, as in the reference
            raise RuntimeError("Dimension out of range")
        mask |= 1 << dd
        if dd not in out:
            out.append(dd)
    return mask, out


def _out_shape(x: torch.Tensor, dims: list[int], keepdim: bool) -> list[int]:
    shape = []
    for i, s in enumerate(x.shape):
        if i in dims:
            if keepdim:
                shape.append(1)
        else:
            shape.append(s)
    return shape


def _check_out(t, shape, dtype, device, what):
    if tuple(t.shape) != tuple(shape) or t.dtype != dtype or t.device != device or not t.is_contiguous():
        raise ValueError(f"{what}: out must be a contiguous {dtype} tensor of shape {tuple(shape)} on {device}")


def _reduce(op: str, x: torch.Tensor, dim, keepdim: bool, correction: int = 1, index_dim: int = -1, out=None):
    _check_input(x, op)
    mask, dims = _dims_mask(x, dim)
    L = _lib.lib()
    nd = x.dim()
    sizes = _lib.i64_array(list(x.shape))
    strides = _lib.i64_array(list(x.stride()))
    shape = _out_shape(x, dims, keepdim)
    want_val = op not in ("argmax", "argmin")
    want_idx = op in ("argmax", "argmin", "max_argmax", "min_argmin")
    val_dtype = torch.bool if op in ("all", "any") else torch.float32
    with torch.cuda.device(x.device):
        if out is not None:
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            ov = outs.pop(0) if want_val else None
            oi = outs.pop(0) if want_idx else None
            if ov is not None:
                _check_out(ov, shape, val_dtype, x.device, op)
            if oi is not None:
                _check_out(oi, shape, torch.int64, x.device, op)
        else:
            ov = torch.empty(shape, dtype=val_dtype, device=x.device) if want_val else None
            oi = torch.empty(shape, dtype=torch.int64, device=x.device) if want_idx else None
        nbytes = L.tpb200_reduce_workspace_bytes(_lib.OP[op], _lib.F32, nd, sizes, strides, mask)
        ws = _workspace(x.device, nbytes)
        rc = L.tpb200_reduce(
            _lib.OP[op], x.data_ptr(), _lib.F32, nd, sizes, strides, mask, index_dim, int(correction),
            ov.data_ptr() if want_val else None, oi.data_ptr() if want_idx else None,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc)
    if want_val and want_idx:
        return ov, oi
    return ov if want_val else oi


def _check_dtype(dtype, what):
    if dtype is not None and dtype != torch.float32:
        raise NotImplementedError(f"{what}: only dtype=float32 (or None) is supported")


def sum(x, dim=None, keepdim=False, *, dtype=None, out=None):
    _check_dtype(dtype, "sum")
    return _reduce("sum", x, dim, keepdim, out=out)


def mean(x, dim=None, keepdim=False, *, dtype=None, out=None):
    _check_dtype(dtype, "mean")
    return _reduce("mean", x, dim, keepdim, out=out)


def var(x, dim=None, correction=1, keepdim=False, *, out=None):
    return _reduce("var", x, dim, keepdim, correction, out=out)


def std(x, dim=None, correction=1, keepdim=False, *, out=None):
    return _reduce("std", x, dim, keepdim, correction, out=out)


def max(x, dim=None, keepdim=False, *, out=None):
    return _reduce("max", x, dim, keepdim, out=out)


def min(x, dim=None, keepdim=False, *, out=None):
    return _reduce("min", x, dim, keepdim, out=out)


def prod(x, dim=None, keepdim=False, *, dtype=None, out=None):
    """prod / prod.dim_IntList (config/native_functions.yaml:735-743)."""
    _check_dtype(dtype, "prod")
    return _reduce("prod", x, dim, keepdim, out=out)


def norm(x, p=2.0, dim=None, keepdim=False, *, out=None):
    """norm / norm.dim (config/native_functions.yaml:801-809).  The reference's CUDA path has
    p = 2 only (p10/src/backend/cuda/ReductionKernels.cu:296-321); its CPU path takes any p
    (p10/src/backend/cpu/ReductionKernels.cpp:858-872).  Here: p = 1, 2, inf, -inf."""
    p = float(p)
    op = {1.0: "norm1", 2.0: "norm2", float("inf"): "norm_inf", float("-inf"): "norm_neg_inf"}.get(p)
    if op is None:
        raise NotImplementedError("norm: only p = 1, 2, inf and -inf are supported")
    return _reduce(op, x, dim, keepdim, out=out)


def all(x, dim=None, keepdim=False, *, out=None):
    """all / all.dim (config/native_functions.yaml:756-764): bool result, true iff every element
    is non-zero."""
    return _reduce("all", x, dim, keepdim, out=out)


def any(x, dim=None, keepdim=False, *, out=None):
    """any / any.dim (config/native_functions.yaml:766-774)."""
    return _reduce("any", x, dim, keepdim, out=out)


def _arg(op, x, dim, keepdim, out=None):
    if dim is None:
        return _reduce(op, x, None, False, index_dim=-1, out=out)
    if not isinstance(dim, int):
        raise TypeError(f"{op}(): dim must be an int or None")
    nd = x.dim()
    d = dim + nd if dim < 0 else dim
    if d < 0 or d >= nd:
        raise RuntimeError("Dimension out of range")
    return _reduce(op, x, d, keepdim, index_dim=d, out=out)


def argmax(x, dim=None, keepdim=False, *, out=None):
    return _arg("argmax", x, dim, keepdim, out)


def argmin(x, dim=None, keepdim=False, *, out=None):
    return _arg("argmin", x, dim, keepdim, out)


def max_with_indices(x, dim, keepdim=False, *, out=None):
    """(max.dim values, argmax indices) from one pass over the input."""
    return _arg("max_argmax", x, dim, keepdim, out)


def min_with_indices(x, dim, keepdim=False, *, out=None):
    return _arg("min_argmin", x, dim, keepdim, out)


def topk(x, k, dim=-1, largest=True, sorted=True, *, out=None):
    """First k entries of each row along `dim`, stably sorted by value (descending if largest),
    ties in ascending index.  Returns (values float32, indices int64).  `out=(values, indices)`
    (contiguous, only for dim = last) makes the call allocation-free."""
    _check_input(x, "topk")
    nd = x.dim()
    d = dim + nd if dim < 0 else dim
    if d < 0 or d >= _py.max(nd, 1):
        raise RuntimeError("Dimension out of range")
    L = _lib.lib()
    sizes = _lib.i64_array(list(x.shape))
    strides = _lib.i64_array(list(x.stride()))
    shape = list(x.shape)
    if nd:
        shape[d] = int(k)
    with torch.cuda.device(x.device):
        if out is not None:
            if nd and d != nd - 1:
                raise ValueError("topk: out= is only supported for dim = last")
            ov, oi = out
            _check_out(ov, shape, torch.float32, x.device, "topk")
            _check_out(oi, shape, torch.int64, x.device, "topk")
        else:
            ov = torch.empty(shape, dtype=torch.float32, device=x.device)
            oi = torch.empty(shape, dtype=torch.int64, device=x.device)
        nbytes = L.tpb200_topk_workspace_bytes(_lib.F32, nd, sizes, strides, d, int(k))
        ws = _workspace(x.device, nbytes)
        # outputs are written as [rows..., k] with k innermost; move k back to `dim` afterwards
        inner_shape = [s for i, s in enumerate(x.shape) if i != d] + [int(k)]
        ov_c = ov if d == nd - 1 or nd == 0 else torch.empty(inner_shape, dtype=torch.float32, device=x.device)
        oi_c = oi if d == nd - 1 or nd == 0 else torch.empty(inner_shape, dtype=torch.int64, device=x.device)
        rc = L.tpb200_topk(
            x.data_ptr(), _lib.F32, nd, sizes, strides, d, int(k), int(bool(largest)), int(bool(sorted)),
            ov_c.data_ptr(), oi_c.data_ptr(), ws.data_ptr() if ws is not None else None,
            ws.numel() if ws is not None else 0, torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc)
    if ov_c is not ov:
        ov = ov_c.movedim(-1, d)
        oi = oi_c.movedim(-1, d)
    return ov, oi


def _softmax(log: bool, x, dim, dtype, out, what):
    _check_input(x, what)
    _check_dtype(dtype, what)
    nd = x.dim()
    if not isinstance(dim, int):
        raise TypeError(f"{what}(): dim must be an int")
    d = dim + nd if dim < 0 else dim
    if d < 0 or d >= nd:     # a 0-dim tensor has no valid dim
        raise RuntimeError("Dimension out of range")
    L = _lib.lib()
    with torch.cuda.device(x.device):
        if out is not None:
            _check_out(out, list(x.shape), torch.float32, x.device, what)
        else:
            out = torch.empty(list(x.shape), dtype=torch.float32, device=x.device)
        rc = L.tpb200_softmax(int(log), x.data_ptr(), _lib.F32, nd, _lib.i64_array(list(x.shape)),
                              _lib.i64_array(list(x.stride())), d, out.data_ptr(),
                              torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc)
    return out


def softmax(x, dim, dtype=None, *, out=None):
    """softmax (config/native_functions.yaml:587-591): exp(x - max) / sum along `dim`."""
    return _softmax(False, x, dim, dtype, out, "softmax")


def log_softmax(x, dim, dtype=None, *, out=None):
    """log_softmax (config/native_functions.yaml:593-597): (x - max) - log(sum exp(x - max))."""
    return _softmax(True, x, dim, dtype, out, "log_softmax")


def median(x, *, out=None):
    """median (config/native_functions.yaml:796-799): element (n - 1) / 2 of the sorted values of the
    whole tensor -- the lower middle one for even n -- as a 0-dim tensor; NaN for an empty tensor."""
    _check_input(x, "median")
    L = _lib.lib()
    with torch.cuda.device(x.device):
        if out is not None:
            _check_out(out, [], torch.float32, x.device, "median")
        else:
            out = torch.empty([], dtype=torch.float32, device=x.device)
        ws = _workspace(x.device, L.tpb200_median_workspace_bytes())
        rc = L.tpb200_median(x.data_ptr() if x.numel() else None, _lib.F32, x.dim(), _lib.i64_array(list(x.shape)),
                             _lib.i64_array(list(x.stride())), out.data_ptr(), ws.data_ptr(), ws.numel(),
                             torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc)
    return out


def copy_(dst, src):
    """dst.copy_(src) for two float32 CUDA views of the same shape with any strides (the reference's
    copy_ on CUDA: p10/src/backend/cuda/CopyKernels.cu:56-160); returns dst."""
    _check_input(src, "copy_")
    _check_input(dst, "copy_")
    if tuple(dst.shape) != tuple(src.shape) or dst.device != src.device:
        raise RuntimeError("Sizes do not match for copy")
    L = _lib.lib()
    with torch.cuda.device(src.device):
        rc = L.tpb200_strided_copy(dst.data_ptr(), _lib.i64_array(list(dst.stride())), src.data_ptr(),
                                   _lib.i64_array(list(src.stride())), _lib.F32, src.dim(), _lib.i64_array(list(src.shape)),
                                   torch.cuda.current_stream(src.device).cuda_stream)
    _lib.check(rc)
    return dst


def contiguous(x):
    """A contiguous copy of a float32 CUDA view (what permute().contiguous() costs the reference a
    div/mod per element for)."""
    _check_input(x, "contiguous")
    out = torch.empty(list(x.shape), dtype=torch.float32, device=x.device)
    return copy_(out, x)
