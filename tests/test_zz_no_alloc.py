"""GPU test of tpb200_reduce_all_noalloc, the entry point for callers that cannot allocate device
memory (their own pool owns the device, or cudaMalloc's hidden device-wide synchronisation is not
acceptable where they run) and therefore cannot pass a workspace either.

It is called through the C ABI twice in a row on different inputs -- the built-in scratch array
keeps the first call's records -- and each result must be bit-identical to what the ordinary entry
point tpb200_reduce returns for the same data with a caller-provided workspace.  The file name
sorts last so that a run stopped at the first failure has already executed every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OPS = ["sum", "mean", "var", "std", "max", "min", "argmax", "argmin", "max_argmax", "min_argmin"]


def _both(lib, _lib, torch, x, op, correction=1):
    """(no-alloc result, ordinary result) as (value bits | None, index | None) pairs."""
    n = x.numel()
    st = torch.cuda.current_stream().cuda_stream
    want_val = op not in ("argmax", "argmin")
    want_idx = op in ("argmax", "argmin", "max_argmax", "min_argmin")
    out = []
    for which in ("noalloc", "ordinary"):
        ov = torch.full((1,), float("nan"), device=x.device)
        oi = torch.full((1,), -7, dtype=torch.int64, device=x.device)
        pv = ov.data_ptr() if want_val else None
        pi = oi.data_ptr() if want_idx else None
        if which == "noalloc":
            rc = lib.tpb200_reduce_all_noalloc(_lib.OP[op], x.data_ptr(), _lib.F32, n, correction, pv, pi, st)
        else:
            sizes, strides = _lib.i64_array([n]), _lib.i64_array([1])
            nb = lib.tpb200_reduce_workspace_bytes(_lib.OP[op], _lib.F32, 1, sizes, strides, 0)
            ws = torch.empty(max(nb, 8), dtype=torch.uint8, device=x.device)
            rc = lib.tpb200_reduce(_lib.OP[op], x.data_ptr(), _lib.F32, 1, sizes, strides, 0, -1, correction,
                                   pv, pi, ws.data_ptr(), ws.numel(), st)
        _lib.check(rc)
        torch.cuda.synchronize()
        out.append((ov.view(torch.int32).item() if want_val else None, oi.item() if want_idx else None))
    return out


def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row(cuda):
    import torch
    from tensorplay_b200 import _lib

    lib = _lib.lib()
    rng = np.random.default_rng(41)
    # first call: large enough for hundreds of slices; second call: fewer slices, so stale records
    # of the first call remain in the scratch array behind the ones it rewrites
    a = rng.uniform(-1, 1, (1 << 24) + 13).astype(np.float32)
    a[rng.choice(a.size, a.size // 100, replace=False)] = 1e4
    a[12345] = a[9_000_000] = 3e4                     # a tie: the lower index must be reported
    b = rng.standard_normal(300_001).astype(np.float32)
    xa, xb = torch.from_numpy(a).to(cuda), torch.from_numpy(b).to(cuda)
    for x in (xa, xb):                                # two calls in a row, per operator
        for op in OPS:
            got, want = _both(lib, _lib, torch, x, op)
            assert got == want, (op, x.numel(), got, want)
    # short inputs, where one warp or one CTA does the whole reduction and the scratch array is not
    # touched at all: still the same bits as the ordinary entry point
    for m in (1, 1000, 20000, 40000):
        xs = torch.from_numpy(rng.standard_normal(m).astype(np.float32)).to(cuda)
        for op in OPS:
            got, want = _both(lib, _lib, torch, xs, op)
            assert got == want, (op, m, got, want)
    empty = torch.empty(0, device=cuda)
    for op in ("sum", "mean", "var"):
        got, want = _both(lib, _lib, torch, empty, op)
        assert got == want, (op, 0, got, want)
    # and the values are right, not merely equal to each other
    st = torch.cuda.current_stream().cuda_stream
    ov = torch.empty(1, device=cuda)
    oi = torch.empty(1, dtype=torch.int64, device=cuda)
    _lib.check(lib.tpb200_reduce_all_noalloc(_lib.OP["max_argmax"], xa.data_ptr(), _lib.F32, xa.numel(), 1,
                                             ov.data_ptr(), oi.data_ptr(), st))
    assert ov.item() == 3e4 and oi.item() == 12345
    _lib.check(lib.tpb200_reduce_all_noalloc(_lib.OP["sum"], xb.data_ptr(), _lib.F32, xb.numel(), 1,
                                             ov.data_ptr(), None, st))
    t = b.astype(np.float64).sum()
    assert abs(ov.item() - t) <= 1e-5 * abs(t)


def test_noalloc_rejects_what_it_cannot_hold(cuda):
    from tensorplay_b200 import _lib

    lib = _lib.lib()
    too_many = (1 << 33) + 1
    rc = lib.tpb200_reduce_all_noalloc(_lib.OP["sum"], ctypes.c_void_p(256), _lib.F32, too_many, 1,
                                       ctypes.c_void_p(256), None, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"at most" in lib.tpb200_last_error()
    assert lib.tpb200_reduce_all_noalloc(_lib.OP["max"], None, _lib.F32, 0, 1, ctypes.c_void_p(256), None, None) == _lib.ERR_EMPTY
    assert lib.tpb200_reduce_all_noalloc(_lib.OP["sum"], None, 3, 4, 1, ctypes.c_void_p(256), None, None) == _lib.ERR_UNSUPPORTED
