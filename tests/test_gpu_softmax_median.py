"""GPU parity of softmax / log_softmax / median against the CPU oracle, through the C ABI.

softmax and log_softmax are float32 chains with exp and log in them: the result must lie within
    |gpu - float64| <= 1e-5 * |float64| + ABS
of a float64 evaluation (ABS = 1e-37 for softmax, whose outputs may be denormal-small; 1e-6 for
log_softmax, whose outputs cross zero at the row maximum), must agree with the reference's own float32
chain (the oracle, pinned bit-for-bit to the compiled reference) to that bound plus the chain's own
distance from float64, and must put NaN and infinities exactly where that chain does.  The median is
one element of the input: bit-exact.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN2 = os.path.join(os.path.dirname(__file__), "golden", "softmax_median_golden.npz")
REL = 1e-5


def close(got, want, abs_tol, what, slack=None):
    """|got - want| <= REL * |want| + abs_tol (+ slack, elementwise), same NaNs, same infinities."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, what
    assert np.array_equal(np.isnan(got), np.isnan(want)), f"{what}: NaN pattern differs"
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf]), f"{what}: infinities differ"
    fin = np.isfinite(want)
    err = np.abs(got[fin] - want[fin])
    tol = REL * np.abs(want[fin]) + abs_tol
    if slack is not None:
        tol = tol + np.asarray(slack, dtype=np.float64)[fin]
    assert np.all(err <= tol), f"{what}: max excess {np.max(err - tol):.3e}"


def check_softmax(cuda, x, dim, what=""):
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O
    xg = torch.from_numpy(np.ascontiguousarray(x)).to(cuda)
    for log in (False, True):
        fn = tpb.log_softmax if log else tpb.softmax
        got = fn(xg, dim).cpu().numpy()
        abs_tol = 1e-6 if log else 1e-37
        name = f"{what} {'log_' if log else ''}softmax shape={x.shape} dim={dim}"
        with np.errstate(all="ignore"):
            truth = O.truth64_softmax(x, dim, log)
            close(got, truth, abs_tol, name + " vs float64")
            # against the reference's float32 chain: the same NaNs and infinities, and no further from it
            # than the bound above plus the chain's own distance from float64 (its sequential float32
            # sum is the less accurate of the two)
            ref = O.softmax(x, dim, log)
            own = np.abs(ref.astype(np.float64) - truth)
            close(got, ref, abs_tol, name + " vs reference chain", slack=np.where(np.isfinite(own), own, 0.0))


def test_softmax_rows_of_every_length(cuda):
    rng = np.random.default_rng(51)
    # (…, 1028) to (…, 16384): the register-resident CTA kernel with four and with eight float4 per
    # thread, partly filled; 16388 and 40000: slices staged in shared memory; 1025 / 4097: unaligned rows
    for shape in ((5, 1), (7, 33), (300, 128), (64, 1000), (33, 1024), (9, 1025), (6, 4097), (17, 40000), (3, 5, 700),
                  (7, 1028), (5, 2048), (4, 5000), (3, 8192), (2, 8196), (4, 12000), (2, 16384), (2, 16388)):
        x = (rng.standard_normal(shape) * 5).astype(np.float32)
        check_softmax(cuda, x, -1)
    # rows not 16-byte aligned and a strided view (every other row of a wider matrix)
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O
    base = (rng.standard_normal((10, 3001)) * 3).astype(np.float32)
    bg = torch.from_numpy(base).to(cuda)
    for vn, vg in ((base[:, 1:], bg[:, 1:]), (base[::2], bg[::2])):
        got = tpb.softmax(vg, 1).cpu().numpy()
        close(got, O.truth64_softmax(np.ascontiguousarray(vn), 1), 1e-37, "strided view")


def test_softmax_other_dims(cuda):
    rng = np.random.default_rng(52)
    x = (rng.standard_normal((6, 50, 37)) * 4).astype(np.float32)
    for d in (0, 1, -2):
        check_softmax(cuda, x, d)
    y = (rng.standard_normal((300, 4, 128)) * 2).astype(np.float32)
    check_softmax(cuda, y, 1)
    check_softmax(cuda, y, 0)


@pytest.mark.parametrize("slices", ["1", "2", "4", "8"])
def test_softmax_long_rows_in_clusters(cuda, slices, monkeypatch):
    """Long rows with 1, 2, 4 and 8 CTAs per row: the (max, sum) pairs cross the cluster through
    distributed shared memory."""
    monkeypatch.setenv("TPB200_SOFTMAX_SLICES", slices)
    rng = np.random.default_rng(53)
    x = (rng.standard_normal((5, 151936)) * 2).astype(np.float32)
    x[0, 100000] = 30.0          # a peaked row: the maximum sits in one slice only
    x[1] = np.sort(x[1])         # the maximum at the very end
    check_softmax(cuda, x, -1, what=f"S={slices}")
    y = (rng.standard_normal((3, 70001)) * 2).astype(np.float32)          # ragged length, scalar tail
    check_softmax(cuda, y, -1, what=f"S={slices}")


def test_softmax_special_rows(cuda):
    """NaN, +inf and all -inf rows give NaN exactly where the reference's float chain does; -inf
    beside numbers counts as exp(-inf) = 0."""
    x = np.zeros((6, 5000), dtype=np.float32)
    rng = np.random.default_rng(54)
    x[:] = rng.standard_normal(x.shape)
    x[0, 4000] = np.nan
    x[1, :] = -np.inf
    x[2, 17] = np.inf
    x[3, :2500] = -np.inf
    x[4, ::2] = -np.inf
    x[5, :] = -np.inf
    x[5, 4999] = 1.0
    check_softmax(cuda, x, 1)
    check_softmax(cuda, np.ascontiguousarray(x[:, :700]), 1)       # the warp-per-row kernel
    check_softmax(cuda, np.ascontiguousarray(x.T), 0)              # the column kernel


def test_softmax_headline_shapes(cuda):
    """[4096, 4096] N(0,1) and [256, 151936] N(0,2) with 64 planted +8.0 per row, full size."""
    from util import config1, config2
    check_softmax(cuda, config1(), -1)
    check_softmax(cuda, config2(), -1)


def test_softmax_and_median_golden(cuda):
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O
    z = np.load(GOLDEN2)
    index = json.loads(bytes(z["index_json"]).decode())
    for e in index:
        x = z[e["x"]]
        xg = torch.from_numpy(x).to(cuda)
        if e["op"] == "median":
            got = tpb.median(xg).cpu().numpy().reshape(1)
            assert got.view(np.uint32)[0] == z[e["out"]].view(np.uint32)[0], e
        else:
            log = e["op"] == "log_softmax"
            got = (tpb.log_softmax if log else tpb.softmax)(xg, e["dim"]).cpu().numpy()
            with np.errstate(all="ignore"):
                own = np.abs(z[e["out"]].astype(np.float64) - O.truth64_softmax(x, e["dim"], log))
            close(got, z[e["out"]], 1e-6 if log else 1e-37, str(e), slack=np.where(np.isfinite(own), own, 0.0))


def test_median(cuda):
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O
    rng = np.random.default_rng(55)
    for n in (1, 2, 3, 10, 1001, 4096, 100000, (1 << 22) + 7):
        x = rng.standard_normal(n).astype(np.float32)
        got = tpb.median(torch.from_numpy(x).to(cuda)).item()
        assert np.float32(got) == O.median(x), n
    # ties around the middle, both zeros, infinities, negative numbers only
    for x in (rng.integers(0, 4, 100001).astype(np.float32), np.array([-0.0, 0.0, -0.0, 0.0, 1.0], dtype=np.float32),
              np.array([-np.inf, np.inf, 1.0, -np.inf], dtype=np.float32), -np.abs(rng.standard_normal(5000)).astype(np.float32)):
        got = tpb.median(torch.from_numpy(x).to(cuda)).item()
        assert np.float32(got) == O.median(x)
    # NaNs rank after all numbers; a strided view is read in place; the empty tensor gives NaN
    y = rng.standard_normal(9999).astype(np.float32)
    y[::10] = np.nan
    assert np.float32(tpb.median(torch.from_numpy(y).to(cuda)).item()) == O.median(y)
    mostly_nan = np.full(101, np.nan, dtype=np.float32)
    mostly_nan[:10] = 1.0
    assert np.isnan(tpb.median(torch.from_numpy(mostly_nan).to(cuda)).item())
    m = rng.standard_normal((300, 400)).astype(np.float32)
    mg = torch.from_numpy(m).to(cuda)
    assert np.float32(tpb.median(mg.t()[::2, 3:]).item()) == O.median(np.ascontiguousarray(m.T[::2, 3:]))
    assert np.isnan(tpb.median(torch.empty(0, device=cuda)).item())
    # two calls in a row on one workspace, and the value is an element of the input
    a = tpb.median(mg).item()
    b = tpb.median(mg).item()
    assert a == b == float(O.median(m))
    from tensorplay_b200 import _lib
    assert _lib.device_status() == 0


def test_errors(cuda):
    import torch
    import tensorplay_b200 as tpb
    x = torch.ones(3, 4, device=cuda)
    with pytest.raises(RuntimeError, match="Dimension out of range"):
        tpb.softmax(x, 2)
    with pytest.raises(RuntimeError, match="Dimension out of range"):
        tpb.log_softmax(torch.tensor(1.0, device=cuda), 0)
    with pytest.raises(NotImplementedError):
        tpb.softmax(x.double(), 1)
    with pytest.raises(NotImplementedError):
        tpb.softmax(torch.ones(4, 6, 8, device=cuda).permute(2, 0, 1), 1)     # not contiguous, dim not last
    assert tpb.softmax(torch.empty(0, 5, device=cuda), 1).shape == (0, 5)
