"""GPU parity of the reduction kernels against the CPU oracle, through the C ABI.

Every case runs the sm_100a kernel (tensorplay_b200.ops -> ctypes -> libtpb200.so) and the plain-C
restatement of the reference's CPU kernels (oracle/) on the same seeded input.
max / min / argmax / argmin: bit-exact.  sum / mean / var / std: within 1e-5 relative of a float64
evaluation, and in condition-aware agreement with the reference (tests/util.py).
"""
import os

import numpy as np
import pytest

from util import (assert_agrees, assert_bits_equal, assert_close64, assert_index_equal, config1, config3)

pytestmark = pytest.mark.gpu

VALUE_OPS = ["sum", "mean", "var", "std"]
EXT_OPS = ["max", "min"]
ARG_OPS = ["argmax", "argmin"]


def gpu_view(x, device):
    """The same strided view of the same bytes, on the GPU."""
    import torch

    base = x
    while isinstance(base.base, np.ndarray):
        base = base.base
    g = torch.from_numpy(np.ascontiguousarray(base).reshape(-1)).to(device)
    if not base.flags.c_contiguous:
        return torch.from_numpy(np.ascontiguousarray(x)).to(device)
    off = (x.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // 4
    return torch.as_strided(g, x.shape, [s // 4 for s in x.strides], off)


def check(device, x, op, dims=None, keepdim=False, correction=1, what=""):
    import tensorplay_b200 as tpb
    from oracle import oracle as O

    xg = gpu_view(x, device)
    what = f"{what} {op} shape={x.shape} strides={x.strides} dims={dims} keepdim={keepdim} corr={correction}"
    if op in ARG_OPS:
        d = None if dims is None else dims[0]
        got = getattr(tpb, op)(xg, d, keepdim).cpu().numpy()
        want = O.reduce(op, x, dims, keepdim)
        assert_index_equal(got, want, what)
        return
    if op in EXT_OPS:
        got = getattr(tpb, op)(xg, dims, keepdim).cpu().numpy()
        want = O.reduce(op, x, dims, keepdim)
        assert_bits_equal(got, want, what)
        return
    if op in ("var", "std"):
        got = getattr(tpb, op)(xg, dims, correction, keepdim).cpu().numpy()
    else:
        got = getattr(tpb, op)(xg, dims, keepdim).cpu().numpy()
    truth = O.truth64(op, x, dims, keepdim, correction)
    ref = O.reduce(op, x, dims, keepdim, correction)
    assert got.shape == ref.shape, what
    assert_close64(got, truth, what)
    if op in ("sum", "mean"):
        ax = None if dims is None else tuple(d % x.ndim for d in dims)
        abs_sum = np.abs(x.astype(np.float64)).sum(axis=ax, keepdims=keepdim)
        if op == "mean":
            n = x.size if ax is None else int(np.prod([x.shape[a] for a in ax]))
            abs_sum = abs_sum / max(n, 1)
        assert_agrees(got, ref, truth, abs_sum, what)
    else:
        # var/std: the reference sums the squared deviations sequentially in float32, so its own
        # distance from float64 grows with the reduction length n (about 1e-4 at n = 3e5)
        n = x.size if dims is None else int(np.prod([x.shape[d % x.ndim] for d in dims]))
        assert_close64(ref, truth, what + " (reference vs float64)", rel=max(1e-4, 2e-9 * n))


# ------------------------------------------------------------------ known answers ------------
def test_reference_known_answers(cuda):
    """The hand-computed cases of the reference's own tests (test/test_reduction.py:35-57,
    test/test_cuda_reductions.py:19-98)."""
    import torch
    import tensorplay_b200 as tpb

    x = torch.tensor([[1.0, 5.0, 2.0], [4.0, 3.0, 6.0]], device=cuda)
    assert tpb.argmax(x).item() == 5 and tpb.argmin(x).item() == 0
    assert tpb.argmax(x, 0).tolist() == [1, 0, 1]
    assert tpb.argmax(x, 1).tolist() == [1, 2]
    y = torch.tensor([[1.0, 2.0], [3.0, 4.0]], device=cuda)
    assert tpb.sum(y).item() == 10.0 and tpb.mean(y).item() == 2.5
    t = torch.ones(3, 4, device=cuda)
    assert tpb.sum(t, [0]).tolist() == [3.0] * 4
    assert tpb.sum(t, [1], keepdim=True).shape == (3, 1)
    assert tpb.mean(t * 2, [0]).tolist() == [2.0] * 4
    z = torch.tensor([1.0, 2.0, 3.0, 4.0], device=cuda)
    assert tpb.max(z.reshape(2, 2)).item() == 4.0 and tpb.min(z.reshape(2, 2)).item() == 1.0
    assert tpb.max(z.reshape(2, 2), [0]).tolist() == [3.0, 4.0]
    assert abs(tpb.var(z).item() - 5.0 / 3.0) < 1e-6
    assert abs(tpb.std(z).item() - (5.0 / 3.0) ** 0.5) < 1e-6
    w = torch.tensor([1.0, 5.0, 2.0, 8.0], device=cuda)
    assert tpb.argmax(w).item() == 3 and tpb.argmin(w).item() == 0


# ------------------------------------------------------------------ small shapes, all dims ---
SMALL = [((10,), [None, [0]]),
         ((5, 5), [None, [0], [1], [-1], [0, 1]]),
         ((2, 3, 4), [None, [0], [1], [2], [0, 2], [1, 2], [0, 1], [0, 1, 2]]),
         ((3, 4, 5, 6), [[1, 3], [0, 2], [2], [3], [0], [1, 2, 3], [0, 3]]),
         ((7, 1001), [None, [0], [1]]),
         ((1, 1), [None, [0], [1]]),
         ((33, 1, 17), [[0], [1], [2], [0, 2]])]


@pytest.mark.parametrize("shape,dimss", SMALL)
def test_small_shapes(cuda, shape, dimss):
    rng = np.random.default_rng(11)
    x = rng.standard_normal(shape).astype(np.float32)
    if x.size > 4:
        x.flat[3] = x.flat[1]
    for dims in dimss:
        for keepdim in (False, True):
            for op in VALUE_OPS + EXT_OPS:
                for corr in ((0, 1, 2) if op in ("var", "std") else (1,)):
                    check(cuda, x, op, dims, keepdim and dims is not None, corr)
            for op in ARG_OPS:
                if dims is None or len(dims) == 1:
                    check(cuda, x, op, dims, keepdim and dims is not None)


def test_many_short_rows(cuda):
    """Thousands of rows of at most 256 elements: several rows share a warp (4, 8 or 16 lanes per row);
    ragged lengths, rows that are not 16-byte aligned, a strided view, ties and NaN."""
    rng = np.random.default_rng(15)
    for shape in ((5000, 64), (4100, 37), (8192, 256), (4097, 130), (6000, 1), (4500, 5), (70000, 16)):
        x = rng.standard_normal(shape).astype(np.float32)
        x[::7, 0] = x[::7, -1]                # ties between the ends of a row
        if shape[1] > 2:
            x[5, 1] = np.nan
        for op in VALUE_OPS + EXT_OPS + ARG_OPS:
            check(cuda, x, op, [1])
            check(cuda, x, op, [-1], True)
    wide = rng.standard_normal((5000, 80)).astype(np.float32)
    for v in (wide[:, 1:65], wide[::2, 3:40]):
        for op in ("sum", "var", "max", "argmin"):
            check(cuda, v, op, [1])


def test_strided_views(cuda):
    rng = np.random.default_rng(12)
    x = rng.standard_normal((6, 8, 10)).astype(np.float32)
    big = rng.standard_normal((40, 67, 131)).astype(np.float32)
    views = [x.transpose(2, 0, 1), x[:, ::2, 1:9], x.transpose(1, 0, 2)[::2], x[1:, :, 3:],
             big[:, 1:, 1:], big.transpose(0, 2, 1), big[::3, :, ::2], big.reshape(-1)[5:][::1]]
    for v in views:
        dimss = [None] + [[d] for d in range(v.ndim)] + ([[0, v.ndim - 1]] if v.ndim > 1 else [])
        for dims in dimss:
            for op in VALUE_OPS + EXT_OPS:
                check(cuda, v, op, dims)
            for op in ARG_OPS:
                if dims is None or len(dims) == 1:
                    check(cuda, v, op, dims)


def test_special_values(cuda):
    nan, inf = np.float32(np.nan), np.float32(np.inf)
    rows = [np.array([nan, 1, 3, nan, -0.0, 0.0, 3, -inf], dtype=np.float32),
            np.array([-0.0, 0.0, -0.0], dtype=np.float32),
            np.array([0.0, -0.0, 0.0], dtype=np.float32),
            np.full(5, nan, dtype=np.float32),
            np.full(700, -inf, dtype=np.float32),
            np.full(700, inf, dtype=np.float32),
            np.array([inf, -inf, 1.0], dtype=np.float32)]
    for r in rows:
        for op in EXT_OPS + ARG_OPS:
            check(cuda, r, op, None)
            check(cuda, r, op, [0])
        tall = np.tile(r, (300, 1))          # [300, n]: row kernels
        wide = np.ascontiguousarray(tall.T)  # [n, 300]: column kernel over dim 0
        for op in EXT_OPS + ARG_OPS:
            check(cuda, tall, op, [1])
            check(cuda, wide, op, [0])
    # sums containing NaN / inf propagate like the reference
    import tensorplay_b200 as tpb
    import torch
    assert np.isnan(tpb.sum(torch.tensor([1.0, float("nan")], device=cuda)).item())
    assert tpb.sum(torch.tensor([1.0, float("inf")], device=cuda)).item() == float("inf")


def test_tie_heavy(cuda):
    rng = np.random.default_rng(13)
    x = rng.integers(0, 4, (257, 3001)).astype(np.float32)
    for op in EXT_OPS + ARG_OPS:
        check(cuda, x, op, [1])
        check(cuda, x, op, [0])
        check(cuda, x, op, None)
    y = rng.integers(0, 3, (5, 70, 33)).astype(np.float32)
    for op in EXT_OPS + ARG_OPS:
        check(cuda, y, op, [1])


def test_empty_and_degenerate(cuda):
    import torch
    import tensorplay_b200 as tpb

    e = torch.empty(0, device=cuda)
    assert tpb.sum(e).item() == 0.0
    assert np.isnan(tpb.mean(e).item())
    assert np.isnan(tpb.var(e).item())
    assert tpb.argmax(e).item() == 0
    with pytest.raises(RuntimeError, match=r"max\(\): Expected reduction dim to be non-empty"):
        tpb.max(e)
    with pytest.raises(RuntimeError, match=r"min\(\): Expected reduction dim to be non-empty"):
        tpb.min(e)
    z = torch.empty(3, 0, device=cuda)
    assert tpb.sum(z, [1]).tolist() == [0.0, 0.0, 0.0]
    assert tpb.max(z, [1]).tolist() == [float("-inf")] * 3     # the reference fills the start value
    assert tpb.min(z, [1]).tolist() == [float("inf")] * 3
    assert tpb.sum(z, [0]).shape == (0,)
    one = torch.tensor([2.0], device=cuda)
    assert np.isnan(tpb.var(one).item())                         # 0 / max(0, 1-1)
    assert tpb.var(one, [0], correction=0).item() == 0.0
    assert tpb.var(torch.tensor([1.0, 3.0], device=cuda), correction=5).item() == float("inf")
    s = torch.tensor(3.5, device=cuda)                           # 0-dim
    assert tpb.sum(s).item() == 3.5 and tpb.max(s).item() == 3.5 and tpb.argmax(s).item() == 0
    with pytest.raises(RuntimeError, match="Dimension out of range"):
        tpb.sum(torch.ones(2, 2, device=cuda), [2])
    with pytest.raises(RuntimeError, match="Dimension out of range"):
        tpb.argmax(torch.ones(2, 2, device=cuda), -3)
    with pytest.raises(NotImplementedError):
        tpb.sum(torch.ones(2, dtype=torch.float64, device=cuda))
    with pytest.raises(RuntimeError):
        tpb.sum(torch.ones(2))


@pytest.mark.parametrize("strategy", ["warp", "cta", "split", "generic"])
def test_forced_row_strategies(cuda, strategy, monkeypatch):
    """The same inputs through every row-kernel family (TPB200_FORCE_STRATEGY)."""
    monkeypatch.setenv("TPB200_FORCE_STRATEGY", strategy)
    rng = np.random.default_rng(14)
    x = rng.standard_normal((19, 40007)).astype(np.float32)
    x[:, 100] = x[:, 7]
    for op in VALUE_OPS + EXT_OPS + ARG_OPS:
        check(cuda, x, op, [1], what=strategy)
        check(cuda, x[:, 1:], op, [1], what=strategy)   # rows not 16-byte aligned
    flat = rng.standard_normal(1_000_003).astype(np.float32)
    for op in VALUE_OPS + EXT_OPS + ARG_OPS:
        check(cuda, flat, op, None, what=strategy)


def test_rowwise_4096x4096(cuda):
    """[4096, 4096] N(0,1), seed 0, full size; sum/mean/var/std/max/min/argmax/argmin over dim -1."""
    x = config1()
    for op in ["sum", "mean", "var", "std", "max", "min", "argmax", "argmin"]:
        check(cuda, x, op, [-1])
    import tensorplay_b200 as tpb
    import torch
    xg = torch.from_numpy(x).to(cuda)
    v, i = tpb.max_with_indices(xg, -1)
    assert torch.equal(v, tpb.max(xg, -1)) and torch.equal(i, tpb.argmax(xg, -1))
    assert torch.equal(v, xg.gather(1, i[:, None])[:, 0])


def test_nonlast_dims_64x4096x512(cuda):
    """[64, 4096, 512] uniform(-1, 1), seed 2, full size: sum/mean/max/argmin (and var, min, argmax)
    over dim 1, sum/std (and mean, max) over dims (0, 2)."""
    x = config3()
    for op in ["sum", "mean", "max", "min", "argmin", "argmax", "var"]:
        check(cuda, x, op, [1])
    for op in ["sum", "std", "mean", "max"]:
        check(cuda, x, op, [0, 2])


def test_whole_tensor_2_to_26(cuda):
    """Whole-tensor reductions of 2^26+5 elements, uniform(-1,1) with 1% of positions +-1e4, against
    the oracle element for element."""
    from util import config4
    x = config4(n=(1 << 26) + 5)
    for op in ["sum", "mean", "var", "std", "max", "min", "argmax", "argmin"]:
        check(cuda, x, op, None)


def test_whole_tensor_2_to_31(cuda):
    """The full 2^31-element tensor (8 GiB; the element count does not fit int32): uniform(-1,1) with
    1% of positions +-1e4, made chunk by chunk on the device.  sum / mean / var / std against a
    float64 evaluation merged over the chunks with Chan's update (torch float64 per chunk, tied to
    numpy float64 on the first and the last chunk); max / min / argmax / argmin exact.  A maximum is
    planted a few hundred elements before the end (the last slice) and tied by an element in the
    first half: the lower index must win; then the tie is removed and the late one must be found."""
    import torch
    import tensorplay_b200 as tpb

    n, chunk = 1 << 31, 1 << 26
    late, early = n - 700, (n >> 1) - 12345
    lo_pos = n - 5                                   # the minimum sits in the very last vector
    xg = torch.empty(n, dtype=torch.float32, device=cuda)
    gen = torch.Generator(device=cuda).manual_seed(3)
    cnt, mean, m2 = 0.0, 0.0, 0.0
    for s in range(0, n, chunk):
        v = torch.rand(chunk, device=cuda, generator=gen) * 2.0 - 1.0
        sel = torch.rand(chunk, device=cuda, generator=gen)
        v = torch.where(sel < 0.005, torch.full_like(v, 1e4), v)
        v = torch.where(sel > 0.995, torch.full_like(v, -1e4), v)
        for p, val in ((late, 3e4), (early, 3e4), (lo_pos, -3e4)):
            if s <= p < s + chunk:
                v[p - s] = val
        xg[s:s + chunk] = v
        v64 = v.double()
        cm = float(v64.mean().item())
        cm2 = float(((v64 - cm) ** 2).sum().item())
        if s == 0 or s + chunk == n:                 # the float64 evaluation itself, against numpy
            h = v.cpu().numpy().astype(np.float64)
            assert abs(h.mean() - cm) <= 1e-12 * max(1.0, abs(cm)) + 1e-9
            assert abs(((h - h.mean()) ** 2).sum() - cm2) <= 1e-9 * cm2
        tot = cnt + chunk
        delta = cm - mean
        m2 = m2 + cm2 + delta * delta * cnt * chunk / tot
        mean = mean + delta * chunk / tot
        cnt = tot
        del v, sel, v64
    truth = {"sum": mean * n, "mean": mean, "var": m2 / (n - 1), "std": float(np.sqrt(m2 / (n - 1)))}
    for op in ("sum", "mean", "var", "std"):
        got = float(getattr(tpb, op)(xg).item())
        assert abs(got - truth[op]) <= 1e-5 * abs(truth[op]), (op, got, truth[op])
    assert tpb.max(xg).item() == 3e4 and tpb.min(xg).item() == -3e4
    assert tpb.argmax(xg).item() == early
    assert tpb.argmin(xg).item() == lo_pos
    v, i = tpb.max_with_indices(xg.view(1, n), 1)
    assert v.item() == 3e4 and i.item() == early
    xg[early] = 0.5
    assert tpb.argmax(xg).item() == late
    from tensorplay_b200 import _lib
    assert _lib.device_status() == 0
    del xg
    torch.cuda.empty_cache()


def test_run_to_run_bit_identity(cuda):
    import torch
    import tensorplay_b200 as tpb
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(3, 5000, 129, generator=g).to(cuda)
    for fn, args in [(tpb.sum, ([1],)), (tpb.var, ([0, 2],)), (tpb.sum, (None,)), (tpb.std, (None,)),
                     (tpb.mean, ([2],))]:
        a = fn(x, *args).clone()
        for _ in range(3):
            assert torch.equal(a.view(torch.int32), fn(x, *args).view(torch.int32))


def _more_cases():
    rng = np.random.default_rng(41)
    x = (rng.standard_normal((37, 1000)) * 0.2 + 1.0).astype(np.float32)      # products stay in range
    y = rng.uniform(-1, 1, (6, 130, 24)).astype(np.float32)
    z = rng.integers(0, 2, (33, 70, 9)).astype(np.float32)
    z[:, ::7, :] = 1.0
    z[3, 5, 2] = np.nan
    return x, y, z


def test_prod_norm_all_any_against_oracle_and_float64(cuda):
    """The other operators of the reference's registration block
    (p10/src/backend/cuda/ReductionKernels.cu:256-267, 296-345): prod and norm within 1e-5 of float64
    (and 1e-4 of the reference's float32 chain), norm(+-inf) and all/any exact."""
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O

    x, y, z = _more_cases()
    for a, dimss in ((x, [None, [1], [0], [-1]]), (y, [None, [0], [1], [2], [0, 2], [1, 2]]),
                     (y.transpose(2, 0, 1), [None, [0], [2], [0, 1]]), (y[:, ::3, 1:23], [[1], [2], None])):
        ag = gpu_view(a, cuda)
        for dims in dimss:
            for kd in (False, True):
                what = f"shape={a.shape} dims={dims} keepdim={kd}"
                got = tpb.prod(ag, dims, kd).cpu().numpy()
                assert_close64(got, O.truth64("prod", a, dims, kd), "prod " + what)
                assert_close64(got, O.reduce("prod", a, dims, kd).astype(np.float64), "prod vs oracle " + what, rel=1e-4)
                for p in (1.0, 2.0):
                    got = tpb.norm(ag, p, dims, kd).cpu().numpy()
                    assert_close64(got, O.truth64("norm", a, dims, kd, p=p), f"norm p={p} " + what)
                    assert_close64(got, O.reduce("norm", a, dims, kd, p=p).astype(np.float64), f"norm p={p} vs oracle " + what, rel=1e-4)
                for p in (float("inf"), float("-inf")):
                    assert_bits_equal(tpb.norm(ag, p, dims, kd).cpu().numpy(), O.reduce("norm", a, dims, kd, p=p), f"norm p={p} " + what)
    zg = torch.from_numpy(z).to(cuda)
    for dims in (None, [0], [1], [2], [0, 2], [1, 2]):
        for op in ("all", "any"):
            got = getattr(tpb, op)(zg, dims).cpu().numpy()
            assert got.dtype == np.bool_ and np.array_equal(got, O.reduce(op, z, dims)), (op, dims)
    zeros = torch.zeros(5, 3000, device=cuda)
    assert not bool(tpb.any(zeros)) and not bool(tpb.all(zeros))
    zeros[2, 2999] = float("nan")                                   # NaN counts as true
    assert bool(tpb.any(zeros)) and tpb.any(zeros, 1).cpu().tolist() == [False, False, True, False, False]
    ones = torch.ones(1 << 22, device=cuda)
    assert bool(tpb.all(ones))
    ones[4_000_001] = 0.0
    assert not bool(tpb.all(ones)) and float(tpb.prod(ones)) == 0.0
    # empty reductions: prod of nothing is 1, norm 0, all true, any false
    e = torch.empty(4, 0, device=cuda)
    assert tpb.prod(e, 1).cpu().tolist() == [1.0] * 4 and tpb.norm(e, 2.0, 1).cpu().tolist() == [0.0] * 4
    assert tpb.all(e, 1).cpu().tolist() == [True] * 4 and tpb.any(e, 1).cpu().tolist() == [False] * 4
    with pytest.raises(NotImplementedError):
        tpb.norm(ones, 3.0)
    with pytest.raises(RuntimeError, match="non-empty"):
        tpb.norm(torch.empty(0, device=cuda), float("inf"))
