"""CPU tests of the checker itself: the C restatement (oracle/tp_oracle.c) against the reference's
known answers, against the golden fixture produced by the reference's compiled CPU code, and --
where that compiled code is present -- against it directly on seeded inputs."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reduce_golden.npz")


def same(a, b):
    if a.shape != b.shape:
        return False
    if a.dtype == np.float32:
        return np.array_equal(a.view(np.uint32), np.asarray(b, dtype=np.float32).view(np.uint32))
    return np.array_equal(a, b)


def test_known_answers_of_the_reference_tests():
    """test/test_reduction.py:35-57 and test/test_cuda_reductions.py:19-98 of the reference."""
    x = np.array([[1.0, 5.0, 2.0], [4.0, 3.0, 6.0]], dtype=np.float32)
    assert O.reduce("argmax", x) == 5 and O.reduce("argmin", x) == 0
    assert O.reduce("argmax", x, [0]).tolist() == [1, 0, 1]
    assert O.reduce("argmax", x, [1]).tolist() == [1, 2]
    y = np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
    assert O.reduce("sum", y) == 10.0 and O.reduce("mean", y) == 2.5
    ones = np.ones((3, 4), dtype=np.float32)
    assert O.reduce("sum", ones) == 12.0
    assert O.reduce("sum", ones, [0]).tolist() == [3.0] * 4
    assert O.reduce("sum", ones, [1], keepdim=True).shape == (3, 1)
    assert O.reduce("mean", ones * 2, [0]).tolist() == [2.0] * 4
    z = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)
    assert O.reduce("max", z.reshape(2, 2)) == 4.0 and O.reduce("min", z.reshape(2, 2)) == 1.0
    assert O.reduce("max", z.reshape(2, 2), [0]).tolist() == [3.0, 4.0]
    assert abs(float(O.reduce("var", z)) - 5.0 / 3.0) < 1e-6
    assert abs(float(O.reduce("std", z)) - (5.0 / 3.0) ** 0.5) < 1e-6
    w = np.array([1.0, 5.0, 2.0, 8.0], dtype=np.float32)
    assert O.reduce("argmax", w) == 3 and O.reduce("argmin", w) == 0
    # test/test_reduction.py:5-33 (prod, all/any), test/test_cuda_reductions.py:66-75 (prod, norm)
    assert O.reduce("prod", y) == 24.0
    assert O.reduce("prod", y, [0]).tolist() == [3.0, 8.0] and O.reduce("prod", y, [1]).tolist() == [2.0, 12.0]
    b = np.array([[1, 0], [1, 1]], dtype=np.float32)
    assert bool(O.reduce("any", b)) and not bool(O.reduce("all", b))
    assert bool(O.reduce("all", np.array([1, 1], dtype=np.float32)))
    assert not bool(O.reduce("any", np.array([0, 0], dtype=np.float32)))
    assert O.reduce("all", b, [0]).tolist() == [True, False]
    assert O.reduce("norm", np.array([3.0, 4.0], dtype=np.float32)) == 5.0


def test_tie_and_nan_rules():
    assert O.reduce("argmax", np.array([1, 5, 2, 5], dtype=np.float32)) == 1
    assert O.reduce("argmax", np.array([-0.0, 0.0, -0.0], dtype=np.float32)) == 0
    assert O.reduce("max", np.array([-0.0, 0.0], dtype=np.float32)).view(np.uint32) == 0x80000000
    x = np.array([np.nan, 1, 3, np.nan], dtype=np.float32)
    assert O.reduce("max", x) == 3.0 and O.reduce("argmax", x) == 2
    allnan = np.full(4, np.nan, dtype=np.float32)
    assert O.reduce("max", allnan) == -np.inf and O.reduce("argmax", allnan) == 0
    with pytest.raises(RuntimeError, match="Dimension out of range"):
        O.reduce("sum", np.ones((2, 2), dtype=np.float32), [2])
    with pytest.raises(RuntimeError, match="non-empty"):
        O.reduce("max", np.empty(0, dtype=np.float32))


def test_against_golden_fixture():
    """Bit-exact against results produced by the reference's compiled CPU code
    (tests/golden/make_golden.py)."""
    z = np.load(GOLDEN)
    index = json.loads(bytes(z["index_json"]).decode())
    assert len(index) > 150
    assert {e["op"] for e in index} >= {"prod", "norm", "all", "any"}
    for e in index:
        got = O.reduce(e["op"], z[e["x"]], e["dims"], False, e["correction"], e.get("p", 2.0))
        assert same(got, z[e["out"]]), e


@pytest.mark.skipif(not O.have_ref(), reason="the reference's CPU path is not compiled here")
def test_against_compiled_reference():
    rng = np.random.default_rng(7)
    cases = [((10,), [None, [0]]), ((5, 5), [None, [0], [1], [-1], [0, 1]]),
             ((2, 3, 4), [None, [0], [1], [2], [0, 2], [1, 2], [0, 1, 2]]),
             ((64, 257), [None, [1], [0]]), ((3, 4, 5, 6), [[1, 3], [0, 2], [2], [3]])]
    for shape, dimss in cases:
        x = rng.standard_normal(shape).astype(np.float32)
        x.flat[3] = x.flat[1]
        for dims in dimss:
            for op in O.OPS:
                if op in ("argmax", "argmin"):
                    if dims is not None and len(dims) != 1:
                        continue
                    if dims is not None and x.ndim >= 3 and dims[0] % x.ndim not in (x.ndim - 1, x.ndim - 2):
                        continue
                for kd in (False, True):
                    if dims is None and kd:
                        continue
                    for corr in ((0, 1, 2) if op in ("var", "std") else (1,)):
                        for p in ((1.0, 2.0, 3.5, np.inf, -np.inf) if op == "norm" else (2.0,)):
                            assert same(O.reduce(op, x, dims, kd, corr, p), O.ref_reduce(op, x, dims, kd, corr, p)), \
                                (shape, dims, op, kd, corr, p)
    x = rng.standard_normal((6, 8, 10)).astype(np.float32)
    for v in (x.transpose(2, 0, 1), x[:, ::2, 1:9], x.transpose(1, 0, 2)[::2]):
        for dims in (None, [0], [1], [2], [0, 2]):
            for op in ("sum", "mean", "var", "max", "min", "prod", "norm", "all", "any"):
                assert same(O.reduce(op, v, dims), O.ref_reduce(op, v, dims)), (v.strides, dims, op)
    z = rng.integers(0, 2, (5, 6, 7)).astype(np.float32)        # zeros decide all / any / prod
    z[0, 0, 0] = np.nan
    for dims in (None, [0], [1], [2], [0, 2]):
        for op in ("all", "any", "prod"):
            assert same(O.reduce(op, z, dims), O.ref_reduce(op, z, dims)), (dims, op)


@pytest.mark.skipif(not O.have_ref(), reason="the reference's CPU path is not compiled here")
def test_known_reference_defect_is_masked():
    """argmax over dim 0 of a 3-D tensor: the reference's CPU code returns a permuted result
    (p10/src/backend/cpu/ReductionKernels.cpp:714-735); the checker returns numpy's."""
    x = np.random.default_rng(3).standard_normal((2, 3, 4)).astype(np.float32)
    assert np.array_equal(O.reduce("argmax", x, [0]), x.argmax(0))
    assert np.array_equal(O.reduce("argmin", x, [0]), x.argmin(0))


def test_topk_forms_agree_and_follow_the_contract():
    rng = np.random.default_rng(9)
    for shape, k in [((4, 100), 7), ((3, 1000), 1000), ((2, 5000), 64), ((5, 17), 1)]:
        x = rng.integers(0, 6, shape).astype(np.float32)      # tie-heavy
        for largest in (True, False):
            v1, i1 = O.topk(x, k, -1, largest)
            v2, i2 = O.topk_sort(x, k, -1, largest)
            assert np.array_equal(i1, i2) and same(v1, v2)
            # numpy restatement: lexsort by (value, index)
            key = -x if largest else x
            order = np.lexsort((np.broadcast_to(np.arange(shape[1]), shape), key), axis=-1)[:, :k]
            assert np.array_equal(i1, order)
    x = np.array([[np.nan, 1.0, -0.0, 0.0, np.nan, 3.0]], dtype=np.float32)
    v, i = O.topk_sort(x, 6, -1, True)
    assert i.tolist() == [[5, 1, 2, 3, 0, 4]]               # zeros tie by index, NaN last
    v, i = O.topk_sort(x, 6, -1, False)
    assert i.tolist() == [[2, 3, 1, 5, 0, 4]]
    # k = 1 equals argmax / argmin
    y = rng.integers(0, 4, (9, 300)).astype(np.float32)
    assert np.array_equal(O.topk(y, 1, -1, True)[1][:, 0], O.reduce("argmax", y, [1]))
    assert np.array_equal(O.topk(y, 1, -1, False)[1][:, 0], O.reduce("argmin", y, [1]))
    with pytest.raises(RuntimeError):
        O.topk(y, 301)


GOLDEN2 = os.path.join(os.path.dirname(__file__), "golden", "softmax_median_golden.npz")


def test_softmax_and_median_against_golden_fixture():
    """softmax / log_softmax / median of the restatement, bit-exact against results of the reference's
    compiled CPU code (tests/golden/make_golden.py)."""
    z = np.load(GOLDEN2)
    index = json.loads(bytes(z["index_json"]).decode())
    assert len(index) >= 20
    for e in index:
        x = z[e["x"]]
        if e["op"] == "median":
            assert same(np.array([O.median(x)], dtype=np.float32), z[e["out"]]), e
        else:
            assert same(O.softmax(x, e["dim"], e["op"] == "log_softmax"), z[e["out"]]), e


def test_softmax_special_rows_and_median_rules():
    x = np.array([[1.0, np.nan, 2.0], [-np.inf, -np.inf, -np.inf], [0.0, np.inf, 1.0], [-np.inf, 0.0, 0.0]], dtype=np.float32)
    s = O.softmax(x, 1)
    assert np.isnan(s[0]).all() and np.isnan(s[1]).all() and np.isnan(s[2]).all()      # the float chain gives NaN
    assert s[3].tolist() == [0.0, 0.5, 0.5]
    ls = O.softmax(x, 1, True)
    assert ls[3][0] == -np.inf and abs(ls[3][1] + np.log(2.0)) < 1e-6
    assert O.median(np.array([3.0, 1.0, 2.0, 4.0], dtype=np.float32)) == 2.0             # lower middle of an even count
    assert O.median(np.array([5.0], dtype=np.float32)) == 5.0
    assert np.isnan(O.median(np.empty(0, dtype=np.float32)))
    assert O.median(np.array([np.nan, 1.0, 2.0], dtype=np.float32)) == 2.0               # NaNs rank last
    assert np.isnan(O.median(np.array([np.nan, np.nan, 2.0], dtype=np.float32)))


@pytest.mark.skipif(not O.have_ref(), reason="the reference's CPU path is not compiled here")
def test_softmax_and_median_against_compiled_reference():
    rng = np.random.default_rng(8)
    for shape in ((9,), (4, 257), (3, 5, 7), (2, 3, 4, 5)):
        x = (rng.standard_normal(shape) * 4).astype(np.float32)
        for d in range(x.ndim):
            for log in (False, True):
                assert same(O.softmax(x, d, log), O.ref_softmax(x, d, log)), (shape, d, log)
        assert O.median(x) == O.ref_median(x), shape
    t = rng.integers(0, 4, 1000).astype(np.float32)       # ties around the middle
    assert O.median(t) == O.ref_median(t)
