"""GPU parity of top-k against the CPU oracle, through the C ABI.  Values and indices must be
bit-exact, including the tie order (ties in ascending index)."""
import numpy as np
import pytest

from util import assert_bits_equal, assert_index_equal, config2, config5

pytestmark = pytest.mark.gpu


def check_topk(device, x, k, dim=-1, largest=True, what="", oracle="heap"):
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O

    xg = torch.from_numpy(np.ascontiguousarray(x)).to(device)
    v, i = tpb.topk(xg, k, dim, largest, True)
    v, i = v.cpu().numpy(), i.cpu().numpy()
    wv, wi = (O.topk if oracle == "heap" else O.topk_sort)(x, k, dim, largest)
    what = f"{what} topk shape={x.shape} k={k} dim={dim} largest={largest}"
    assert_index_equal(np.ascontiguousarray(i), np.ascontiguousarray(wi), what)
    assert_bits_equal(np.ascontiguousarray(v), np.ascontiguousarray(wv), what)


def test_small_rows_sorted_whole(cuda):
    rng = np.random.default_rng(21)
    for shape, ks in [((5, 10), [1, 3, 10]), ((3, 1), [1]), ((64, 257), [1, 17, 257]),
                      ((9, 4096), [1, 50, 1000, 4096]), ((2, 3, 40), [5])]:
        x = rng.standard_normal(shape).astype(np.float32)
        for k in ks:
            for largest in (True, False):
                check_topk(cuda, x, k, -1, largest, oracle="sort")


def test_k1_equals_argmax(cuda):
    import torch
    import tensorplay_b200 as tpb
    rng = np.random.default_rng(22)
    x = rng.integers(0, 5, (33, 20000)).astype(np.float32)
    xg = torch.from_numpy(x).to(cuda)
    v, i = tpb.topk(xg, 1, -1, True)
    assert torch.equal(i[:, 0], tpb.argmax(xg, 1)) and torch.equal(v[:, 0], tpb.max(xg, 1))
    v, i = tpb.topk(xg, 1, -1, False)
    assert torch.equal(i[:, 0], tpb.argmin(xg, 1)) and torch.equal(v[:, 0], tpb.min(xg, 1))


@pytest.mark.parametrize("k", [1, 50, 512, 513, 1024, 2048])
def test_streaming_path(cuda, k):
    rng = np.random.default_rng(23)
    x = rng.standard_normal((7, 100003)).astype(np.float32)
    for largest in (True, False):
        check_topk(cuda, x, k, -1, largest)


@pytest.mark.parametrize("slices", ["1", "2", "5"])
def test_streaming_slices(cuda, slices, monkeypatch):
    monkeypatch.setenv("TPB200_TOPK_SLICES", slices)
    rng = np.random.default_rng(24)
    x = rng.standard_normal((5, 300001)).astype(np.float32)
    for k in (50, 1024):
        check_topk(cuda, x, k, -1, True, what=f"S={slices}")
        check_topk(cuda, x, k, -1, False, what=f"S={slices}")


def test_tie_heavy(cuda):
    """Massive duplicates: the answer is decided by the tie rule alone."""
    rng = np.random.default_rng(25)
    x = rng.integers(0, 1000, (6, 1 << 18)).astype(np.float32)
    for k in (1024, 100):
        check_topk(cuda, x, k, -1, True)
        check_topk(cuda, x, k, -1, False)
    y = rng.integers(0, 3, (4, 70001)).astype(np.float32)     # thousands of copies of each value
    for k in (10, 2000):
        check_topk(cuda, y, k, -1, True)
        check_topk(cuda, y, k, -1, False)
    z = np.full((3, 50000), 7.0, dtype=np.float32)             # every element ties
    check_topk(cuda, z, 1500, -1, True)
    check_topk(cuda, z, 1500, -1, False)


def test_adversarial_orders(cuda):
    """Ascending rows force a buffer cut at almost every tile; descending rows never append."""
    n = 120000
    asc = np.arange(n, dtype=np.float32)[None, :].repeat(2, 0)
    for x in (asc, asc[:, ::-1].copy()):
        for k in (64, 1024):
            check_topk(cuda, x, k, -1, True)
            check_topk(cuda, x, k, -1, False)


def test_special_values(cuda):
    rng = np.random.default_rng(26)
    x = rng.standard_normal((4, 30000)).astype(np.float32)
    x[:, ::7] = np.nan
    x[:, 5::11] = 0.0
    x[:, 6::11] = -0.0
    x[0, 100] = np.inf
    x[1, 200] = -np.inf
    for k in (5, 300):
        check_topk(cuda, x, k, -1, True)
        check_topk(cuda, x, k, -1, False)
    few = np.full((2, 20000), np.nan, dtype=np.float32)        # fewer numbers than k: NaNs fill up
    few[:, 3] = 1.0
    few[:, 17000] = 2.0
    check_topk(cuda, few, 10, -1, True)
    check_topk(cuda, few, 10, -1, False)
    short = np.array([[np.nan, 1.0, -0.0, 0.0, np.nan, 3.0]], dtype=np.float32)
    check_topk(cuda, short, 6, -1, True, oracle="sort")
    check_topk(cuda, short, 6, -1, False, oracle="sort")


def test_other_dims_and_views(cuda):
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O
    rng = np.random.default_rng(27)
    x = rng.standard_normal((6, 5000, 9)).astype(np.float32)
    for dim in (0, 1, 2, -2):
        k = min(4, x.shape[dim])
        check_topk(cuda, x, k, dim, True)
    # a strided view: every other column of a wider matrix, rows not 16-byte aligned
    base = rng.standard_normal((5, 40011)).astype(np.float32)
    bg = torch.from_numpy(base).to(cuda)
    for view_np, view_g in [(base[:, 1:], bg[:, 1:]), (base[:, ::2], bg[:, ::2])]:
        v, i = tpb.topk(view_g, 33, -1, True)
        wv, wi = O.topk(np.ascontiguousarray(view_np), 33, -1, True)
        assert_index_equal(i.cpu().numpy(), wi)
        assert_bits_equal(v.cpu().numpy(), wv)


@pytest.mark.parametrize("warps,slices", [("4", "1"), ("4", "3"), ("8", "2"), ("16", "1")])
def test_small_k_kernel_geometries(cuda, warps, slices, monkeypatch):
    """k <= 64 runs the barrier-free ring kernel; every CTA width and a row split give the same
    bit-exact answer, and no device-side wait gives up."""
    from tensorplay_b200 import _lib
    monkeypatch.setenv("TPB200_TOPK_WARPS", warps)
    monkeypatch.setenv("TPB200_TOPK_SLICES", slices)
    rng = np.random.default_rng(31)
    x = rng.standard_normal((3, 70001)).astype(np.float32)
    x[0, ::5] = 3.0                                   # 14001 ties above the threshold: chunk after chunk is cut
    x[1, 60000:] = np.nan
    x[2] = np.sort(x[2])                              # ascending: every element beats the threshold
    for k in (1, 8, 33, 64):
        check_topk(cuda, x, k, -1, True, what=f"warps={warps} S={slices}")
        check_topk(cuda, x, k, -1, False, what=f"warps={warps} S={slices}")
    nan_rows = np.full((2, 50000), np.nan, dtype=np.float32)   # fewer numbers than k: NaNs fill up by index
    nan_rows[:, 7] = 1.0
    nan_rows[:, 49999] = -2.0
    check_topk(cuda, nan_rows, 40, -1, True)
    check_topk(cuda, nan_rows, 40, -1, False)
    zeros = np.zeros((2, 30000), dtype=np.float32)              # the sign of zero must come back bit-exact
    zeros[:, 1::2] = -0.0
    check_topk(cuda, zeros, 16, -1, True)
    check_topk(cuda, zeros, 16, -1, False)
    assert _lib.device_status() == 0


def test_large_k_on_strided_rows(cuda):
    """k in the hundreds along a strided dim: the rendezvous kernel's scalar-load path, with the
    bootstrap that takes four values per lane, on rows with ties, NaNs and both zeros."""
    rng = np.random.default_rng(33)
    x = rng.integers(-50, 50, (40000, 6)).astype(np.float32)
    x[::13, 2] = np.nan
    x[5::17, 3] = -0.0
    for k in (200, 700):
        check_topk(cuda, x, k, 0, True)
        check_topk(cuda, x, k, 0, False)
    y = rng.standard_normal((3, 90001)).astype(np.float32)[:, 1:]      # rows not 16-byte aligned
    check_topk(cuda, np.ascontiguousarray(y), 1000, -1, True)


def test_errors(cuda):
    import torch
    import tensorplay_b200 as tpb
    x = torch.ones(3, 10, device=cuda)
    with pytest.raises(RuntimeError, match="selected index k out of range"):
        tpb.topk(x, 11)
    with pytest.raises(RuntimeError, match="Dimension out of range"):
        tpb.topk(x, 1, 2)
    v, i = tpb.topk(x, 0)
    assert v.shape == (3, 0) and i.shape == (3, 0)
    with pytest.raises(NotImplementedError):
        tpb.topk(torch.ones(2, 100000, device=cuda), 3000)


def test_config2_logits(cuda):
    """BASELINE config 2: [256, 151936] N(0, 2), 64 planted +8.0 per row, k = 50."""
    x = config2()
    check_topk(cuda, x, 50, -1, True)


def test_config5_tie_heavy_rows(cuda):
    """BASELINE config 5 at 64 of its 512 rows (one GPU's share at 8 GPUs; same generator and seed):
    integers 0..999 as float, k = 1024, both directions."""
    x = config5(rows=64)
    check_topk(cuda, x, 1024, -1, True)
    check_topk(cuda, x, 1024, -1, False)
