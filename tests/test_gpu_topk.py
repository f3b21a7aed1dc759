"""GPU parity of top-k against the CPU oracle, through the C ABI.  Values and indices must be
bit-exact, including the tie order (ties in ascending index)."""
import numpy as np
import pytest

from util import assert_bits_equal, assert_index_equal, config2, config5

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["select", "scan"], autouse=True)
def topk_path(request, monkeypatch):
    """Every test runs twice: with the sampled-threshold kernel (the default for long rows; it redoes
    the rows that fail its check with the scanning kernel's body) and with the scanning kernels alone."""
    # "2": the sampled-threshold kernel wherever it applies, also where the planner would prefer the ring
    # kernel (k <= 64 with rows enough to fill the GPU)
    monkeypatch.setenv("TPB200_TOPK_SELECT", "2" if request.param == "select" else "0")
    return request.param


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


def test_warp_per_row_kernel(cuda):
    """Rows of at most 4096 elements with k <= 64 (a warp per row): every tile count, ragged lengths,
    strided and unaligned rows, k at both ends, ties, NaN and zeros of both signs, and rows with more
    than 256 elements at the threshold (all equal, two values), which take the selection path."""
    import torch
    import tensorplay_b200 as tpb
    from tensorplay_b200 import _lib
    rng = np.random.default_rng(29)
    assert _lib.topk_plan_info([4100, 1000], [1000, 1], 1, 10)["scan_kernel"] == 4
    for shape, ks in [((4100, 100), [1, 10, 64]), ((300, 1000), [1, 7, 33, 64]), ((70, 1024), [64]), ((50, 1025), [5, 40]),
                      ((33, 2048), [50]), ((17, 3000), [32, 64]), ((9, 4096), [1, 64]), ((5, 40), [40]), ((3, 64), [64]),
                      ((6, 70), [64])]:
        x = rng.standard_normal(shape).astype(np.float32)
        x[::3, 1] = x[::3, 0]                         # a tie at the front of some rows
        if shape[1] > 8:
            x[1, 3] = np.nan
            x[2, 5] = 0.0
            x[2, 6] = -0.0
        for k in ks:
            for largest in (True, False):
                check_topk(cuda, x, k, -1, largest, oracle="sort")
    # tie-heavy rows: more than 256 elements reach the threshold
    for x in (np.ones((6, 3000), dtype=np.float32), rng.integers(0, 2, (8, 4096)).astype(np.float32),
              rng.integers(0, 3, (5, 700)).astype(np.float32)):
        for k in (1, 20, 64):
            for largest in (True, False):
                check_topk(cuda, x, k, -1, largest, oracle="sort")
    # a strided view (every other column) and rows that are not 16-byte aligned
    from oracle import oracle as O
    wide = rng.standard_normal((200, 2051)).astype(np.float32)
    wg = torch.from_numpy(wide).to(cuda)
    for vn, vg in ((wide[:, ::2], wg[:, ::2]), (wide[:, 1:1026], wg[:, 1:1026]), (wide[::2, 3:], wg[::2, 3:])):
        gv, gi = tpb.topk(vg, 16, -1, True, True)        # the views are read in place
        wv, wi = O.topk_sort(np.ascontiguousarray(vn), 16, -1, True)
        assert_index_equal(gi.cpu().numpy(), wi, "strided view")
        assert_bits_equal(gv.cpu().numpy(), wv, "strided view")
    # a middle dim
    y = rng.standard_normal((12, 500, 7)).astype(np.float32)
    check_topk(cuda, y, 9, 1, False, oracle="sort")
    assert _lib.device_status() == 0


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
    monkeypatch.setenv("TPB200_TOPK_SLICES", slices)   # slices of the scanning kernels (second launch / alone)
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


@pytest.mark.parametrize("warps,slices", [("16", "1"), ("16", "2"), ("8", "4"), ("4", "8"), ("8", "1")])
def test_select_kernel_geometries(cuda, warps, slices, monkeypatch, topk_path):
    """The sampled-threshold kernel with one CTA per row and with clusters of 2, 4 and 8 CTAs per row
    (candidates merged through distributed shared memory), on rows that pass its check and on rows
    it has to scan a second time: ascending rows (the sample says nothing about the rest),
    all-equal rows (every element is a candidate) and rows with fewer numbers than k."""
    if topk_path != "select":
        pytest.skip("select path only")
    from tensorplay_b200 import _lib
    monkeypatch.setenv("TPB200_SEL_WARPS", warps)
    monkeypatch.setenv("TPB200_SEL_SLICES", slices)
    rng = np.random.default_rng(41)
    n = 300007
    x = rng.standard_normal((6, n)).astype(np.float32)
    x[1, ::3] = 2.5                                    # 100 k ties far above the threshold: overflow, redone
    x[2] = np.sort(x[2])                               # ascending
    x[3] = rng.integers(0, 1000, n).astype(np.float32)  # tie-heavy
    x[4, 5000:] = np.nan                               # numbers only at the start
    x[5, :] = np.nan
    x[5, 123456] = 1.0                                 # fewer numbers than k
    for k in (1, 50, 64, 300, 1024, 2048):
        for largest in (True, False):
            check_topk(cuda, x, k, -1, largest, what=f"select warps={warps} S={slices}")
    y = rng.standard_normal((3, 100003)).astype(np.float32)[:, 3:]     # rows not 16-byte aligned: scalar loads
    check_topk(cuda, np.ascontiguousarray(y), 40, -1, True)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("rank,pdl", [("1", "1"), ("1", "0"), ("90", "1")])
def test_select_rows_redone(cuda, rank, pdl, monkeypatch, topk_path):
    """A threshold taken too high (rank 1: the sample's maximum) leaves fewer than k candidates in
    every row, one taken too low overflows the candidate buffer: either way the check fails and the
    CTA scans the row again -- launched as a dependent launch and as an ordinary one."""
    if topk_path != "select":
        pytest.skip("select path only")
    from tensorplay_b200 import _lib
    monkeypatch.setenv("TPB200_SEL_RANK", rank)
    monkeypatch.setenv("TPB200_PDL", pdl)
    rng = np.random.default_rng(42)
    x = rng.standard_normal((9, 200000)).astype(np.float32)
    for k in (50, 700):
        check_topk(cuda, x, k, -1, True, what=f"rank={rank} pdl={pdl}")
        check_topk(cuda, x, k, -1, False, what=f"rank={rank} pdl={pdl}")
    assert _lib.device_status() == 0


def test_select_many_calls_in_one_graph(cuda, topk_path):
    """Several calls captured in one CUDA graph (cluster launches, each a dependent launch of the one
    before) give the same bits as eager calls."""
    if topk_path != "select":
        pytest.skip("select path only")
    import torch
    import tensorplay_b200 as tpb
    rng = np.random.default_rng(43)
    xs = [torch.from_numpy(rng.standard_normal((16, 150000)).astype(np.float32)).to(cuda) for _ in range(3)]
    xs[1][3] = torch.sort(xs[1][3]).values          # one row of one input fails the check and is scanned again
    eager = [tpb.topk(x, 50) for x in xs]
    outs = [(torch.empty(16, 50, device=cuda), torch.empty(16, 50, dtype=torch.int64, device=cuda)) for _ in xs]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for x, o in zip(xs, outs):
            tpb.topk(x, 50, out=o)                  # warm-up outside the capture (workspace allocation)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for x, o in zip(xs, outs):
                tpb.topk(x, 50, out=o)
        for o in outs:
            o[0].zero_(); o[1].zero_()
        graph.replay()
        stream.synchronize()
    for (ev, ei), (gv, gi) in zip(eager, outs):
        assert torch.equal(ei, gi) and torch.equal(ev.view(torch.int32), gv.view(torch.int32))


def test_one_long_row_small_k(cuda):
    """One row of 2^26 elements, k = 56 and 64: the slices of the ring kernel are limited by what
    the merge kernel can sort in shared memory."""
    rng = np.random.default_rng(44)
    x = rng.standard_normal((1, 1 << 26)).astype(np.float32)
    for k in (56, 64):
        check_topk(cuda, x, k, -1, True)
        check_topk(cuda, x, k, -1, False)


def test_more_rows_than_a_grid_dimension(cuda):
    """70 000 rows of 4100 elements: rows ride on grid.x, so the 65 535 limit of grid.y is gone."""
    rng = np.random.default_rng(45)
    x = rng.integers(0, 50, (70000, 4100)).astype(np.float32)
    check_topk(cuda, x, 5, -1, True)
    check_topk(cuda, x, 100, -1, False)


def test_logits_256x151936_k50(cuda):
    """[256, 151936] N(0, 2) with 64 planted +8.0 per row, k = 50 (the headline shape, full size)."""
    x = config2()
    check_topk(cuda, x, 50, -1, True)


def test_tie_heavy_512x1048576_k1024(cuda):
    """[512, 1048576] integers 0..999 as float, k = 1024, both directions, all 512 rows: the answer is
    decided by the tie rule alone."""
    x = config5()
    check_topk(cuda, x, 1024, -1, True)
    check_topk(cuda, x, 1024, -1, False)
