"""CPU tests of the C ABI: the shared library loads, exports every symbol include/tpb200.h
declares, and its argument checks and planners answer without a GPU (no kernel is launched)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from tensorplay_b200 import build, _lib
    build.build_library()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tpb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tpb200_[a-z_0-9]+)\s*\(", text)))


def test_exports_every_declared_symbol(lib):
    from tensorplay_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 11
    assert sorted(_lib.SYMBOLS) == names
    for n in names:
        assert hasattr(lib, n), n
    assert lib.tpb200_version() == 100


def test_argument_checks_need_no_gpu(lib):
    from tensorplay_b200 import _lib
    i64 = _lib.i64_array
    # unsupported dtype
    rc = lib.tpb200_reduce(0, None, 7, 1, i64([4]), i64([1]), 0, -1, 1, None, None, None, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"float32" in lib.tpb200_last_error()
    # unknown op
    assert lib.tpb200_reduce(99, None, 0, 1, i64([4]), i64([1]), 0, -1, 1, None, None, None, 0, None) == _lib.ERR_INVALID
    # dim out of range
    rc = lib.tpb200_reduce(0, None, 0, 2, i64([4, 4]), i64([4, 1]), 1 << 2, -1, 1, None, None, None, 0, None)
    assert rc == _lib.ERR_DIM_RANGE and lib.tpb200_last_error() == b"Dimension out of range"
    # whole-tensor max of an empty tensor
    rc = lib.tpb200_reduce(_lib.OP["max"], None, 0, 1, i64([0]), i64([1]), 0, -1, 1, None, None, None, 0, None)
    assert rc == _lib.ERR_EMPTY and b"max(): Expected reduction dim to be non-empty" in lib.tpb200_last_error()
    # missing output
    rc = lib.tpb200_reduce(0, ctypes.c_void_p(16), 0, 1, i64([4]), i64([1]), 0, -1, 1, None, None, None, 0, None)
    assert rc == _lib.ERR_INVALID
    # top-k: k out of range, bad dim, unsupported k
    assert lib.tpb200_topk(None, 0, 2, i64([3, 10]), i64([10, 1]), 1, 11, 1, 1, None, None, None, 0, None) == _lib.ERR_INVALID
    assert b"selected index k out of range" in lib.tpb200_last_error()
    assert lib.tpb200_topk(None, 0, 2, i64([3, 10]), i64([10, 1]), 2, 1, 1, 1, None, None, None, 0, None) == _lib.ERR_DIM_RANGE
    assert lib.tpb200_topk(None, 0, 2, i64([3, 100000]), i64([100000, 1]), 1, 3000, 1, 1, None, None, None, 0, None) == _lib.ERR_UNSUPPORTED
    # merge limits
    assert lib.tpb200_topk_merge(None, None, 9000, 10, 1, None, 1, None, None, None) == _lib.ERR_UNSUPPORTED
    assert lib.tpb200_reduce_combine(0, None, 0, 0, 1, None, None, None) == _lib.ERR_INVALID
    assert lib.tpb200_reduce_partial(0, None, 0, -1, 0, None, None, 0, None) == _lib.ERR_INVALID


def test_workspace_planner(lib, monkeypatch):
    from tensorplay_b200 import _lib
    i64 = _lib.i64_array
    P = _lib.PARTIAL_BYTES
    # row kernels with many rows need no scratch
    assert lib.tpb200_reduce_workspace_bytes(0, 0, 2, i64([4096, 4096]), i64([4096, 1]), 1 << 1) == 0
    # the whole tensor of 2^31 elements is split over 16 CTAs per SM, one packed record each
    n = lib.tpb200_reduce_workspace_bytes(0, 0, 1, i64([1 << 31]), i64([1]), 0)
    assert n > 0 and n % P == 0 and n // P >= 148
    assert lib.tpb200_reduce_partial_workspace_bytes(0, 0, 1 << 28) % P == 0
    # column reduction over dim 1 of [64, 4096, 512]: records for [64, S, 512]
    n = lib.tpb200_reduce_workspace_bytes(0, 0, 3, i64([64, 4096, 512]), i64([4096 * 512, 512, 1]), 1 << 1)
    assert n % (64 * 512 * P) == 0
    # top-k: short rows and the sampled-threshold kernel need no scratch; the scanning kernels alone
    # need S*k words per row when they split rows into slices
    assert lib.tpb200_topk_workspace_bytes(0, 2, i64([4, 1000]), i64([1000, 1]), 1, 5) == 0
    assert lib.tpb200_topk_workspace_bytes(0, 2, i64([8, 1 << 22]), i64([1 << 22, 1]), 1, 64) == 0
    assert _lib.topk_plan_info([8, 1 << 22], [1 << 22, 1], 1, 64)["launches"] == 1
    monkeypatch.setenv("TPB200_TOPK_SELECT", "0")
    n = lib.tpb200_topk_workspace_bytes(0, 2, i64([8, 1 << 22]), i64([1 << 22, 1]), 1, 64)
    assert n > 0 and n % (8 * 64 * 8) == 0
    assert _lib.topk_plan_info([8, 1 << 22], [1 << 22, 1], 1, 64)["launches"] == 2
    monkeypatch.delenv("TPB200_TOPK_SELECT")
    # too small a workspace is refused before any launch
    rc = lib.tpb200_reduce(0, ctypes.c_void_p(16), 0, 1, i64([1 << 31]), i64([1]), 0, -1, 1,
                           ctypes.c_void_p(16), None, ctypes.c_void_p(256), 8, None)
    assert rc == _lib.ERR_WORKSPACE


def test_topk_slices_fit_the_merge_kernel(lib, monkeypatch):
    """One very long row, k <= 64: the number of slices times k must stay within what the merge
    kernel sorts in shared memory (16384 words), whatever the row length."""
    from tensorplay_b200 import _lib
    i64 = _lib.i64_array
    monkeypatch.setenv("TPB200_TOPK_SELECT", "0")      # the scanning kernels' own workspace only
    for n in (1 << 22, 1 << 25, 1 << 26, 1 << 28, (1 << 31) + 5):
        for k in range(1, 65):
            nb = lib.tpb200_topk_workspace_bytes(0, 1, i64([n]), i64([1]), 0, k)
            words = nb // 8
            assert words % k == 0 and words <= 16384, (n, k, words)
            mergeN = 2
            while mergeN < words:
                mergeN *= 2
            assert mergeN * 8 <= 227 * 1024
    # rows ride on grid.x: more than 65535 long rows plan without an error
    assert lib.tpb200_topk(None, 0, 2, i64([70000, 8192]), i64([8192, 1]), 1, 5, 1, 1, None, None, None, 0, None) == _lib.ERR_INVALID
    assert b"input pointer is NULL" in lib.tpb200_last_error()


def test_comm_argument_checks_need_no_gpu(lib):
    """The single-process multi-GPU host refuses bad arguments before it touches a device."""
    from tensorplay_b200 import _lib
    comm = ctypes.c_void_p()
    devs = (ctypes.c_int * 1)(0)
    assert lib.tpb200_comm_create(0, devs, ctypes.byref(comm)) == _lib.ERR_UNSUPPORTED
    assert lib.tpb200_comm_create(17, devs, ctypes.byref(comm)) == _lib.ERR_UNSUPPORTED
    assert lib.tpb200_comm_create(1, None, ctypes.byref(comm)) == _lib.ERR_INVALID
    assert lib.tpb200_comm_create(1, devs, None) == _lib.ERR_INVALID
    assert lib.tpb200_comm_size(None) == 0 and lib.tpb200_comm_destroy(None) == _lib.OK
    assert lib.tpb200_reduce_sharded(None, 0, None, None, 0, 1, None, None) == _lib.ERR_INVALID
    assert lib.tpb200_topk_sharded(None, None, None, 0, 4, 1, None, None) == _lib.ERR_INVALID
