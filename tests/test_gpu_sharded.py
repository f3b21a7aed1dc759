"""GPU tests of the sharded paths.  The per-rank kernels never wait on one another, so G ranks are
emulated on one GPU by running them one after the other into the slots of the gather buffer; with
two or more GPUs the real one-process-per-GPU path over NCCL is run as well."""
import os
import socket
import sys

import numpy as np
import pytest

from util import assert_close64, config4

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_whole_tensor_partials_and_rank_ordered_combine(cuda, G):
    import torch
    import tensorplay_b200 as tpb
    from tensorplay_b200 import _lib
    from oracle import oracle as O

    n = (1 << 24) + 1237
    x = config4(n=n)
    x[n // 2] = 3e4
    x[n // 2 + G * 1000 + 1] = 3e4         # tie in a later partition: the lower global index must win
    xg = torch.from_numpy(x).to(cuda)
    L = _lib.lib()
    records = torch.zeros(G, _lib.PARTIAL_BYTES, dtype=torch.uint8, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    for fam, ops in [("sum", ["sum", "mean"]), ("var", ["var", "std"]),
                     ("max_argmax", ["max", "argmax", "max_argmax"]), ("min_argmin", ["min", "argmin"])]:
        for g in range(G):
            a, b = tpb.flat_partition(n, g, G)
            part = xg[a:b]
            nb = L.tpb200_reduce_partial_workspace_bytes(_lib.OP[fam], 0, b - a)
            ws = torch.empty(max(nb, 8), dtype=torch.uint8, device=cuda)
            _lib.check(L.tpb200_reduce_partial(_lib.OP[fam], part.data_ptr(), 0, b - a, a, records[g].data_ptr(),
                                               ws.data_ptr(), ws.numel(), st))
        for op in ops:
            ov = torch.empty(1, device=cuda)
            oi = torch.empty(1, dtype=torch.int64, device=cuda)
            want_val = op not in ("argmax", "argmin")
            want_idx = op in ("argmax", "argmin", "max_argmax")
            _lib.check(L.tpb200_reduce_combine(_lib.OP[op], records.data_ptr(), G, n, 1,
                                               ov.data_ptr() if want_val else None,
                                               oi.data_ptr() if want_idx else None, st))
            if op in ("sum", "mean", "var", "std"):
                assert_close64(ov.cpu().numpy()[0], O.truth64(op, x), f"G={G} {op}")
            else:
                base = op.replace("_argmax", "")
                if want_val:
                    assert ov.item() == float(O.reduce("max" if "max" in op else "min", x))
                if want_idx:
                    assert oi.item() == int(O.reduce("argmax" if "max" in op else "argmin", x)), (G, op)


@pytest.mark.parametrize("G", [1, 2, 8])
def test_global_topk_merge(cuda, G):
    import torch
    import tensorplay_b200 as tpb
    from tensorplay_b200 import _lib
    from oracle import oracle as O

    rng = np.random.default_rng(31)
    n = 400000
    x = rng.integers(0, 500, n).astype(np.float32)       # tie-heavy: global index order decides
    xg = torch.from_numpy(x).to(cuda)
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    for k, largest in [(64, True), (64, False), (1024, True)]:
        if G * k > 8192:
            continue
        cv = torch.empty(G, k, device=cuda)
        ci = torch.empty(G, k, dtype=torch.int64, device=cuda)
        offs = torch.empty(G, dtype=torch.int64, device=cuda)
        for g in range(G):
            a, b = tpb.flat_partition(n, g, G)
            v, i = tpb.topk(xg[a:b], k, 0, largest)
            cv[g], ci[g] = v, i
            offs[g] = a
        ov = torch.empty(k, device=cuda)
        oi = torch.empty(k, dtype=torch.int64, device=cuda)
        _lib.check(L.tpb200_topk_merge(cv.data_ptr(), ci.data_ptr(), G * k, k, int(largest), offs.data_ptr(), k,
                                       ov.data_ptr(), oi.data_ptr(), st))
        wv, wi = O.topk(x[None, :], k, -1, largest)
        assert np.array_equal(oi.cpu().numpy(), wi[0]), (G, k, largest)
        assert np.array_equal(ov.cpu().numpy().view(np.uint32), wv[0].view(np.uint32))


def test_sharded_reducer_one_rank(cuda):
    import torch
    import tensorplay_b200 as tpb
    x = torch.arange(1 << 20, dtype=torch.float32, device=cuda)
    red = tpb.ShardedReducer(cuda)
    v, i = red.reduce("max_argmax", x, 0, x.numel())
    assert v.item() == float((1 << 20) - 1) and i.item() == (1 << 20) - 1
    v, _ = red.reduce("mean", x, 0, x.numel())
    assert abs(v.item() - ((1 << 20) - 1) / 2) <= 1e-5 * ((1 << 20) - 1) / 2
    tv, ti = red.topk(x, 8, 0, True)
    assert ti.tolist() == list(range((1 << 20) - 1, (1 << 20) - 9, -1))


def test_fused_exchange_one_rank(cuda):
    """The fused kernel with a single rank exchanges with itself: ticket, epoch and parity logic over
    several calls in a row, bit-identical to the unfused path."""
    import torch
    import tensorplay_b200 as tpb
    from util import config4
    x = torch.from_numpy(config4(n=(1 << 22) + 77)).to(cuda)
    plain = tpb.ShardedReducer(cuda)
    fused = tpb.ShardedReducer(cuda, fused=True)
    for rep in range(3):
        for op in ("sum", "mean", "var", "std", "max", "argmax", "min_argmin"):
            pv, pi = plain.reduce(op, x, 0, x.numel())
            pv = None if pv is None else pv.clone()
            pi = None if pi is None else pi.clone()
            fv, fi = fused.reduce(op, x, 0, x.numel())
            if pv is not None:
                assert torch.equal(pv.view(torch.int32), fv.view(torch.int32)), (rep, op)
            if pi is not None:
                assert torch.equal(pi, fi), (rep, op)
    from tensorplay_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_single_process_comm(cuda, G):
    """tpb200_comm_*: the torch-free multi-GPU host of the C ABI.  With one physical GPU the G ranks
    are the same device listed G times (records and candidates are then copied between the gather
    buffers; no kernel waits for another); with G real GPUs the reductions exchange by peer stores."""
    import ctypes
    import torch
    import tensorplay_b200 as tpb
    from tensorplay_b200 import _lib
    from oracle import oracle as O
    L = _lib.lib()
    ndev = torch.cuda.device_count()
    devices = list(range(G)) if ndev >= G else [0] * G
    comm = ctypes.c_void_p()
    _lib.check(L.tpb200_comm_create(G, (ctypes.c_int * G)(*devices), ctypes.byref(comm)))
    try:
        assert L.tpb200_comm_size(comm) == G
        assert L.tpb200_comm_fused(comm) == (1 if (G == 1 or ndev >= G) else 0)
        n = (1 << 22) + 13 * G + 5
        x = config4(n=n)
        x[n - 77] = 3e4                      # the maximum in the last partition ...
        x[n // 3] = 3e4                      # ... tied by an earlier element: the lower index wins
        bounds = [tpb.flat_partition(n, g, G) for g in range(G)]
        parts = [torch.from_numpy(x[a:b].copy()).to(torch.device("cuda", devices[g])) for g, (a, b) in enumerate(bounds)]
        torch.cuda.synchronize()
        pp = (ctypes.c_void_p * G)(*[p.data_ptr() for p in parts])
        cc = (ctypes.c_int64 * G)(*[b - a for a, b in bounds])

        for rep in range(2):
            for op in ("sum", "mean", "var", "std", "max_argmax", "argmin"):
                want_val = op != "argmin"
                want_idx = op in ("max_argmax", "argmin")
                ovs = [torch.full((1,), float("nan"), device=torch.device("cuda", devices[g])) for g in range(G)]
                ois = [torch.full((1,), -5, dtype=torch.int64, device=torch.device("cuda", devices[g])) for g in range(G)]
                torch.cuda.synchronize()
                pv = (ctypes.c_void_p * G)(*[t.data_ptr() for t in ovs]) if want_val else None
                pi = (ctypes.c_void_p * G)(*[t.data_ptr() for t in ois]) if want_idx else None
                _lib.check(L.tpb200_reduce_sharded(comm, _lib.OP[op], pp, cc, 0, 1, pv, pi))
                _lib.check(L.tpb200_comm_synchronize(comm))
                for g in range(G):
                    if op in ("sum", "mean", "var", "std"):
                        assert_close64(ovs[g].cpu().numpy()[0], O.truth64(op, x), f"comm G={G} {op} gpu {g}")
                        assert ovs[g].cpu().view(torch.int32).item() == ovs[0].cpu().view(torch.int32).item()
                    if op == "max_argmax":
                        assert ovs[g].item() == 3e4 and ois[g].item() == n // 3
                    if op == "argmin":
                        assert ois[g].item() == int(np.argmin(x))
        # global top-k, tie-heavy: global index order decides
        y = np.random.default_rng(61).integers(0, 300, n).astype(np.float32)
        yparts = [torch.from_numpy(y[a:b].copy()).to(torch.device("cuda", devices[g])) for g, (a, b) in enumerate(bounds)]
        torch.cuda.synchronize()
        yp = (ctypes.c_void_p * G)(*[p.data_ptr() for p in yparts])
        for k, largest in ((64, True), (1000, False)):
            if G * k > 8192:
                continue
            tvs = [torch.empty(k, device=torch.device("cuda", devices[g])) for g in range(G)]
            tis = [torch.empty(k, dtype=torch.int64, device=torch.device("cuda", devices[g])) for g in range(G)]
            torch.cuda.synchronize()
            pv = (ctypes.c_void_p * G)(*[t.data_ptr() for t in tvs])
            pi = (ctypes.c_void_p * G)(*[t.data_ptr() for t in tis])
            _lib.check(L.tpb200_topk_sharded(comm, yp, cc, 0, k, int(largest), pv, pi))
            _lib.check(L.tpb200_comm_synchronize(comm))
            wv, wi = O.topk(y[None, :], k, -1, largest)
            for g in range(G):
                assert np.array_equal(tis[g].cpu().numpy(), wi[0]), (G, k, g)
                assert np.array_equal(tvs[g].cpu().numpy().view(np.uint32), wv[0].view(np.uint32))
        assert L.tpb200_topk_sharded(comm, yp, cc, 0, 5000, 1, None, None) == _lib.ERR_UNSUPPORTED
    finally:
        _lib.check(L.tpb200_comm_destroy(comm))
    assert _lib.device_status() == 0


def test_fused_exchange_wait_runs_out(cuda):
    """A rank whose peer never arrives: the wait is bounded, the kernel returns by itself with status 5
    and poisoned outputs (NaN / -1, not the previous call's answer), and the next call works.  Rank 1
    of a two-rank exchange simply never runs here; nothing faults or hangs."""
    import ctypes
    import torch
    import tensorplay_b200 as tpb
    from tensorplay_b200 import _lib
    L = _lib.lib()
    x = torch.arange(1 << 20, dtype=torch.float32, device=cuda)
    n = x.numel()
    nb = L.tpb200_exchange_buffer_bytes()
    bufs = [torch.zeros(nb, dtype=torch.uint8, device=cuda) for _ in range(2)]
    peers = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    ws = torch.empty(max(8, L.tpb200_reduce_partial_workspace_bytes(_lib.OP["sum"], 0, n)), dtype=torch.uint8, device=cuda)
    ov = torch.full((1,), 123.0, device=cuda)          # stands for the previous call's answer
    oi = torch.full((1,), 456, dtype=torch.int64, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    assert _lib.device_status() == 0
    _lib.check(L.tpb200_set_exchange_wait_polls(2000))          # a fraction of a millisecond
    try:
        _lib.check(L.tpb200_reduce_fused_exchange(_lib.OP["max_argmax"], x.data_ptr(), 0, n, 0, 2 * n, 1, 0, 2, peers,
                                                  ov.data_ptr(), oi.data_ptr(), ws.data_ptr(), ws.numel(), st))
        assert _lib.device_status() == 5                           # synchronises; reads and clears the word
        assert torch.isnan(ov).item() and oi.item() == -1
        assert _lib.device_status() == 0
    finally:
        _lib.check(L.tpb200_set_exchange_wait_polls(1 << 22))
    assert L.tpb200_set_exchange_wait_polls(0) == _lib.ERR_INVALID
    # a fresh single-rank exchange right after it
    red = tpb.ShardedReducer(cuda, fused=True)
    v, i = red.reduce("max_argmax", x, 0, n)
    assert v.item() == float(n - 1) and i.item() == n - 1
    assert _lib.device_status() == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _nccl_worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import tensorplay_b200 as tpb
        from util import config4
        n = (1 << 22) + 11
        x = config4(n=n)
        a, b = tpb.flat_partition(n, rank, world)
        local = torch.from_numpy(x[a:b].copy()).to(dev)
        red = tpb.ShardedReducer(dev)
        out = {}
        for op in ("sum", "var", "max_argmax", "argmin"):
            v, i = red.reduce(op, local, a, n)
            out[op] = (None if v is None else float(v.item()), None if i is None else int(i.item()))
        tv, ti = red.topk(local, 32, a, True)
        out["topk"] = ti.tolist()
        # the fused peer-to-peer exchange must give bit-identical results, call after call
        fused = tpb.ShardedReducer(dev, fused=True)
        for rep in range(3):
            for op in ("sum", "var", "max_argmax", "argmin"):
                v, i = fused.reduce(op, local, a, n)
                got = (None if v is None else float(v.item()), None if i is None else int(i.item()))
                assert got == out[op], (rank, rep, op, got, out[op])
        from tensorplay_b200 import _lib
        assert _lib.device_status() == 0
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_nccl(cuda):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from oracle import oracle as O
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_nccl_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret[0] == ret[1]
    n = (1 << 22) + 11
    x = config4(n=n)
    assert_close64(np.float32(ret[0]["sum"][0]), O.truth64("sum", x), "nccl sum")
    assert_close64(np.float32(ret[0]["var"][0]), O.truth64("var", x), "nccl var")
    assert ret[0]["max_argmax"][1] == int(O.reduce("argmax", x))
    assert ret[0]["argmin"][1] == int(O.reduce("argmin", x))
    assert ret[0]["topk"] == O.topk(x[None, :], 32, -1, True)[1][0].tolist()
