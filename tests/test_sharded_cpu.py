"""CPU tests of the multi-GPU host logic: partition arithmetic, and the ShardedReducer protocol
(record slot per rank -> all-gather -> rank-ordered merge) on two gloo ranks with a numpy
stand-in for the kernels (tests/fake_backend.py)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def test_row_block_and_flat_partition_cover_exactly():
    from tensorplay_b200 import flat_partition, row_block
    for rows in (0, 1, 7, 256, 512, 4096, 1000003):
        for world in (1, 2, 3, 4, 8):
            blocks = [row_block(rows, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
            sizes = [b - a for a, b in blocks]
            assert max(sizes) - min(sizes) <= 1
    for numel in (0, 5, 4096, (1 << 31), (1 << 31) + 3, 12345677):
        for world in (1, 2, 4, 8):
            parts = [flat_partition(numel, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == numel
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            assert all(a % 4 == 0 for a, b in parts if b > a)   # non-empty parts start 16-byte aligned
    assert flat_partition(1 << 31, 3, 8) == (3 << 28, 4 << 28)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total, ret):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fake_backend import NumpyBackend
        from tensorplay_b200 import ShardedReducer, flat_partition
        rng = np.random.default_rng(3)
        full = rng.uniform(-1, 1, total).astype(np.float32)
        full[rng.choice(total, total // 100, replace=False)] = 1e4
        full[total // 2 + 5] = 2e4
        full[total // 2 + 900] = 2e4          # tie across the partition boundary region: lowest index wins
        a, b = flat_partition(total, rank, world)
        local = torch.from_numpy(full[a:b].copy())
        red = ShardedReducer(device=torch.device("cpu"), backend=NumpyBackend())
        out = {}
        for op in ("sum", "mean", "var", "std", "max", "argmax", "min", "argmin", "max_argmax"):
            v, i = red.reduce(op, local, a, total)
            out[op] = (None if v is None else float(v[0]), None if i is None else int(i[0]))
        tv, ti = red.topk(local, 16, a, True)
        out["topk"] = (tv.numpy().tolist(), ti.numpy().tolist())
        sv, si = red.topk(local, 16, a, False)
        out["topk_small"] = (sv.numpy().tolist(), si.numpy().tolist())
        ret[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_reducer_protocol_on_gloo(world):
    total = 100003
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, total, ret), nprocs=world, join=True)
    assert len(ret) == world
    # every rank holds the same answer
    assert all(ret[r] == ret[0] for r in range(world))
    rng = np.random.default_rng(3)
    full = rng.uniform(-1, 1, total).astype(np.float32)
    full[rng.choice(total, total // 100, replace=False)] = 1e4
    full[total // 2 + 5] = 2e4
    full[total // 2 + 900] = 2e4
    f64 = full.astype(np.float64)
    got = ret[0]
    assert abs(got["sum"][0] - f64.sum()) <= 1e-5 * abs(f64.sum())
    assert abs(got["mean"][0] - f64.mean()) <= 1e-5 * abs(f64.mean())
    assert abs(got["var"][0] - f64.var(ddof=1)) <= 1e-5 * f64.var(ddof=1)
    assert abs(got["std"][0] - f64.std(ddof=1)) <= 1e-5 * f64.std(ddof=1)
    assert got["max"] == (2e4, None) and got["argmax"] == (None, total // 2 + 5)
    assert got["max_argmax"] == (2e4, total // 2 + 5)
    assert got["argmin"][1] == int(np.argmin(full)) and got["min"][0] == float(full.min())
    from oracle import oracle as O
    wv, wi = O.topk(full[None, :], 16, -1, True)
    assert got["topk"][1] == wi[0].tolist() and got["topk"][0] == wv[0].tolist()
    wv, wi = O.topk(full[None, :], 16, -1, False)
    assert got["topk_small"][1] == wi[0].tolist()


def test_sharded_reducer_single_process_uses_no_collective():
    sys.path.insert(0, HERE)
    from fake_backend import NumpyBackend
    from tensorplay_b200 import ShardedReducer
    x = torch.arange(1000, dtype=torch.float32)
    red = ShardedReducer(device=torch.device("cpu"), backend=NumpyBackend())
    assert red.world == 1
    v, i = red.reduce("max_argmax", x, 0, 1000)
    assert float(v[0]) == 999.0 and int(i[0]) == 999
    v, _ = red.reduce("sum", x, 0, 1000)
    assert float(v[0]) == 499500.0
    with pytest.raises(ValueError):
        red.reduce("sum", x.reshape(10, 100), 0, 1000)
    with pytest.raises(ValueError):
        red.topk(x[:5], 6, 0)
