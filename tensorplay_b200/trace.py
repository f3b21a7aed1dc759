"""Phase timing of the whole-tensor exchange from the development build with %globaltimer stamps.

    python -m tensorplay_b200.build --trace
    TPB200_TRACE=1 python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29533 -m tensorplay_b200.trace exchange --elements 2147483648 --steps 20

Every rank reduces its flat partition of a tensor of `--elements` floats with the fused exchange
(slice kernel, then the kernel that merges the slices, stores its 40-byte record and flag into every
rank's buffer, waits for all flags and merges the records), one step at a time, and reads the stamps
after each step.  Rank 0 prints, per phase, the median over steps of each rank's duration, and the step
time seen by CUDA events.  Stamps are each GPU's own %globaltimer: only differences on one GPU are
used.  The stamped build is a diagnostic: its numbers are not benchmark values (a stamp costs about
half a microsecond).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics


def exchange(args) -> None:
    import torch
    import torch.distributed as dist

    import tensorplay_b200 as tpb
    from tensorplay_b200 import _lib

    if not _lib.TRACE:
        raise SystemExit("set TPB200_TRACE=1 (and build with `python -m tensorplay_b200.build --trace`)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    L.tpb200_debug_reduce_trace.restype = ctypes.c_int
    L.tpb200_debug_reduce_trace.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int]
    total = int(args.elements)
    start, stop = tpb.flat_partition(total, rank, world)
    x = torch.empty(stop - start, device=dev)
    step = 1 << 26
    gen = torch.Generator(device=dev).manual_seed(99 + rank)
    for s in range(0, stop - start, step):
        x[s:s + step] = torch.rand(min(step, stop - start - s), device=dev, generator=gen) * 2.0 - 1.0
    red = tpb.ShardedReducer(dev, fused=True)
    buf = (ctypes.c_uint64 * 8)()
    phases = {k: [] for k in ("slice_kernel", "gap_to_exchange_kernel", "merge_own_slices", "publish_to_peers",
                             "wait_for_all_flags", "merge_records_and_write", "first_cta_to_result", "event_step")}
    for it in range(args.steps + 3):
        torch.cuda.synchronize()
        assert L.tpb200_debug_reduce_trace(buf, 8) == 0        # re-arm
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        red.reduce(args.op, x, start, total)
        e1.record()
        torch.cuda.synchronize()
        assert L.tpb200_debug_reduce_trace(buf, 8) == 0
        t = [int(v) for v in buf]
        if it < 3:
            continue
        phases["slice_kernel"].append((t[1] - t[0]) / 1e3)
        phases["gap_to_exchange_kernel"].append((t[2] - t[1]) / 1e3)
        phases["merge_own_slices"].append((t[3] - t[2]) / 1e3)
        phases["publish_to_peers"].append((t[4] - t[3]) / 1e3)
        phases["wait_for_all_flags"].append((t[5] - t[4]) / 1e3)
        phases["merge_records_and_write"].append((t[6] - t[5]) / 1e3)
        phases["first_cta_to_result"].append((t[6] - t[0]) / 1e3)
        phases["event_step"].append(e0.elapsed_time(e1) * 1e3)
    mine = {k: round(statistics.median(v), 2) for k, v in phases.items()}
    rows = [None] * world
    if world > 1:
        dist.all_gather_object(rows, mine)
    else:
        rows = [mine]
    if rank == 0:
        out = {"op": args.op, "elements": total, "world": world, "steps": args.steps, "unit": "us (median over steps)",
               "per_rank": rows,
               "max_over_ranks": {k: max(r[k] for r in rows) for k in mine},
               "min_over_ranks": {k: min(r[k] for r in rows) for k in mine}}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    ex = sub.add_parser("exchange")
    ex.add_argument("--elements", type=int, default=1 << 31)
    ex.add_argument("--steps", type=int, default=20)
    ex.add_argument("--op", default="sum")
    args = ap.parse_args()
    exchange(args)


if __name__ == "__main__":
    main()
