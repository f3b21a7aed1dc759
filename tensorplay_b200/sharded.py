"""Single-box multi-GPU layer: one process per GPU, torch.distributed for the plumbing.

The reference has no multi-GPU support of any kind (its allocator pins device 0:
p10/src/backend/cuda/CUDAAllocator.cpp:87-88), so the contract here is "the same answer as the
one-GPU kernel on the un-sharded tensor".

* Independent rows (last-dim reductions, top-k along a dim): rows are split in contiguous blocks,
  every rank runs the ordinary kernels on its block, nothing is exchanged (`row_block`).
* Whole-tensor reductions: rank g owns the flat partition [offset_g, offset_g + n_g).  Its kernel
  writes ONE packed 40-byte record straight into slot g of the all-gather buffer
  (tpb200_reduce_partial), one all-gather moves the records, and every rank merges the G records
  in rank order (tpb200_reduce_combine): Chan's update for (count, mean, M2), lowest global index
  on extremum ties.  Rank order is fixed, so all ranks get bit-identical results.  An all-reduce
  could not express the Welford / arg-extremum merges and would make the float sum order
  depend on the collective algorithm.
* Global top-k over a flat sharded tensor: local top-k per rank, one all-gather of k (value,
  local index) pairs per rank, then tpb200_topk_merge over the G*k candidates with the rank
  offsets applied in the kernel.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib

_FAMILY = {"sum": "sum", "mean": "sum", "var": "var", "std": "var",
           "max": "max_argmax", "argmax": "max_argmax", "max_argmax": "max_argmax",
           "min": "min_argmin", "argmin": "min_argmin", "min_argmin": "min_argmin"}


def row_block(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block [start, stop) of `rows` owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def flat_partition(numel: int, rank: int, world: int, align: int = 4) -> tuple[int, int]:
    """Flat partition [start, stop) of a tensor of `numel` elements; starts are multiples of
    `align` elements so that every partition keeps 16-byte aligned vector loads."""
    per = -(-numel // world)
    per = -(-per // align) * align
    start = min(rank * per, numel)
    return start, min(start + per, numel)


class _CudaBackend:
    """The product backend: libtpb200.so kernels on the current CUDA stream."""

    def __init__(self, device: torch.device):
        self.device = device
        self.lib = _lib.lib()
        self._ws = None

    def workspace(self, nbytes: int):
        if nbytes == 0:
            return None, 0
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return self._ws.data_ptr(), self._ws.numel()

    def stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def partial(self, family: str, x: torch.Tensor, offset: int, slot: torch.Tensor) -> None:
        n = x.numel()
        fam = _lib.OP[family]
        ws, wsn = self.workspace(self.lib.tpb200_reduce_partial_workspace_bytes(fam, _lib.F32, n))
        _lib.check(self.lib.tpb200_reduce_partial(fam, x.data_ptr() if n else None, _lib.F32, n, offset,
                                                  slot.data_ptr(), ws, wsn, self.stream()))

    def fused(self, op: str, x: torch.Tensor, offset: int, total: int, correction: int, rank: int, world: int,
              peer_ptrs, out_val, out_idx) -> None:
        import ctypes
        n = x.numel()
        fam = _lib.OP[op]
        ws, wsn = self.workspace(self.lib.tpb200_reduce_partial_workspace_bytes(fam, _lib.F32, n))
        arr = (ctypes.c_void_p * world)(*peer_ptrs)
        _lib.check(self.lib.tpb200_reduce_fused_exchange(
            fam, x.data_ptr() if n else None, _lib.F32, n, offset, total, correction, rank, world, arr,
            out_val.data_ptr() if out_val is not None else None,
            out_idx.data_ptr() if out_idx is not None else None, ws, wsn, self.stream()))

    def combine(self, op: str, records: torch.Tensor, n_parts: int, total: int, correction: int,
                out_val, out_idx) -> None:
        _lib.check(self.lib.tpb200_reduce_combine(
            _lib.OP[op], records.data_ptr(), n_parts, total, correction,
            out_val.data_ptr() if out_val is not None else None,
            out_idx.data_ptr() if out_idx is not None else None, self.stream()))

    def topk_local(self, x: torch.Tensor, k: int, largest: bool, out_val, out_idx) -> None:
        sizes = _lib.i64_array([x.numel()])
        strides = _lib.i64_array([1])
        ws, wsn = self.workspace(self.lib.tpb200_topk_workspace_bytes(_lib.F32, 1, sizes, strides, 0, k))
        _lib.check(self.lib.tpb200_topk(x.data_ptr(), _lib.F32, 1, sizes, strides, 0, k, int(largest), 1,
                                        out_val.data_ptr(), out_idx.data_ptr(), ws, wsn, self.stream()))

    def topk_merge(self, cand_val, cand_idx, n_cand, k, largest, offsets, list_len, out_val, out_idx):
        _lib.check(self.lib.tpb200_topk_merge(
            cand_val.data_ptr(), cand_idx.data_ptr(), n_cand, k, int(largest),
            offsets.data_ptr() if offsets is not None else None, list_len,
            out_val.data_ptr(), out_idx.data_ptr(), self.stream()))


class ShardedReducer:
    """Whole-tensor reductions and global top-k over a flat tensor sharded across the ranks of a
    process group.  Buffers are allocated once; a call enqueues kernel -> all-gather -> kernel.

    `backend` exists so that the host logic (partitioning, record exchange, rank-ordered merge)
    can be driven by CPU ranks over gloo in tests; the default is the CUDA library and there is
    no other product backend.
    """

    def __init__(self, device: torch.device | None = None, group=None, backend=None, fused: bool = False):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if backend is None:
            if device is None:
                device = torch.device("cuda", torch.cuda.current_device())
            backend = _CudaBackend(device)
        self.backend = backend
        self.device = device if device is not None else torch.device("cpu")
        # all-gather buffer: one packed record per rank; slot `rank` is the kernel's output
        self.records = torch.zeros(self.world, _lib.PARTIAL_BYTES, dtype=torch.uint8, device=self.device)
        self.out_val = torch.empty(1, dtype=torch.float32, device=self.device)
        self.out_idx = torch.empty(1, dtype=torch.int64, device=self.device)
        self._cand = {}
        # fused = True: whole-tensor reductions exchange their records inside the reduction kernel,
        # by peer-to-peer stores into symmetric memory (NVLink), instead of an NCCL all-gather
        self.peer_ptrs = None
        if fused:
            self._setup_exchange()

    def _setup_exchange(self) -> None:
        nbytes = self.backend.lib.tpb200_exchange_buffer_bytes()
        if self.world == 1:
            self._xbuf = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            self.peer_ptrs = [self._xbuf.data_ptr()]
            return
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer mappings only
        import torch.distributed._symmetric_memory as symm_mem
        self._xbuf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._xhdl = symm_mem.rendezvous(self._xbuf, self.group if self.group is not None else dist.group.WORLD)
        self._xbuf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.peer_ptrs = [int(p) for p in self._xhdl.buffer_ptrs]

    # -- whole-tensor reductions ---------------------------------------------------------
    def reduce(self, op: str, local: torch.Tensor, global_offset: int, total_count: int, correction: int = 1):
        """`local` is this rank's contiguous flat partition, starting at element `global_offset`
        of a tensor with `total_count` elements.  Returns (value tensor | None, index tensor | None),
        identical on every rank."""
        if op not in _FAMILY:
            raise ValueError(f"unknown reduction {op!r}")
        if local.dim() != 1 or not local.is_contiguous():
            raise ValueError("the local partition must be a contiguous 1-D tensor")
        want_val = op not in ("argmax", "argmin")
        want_idx = op in ("argmax", "argmin", "max_argmax", "min_argmin")
        if self.peer_ptrs is not None:
            self.backend.fused(op, local, int(global_offset), int(total_count), int(correction), self.rank,
                               self.world, self.peer_ptrs, self.out_val if want_val else None,
                               self.out_idx if want_idx else None)
            return (self.out_val if want_val else None), (self.out_idx if want_idx else None)
        self.backend.partial(_FAMILY[op], local, int(global_offset), self.records[self.rank])
        if self.world > 1:
            dist.all_gather_into_tensor(self.records.view(-1), self.records[self.rank], group=self.group)
        want_val = op not in ("argmax", "argmin")
        want_idx = op in ("argmax", "argmin", "max_argmax", "min_argmin")
        self.backend.combine(op, self.records, self.world, int(total_count), int(correction),
                             self.out_val if want_val else None, self.out_idx if want_idx else None)
        return (self.out_val if want_val else None), (self.out_idx if want_idx else None)

    # -- global top-k ----------------------------------------------------------------------
    def topk(self, local: torch.Tensor, k: int, global_offset: int, largest: bool = True):
        """Top-k of the whole flat tensor; `local` as in reduce().  Every rank must hold at least
        k elements.  Returns (values [k], global indices [k]), identical on every rank."""
        if local.dim() != 1 or not local.is_contiguous():
            raise ValueError("the local partition must be a contiguous 1-D tensor")
        if k > local.numel():
            raise ValueError("every rank must hold at least k elements")
        key = int(k)
        if key not in self._cand:
            self._cand[key] = (
                torch.empty(self.world, k, dtype=torch.float32, device=self.device),
                torch.empty(self.world, k, dtype=torch.int64, device=self.device),
                torch.empty(self.world, dtype=torch.int64, device=self.device),
                torch.empty(k, dtype=torch.float32, device=self.device),
                torch.empty(k, dtype=torch.int64, device=self.device),
                torch.empty(1, dtype=torch.int64, device=self.device),
            )
        cv, ci, offs, ov, oi, my_off = self._cand[key]
        self.backend.topk_local(local, k, largest, cv[self.rank], ci[self.rank])
        if self.world > 1:
            my_off.fill_(int(global_offset))
            dist.all_gather_into_tensor(cv.view(-1), cv[self.rank], group=self.group)
            dist.all_gather_into_tensor(ci.view(-1), ci[self.rank], group=self.group)
            dist.all_gather_into_tensor(offs, my_off, group=self.group)
        else:
            offs.fill_(int(global_offset))
        self.backend.topk_merge(cv, ci, self.world * k, k, largest, offs, k, ov, oi)
        return ov, oi
