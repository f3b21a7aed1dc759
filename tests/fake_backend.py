"""Test-only stand-in for the CUDA backend of tensorplay_b200.sharded.ShardedReducer: produces and
merges the same 40-byte packed records with numpy, so the host logic (partitioning, record
exchange, rank-ordered merge, index offsets) can run on CPU ranks over gloo."""
import struct

import numpy as np
import torch

FMT = "<dddqfI"
NO_INDEX = 0x7FFFFFFFFFFFFFFF
assert struct.calcsize(FMT) == 40


class NumpyBackend:
    def partial(self, family, x, offset, slot):
        a = x.numpy().astype(np.float64)
        n = a.size
        if family == "sum":
            rec = (a.sum(), 0.0, 0.0, 0, 0.0, 0)
        elif family == "var":
            m = a.mean() if n else 0.0
            rec = (float(n), m, ((a - m) ** 2).sum() if n else 0.0, 0, 0.0, 0)
        else:
            x32 = x.numpy()
            if family == "max_argmax":
                ok = x32 > -np.inf
                i = int(np.argmax(np.where(np.isnan(x32), -np.inf, x32))) if ok.any() else -1
            else:
                ok = x32 < np.inf
                i = int(np.argmin(np.where(np.isnan(x32), np.inf, x32))) if ok.any() else -1
            if i < 0:
                rec = (0.0, 0.0, 0.0, NO_INDEX, -np.inf if family == "max_argmax" else np.inf, 0)
            else:
                rec = (0.0, 0.0, 0.0, i + offset, float(x32[i]), 0)
        slot.copy_(torch.frombuffer(bytearray(struct.pack(FMT, *rec)), dtype=torch.uint8))

    def combine(self, op, records, n_parts, total, correction, out_val, out_idx):
        recs = [struct.unpack(FMT, bytes(records[i].numpy().tobytes())) for i in range(n_parts)]
        if op in ("sum", "mean"):
            s = 0.0
            for r in recs:
                s += r[0]
            out_val[0] = float(np.float32(s / total if op == "mean" else s))
        elif op in ("var", "std"):
            n, mean, m2 = 0.0, 0.0, 0.0
            for r in recs:
                if r[0] == 0:
                    continue
                if n == 0:
                    n, mean, m2 = r[0], r[1], r[2]
                    continue
                nt = n + r[0]
                d = r[1] - mean
                w = r[0] / nt
                mean += d * w
                m2 += r[2] + d * d * n * w
                n = nt
            dv = max(0.0, total - correction)
            v = np.float32(m2 / dv) if dv > 0 else np.float32(np.inf if m2 > 0 else np.nan)
            out_val[0] = float(np.sqrt(v) if op == "std" else v)
        else:
            is_max = op in ("max", "argmax", "max_argmax")
            bv, bi = (-np.inf if is_max else np.inf), NO_INDEX
            for r in recs:
                v, i = r[4], r[3]
                better = v > bv if is_max else v < bv
                if better or (v == bv and i < bi):
                    bv, bi = v, i
            if out_val is not None:
                out_val[0] = float(np.float32(bv))
            if out_idx is not None:
                out_idx[0] = int(0 if bi == NO_INDEX else bi)

    def topk_local(self, x, k, largest, out_val, out_idx):
        from oracle import oracle as O
        v, i = O.topk(x.numpy()[None, :], k, -1, largest)
        out_val.copy_(torch.from_numpy(v[0]))
        out_idx.copy_(torch.from_numpy(i[0]))

    def topk_merge(self, cand_val, cand_idx, n_cand, k, largest, offsets, list_len, out_val, out_idx):
        v = cand_val.numpy().reshape(-1)[:n_cand]
        i = cand_idx.numpy().reshape(-1)[:n_cand].copy()
        if offsets is not None:
            i += np.repeat(offsets.numpy(), list_len)
        key = np.where(np.isnan(v), -np.inf if largest else np.inf, v)
        order = np.lexsort((i, -key if largest else key))[:k]
        out_val.copy_(torch.from_numpy(v[order]))
        out_idx.copy_(torch.from_numpy(i[order]))
