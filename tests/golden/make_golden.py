"""Generates tests/golden/reduce_golden.npz and tests/golden/softmax_median_golden.npz from the REFERENCE's own compiled CPU code
(oracle/_ref/libtpref.so, built by oracle/build_ref.sh from a TensorPlay checkout).

Run where the checkout exists:   python tests/golden/make_golden.py
The fixture pins the CPU restatement (tests/test_oracle.py) and the GPU kernels
(tests/test_gpu_golden.py) on machines where the reference cannot be built.
Inputs are seeded; every array is stored, so the fixture is self-contained.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402

OPS = ["sum", "mean", "var", "std", "max", "min", "argmax", "argmin", "prod", "norm", "all", "any"]


def cases():
    rng = np.random.default_rng(2024)
    shapes = [((10,), [None, [0]]),
              ((5, 5), [None, [0], [1], [0, 1]]),
              ((2, 3, 4), [None, [0], [1], [2], [0, 2], [1, 2]]),
              ((16, 257), [None, [0], [1]]),
              ((4, 33, 20), [[1], [2], [0, 2]])]
    for shape, dimss in shapes:
        x = rng.standard_normal(shape).astype(np.float32)
        if x.size > 8:
            x.flat[5] = x.flat[2]          # a tie
            x.flat[7] = np.float32(-0.0)
        for dims in dimss:
            yield x, dims
    # tie-heavy and special values
    t = rng.integers(0, 3, (6, 40)).astype(np.float32)
    for dims in (None, [0], [1]):
        yield t, dims
    s = np.array([np.nan, 1, 3, np.nan, -0.0, 0.0, 3, -np.inf], dtype=np.float32)
    for dims in (None, [0]):
        yield s, dims


def main():
    arrays, index = {}, []
    n = 0
    for x, dims in cases():
        xi = f"x{n}"
        arrays[xi] = x
        for op in OPS:
            if op in ("argmax", "argmin"):
                if dims is not None and len(dims) != 1:
                    continue
                # the reference's CPU argmax/argmin is only well-formed for the last or the
                # second-to-last dim of a >= 3-D tensor (p10/src/backend/cpu/ReductionKernels.cpp:714-735)
                if dims is not None and x.ndim >= 3 and dims[0] % x.ndim not in (x.ndim - 1, x.ndim - 2):
                    continue
            if op in ("sum", "mean", "var", "std", "prod", "norm") and not np.all(np.isfinite(x)):
                continue
            for corr in ((0, 1) if op in ("var", "std") else (1,)):
                for p in ((1.0, 2.0, "inf", "-inf") if op == "norm" else (2.0,)):
                    key = f"r{len(index)}"
                    arrays[key] = O.ref_reduce(op, x, dims, False, corr, float(p))
                    index.append({"x": xi, "op": op, "dims": dims, "correction": corr, "p": float(p), "out": key})
        n += 1
    arrays["index_json"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    out = os.path.join(HERE, "reduce_golden.npz")
    np.savez_compressed(out, **arrays)
    print(f"wrote {out}: {len(index)} results, {os.path.getsize(out)} bytes")
    more()


def more():
    """softmax / log_softmax along every dim and the whole-tensor median, from the reference's
    compiled CPU kernels (PointwiseKernels.cpp:519-546, ReductionKernels.cpp:874-901)."""
    rng = np.random.default_rng(2025)
    arrays, index = {}, []
    xs = [rng.standard_normal((7,)).astype(np.float32), (rng.standard_normal((6, 130)) * 3).astype(np.float32),
          rng.standard_normal((3, 9, 5)).astype(np.float32), rng.uniform(-30, 30, (4, 1500)).astype(np.float32)]
    xs[1][2, 5] = xs[1][2, 9] = xs[1][2].max() + 1.0            # tied maxima
    xs[2][1, :, 2] = -np.inf
    xs[2][1, 3, 2] = 0.5                                        # -inf beside one number
    for n, x in enumerate(xs):
        arrays[f"x{n}"] = x
        for d in range(x.ndim):
            for log in (0, 1):
                key = f"s{len(index)}"
                arrays[key] = O.ref_softmax(x, d, bool(log))
                index.append({"x": f"x{n}", "op": "log_softmax" if log else "softmax", "dim": d, "out": key})
        key = f"s{len(index)}"
        arrays[key] = np.array([O.ref_median(x[np.isfinite(x)].copy())], dtype=np.float32)   # numbers only: nth_element and NaN / inf ties
        arrays[f"m{n}"] = x[np.isfinite(x)].copy()
        index.append({"x": f"m{n}", "op": "median", "dim": None, "out": key})
    arrays["index_json"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    out = os.path.join(HERE, "softmax_median_golden.npz")
    np.savez_compressed(out, **arrays)
    print(f"wrote {out}: {len(index)} results, {os.path.getsize(out)} bytes")


if __name__ == "__main__":
    main()
