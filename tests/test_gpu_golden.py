"""GPU kernels against the golden fixture produced by the reference's compiled CPU code
(tests/golden/make_golden.py): extrema and indices bit-exact, sums and variances within 1e-5
relative of float64 and in condition-aware agreement with the stored reference result."""
import json
import os

import numpy as np
import pytest

from util import assert_agrees, assert_bits_equal, assert_close64, assert_index_equal

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reduce_golden.npz")


def test_gpu_matches_reference_golden(cuda):
    import torch
    import tensorplay_b200 as tpb
    from oracle import oracle as O

    z = np.load(GOLDEN)
    index = json.loads(bytes(z["index_json"]).decode())
    for e in index:
        x = z[e["x"]]
        want = z[e["out"]]
        xg = torch.from_numpy(x).to(cuda)
        op, dims, corr = e["op"], e["dims"], e["correction"]
        what = f"golden {op} shape={x.shape} dims={dims} corr={corr}"
        if op in ("argmax", "argmin"):
            got = getattr(tpb, op)(xg, None if dims is None else dims[0]).cpu().numpy()
            assert_index_equal(got, want, what)
        elif op in ("max", "min"):
            assert_bits_equal(getattr(tpb, op)(xg, dims).cpu().numpy(), want, what)
        elif op in ("all", "any"):
            got = getattr(tpb, op)(xg, dims).cpu().numpy()
            assert got.dtype == np.bool_ and np.array_equal(got, want.astype(bool)), what
        elif op == "norm" and np.isinf(e["p"]):
            assert_bits_equal(tpb.norm(xg, e["p"], dims).cpu().numpy(), want, what)     # an extremum of |x|: exact
        elif op in ("prod", "norm"):
            got = (tpb.prod(xg, dims) if op == "prod" else tpb.norm(xg, e["p"], dims)).cpu().numpy()
            truth = O.truth64(op, x, dims, False, corr, e["p"])
            assert_close64(got, truth, what)
            # the reference multiplies / adds in float32 one element after the other
            assert_close64(got, want.astype(np.float64), what + " vs reference", rel=1e-4)
        else:
            got = (getattr(tpb, op)(xg, dims, corr) if op in ("var", "std") else getattr(tpb, op)(xg, dims)).cpu().numpy()
            truth = O.truth64(op, x, dims, False, corr)
            assert_close64(got, truth, what)
            if op in ("sum", "mean"):
                ax = None if dims is None else tuple(dims)
                abs_sum = np.abs(x.astype(np.float64)).sum(axis=ax)
                if op == "mean":
                    abs_sum = abs_sum / (x.size if ax is None else np.prod([x.shape[a] for a in ax]))
                assert_agrees(got, want, truth, abs_sum, what)
            else:
                assert_close64(got, want.astype(np.float64), what + " vs reference", rel=1e-4)
