"""The range-checking build of the library (libtpb200_checked.so, -DTPB200_CHECKED): the same sources
with every access to global memory compared against the ranges that the entry point registered for its
call.  A violation is recorded and the access skipped; nothing traps.

Run the whole GPU suite under it with `TPB200_CHECKED=1 python -m pytest tests -m gpu` (tests/conftest.py
then asserts a clean record after every test).  This file keeps two things in the ordinary run: the
checker's own test, and a pass of the reduction / top-k / softmax / median / copy parity tests under
the checker in a child process."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED_LIB = os.path.join(ROOT, "tensorplay_b200", "libtpb200_checked.so")


def _child(args, timeout):
    env = dict(os.environ, TPB200_CHECKED="1")
    r = subprocess.run([sys.executable, "-m", "pytest", *args, "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (r.stdout[-3000:] + r.stderr[-2000:])
    return r.stdout


def test_checker_catches_a_trimmed_range(cuda):
    """The checker's own test.  Every range of one call is registered 64 bytes short: the kernel's reads
    of the input's last 16 floats and its write of the last outputs are caught, counted and NOT made;
    the status word says so; the next call is clean and correct."""
    from tensorplay_b200 import _lib
    if not _lib.CHECKED:
        assert os.path.exists(CHECKED_LIB), "libtpb200_checked.so was not built"
        out = _child([os.path.join("tests", "test_gpu_checked.py"), "-k", "trimmed_range"], 600)
        assert "1 passed" in out, out
        return
    import torch
    import tensorplay_b200 as tpb
    assert _lib.check_report()["checked_build"] == 1
    rng = np.random.default_rng(7)
    x = rng.standard_normal((300, 4096)).astype(np.float32)
    xg = torch.from_numpy(x).to(cuda)
    out = torch.full((300,), -7.0, device=cuda)
    _lib.check_trim_next(64)
    tpb.sum(xg, dim=1, out=out)
    assert _lib.device_status() == 0x40000000
    rep = _lib.check_report()
    assert rep["violations"] >= 2 and rep["line"] > 0 and rep["bytes"] in (4, 16), rep
    got = out.cpu().numpy()
    assert np.all(got[-16:] == -7.0)                  # the skipped stores: the outputs keep what they held
    want = x.astype(np.float64).sum(axis=1)
    assert np.allclose(got[:-16][:200], want[:200], rtol=1e-5, atol=1e-4)
    # the next call registers the full ranges again
    tpb.sum(xg, dim=1, out=out)
    assert _lib.device_status() == 0
    assert _lib.check_report()["violations"] == 0
    assert np.allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-4)
    # top-k: values, indices and the row re-reads
    v, i = tpb.topk(xg, 5, dim=1)
    assert _lib.check_report()["violations"] == 0
    _lib.check_trim_next(8)
    tpb.topk(xg, 5, dim=1)
    assert _lib.check_report()["violations"] >= 1
    assert _lib.device_status() == 0x40000000


def test_parity_suites_under_the_checker(cuda):
    """Reductions, top-k (scanning and select kernels), softmax, median and strided copy at the sizes of the
    ordinary parity tests, every global access range-checked.  Full-size cases are left to the run of
    the whole suite under TPB200_CHECKED=1."""
    from tensorplay_b200 import _lib
    if _lib.CHECKED:
        pytest.skip("already running under the checked build")
    assert os.path.exists(CHECKED_LIB), "libtpb200_checked.so was not built"
    out = _child([os.path.join("tests", f) for f in ("test_gpu_reduce.py", "test_gpu_topk.py", "test_gpu_softmax_median.py",
                                                      "test_gpu_copy.py", "test_zz_no_alloc.py")]
                 + ["-k", "not 2_to_31 and not 64x4096x512 and not 512x1048576 and not one_long_row and not more_rows_than and not headline"], 1500)
    assert " passed" in out and "failed" not in out, out[-2000:]
