import os
import sys

import pytest

# the planner overrides that some tests set (TPB200_TOPK_SLICES, TPB200_FORCE_STRATEGY, ...) are only
# honoured when this switch is in the environment at the library's first call
os.environ.setdefault("TPB200_EXPERIMENTS", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tensorplay_b200 import _lib

    _lib.lib()  # fail loudly if the extension is missing
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _no_range_violation(request):
    """Under TPB200_CHECKED=1 (the range-checking build of the library) every GPU test also asserts that
    no kernel touched memory outside the ranges its entry point registered."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    from tensorplay_b200 import _lib

    if not _lib.CHECKED or _lib._lib is None:
        return
    rep = _lib.check_report()
    assert rep["violations"] == 0, f"range violations under the checked build: {rep}"
