"""CPU tests of the host-side mirror of the reference interface: argument handling and error
behaviour that needs no GPU, and the loud failure when the CUDA path is unavailable."""
import pytest
import torch


def test_no_cpu_fallback():
    import tensorplay_b200 as tpb
    x = torch.ones(4, 4)
    for fn in (tpb.sum, tpb.mean, tpb.var, tpb.std, tpb.max, tpb.min, tpb.argmax, tpb.argmin, tpb.prod, tpb.norm,
               tpb.all, tpb.any):
        with pytest.raises(RuntimeError, match="CUDA tensors only"):
            fn(x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tpb.topk(x, 2)
    # norm: the exponents the kernels have; anything else is refused before a tensor is looked at
    with pytest.raises(NotImplementedError, match="p = 1, 2, inf and -inf"):
        tpb.norm(x, 3.0)


def test_dim_handling_matches_the_reference_rules():
    from tensorplay_b200 import ops
    x = torch.empty(2, 3, 4)
    assert ops._dims_mask(x, None) == (0, [0, 1, 2])
    assert ops._dims_mask(x, []) == (0, [0, 1, 2])          # empty list = reduce all
    assert ops._dims_mask(x, -1) == (1 << 2, [2])
    assert ops._dims_mask(x, [0, -1, 0]) == ((1 << 0) | (1 << 2), [0, 2])   # duplicates are harmless
    for bad in (3, -4, [0, 5]):
        with pytest.raises(RuntimeError, match="Dimension out of range"):
            ops._dims_mask(x, bad)
    assert ops._out_shape(x, [0, 2], False) == [3]
    assert ops._out_shape(x, [0, 2], True) == [1, 3, 1]
    assert ops._out_shape(x, [0, 1, 2], False) == []
    s = torch.empty(())
    assert ops._dims_mask(s, None) == (0, [])
    for bad in (0, -1, 1):      # compute_reduction_shape rejects every dim of a 0-dim tensor
        with pytest.raises(RuntimeError, match="Dimension out of range"):
            ops._dims_mask(s, bad)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tensorplay_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libtpb200.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()
