"""GPU test of the strided copy (tpb200_strided_copy) against numpy: bit-exact, every kernel path."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_strided_copy_paths(cuda):
    import torch
    import tensorplay_b200 as tpb
    rng = np.random.default_rng(71)
    base = rng.standard_normal((6, 50, 70)).astype(np.float32)
    bg = torch.from_numpy(base).to(cuda)
    # (name, the view in numpy, the same view in torch)
    views = [
        ("contiguous", lambda a: a, lambda t: t),
        ("transpose of the last two dims", lambda a: a.transpose(0, 2, 1), lambda t: t.transpose(1, 2)),
        ("permute (2, 0, 1)", lambda a: a.transpose(2, 0, 1), lambda t: t.permute(2, 0, 1)),
        ("permute (1, 2, 0)", lambda a: a.transpose(1, 2, 0), lambda t: t.permute(1, 2, 0)),
        ("slices, rows not aligned", lambda a: a[1:5, 3:40, 1:69], lambda t: t[1:5, 3:40, 1:69]),
        ("every other column (no unit stride)", lambda a: a[:, :, ::2], lambda t: t[:, :, ::2]),
        ("one row", lambda a: a[2, 7], lambda t: t[2, 7]),
    ]
    for name, fn, ft in views:
        want = np.ascontiguousarray(fn(base))
        got = tpb.contiguous(ft(bg))
        assert got.is_contiguous() and np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32)), name
    # strided destination: write a transposed view into a slice of a larger buffer
    big = torch.zeros(80, 60, device=cuda)
    src = bg[0]                                        # [50, 70]
    tpb.copy_(big[5:75, 3:53], src.t())
    want = np.zeros((80, 60), dtype=np.float32)
    want[5:75, 3:53] = base[0].T
    assert np.array_equal(big.cpu().numpy(), want)
    # NaN payloads and -0.0 travel as bits
    odd = np.array([np.nan, -0.0, 0.0, np.inf], dtype=np.float32)
    odd.view(np.uint32)[0] = 0x7FC12345
    og = torch.from_numpy(np.tile(odd, (33, 1))).to(cuda)
    assert np.array_equal(tpb.contiguous(og.t()).cpu().numpy().view(np.uint32), np.ascontiguousarray(np.tile(odd, (33, 1)).T).view(np.uint32))
    assert tpb.contiguous(torch.empty(0, 4, device=cuda)).shape == (0, 4)
    with pytest.raises(RuntimeError, match="Sizes do not match"):
        tpb.copy_(torch.empty(3, 4, device=cuda), torch.empty(4, 3, device=cuda))


def test_permute_64x4096x512(cuda):
    """The copy the reference makes before argmin over dim 1 of [64, 4096, 512] (512 MiB through a
    one-element-per-thread kernel): permute to [64, 512, 4096], bit-exact against torch."""
    import torch
    import tensorplay_b200 as tpb
    g = torch.Generator(device=cuda).manual_seed(7)
    x = torch.rand(64, 4096, 512, device=cuda, generator=g)
    got = tpb.contiguous(x.permute(0, 2, 1))
    assert torch.equal(got, x.permute(0, 2, 1).contiguous())
