"""Sub-byte tensor wrappers."""
import pytest
import torch

from torchrec_b200.tensor_types import UInt2Tensor, UInt4Tensor, fill_defaults


def test_fill_defaults():
    assert fill_defaults([1, 2, 3], 5, [3, 4, 5]) == [1, 2, 3, 4, 5]
    assert fill_defaults([1, 2, 3], 5, [None, None, None]) == [1, 2, 3, None, None]
    assert fill_defaults([1, 2], 2, [9]) == [1, 2]
    with pytest.raises(RuntimeError):
        fill_defaults([1], 5, [0])


def test_uint4_shape_slice_view():
    raw = torch.arange(4 * 8, dtype=torch.uint8).reshape(4, 8)
    t = UInt4Tensor(raw)
    assert t.shape == (4, 16) and t.dtype == torch.uint8
    assert torch.equal(t.view(torch.uint8), raw)
    s = t[:, 4:12]
    assert isinstance(s, UInt4Tensor) and s.shape == (4, 8) and torch.equal(s.view(torch.uint8), raw[:, 2:6])
    r = t[1:3]
    assert r.shape == (2, 16) and torch.equal(r.view(torch.uint8), raw[1:3])
    v = t.view(8, 8)
    assert v.shape == (8, 8) and torch.equal(v.view(torch.uint8), raw.reshape(8, 4))
    assert t[2].shape == (16,) and torch.equal(t[2].view(torch.uint8), raw[2])
    with pytest.raises(AssertionError):
        t[:, 1:5]
    with pytest.raises(NotImplementedError):
        t + 1


def test_uint2_clone_copy_detach():
    raw = torch.randint(0, 255, (3, 4), dtype=torch.uint8)
    t = UInt2Tensor(raw)
    assert t.shape == (3, 16)
    c = t.clone()
    assert isinstance(c, UInt2Tensor) and torch.equal(c.view(torch.uint8), raw) and c.view(torch.uint8).data_ptr() != raw.data_ptr()
    d = UInt2Tensor(torch.zeros(3, 4, dtype=torch.uint8))
    d.copy_(t)
    assert torch.equal(d.view(torch.uint8), raw)
    assert torch.equal(t.detach().view(torch.uint8), raw)
    assert "UInt2Tensor" in repr(t)
