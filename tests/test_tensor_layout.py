"""Layout algebra, mirroring the reference's own unit tests
(adrastea_models/src/tensor.rs:587-664)."""
import pytest
import torch

from adrastea_b200 import TensorLayout, TensorView


def iota(n):
    return TensorView.of(torch.arange(n, dtype=torch.int32))


def test_row_and_column_major():
    rm = TensorLayout.row_major([2, 3, 4])
    assert rm.strides == (12, 4, 1)
    cm = TensorLayout.column_major([2, 3, 4])
    assert cm.strides == (12, 1, 4)
    assert rm.largest_address() == 23


def test_permute_is_transpose():
    t = TensorView.of(torch.arange(9, dtype=torch.float32).reshape(3, 3))
    tr = t.permute([1, 0])
    assert tr.layout.dims == (3, 3) and tr.layout.strides == (1, 3)
    assert tr.as_torch().tolist() == [[0, 3, 6], [1, 4, 7], [2, 5, 8]]


def test_shape_cast():
    t = TensorView.of(torch.arange(1, 17, dtype=torch.float32).reshape(4, 4))
    v = t.shape_cast([-1, 8])
    assert v.layout.dims == (2, 8) and v.layout.strides == (8, 1)
    assert v.as_torch()[1].tolist() == list(range(9, 17))


def test_shape_cast_must_preserve_volume():
    with pytest.raises(AssertionError):
        iota(256).shape_cast([16, 1])


def test_skip_and_take():
    reshaped = iota(256).shape_cast([16, 16])
    skipped = reshaped.skip([15, 0])
    assert skipped.size(-2) == 1 and skipped.size(-1) == 16
    assert skipped.as_cpu_list() == list(range(240, 256))
    taken = reshaped.skip([1, 0]).take([1, 16])
    assert taken.size(-2) == 1 and taken.size(-1) == 16
    assert taken.as_cpu_list() == list(range(16, 32))


def test_zero_dims_rejected():
    with pytest.raises(AssertionError):
        TensorLayout.new([0, 4], [4, 1])
    with pytest.raises(AssertionError):
        TensorLayout.new([2, 4], [4])


def test_attention_views_match_reference_strides():
    # llama.rs:530-536: [S, D] -> shape_cast [S, H, hd] -> permute
    S, H, hd = 5, 4, 8
    q = TensorView.of(torch.zeros(S, H * hd, dtype=torch.float16))
    q_view = q.shape_cast([S, H, -1]).permute([1, 0, 2])
    k_view = q.shape_cast([S, H, -1]).permute([1, 2, 0])
    assert q_view.layout.dims == (H, S, hd) and q_view.layout.strides == (hd, H * hd, 1)
    assert k_view.layout.dims == (H, hd, S) and k_view.layout.strides == (hd, 1, H * hd)
