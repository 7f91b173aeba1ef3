"""Layout and view algebra feeding the matmul strides.

Mirror of the reference's ``TensorLayout`` / ``TensorView(Mut)``
(adrastea_models/src/tensor.rs:25-150, 373-575): dims and strides are in
elements, views never copy, ``permute`` / ``shape_cast`` / ``skip`` / ``take``
have the reference's meaning and failure behaviour (an ``AssertionError``
where the reference panics).  A view sits on a torch tensor's storage (device
memory and streams come from PyTorch; the arithmetic does not).
"""
from __future__ import annotations

from dataclasses import dataclass
from math import prod
from typing import Sequence

import torch

MAX_DIMS = 7  # SmallVec<[usize; 7]>, tensor.rs:27-28; device descriptor compat.h:40-45


@dataclass(frozen=True)
class TensorLayout:
    dims: tuple[int, ...]
    strides: tuple[int, ...]

    def __post_init__(self):
        # tensor.rs:32-38
        assert len(self.dims) == len(self.strides)
        assert len(self.dims) != 0
        assert all(d != 0 for d in self.dims)
        assert all(s != 0 for s in self.strides)

    @staticmethod
    def new(dims: Sequence[int], strides: Sequence[int]) -> "TensorLayout":
        return TensorLayout(tuple(int(d) for d in dims), tuple(int(s) for s in strides))

    @staticmethod
    def row_major(dims: Sequence[int]) -> "TensorLayout":
        # tensor.rs:41-50
        strides = []
        stride = 1
        for d in reversed(dims):
            strides.append(stride)
            stride *= d
        return TensorLayout.new(dims, list(reversed(strides)))

    @staticmethod
    def column_major(dims: Sequence[int]) -> "TensorLayout":
        # tensor.rs:52-60: swap the last two strides of the row-major layout
        rm = TensorLayout.row_major(dims)
        s = list(rm.strides)
        s[-2], s[-1] = s[-1], s[-2]
        return TensorLayout.new(dims, s)

    def largest_address(self) -> int:
        return sum((d - 1) * s for d, s in zip(self.dims, self.strides))

    def permute(self, dim_order: Sequence[int]) -> "TensorLayout":
        # tensor.rs:70-79
        assert len(dim_order) == len(self.dims)
        return TensorLayout.new([self.dims[i] for i in dim_order],
                                [self.strides[i] for i in dim_order])

    def shape_cast(self, dims: Sequence[int]) -> "TensorLayout":
        """Re-stride as row-major with new dims; one dim may be -1.

        Like the reference (tensor.rs:81-105) this does not check that the
        source was contiguous: it is a "poor man's view".
        """
        dims = list(dims)
        vol = prod(self.dims)
        neg = [i for i, d in enumerate(dims) if d < 0]
        assert len(neg) <= 1
        if neg:
            known = prod(d for d in dims if d >= 0)
            dims[neg[0]] = vol // known
        assert prod(dims) == vol
        strides = []
        stride = 1
        for d in reversed(dims):
            strides.append(stride)
            stride *= d
        # the reference builds this one without the non-zero checks
        return TensorLayout(tuple(dims), tuple(reversed(strides)))

    def size(self, dim: int) -> int:
        return self.dims[dim]

    def stride(self, dim: int) -> int:
        return self.strides[dim]

    def skip(self, sizes: Sequence[int]) -> tuple[int, "TensorLayout"]:
        # tensor.rs:123-136
        offset = 0
        nd, ns = [], []
        for d, s, size in zip(self.dims, self.strides, sizes):
            size = d if size == -1 else size
            assert 0 <= size <= d
            offset += s * size
            nd.append(d - size)
            ns.append(s)
        return offset, TensorLayout.new(nd, ns)

    def take(self, sizes: Sequence[int]) -> "TensorLayout":
        # tensor.rs:138-149
        nd, ns = [], []
        for d, s, size in zip(self.dims, self.strides, sizes):
            size = d if size == -1 else size
            assert 0 <= size <= d
            nd.append(size)
            ns.append(s)
        return TensorLayout.new(nd, ns)


class TensorView:
    """A strided window on a torch tensor's storage (tensor.rs:373-575).

    ``base`` keeps the storage alive; ``offset`` is in elements from the
    start of ``base``'s first element.
    """

    __slots__ = ("base", "offset", "layout")

    def __init__(self, base: torch.Tensor, layout: TensorLayout, offset: int = 0):
        assert len(layout.dims) <= MAX_DIMS
        self.base = base
        self.layout = layout
        self.offset = offset

    # -- construction --------------------------------------------------
    @staticmethod
    def of(t: torch.Tensor) -> "TensorView":
        """View with the torch tensor's own dims and strides."""
        assert t.dim() >= 1
        return TensorView(t, TensorLayout.new(t.shape, t.stride()), 0)

    # -- reference API --------------------------------------------------
    def size(self, dim: int) -> int:
        return self.layout.size(dim)

    def stride(self, dim: int) -> int:
        return self.layout.stride(dim)

    @property
    def dtype(self):
        return self.base.dtype

    @property
    def device(self):
        return self.base.device

    def permute(self, dim_order: Sequence[int]) -> "TensorView":
        return TensorView(self.base, self.layout.permute(dim_order), self.offset)

    def shape_cast(self, dims: Sequence[int]) -> "TensorView":
        return TensorView(self.base, self.layout.shape_cast(dims), self.offset)

    def skip(self, sizes: Sequence[int]) -> "TensorView":
        off, lay = self.layout.skip(sizes)
        return TensorView(self.base, lay, self.offset + off)

    def take(self, sizes: Sequence[int]) -> "TensorView":
        return TensorView(self.base, self.layout.take(sizes), self.offset)

    def data_ptr(self) -> int:
        """Address of element 0 of the view (as_gpu_ptr, tensor.rs:417-419)."""
        return self.base.data_ptr() + self.offset * self.base.element_size()

    def as_torch(self) -> torch.Tensor:
        """The same window as a torch strided tensor (for checks and glue ops)."""
        return torch.as_strided(self.base, self.layout.dims, self.layout.strides,
                                self.base.storage_offset() + self.offset)

    def as_cpu_list(self) -> list:
        """Elements in logical (row-major iteration) order, like as_cpu_slice on
        a contiguous view."""
        return self.as_torch().cpu().reshape(-1).tolist()

    def __repr__(self):
        return f"TensorView(dims={self.layout.dims}, strides={self.layout.strides}, offset={self.offset})"


# The reference distinguishes TensorView and TensorViewMut only by borrow
# rules; in Python they are the same object.
TensorViewMut = TensorView
