"""Host-side marshalling (GpuKernels::matmul_f16, kernels.rs:821-890) and the
C ABI's exported symbols.  No GPU needed."""
import re
from pathlib import Path

import pytest
import torch

from adrastea_b200 import (MatmulLoad, MatmulMask, MatmulOptions, MatmulStore, MatmulStoreOp,
                           TensorView, lower_matmul)

ROOT = Path(__file__).resolve().parents[1]


def tv(*shape):
    return TensorView.of(torch.zeros(*shape, dtype=torch.float16))


def test_lowering_of_a_linear_layer():
    x, w, out = tv(7, 64), tv(48, 64), tv(7, 48)
    args = lower_matmul(out, x, w.permute([1, 0]), MatmulOptions.new())
    (batches, m, k, n, sox, soy, soz, slx, sly, slz, srx, sry, srz, bias, beta, scale, store, load,
     mask) = args
    assert (batches, m, k, n) == (1, 7, 64, 48)
    assert (sox, soy, soz) == (1, 48, 0)
    assert (slx, sly, slz) == (1, 64, 0)
    assert (srx, sry, srz) == (64, 1, 0)  # NT: K-contiguous weight
    assert bias is None and beta == 0.0 and scale == 1.0 and (store, load, mask) == (0, 0, 0)


def test_lowering_batched_with_broadcast_and_scales():
    H, S, hd = 4, 9, 16
    q = tv(S, H * hd).shape_cast([S, H, -1]).permute([1, 0, 2])
    k = tv(S, H * hd).shape_cast([S, H, -1]).permute([1, 2, 0])
    out = tv(H, S, S)
    opts = (MatmulOptions.new().load(MatmulLoad.Scale(0.5)).store(MatmulStore.Scale(0.25))
            .mask(MatmulMask.Causal))
    args = lower_matmul(out, q, k, opts)
    assert args[0] == H and args[1:4] == (S, hd, S)
    assert args[4:7] == (1, S, S * S)
    assert args[7:10] == (1, H * hd, hd)
    assert args[10:13] == (H * hd, 1, hd)
    assert args[15] == pytest.approx(0.125)  # load scale x store scale, kernels.rs:837-843
    assert args[16:] == (int(MatmulStoreOp.Scale), 1, 1)
    # a 2-D right operand broadcasts over the batch: z-stride 0 (kernels.rs:878-880)
    args = lower_matmul(out, q, tv(hd, S), MatmulOptions.new())
    assert args[12] == 0


def test_lowering_beta_and_bias():
    out, x, w, b = tv(4, 8), tv(4, 16), tv(8, 16), tv(8)
    a = lower_matmul(out, x, w.permute([1, 0]), MatmulOptions.new().store(MatmulStore.BetaBias(1.0, b)))
    assert a[13] is b and a[14] == 1.0 and a[16] == 3
    a = lower_matmul(out, x, w.permute([1, 0]), MatmulOptions.new().store(MatmulStore.QuickGeluBias(b)))
    assert a[13] is b and a[14] == 0.0 and a[16] == 6
    a = lower_matmul(out, x, w.permute([1, 0]), MatmulOptions.new().store(MatmulStore.Add()))
    assert a[13] is None and a[16] == 5


def test_shape_mismatch_panics_like_the_reference():
    with pytest.raises(AssertionError):
        lower_matmul(tv(4, 8), tv(4, 16), tv(15, 8), MatmulOptions.new())
    with pytest.raises(AssertionError):
        lower_matmul(tv(5, 8), tv(4, 16), tv(16, 8), MatmulOptions.new())
    with pytest.raises(AssertionError):
        lower_matmul(tv(4, 9), tv(4, 16), tv(16, 8), MatmulOptions.new())


def declared_symbols():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"\b(adr_[a-z0-9_]+)\s*\(", h.read_text()))
    return names


def test_library_exports_every_declared_symbol():
    from adrastea_b200 import _lib
    from adrastea_b200.build import build_library
    build_library()
    lib = _lib.load()
    declared = declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_no_cpu_fallback_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from adrastea_b200 import GpuKernels
    with pytest.raises(RuntimeError):
        GpuKernels(0)


def test_strerror_needs_no_gpu():
    from adrastea_b200 import _lib
    lib = _lib.load()
    assert lib.adr_strerror(0) == b"ok"
    assert b"shape" in lib.adr_strerror(2)
