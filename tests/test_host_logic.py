"""Host-side marshalling (GpuKernels::matmul_f16, kernels.rs:821-890) and the
C ABI's exported symbols.  No GPU needed."""
import re
from pathlib import Path

import pytest
import torch

from adrastea_b200 import (MatmulLoad, MatmulMask, MatmulOptions, MatmulStore, MatmulStoreOp,
                           TensorLayout, TensorView, lower_matmul)

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


def test_every_error_code_has_its_own_text():
    from adrastea_b200 import _lib
    lib = _lib.load()
    texts = [lib.adr_strerror(c) for c in range(8)]
    assert len(set(texts)) == 8 and b"unknown" not in b" ".join(texts)
    assert b"built-in scratch" in lib.adr_strerror(7)
    assert lib.adr_strerror(99) == b"unknown error"


def test_entry_points_refuse_a_missing_context_before_touching_a_gpu():
    """Argument checks come first: with no context (and no GPU) the calls return ADR_ERR_INVALID."""
    import ctypes as C
    from adrastea_b200 import _lib
    lib = _lib.load()
    buf = C.create_string_buffer(64)
    p = C.cast(buf, C.c_void_p)
    ptrs = (C.c_void_p * 2)(p, p)
    ns = (C.c_int * 2)(16, 16)
    assert lib.adr_matmul_nt_fp16u8(None, None, p, p, p, p, None, 1, 128, 16, 128, 0.0) == 1
    assert lib.adr_matmul_nt_fp16u8_ws(None, None, p, p, p, p, None, 1, 128, 16, 128, 0.0, p, 64) == 1
    assert lib.adr_matmul_nt_fp16u8_noalloc(None, None, p, p, p, p, None, 1, 128, 16, 128, 0.0) == 1
    assert lib.adr_matmul_nt_fp16u8_grouped(None, None, 2, ptrs, p, ptrs, ptrs, None, 1, 128, ns, 128, 0.0) == 1
    assert lib.adr_silu_mul_matmul_nt_fp16u8(None, None, p, p, p, p, None, p, p, None, 1, 128, 16, 128) == 1
    assert lib.adr_set_tunable(None, b"pdl", 1) != 0


def test_lowering_of_rank_four_views_keeps_the_inner_batch():
    """A rank-4 output lowers to the inner batch count and z strides; the outer dimension's
    stride is what adr_matmul_f16_b2 takes next to them."""
    o = TensorView(None, TensorLayout.new((3, 4, 72, 72), (4 * 72 * 72, 72 * 72, 72, 1)))
    q = TensorView(None, TensorLayout.new((3, 4, 72, 64), (72 * 256, 64, 256, 1)))
    k = TensorView(None, TensorLayout.new((3, 4, 64, 72), (72 * 256, 64, 1, 256)))
    low = lower_matmul(o, q, k, MatmulOptions.new())
    assert low[:4] == (4, 72, 64, 72)
    assert low[4:13] == (1, 72, 72 * 72, 1, 256, 64, 256, 1, 64)
    assert (o.stride(-4), q.stride(-4), k.stride(-4)) == (4 * 72 * 72, 72 * 256, 72 * 256)
