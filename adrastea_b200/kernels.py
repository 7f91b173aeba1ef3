"""Host-side mirror of the reference's kernel-call interface for the matmul path.

Same names, argument meaning and error behaviour as
adrastea_models/src/kernels.rs: ``MatmulOptions`` / ``MatmulStore`` /
``MatmulLoad`` / ``MatmulMask`` (kernels.rs:80-167), ``GpuKernels.matmul_f16``
and ``matmul_f16_slow`` (kernels.rs:753-890), ``MatmulTracer``
(kernels.rs:231-248, 306-333).  Every call goes through the C ABI of
libadrastea_b200.so; there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import enum
import json
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib
from .tensor import TensorLayout, TensorView


class AdrError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"adrastea_b200 error {code}: {msg}")
        self.code = code


# -- enums (kernels.rs:80-139; matmul.cu:26-36) ---------------------------
class MatmulLoadOp(enum.IntEnum):
    Identity = 0
    Scale = 1


class MatmulStoreOp(enum.IntEnum):
    Identity = 0
    GeluBias = 1
    BetaGeluBias = 2
    BetaBias = 3
    Scale = 4
    Add = 5
    QuickGeluBias = 6


class MatmulMask(enum.IntEnum):
    None_ = 0
    Causal = 1


class BinaryOp(enum.IntEnum):
    """enum BinaryOp (kernels.rs:70-74, elementwise.cu:16-19)."""
    Add = 1
    SiluMul = 2


class Kernel(enum.IntEnum):
    Auto = 0
    F16Simt = 1
    F16Tc = 2
    U8Gemv = 3
    U8Mma = 4
    U8Tc = 5
    U8Simt = 6
    U8Stream = 7
    U8Ring = 8
    F16TcGather = 9
    U8Ts = 10
    U8KSplit = 11


@dataclass(frozen=True)
class MatmulLoad:
    op: MatmulLoadOp = MatmulLoadOp.Identity
    scale: float = 1.0

    @staticmethod
    def Identity() -> "MatmulLoad":
        return MatmulLoad(MatmulLoadOp.Identity, 1.0)

    @staticmethod
    def Scale(scale: float) -> "MatmulLoad":
        return MatmulLoad(MatmulLoadOp.Scale, float(scale))

    def lower(self) -> MatmulLoadOp:
        return self.op


@dataclass(frozen=True)
class MatmulStore:
    op: MatmulStoreOp = MatmulStoreOp.Identity
    beta: float = 0.0
    scale: float = 1.0
    bias: Optional[TensorView] = None

    @staticmethod
    def Identity() -> "MatmulStore":
        return MatmulStore()

    @staticmethod
    def GeluBias(bias: TensorView) -> "MatmulStore":
        return MatmulStore(MatmulStoreOp.GeluBias, bias=bias)

    @staticmethod
    def QuickGeluBias(bias: TensorView) -> "MatmulStore":
        return MatmulStore(MatmulStoreOp.QuickGeluBias, bias=bias)

    @staticmethod
    def BetaGeluBias(beta: float, bias: TensorView) -> "MatmulStore":
        return MatmulStore(MatmulStoreOp.BetaGeluBias, beta=float(beta), bias=bias)

    @staticmethod
    def BetaBias(beta: float, bias: TensorView) -> "MatmulStore":
        return MatmulStore(MatmulStoreOp.BetaBias, beta=float(beta), bias=bias)

    @staticmethod
    def Scale(scale: float) -> "MatmulStore":
        return MatmulStore(MatmulStoreOp.Scale, scale=float(scale))

    @staticmethod
    def Add() -> "MatmulStore":
        return MatmulStore(MatmulStoreOp.Add)

    def lower(self) -> MatmulStoreOp:
        return self.op


@dataclass
class MatmulOptions:
    """Builder with the reference's defaults (kernels.rs:148-167)."""
    load_: MatmulLoad = field(default_factory=MatmulLoad.Identity)
    store_: MatmulStore = field(default_factory=MatmulStore.Identity)
    mask_: MatmulMask = MatmulMask.None_

    @staticmethod
    def new() -> "MatmulOptions":
        return MatmulOptions()

    def load(self, load: MatmulLoad) -> "MatmulOptions":
        self.load_ = load
        return self

    def store(self, store: MatmulStore) -> "MatmulOptions":
        self.store_ = store
        return self

    def mask(self, mask: MatmulMask) -> "MatmulOptions":
        self.mask_ = mask
        return self


def lower_matmul(output: TensorView, left: TensorView, right: TensorView,
                 options: MatmulOptions) -> tuple:
    """The marshalling of GpuKernels::matmul_f16 (kernels.rs:825-887).

    Returns the 19 scalar arguments that follow the three pointers:
    (batches, m, k, n, 9 strides, bias_view_or_None, beta, scale, store, load, mask).
    Shape mismatches raise AssertionError where the reference's assert_eq!
    panics (kernels.rs:825-827).
    """
    assert left.size(-1) == right.size(-2), "K mismatch"
    assert output.size(-2) == left.size(-2), "M mismatch"
    assert output.size(-1) == right.size(-1), "N mismatch"
    store = options.store_
    bias = store.bias  # kernels.rs:828-836
    scale = options.load_.scale if options.load_.op == MatmulLoadOp.Scale else 1.0
    if store.op == MatmulStoreOp.Scale:
        scale *= store.scale  # kernels.rs:837-843
    beta = store.beta if store.op in (MatmulStoreOp.BetaGeluBias, MatmulStoreOp.BetaBias) else 0.0
    out_rank = len(output.layout.dims)
    batches = output.size(-3) if out_rank > 2 else 1

    def zstride(v: TensorView) -> int:
        return v.stride(-3) if len(v.layout.dims) > 2 else 0

    return (batches, left.size(-2), left.size(-1), right.size(-1),
            output.stride(-1), output.stride(-2), zstride(output),
            left.stride(-1), left.stride(-2), zstride(left),
            right.stride(-1), right.stride(-2), zstride(right),
            bias, beta, scale, int(store.lower()), int(options.load_.lower()),
            int(options.mask_))


def _stream_handle(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


class GpuKernels:
    """Mirror of ``GpuKernels`` (kernels.rs:361-502) for the matmul path.

    The reference's constructor takes the device capability and loads the
    embedded cubins; here it takes a CUDA device ordinal and opens the
    library.  Calls are enqueued on torch's current stream (the reference
    uses the NULL stream) and are asynchronous.
    """

    def __init__(self, device: int | torch.device | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("adrastea_b200 needs a CUDA device (sm_100a); there is no CPU path")
        if device is None:
            device = torch.cuda.current_device()
        if isinstance(device, torch.device):
            device = device.index if device.index is not None else torch.cuda.current_device()
        self.device = int(device)
        self._lib = _lib.load()
        ctx = C.c_void_p()
        with torch.cuda.device(self.device):
            torch.cuda.current_stream()  # make sure the primary context exists
            rc = self._lib.adr_init(self.device, C.byref(ctx))
        self._ctx = ctx
        self._check(rc)

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.adr_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers ----------------------------------------------------------
    def _check(self, rc: int):
        if rc != 0:
            msg = self._lib.adr_strerror(rc).decode()
            if rc == 4 and self._ctx:
                msg += f" (cudaError {self._lib.adr_last_cuda_error(self._ctx)})"
            raise AdrError(rc, msg)

    def force_kernel(self, kernel: Kernel | int):
        self._check(self._lib.adr_force_kernel(self._ctx, int(kernel)))

    def set_tunable(self, name: str, value: int):
        self._check(self._lib.adr_set_tunable(self._ctx, name.encode(), int(value)))

    def device_status(self):
        """Synchronise and raise if a kernel gave up on a bounded wait."""
        self._check(self._lib.adr_device_status(self._ctx))

    def last_kernel(self) -> Kernel:
        return Kernel(self._lib.adr_last_kernel(self._ctx))

    def launch_count(self) -> int:
        return int(self._lib.adr_launch_count(self._ctx))

    @staticmethod
    def _f16(v: TensorView, what: str):
        if v.dtype != torch.float16:
            raise TypeError(f"{what} must be float16, got {v.dtype}")

    # -- the reference's matmul methods -----------------------------------
    def _matmul(self, fn, output: TensorView, left: TensorView, right: TensorView,
                options: MatmulOptions, stream=None):
        for v, w in ((output, "output"), (left, "left"), (right, "right")):
            self._f16(v, w)
        (batches, m, k, n, sox, soy, soz, slx, sly, slz, srx, sry, srz,
         bias, beta, scale, store, load, mask) = lower_matmul(output, left, right, options)
        bias_ptr = None
        if bias is not None:
            self._f16(bias, "bias")
            bias_ptr = bias.data_ptr()
        rc = fn(self._ctx, _stream_handle(stream), output.data_ptr(), left.data_ptr(),
                right.data_ptr(), batches, m, k, n, sox, soy, soz, slx, sly, slz, srx, sry, srz,
                bias_ptr, beta, scale, store, load, mask)
        self._check(rc)

    def matmul_f16(self, output: TensorView, left: TensorView, right: TensorView,
                   options: MatmulOptions | None = None, stream=None):
        """CommonKernels::matmul_f16 (kernels.rs:210-213, 821-890)."""
        self._matmul(self._lib.adr_matmul_f16, output, left, right, options or MatmulOptions(),
                     stream)

    def matmul_f16_b2(self, output: TensorView, left: TensorView, right: TensorView,
                      options: MatmulOptions | None = None, stream=None):
        """adr_matmul_f16_b2: matmul_f16 for rank-4 views (two batch dimensions; an operand of
        lower rank is broadcast), which the reference's launch cannot take (kernels.rs:858)."""
        options = options or MatmulOptions()
        for v, w in ((output, "output"), (left, "left"), (right, "right")):
            self._f16(v, w)
        assert len(output.layout.dims) == 4
        (batches, m, k, n, sox, soy, soz, slx, sly, slz, srx, sry, srz,
         bias, beta, scale, store, load, mask) = lower_matmul(output, left, right, options)

        def wstride(v: TensorView) -> int:
            return v.stride(-4) if len(v.layout.dims) > 3 else 0

        for v in (left, right):
            if len(v.layout.dims) > 3:
                assert v.size(-4) == output.size(-4), "outer batch mismatch"
        bias_ptr = None
        if bias is not None:
            self._f16(bias, "bias")
            bias_ptr = bias.data_ptr()
        rc = self._lib.adr_matmul_f16_b2(
            self._ctx, _stream_handle(stream), output.data_ptr(), left.data_ptr(), right.data_ptr(),
            output.size(-4), batches, m, k, n, sox, soy, soz, wstride(output), slx, sly, slz,
            wstride(left), srx, sry, srz, wstride(right), bias_ptr, beta, scale, store, load, mask)
        self._check(rc)

    def matmul_f16_slow(self, output: TensorView, left: TensorView, right: TensorView,
                        options: MatmulOptions | None = None, stream=None):
        """CommonKernels::matmul_f16_slow (kernels.rs:206-209, 753-819)."""
        self._matmul(self._lib.adr_matmul_f16_slow, output, left, right,
                     options or MatmulOptions(), stream)

    # -- kernels the reference ships without a Rust call site ---------------
    def matmul_nt_fp16u8(self, output: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor,
                         scales: torch.Tensor, block_size: int, beta: float = 0.0,
                         zeros: torch.Tensor | None = None, stream=None):
        """matmul_nt_fp16u8 / matmul_nt_wmma_16x128x256_fp16u8
        (matmul_nt_fp16u8.cu:4-12): out[m,n] = lhs[m,p] . deq(rhs[n,p])^T + beta*out."""
        m, p = lhs.shape
        n = rhs.shape[0]
        assert rhs.shape == (n, p) and output.shape == (m, n)
        assert scales.shape == (n, p // block_size)
        for t in (output, lhs, rhs, scales) + ((zeros,) if zeros is not None else ()):
            assert t.is_contiguous() and t.is_cuda
        assert rhs.dtype == torch.uint8 and lhs.dtype == torch.float16
        assert output.dtype == torch.float16 and scales.dtype == torch.float16
        zp = None
        if zeros is not None:
            assert zeros.shape == scales.shape and zeros.dtype == torch.float16
            zp = zeros.data_ptr()
        rc = self._lib.adr_matmul_nt_fp16u8(self._ctx, _stream_handle(stream), output.data_ptr(),
                                            lhs.data_ptr(), rhs.data_ptr(), scales.data_ptr(), zp,
                                            m, p, n, block_size, beta)
        self._check(rc)

    def matmul_nt_fp16u8_grouped(self, outputs, lhs: torch.Tensor, rhss, scaless, block_size: int,
                                 beta: float = 0.0, zeross=None, stream=None):
        """adr_matmul_nt_fp16u8_grouped: several u8 products over the same activations (q/k/v,
        gate/up), as one launch of the decode kernel where it takes them."""
        import ctypes as C
        count = len(outputs)
        m, p = lhs.shape
        assert len(rhss) == count and len(scaless) == count and (zeross is None or len(zeross) == count)
        for o, q, s in zip(outputs, rhss, scaless):
            assert q.shape[1] == p and o.shape == (m, q.shape[0]) and s.shape == (q.shape[0], p // block_size)
            for t in (o, q, s):
                assert t.is_contiguous() and t.is_cuda
        assert lhs.is_contiguous() and lhs.dtype == torch.float16

        def arr(ts):
            return (C.c_void_p * count)(*[t.data_ptr() for t in ts])

        ns = (C.c_int * count)(*[q.shape[0] for q in rhss])
        rc = self._lib.adr_matmul_nt_fp16u8_grouped(
            self._ctx, _stream_handle(stream), count, arr(outputs), lhs.data_ptr(), arr(rhss),
            arr(scaless), arr(zeross) if zeross is not None else None, m, p, ns, block_size, beta)
        self._check(rc)

    def silu_mul_matmul_nt_fp16u8(self, output: torch.Tensor, lhs: torch.Tensor, rhs_gate: torch.Tensor,
                                  scales_gate: torch.Tensor, rhs_up: torch.Tensor,
                                  scales_up: torch.Tensor, block_size: int,
                                  zeros_gate: torch.Tensor | None = None,
                                  zeros_up: torch.Tensor | None = None, stream=None):
        """adr_silu_mul_matmul_nt_fp16u8: SiluMul(lhs . gate^T, lhs . up^T) in one launch of the
        decode kernel (raises AdrError code 2 for shapes it does not take)."""
        m, p = lhs.shape
        n = rhs_gate.shape[0]
        assert rhs_gate.shape == (n, p) and rhs_up.shape == (n, p) and output.shape == (m, n)
        for t in (output, lhs, rhs_gate, rhs_up, scales_gate, scales_up):
            assert t.is_contiguous() and t.is_cuda
        rc = self._lib.adr_silu_mul_matmul_nt_fp16u8(
            self._ctx, _stream_handle(stream), output.data_ptr(), lhs.data_ptr(), rhs_gate.data_ptr(),
            scales_gate.data_ptr(), zeros_gate.data_ptr() if zeros_gate is not None else None,
            rhs_up.data_ptr(), scales_up.data_ptr(),
            zeros_up.data_ptr() if zeros_up is not None else None, m, p, n, block_size)
        self._check(rc)

    def qkv_rope_append_matmul_nt_fp16u8(self, q_out: torch.Tensor, lhs: torch.Tensor,
                                         rhs: torch.Tensor, scales: torch.Tensor, block_size: int,
                                         n_heads: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                         pos: torch.Tensor, theta: float,
                                         norm_weights: torch.Tensor | None = None, eps: float = 0.0,
                                         zeros: torch.Tensor | None = None, stream=None):
        """adr_qkv_rope_append_matmul_nt_fp16u8: fused q/k/v product (+ rms_norm) + rotary + cache
        append in one launch; q_out is a [m, width] view (row pitch q_out.stride(0))."""
        m, p = lhs.shape
        width = rhs.shape[0] // 3
        assert rhs.shape == (3 * width, p) and q_out.shape == (m, width) and q_out.stride(1) == 1
        assert k_cache.shape[2] == width and v_cache.shape == k_cache.shape and k_cache.shape[0] >= m
        assert pos.dtype == torch.int32 and pos.is_cuda
        rc = self._lib.adr_qkv_rope_append_matmul_nt_fp16u8(
            self._ctx, _stream_handle(stream), q_out.data_ptr(), q_out.stride(0), lhs.data_ptr(),
            norm_weights.data_ptr() if norm_weights is not None else None, eps, rhs.data_ptr(),
            scales.data_ptr(), zeros.data_ptr() if zeros is not None else None, m, p, width, n_heads,
            block_size, k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[1], pos.data_ptr(), theta)
        self._check(rc)

    def matmul_nt_fp16u8_ws(self, output: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor,
                            scales: torch.Tensor, block_size: int, workspace: torch.Tensor,
                            beta: float = 0.0, zeros: torch.Tensor | None = None, stream=None):
        """adr_matmul_nt_fp16u8_ws: the same product with a scratch buffer to expand weight panels
        into (any contiguous CUDA tensor; its bytes are clobbered)."""
        m, p = lhs.shape
        n = rhs.shape[0]
        assert rhs.shape == (n, p) and output.shape == (m, n) and scales.shape == (n, p // block_size)
        for t in (output, lhs, rhs, scales, workspace) + ((zeros,) if zeros is not None else ()):
            assert t.is_contiguous() and t.is_cuda
        rc = self._lib.adr_matmul_nt_fp16u8_ws(
            self._ctx, _stream_handle(stream), output.data_ptr(), lhs.data_ptr(), rhs.data_ptr(),
            scales.data_ptr(), zeros.data_ptr() if zeros is not None else None, m, p, n, block_size,
            beta, workspace.data_ptr(), workspace.numel() * workspace.element_size())
        self._check(rc)

    def matmul_nt_fp16u8_noalloc(self, output: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor,
                                 scales: torch.Tensor, block_size: int, beta: float = 0.0,
                                 zeros: torch.Tensor | None = None, stream=None):
        """adr_matmul_nt_fp16u8_noalloc: the product of matmul_nt_fp16u8_ws over the library's
        built-in 16 MiB scratch array (one per device: calls that overlap in time race on it)."""
        m, p = lhs.shape
        n = rhs.shape[0]
        assert rhs.shape == (n, p) and output.shape == (m, n) and scales.shape == (n, p // block_size)
        for t in (output, lhs, rhs, scales) + ((zeros,) if zeros is not None else ()):
            assert t.is_contiguous() and t.is_cuda
        rc = self._lib.adr_matmul_nt_fp16u8_noalloc(
            self._ctx, _stream_handle(stream), output.data_ptr(), lhs.data_ptr(), rhs.data_ptr(),
            scales.data_ptr(), zeros.data_ptr() if zeros is not None else None, m, p, n, block_size,
            beta)
        self._check(rc)

    def matmul_nt_f16(self, output: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor,
                      beta: float = 0.0, stream=None):
        """matmul_nt_wmma_128x64x64 / matmul_nt_wmma_16x128x256
        (matmul_nt_wmma_128x64x64.cu:8-14): out = lhs . rhs^T + beta*out."""
        m, p = lhs.shape
        n = rhs.shape[0]
        assert rhs.shape == (n, p) and output.shape == (m, n)
        for t in (output, lhs, rhs):
            assert t.is_contiguous() and t.is_cuda and t.dtype == torch.float16
        rc = self._lib.adr_matmul_nt_f16(self._ctx, _stream_handle(stream), output.data_ptr(),
                                         lhs.data_ptr(), rhs.data_ptr(), m, p, n, beta)
        self._check(rc)

    def dequantize_absmax_uint8(self, output: torch.Tensor, scales: torch.Tensor,
                                q: torch.Tensor, zeros: torch.Tensor | None = None, stream=None):
        """dequantize_absmax_uint8 (quantize.cu:46-56)."""
        rows, k = q.shape
        bs = k // scales.shape[1]
        assert output.shape == (rows, k) and output.dtype == torch.float16
        rc = self._lib.adr_dequantize_absmax_uint8(
            self._ctx, _stream_handle(stream), output.data_ptr(), scales.data_ptr(),
            zeros.data_ptr() if zeros is not None else None, q.data_ptr(), rows, k, bs)
        self._check(rc)

    def quantize_absmax_uint8(self, q: torch.Tensor, scales: torch.Tensor, inp: torch.Tensor,
                              stream=None):
        """quantize_absmax_uint8 (quantize.cu:3-44)."""
        rows, k = inp.shape
        bs = k // scales.shape[1]
        assert q.shape == (rows, k) and q.dtype == torch.uint8 and inp.dtype == torch.float16
        rc = self._lib.adr_quantize_absmax_uint8(self._ctx, _stream_handle(stream), q.data_ptr(),
                                                 scales.data_ptr(), inp.data_ptr(), rows, k, bs)
        self._check(rc)

    # -- the kernels either side of the matmuls ------------------------------
    def rms_norm(self, output: TensorView, input: TensorView, weight: TensorView, eps: float,
                 stream=None):
        """CommonKernels::rms_norm (kernels.rs:198-201, 680-706)."""
        assert input.size(-1) == output.size(-1) and input.size(-2) == output.size(-2)
        assert weight.stride(-1) == 1 and weight.size(-1) == output.size(-1)
        rc = self._lib.adr_rms_norm(self._ctx, _stream_handle(stream), output.data_ptr(),
                                    input.data_ptr(), weight.data_ptr(), output.size(-1),
                                    output.size(-2), output.stride(-1), output.stride(-2),
                                    input.stride(-1), input.stride(-2), eps)
        self._check(rc)

    def layer_norm(self, output: TensorView, input: TensorView, weight: TensorView,
                   bias: TensorView, eps: float, stream=None):
        """CommonKernels::layer_norm (kernels.rs:194-197, 652-678)."""
        assert input.size(-1) == output.size(-1) and input.size(-2) == output.size(-2)
        assert weight.stride(-1) == 1 and weight.size(-1) == output.size(-1)
        assert bias.stride(-1) == 1 and bias.size(-1) == output.size(-1)
        rc = self._lib.adr_layer_norm(self._ctx, _stream_handle(stream), output.data_ptr(),
                                      input.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                      output.size(-1), output.size(-2), output.stride(-1),
                                      output.stride(-2), input.stride(-1), input.stride(-2), eps)
        self._check(rc)

    def rotary_inplace(self, inout: TensorView, n_heads: int, pos_offset: int, theta: float,
                       stream=None):
        """CommonKernels::rotary_inplace (kernels.rs:203-205, 722-751)."""
        rc = self._lib.adr_rotary(self._ctx, _stream_handle(stream), inout.data_ptr(),
                                  inout.data_ptr(), inout.size(-1), inout.size(-2),
                                  inout.stride(-1), inout.stride(-2), inout.stride(-1),
                                  inout.stride(-2), n_heads, pos_offset, theta)
        self._check(rc)

    def softmax_rows_inplace(self, output: TensorView, temperature: float = 1.0, stream=None):
        """CommonKernels::softmax_rows_inplace (kernels.rs:214-216, 892-915); rows may be
        padded (stride(-2) >= size(-1)), matrices must follow one another."""
        nd = len(output.layout.dims)
        heads = output.size(-3) if nd > 2 else 1
        h, w, pitch = output.size(-2), output.size(-1), output.stride(-2)
        assert output.stride(-1) == 1 and (nd <= 2 or output.stride(-3) == h * pitch)
        rc = self._lib.adr_softmax_rows(self._ctx, _stream_handle(stream), output.data_ptr(),
                                        output.data_ptr(), heads, h, w, pitch, temperature)
        self._check(rc)

    def elementwise_binary_2d_f16(self, output: TensorView, left: TensorView, right: TensorView,
                                  op: "BinaryOp", stream=None):
        """The kernel behind elementwise_binary_2d_f16_inplace with a separate output
        (elementwise.cu `elementwise_binary_2d_f16` takes one: kernels.rs:647)."""
        for t in (output, left, right):
            assert t.stride(-1) == 1 and t.size(-1) == output.size(-1) and t.size(-2) == output.size(-2)
        rc = self._lib.adr_elementwise_binary_2d_f16(
            self._ctx, _stream_handle(stream), output.data_ptr(), left.data_ptr(), right.data_ptr(),
            output.size(-2), output.size(-1), output.stride(-2), left.stride(-2), right.stride(-2),
            int(op))
        self._check(rc)

    def elementwise_binary_2d_f16_inplace(self, inout_left: TensorView, right: TensorView,
                                          op: "BinaryOp", stream=None):
        """CommonKernels::elementwise_binary_2d_f16_inplace (kernels.rs:191-193, 633-650)."""
        assert inout_left.stride(-1) == 1 and right.stride(-1) == 1
        assert inout_left.size(-1) == right.size(-1) and inout_left.size(-2) == right.size(-2)
        rc = self._lib.adr_elementwise_binary_2d_f16(
            self._ctx, _stream_handle(stream), inout_left.data_ptr(), inout_left.data_ptr(),
            right.data_ptr(), inout_left.size(-2), inout_left.size(-1), inout_left.stride(-2),
            inout_left.stride(-2), right.stride(-2), int(op))
        self._check(rc)

    def decode_rope_append(self, q: TensorView, k: TensorView, v: TensorView,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int,
                           pos_dev: torch.Tensor, theta: float, stream=None):
        """No reference counterpart (the reference keeps no cache): q[b] rotated in place,
        k[b] rotated into k_cache[b, pos], v[b] copied into v_cache[b, pos]; caches
        [B, S, n_heads*head_dim], pos_dev an int32 device scalar."""
        B, width = q.size(-2), q.size(-1)
        assert k_cache.shape == v_cache.shape and k_cache.shape[0] == B and k_cache.shape[2] == width
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and pos_dev.dtype == torch.int32
        rc = self._lib.adr_decode_rope_append(
            self._ctx, _stream_handle(stream), q.data_ptr(), k.data_ptr(), v.data_ptr(),
            k_cache.data_ptr(), v_cache.data_ptr(), B, n_heads, width // n_heads, k_cache.shape[1],
            q.stride(-2), k.stride(-2), v.stride(-2), pos_dev.data_ptr(), theta)
        self._check(rc)

    def decode_attention(self, out: TensorView, q: TensorView, k_cache: torch.Tensor,
                         v_cache: torch.Tensor, n_heads: int, pos_dev: torch.Tensor, scale: float,
                         stream=None):
        """No reference counterpart: one new token per sequence against the cache, with the
        rounding points of matmul(Scale) -> softmax_rows -> matmul (llama.rs:538-554)."""
        B, width = q.size(-2), q.size(-1)
        assert k_cache.shape == v_cache.shape and k_cache.shape[0] == B and k_cache.shape[2] == width
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and pos_dev.dtype == torch.int32
        rc = self._lib.adr_decode_attention(
            self._ctx, _stream_handle(stream), out.data_ptr(), q.data_ptr(), k_cache.data_ptr(),
            v_cache.data_ptr(), B, n_heads, width // n_heads, k_cache.shape[1], q.stride(-2),
            out.stride(-2), pos_dev.data_ptr(), scale)
        self._check(rc)

    def attention_f16(self, out: TensorView, q: TensorView, k: TensorView, v: TensorView,
                      scale: float, mask: MatmulMask = MatmulMask.None_, stream=None):
        """adr_attention_f16: softmax(scale * q.k^T [causal]) . v in one launch, for views of rank
        2 ([S, hd]), 3 ([heads, S, hd]) or 4 ([outer, inner, S, hd]) with unit innermost stride:
        the reference's matmul(Scale) -> softmax_rows -> matmul chain (llama.rs:538-554,
        clip.rs:374-388).  Raises AdrError(ADR_ERR_SHAPE) for layouts it does not take."""
        def lower(t: TensorView):
            self._f16(t, "attention operand")
            nd = len(t.layout.dims)
            assert 2 <= nd <= 4 and t.stride(-1) == 1
            st = [t.stride(-2), t.stride(-3) if nd > 2 else 0, t.stride(-4) if nd > 3 else 0]
            return (C.c_longlong * 3)(*st)
        nd = len(out.layout.dims)
        inner = out.size(-3) if nd > 2 else 1
        outer = out.size(-4) if nd > 3 else 1
        s_q, hd, s_k = q.size(-2), q.size(-1), k.size(-2)
        assert out.size(-2) == s_q and out.size(-1) == hd and k.size(-1) == hd
        assert v.size(-2) == s_k and v.size(-1) == hd
        rc = self._lib.adr_attention_f16(self._ctx, _stream_handle(stream), out.data_ptr(),
                                         q.data_ptr(), k.data_ptr(), v.data_ptr(), outer, inner,
                                         s_q, s_k, hd, lower(q), lower(k), lower(v), lower(out),
                                         float(scale), int(mask))
        self._check(rc)

    def rms_norm_matmul_nt_fp16u8(self, output: torch.Tensor, lhs: torch.Tensor,
                                  norm_weight: torch.Tensor, eps: float, rhs: torch.Tensor,
                                  scales: torch.Tensor, block_size: int, beta: float = 0.0,
                                  zeros: torch.Tensor | None = None, stream=None):
        """adr_rms_norm_matmul_nt_fp16u8: rms_norm of the rows of lhs, then the u8 product, in one
        launch; raises AdrError(ADR_ERR_SHAPE) for shapes it does not take."""
        m, p = lhs.shape
        n = rhs.shape[0]
        assert rhs.shape == (n, p) and output.shape == (m, n) and norm_weight.shape == (p,)
        for t in (output, lhs, rhs, scales, norm_weight):
            assert t.is_contiguous() and t.is_cuda
        rc = self._lib.adr_rms_norm_matmul_nt_fp16u8(
            self._ctx, _stream_handle(stream), output.data_ptr(), lhs.data_ptr(),
            norm_weight.data_ptr(), eps, rhs.data_ptr(), scales.data_ptr(),
            zeros.data_ptr() if zeros is not None else None, m, p, n, block_size, beta)
        self._check(rc)

    def matmul_nt_fp16u8_allreduce(self, output: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor,
                                   scales: torch.Tensor, block_size: int, residual: bool,
                                   inbox_ptrs, flag_ptrs, epochs: torch.Tensor, max_ctas: int,
                                   rank: int, world: int, zeros: torch.Tensor | None = None,
                                   stream=None):
        """adr_matmul_nt_fp16u8_allreduce: the row-split u8 product with its all-reduce in the same
        kernel; raises AdrError(ADR_ERR_SHAPE) for shapes the decode kernel does not take."""
        m, p = lhs.shape
        n = rhs.shape[0]
        assert rhs.shape == (n, p) and output.shape == (m, n) and scales.shape == (n, p // block_size)
        for t in (output, lhs, rhs, scales):
            assert t.is_contiguous() and t.is_cuda
        boxes = (C.c_void_p * world)(*[int(x) for x in inbox_ptrs])
        flags = (C.c_void_p * world)(*[int(x) for x in flag_ptrs])
        rc = self._lib.adr_matmul_nt_fp16u8_allreduce(
            self._ctx, _stream_handle(stream), output.data_ptr(), lhs.data_ptr(), rhs.data_ptr(),
            scales.data_ptr(), zeros.data_ptr() if zeros is not None else None, m, p, n, block_size,
            int(residual), boxes, flags, epochs.data_ptr(), max_ctas, rank, world)
        self._check(rc)

    def allreduce_oneshot(self, out: torch.Tensor, buf_ptrs, flag_ptrs, epochs: torch.Tensor,
                          blocks: int, rank: int, world: int, count: int, residual: bool,
                          stream=None):
        """adr_allreduce_oneshot: buf_ptrs / flag_ptrs are per-rank device addresses (ints)."""
        bufs = (C.c_void_p * world)(*[int(x) for x in buf_ptrs])
        flags = (C.c_void_p * world)(*[int(x) for x in flag_ptrs])
        rc = self._lib.adr_allreduce_oneshot(self._ctx, _stream_handle(stream), out.data_ptr(), bufs,
                                             flags, epochs.data_ptr(), blocks, rank, world, count,
                                             int(residual))
        self._check(rc)

    def embed_uint8(self, output: torch.Tensor, ids: torch.Tensor, table: torch.Tensor,
                    scales: torch.Tensor, block_size: int, stream=None):
        """embed_uint8 (embed_uint8.cu:3-19): rows `ids` (int16) of the u8 table, dequantised."""
        n_ids, n_dim = output.shape
        assert ids.dtype == torch.int16 and ids.shape == (n_ids,) and table.shape[1] == n_dim
        assert table.dtype == torch.uint8 and output.dtype == torch.float16
        for t in (output, ids, table, scales):
            assert t.is_contiguous() and t.is_cuda
        rc = self._lib.adr_embed_uint8(self._ctx, _stream_handle(stream), n_dim, n_ids, ids.data_ptr(),
                                       output.data_ptr(), table.data_ptr(), scales.data_ptr(), block_size)
        self._check(rc)

    # -- library-side trace (kernel family per distinct call) -------------
    def trace_enable(self, on: bool = True):
        self._check(self._lib.adr_trace_enable(self._ctx, int(on)))

    def trace_dump(self) -> list[dict]:
        need = self._lib.adr_trace_dump(self._ctx, None, 0)
        buf = C.create_string_buffer(need)
        self._lib.adr_trace_dump(self._ctx, buf, need)
        return [json.loads(l) for l in buf.value.decode().splitlines() if l]


class MatmulTracer:
    """Decorator that records the distinct (left, right, out) layouts seen by
    the matmul methods (kernels.rs:231-248, 306-333) and forwards everything."""

    def __init__(self, kernels: GpuKernels):
        self.kernels = kernels
        self.shape_set: set[tuple[TensorLayout, TensorLayout, TensorLayout]] = set()

    def clear(self):
        self.shape_set.clear()

    def shapes(self):
        return list(self.shape_set)

    def matmul_f16(self, output, left, right, options=None, stream=None):
        self.shape_set.add((left.layout, right.layout, output.layout))
        return self.kernels.matmul_f16(output, left, right, options, stream)

    def matmul_f16_slow(self, output, left, right, options=None, stream=None):
        self.shape_set.add((left.layout, right.layout, output.layout))
        return self.kernels.matmul_f16_slow(output, left, right, options, stream)

    def __getattr__(self, name):
        return getattr(self.kernels, name)
