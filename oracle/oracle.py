"""ctypes/numpy front end of oracle/liboracle.so (see adr_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline legs of bench.py.  fp16 arrays travel as numpy float16.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"

_lib = None


def build(with_reference: bool = True) -> None:
    """Run oracle/Makefile (liboracle.so; reference cubins when the tree is there)."""
    target = ["all"] if with_reference else ["liboracle.so"]
    res = subprocess.run(["make", "-C", str(HERE), *target], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + res.stdout + res.stderr)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build(with_reference=False)
        _lib = C.CDLL(str(LIB))
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f64_to_f16.restype = C.c_uint16
        _lib.orc_f64_to_f16.argtypes = [C.c_double]
        _lib.orc_hmul.restype = C.c_uint16
        _lib.orc_hmul.argtypes = [C.c_uint16, C.c_uint16]
        _lib.orc_hadd.restype = C.c_uint16
        _lib.orc_hadd.argtypes = [C.c_uint16, C.c_uint16]
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_set_num_threads.restype = C.c_int
        _lib.orc_set_num_threads.argtypes = [C.c_int]
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _chk16(a: np.ndarray):
    assert a.dtype == np.float16, a.dtype


def matmul_f16(out: np.ndarray, lhs: np.ndarray, rhs: np.ndarray, batches, m, k, n, strides,
               bias: np.ndarray | None = None, beta=0.0, scale=1.0, store=0, load=0, mask=0,
               ideal=False, offsets=(0, 0, 0)) -> int:
    """Run the restated kernel on flat fp16 buffers.

    `out`, `lhs`, `rhs` are 1-D float16 storage arrays; `strides` is the
    9-tuple (ox, oy, oz, lx, ly, lz, rx, ry, rz) in elements; `offsets` are
    element offsets of the three views into their storage.  `out` is updated
    in place.  Returns the status (0 ok, 3 unsupported op).
    """
    for a in (out, lhs, rhs):
        _chk16(a)
        assert a.ndim == 1 and a.flags.c_contiguous
    fn = lib().orc_matmul_f16_ideal if ideal else lib().orc_matmul_f16_ref
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 3 + [C.c_int] * 13 + [C.c_void_p, C.c_float, C.c_float,
                                                        C.c_uint, C.c_uint, C.c_uint]
    base = lambda a, off: C.c_void_p(a.ctypes.data + 2 * off)
    if bias is not None:
        _chk16(bias)
    return fn(base(out, offsets[0]), base(lhs, offsets[1]), base(rhs, offsets[2]), batches, m, k, n,
              *[int(s) for s in strides], _p(bias), float(beta), float(scale), int(store),
              int(load), int(mask))


def dequantize(q: np.ndarray, scales: np.ndarray, block_size: int,
               zeros: np.ndarray | None = None) -> np.ndarray:
    rows, k = q.shape
    assert q.dtype == np.uint8 and q.flags.c_contiguous
    _chk16(scales)
    out = np.empty((rows, k), np.float16)
    f = lib().orc_dequantize_absmax_uint8
    f.restype = None
    f.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3
    f(_p(out), _p(np.ascontiguousarray(scales)), _p(zeros), _p(q), rows, k, block_size)
    return out


def quantize(x: np.ndarray, block_size: int) -> tuple[np.ndarray, np.ndarray]:
    rows, k = x.shape
    _chk16(x)
    q = np.empty((rows, k), np.uint8)
    s = np.empty((rows, k // block_size), np.float16)
    f = lib().orc_quantize_absmax_uint8
    f.restype = None
    f.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3
    f(_p(q), _p(s), _p(np.ascontiguousarray(x)), rows, k, block_size)
    return q, s


def matmul_nt_fp16u8(lhs: np.ndarray, q: np.ndarray, scales: np.ndarray, block_size: int,
                     beta=0.0, out: np.ndarray | None = None, zeros: np.ndarray | None = None,
                     faithful=False) -> np.ndarray:
    """faithful=True: matmul_nt_fp16u8.cu's own arithmetic (no zeros);
    faithful=False: bit-exact fp16 dequantisation, exact products, wide accumulation."""
    m, p = lhs.shape
    n = q.shape[0]
    _chk16(lhs)
    _chk16(scales)
    res = np.zeros((m, n), np.float16) if out is None else np.ascontiguousarray(out).copy()
    if faithful:
        assert zeros is None
        f = lib().orc_matmul_nt_fp16u8_ref
        f.restype = None
        f.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float]
        f(_p(res), _p(np.ascontiguousarray(lhs)), _p(q), _p(np.ascontiguousarray(scales)), m, p, n,
          block_size, float(beta))
    else:
        f = lib().orc_matmul_nt_fp16u8_ideal
        f.restype = None
        f.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4 + [C.c_float]
        f(_p(res), _p(np.ascontiguousarray(lhs)), _p(q), _p(np.ascontiguousarray(scales)),
          _p(zeros), m, p, n, block_size, float(beta))
    return res


def matmul_nt_f16(lhs: np.ndarray, rhs: np.ndarray, beta=0.0, out: np.ndarray | None = None):
    m, p = lhs.shape
    n = rhs.shape[0]
    res = np.zeros((m, n), np.float16) if out is None else np.ascontiguousarray(out).copy()
    f = lib().orc_matmul_nt_f16_ideal
    f.restype = None
    f.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_float]
    f(_p(res), _p(np.ascontiguousarray(lhs)), _p(np.ascontiguousarray(rhs)), m, p, n, float(beta))
    return res


def error_stats(a: np.ndarray, b: np.ndarray) -> tuple[float, float, float]:
    """[MSE, max|d|, MAE] as error_stats.cu:13 defines them."""
    a = np.ascontiguousarray(a, np.float16).reshape(-1)
    b = np.ascontiguousarray(b, np.float16).reshape(-1)
    out = (C.c_float * 3)()
    f = lib().orc_error_stats_f16
    f.restype = None
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
    f(out, _p(a), _p(b), a.size)
    return float(out[0]), float(out[1]), float(out[2])


def sgemm(a: np.ndarray, b: np.ndarray, c: np.ndarray | None = None, alpha=1.0, beta=0.0):
    """C = alpha*A.B + beta*C on f32 arrays of any 2-D strides (mel.rs:140-158 convention)."""
    m, k = a.shape
    k2, n = b.shape
    assert k == k2 and a.dtype == np.float32 and b.dtype == np.float32
    if c is None:
        c = np.zeros((m, n), np.float32)
    f = lib().orc_sgemm
    f.restype = None
    f.argtypes = [C.c_int] * 3 + [C.c_float, C.c_void_p, C.c_ssize_t, C.c_ssize_t, C.c_void_p,
                                  C.c_ssize_t, C.c_ssize_t, C.c_float, C.c_void_p, C.c_ssize_t,
                                  C.c_ssize_t]
    es = 4
    f(m, k, n, float(alpha), _p(a), a.strides[0] // es, a.strides[1] // es, _p(b),
      b.strides[0] // es, b.strides[1] // es, float(beta), _p(c), c.strides[0] // es,
      c.strides[1] // es)
    return c


def max_rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max |got-ref| / max(|ref|, rms(ref)): relative error with a floor that keeps
    near-zero outputs from dominating."""
    g = got.astype(np.float64).reshape(-1)
    r = ref.astype(np.float64).reshape(-1)
    fin = np.isfinite(r)
    if not np.array_equal(np.isfinite(g), fin):
        return float("inf")
    if (~fin).any() and not np.array_equal(np.nan_to_num(g[~fin], nan=7e300),
                                           np.nan_to_num(r[~fin], nan=7e300)):
        return float("inf")
    g, r = g[fin], r[fin]
    if r.size == 0:
        return 0.0
    rms = float(np.sqrt(np.mean(r * r)))
    den = np.maximum(np.abs(r), max(rms, 1e-30))
    return float(np.max(np.abs(g - r) / den))


# ---------------------------------------------------------------------------
# row ops (the kernels either side of the matmuls)
# ---------------------------------------------------------------------------
def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    ly, lx = x.shape
    x = np.ascontiguousarray(x)
    _chk16(x)
    out = np.zeros_like(x)
    f = lib().orc_rms_norm
    f.restype = None
    f.argtypes = [C.c_void_p] * 3 + [C.c_int] * 6 + [C.c_float]
    f(_p(out), _p(x), _p(np.ascontiguousarray(w)), lx, ly, 1, lx, 1, lx, float(eps))
    return out


def layer_norm(x: np.ndarray, w: np.ndarray, b: np.ndarray, eps: float) -> np.ndarray:
    ly, lx = x.shape
    x = np.ascontiguousarray(x)
    _chk16(x)
    out = np.zeros_like(x)
    f = lib().orc_layer_norm
    f.restype = None
    f.argtypes = [C.c_void_p] * 4 + [C.c_int] * 6 + [C.c_float]
    f(_p(out), _p(x), _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(b)), lx, ly, 1, lx, 1, lx,
      float(eps))
    return out


def softmax_rows(x: np.ndarray, w: int | None = None, temp: float = 1.0) -> np.ndarray:
    """x: [heads, h, pitch]; softmax over the first w elements of every row (others kept)."""
    heads, h, pitch = x.shape
    x = np.ascontiguousarray(x)
    _chk16(x)
    out = x.copy()
    f = lib().orc_softmax_rows
    f.restype = None
    f.argtypes = [C.c_void_p] * 2 + [C.c_int] * 4 + [C.c_float]
    f(_p(out), _p(x), heads, h, pitch if w is None else w, pitch, float(temp))
    return out


def rotary(x: np.ndarray, n_heads: int, pos_offset: int, theta: float, same_pos=False) -> np.ndarray:
    ly, lx = x.shape
    x = np.ascontiguousarray(x)
    _chk16(x)
    out = np.zeros_like(x)
    f = lib().orc_rotary
    f.restype = None
    f.argtypes = [C.c_void_p] * 2 + [C.c_int] * 8 + [C.c_float, C.c_int]
    f(_p(out), _p(x), lx, ly, 1, lx, 1, lx, n_heads, pos_offset, float(theta), int(same_pos))
    return out


def elementwise_binary(left: np.ndarray, right: np.ndarray, op: int) -> np.ndarray:
    rows, cols = left.shape
    left, right = np.ascontiguousarray(left), np.ascontiguousarray(right)
    _chk16(left)
    _chk16(right)
    out = np.zeros_like(left)
    f = lib().orc_elementwise_binary_2d_f16
    f.restype = C.c_int
    f.argtypes = [C.c_void_p] * 3 + [C.c_int] * 6
    rc = f(_p(out), _p(left), _p(right), rows, cols, cols, cols, cols, op)
    if rc != 0:
        raise ValueError(f"unsupported binary op {op}")
    return out


def decode_attention(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, n_heads: int,
                     pos: int, scale: float) -> np.ndarray:
    """q: [B, H*hd]; caches: [B, S, H*hd] -> [B, H*hd]."""
    B, width = q.shape
    S = k_cache.shape[1]
    q, k_cache, v_cache = (np.ascontiguousarray(a) for a in (q, k_cache, v_cache))
    for a in (q, k_cache, v_cache):
        _chk16(a)
    out = np.zeros_like(q)
    f = lib().orc_decode_attention
    f.restype = None
    f.argtypes = [C.c_void_p] * 4 + [C.c_int] * 7 + [C.c_float]
    f(_p(out), _p(q), _p(k_cache), _p(v_cache), B, n_heads, width // n_heads, S, width, width,
      pos, float(scale))
    return out


def embed_uint8(ids: np.ndarray, table: np.ndarray, scales: np.ndarray, block_size: int) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.int16)
    out = np.zeros((ids.shape[0], table.shape[1]), np.float16)
    _chk16(scales)
    f = lib().orc_embed_uint8
    f.restype = None
    f.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 4 + [C.c_int]
    f(table.shape[1], ids.shape[0], _p(ids), _p(out), _p(np.ascontiguousarray(table)),
      _p(np.ascontiguousarray(scales)), block_size)
    return out
