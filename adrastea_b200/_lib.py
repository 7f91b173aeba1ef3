"""ctypes binding of libadrastea_b200.so (the C ABI in include/adrastea_b200.h).

There is no fallback: if the shared object is missing or a symbol cannot be
resolved, importing or calling fails with an error that says so.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from .build import LIB_PATH

_c_int = C.c_int
_vp = C.c_void_p

# name -> (restype, argtypes); one entry per declaration in include/adrastea_b200.h
_MATMUL_F16_ARGS = [_vp, _vp, _vp, _vp, _vp] + [_c_int] * 13 + [_vp, C.c_float, C.c_float,
                                                               C.c_uint32, C.c_uint32, C.c_uint32]
SIGNATURES = {
    "adr_init": (_c_int, [_c_int, C.POINTER(_vp)]),
    "adr_destroy": (None, [_vp]),
    "adr_strerror": (C.c_char_p, [_c_int]),
    "adr_last_cuda_error": (_c_int, [_vp]),
    "adr_force_kernel": (_c_int, [_vp, _c_int]),
    "adr_last_kernel": (_c_int, [_vp]),
    "adr_set_tunable": (_c_int, [_vp, C.c_char_p, _c_int]),
    "adr_device_status": (_c_int, [_vp]),
    "adr_launch_count": (C.c_uint64, [_vp]),
    "adr_matmul_f16": (_c_int, _MATMUL_F16_ARGS),
    "adr_matmul_f16_slow": (_c_int, _MATMUL_F16_ARGS),
    # (ctx, stream, out, lhs, rhs) + outer batches + (batches, m, k, n) + 12 strides + bias + ...
    "adr_matmul_f16_b2": (_c_int, [_vp] * 5 + [_c_int] * 17 + [_vp, C.c_float, C.c_float, C.c_uint32,
                                                         C.c_uint32, C.c_uint32]),
    "adr_matmul_f16_raw": (_c_int, [_vp, _vp, _vp, _vp, _vp] + [_c_int] * 13),
    "adr_matmul_nt_fp16u8": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int,
                                      _c_int, C.c_float]),
    "adr_matmul_nt_fp16u8_ws": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int,
                                         _c_int, C.c_float, _vp, C.c_size_t]),
    "adr_matmul_nt_fp16u8_noalloc": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int,
                                              _c_int, _c_int, C.c_float]),
    "adr_matmul_nt_fp16u8_grouped": (_c_int, [_vp, _vp, _c_int, C.POINTER(_vp), _vp, C.POINTER(_vp),
                                              C.POINTER(_vp), C.POINTER(_vp), _c_int, _c_int,
                                              C.POINTER(_c_int), _c_int, C.c_float]),
    "adr_silu_mul_matmul_nt_fp16u8": (_c_int, [_vp] * 10 + [_c_int] * 4),
    "adr_qkv_rope_append_matmul_nt_fp16u8": (_c_int, [_vp, _vp, _vp, _c_int, _vp, _vp, C.c_float, _vp,
                                                      _vp, _vp, _c_int, _c_int, _c_int, _c_int,
                                                      _c_int, _vp, _vp, _c_int, _vp, C.c_float]),
    "adr_matmul_nt_f16": (_c_int, [_vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, C.c_float]),
    "adr_dequantize_absmax_uint8": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int]),
    "adr_quantize_absmax_uint8": (_c_int, [_vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int]),
    "adr_embed_uint8": (_c_int, [_vp, _vp, _c_int, _c_int, _vp, _vp, _vp, _vp, _c_int]),
    "adr_rms_norm": (_c_int, [_vp, _vp, _vp, _vp, _vp] + [_c_int] * 6 + [C.c_float]),
    "adr_layer_norm": (_c_int, [_vp] * 6 + [_c_int] * 6 + [C.c_float]),
    "adr_softmax_rows": (_c_int, [_vp, _vp, _vp, _vp] + [_c_int] * 4 + [C.c_float]),
    "adr_rotary": (_c_int, [_vp, _vp, _vp, _vp] + [_c_int] * 8 + [C.c_float]),
    "adr_elementwise_binary_2d_f16": (_c_int, [_vp, _vp, _vp, _vp, _vp] + [_c_int] * 5 + [C.c_uint32]),
    "adr_decode_rope_append": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp] + [_c_int] * 7
                               + [_vp, C.c_float]),
    "adr_decode_attention": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp] + [_c_int] * 6
                             + [_vp, C.c_float]),
    "adr_attention_f16": (_c_int, [_vp] * 6 + [_c_int] * 5 + [_vp] * 4 + [C.c_float, C.c_uint32]),
    "adr_allreduce_oneshot": (_c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int,
                                       C.c_longlong, _c_int]),
    "adr_rms_norm_matmul_nt_fp16u8": (_c_int, [_vp, _vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _vp,
                                             _c_int, _c_int, _c_int, _c_int, C.c_float]),
    "adr_matmul_nt_fp16u8_allreduce": (_c_int, [_vp] * 7 + [_c_int] * 5 + [_vp, _vp, _vp]
                                       + [_c_int] * 3),
    "adr_trace_enable": (_c_int, [_vp, _c_int]),
    "adr_trace_clear": (None, [_vp]),
    "adr_trace_dump": (C.c_size_t, [_vp, C.c_char_p, C.c_size_t]),
}

_lib = None


def load(path: str | Path | None = None) -> C.CDLL:
    """Load the shared object and bind every declared symbol."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else LIB_PATH
    if not p.exists():
        raise ImportError(
            f"{p} is missing: build it with `python -m adrastea_b200.build` "
            "(there is no CPU or PyTorch fallback for this library)")
    lib = C.CDLL(str(p))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(f"{p} does not export {name}") from e
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _lib = lib
    return lib
