"""Launcher for the reference's own device kernels (oracle/_ref/*.cubin).

TEST INFRASTRUCTURE ONLY.  The cubins are compiled by oracle/Makefile from the
unmodified reference sources; this module loads them with the CUDA driver API
and launches them with the geometry the reference's host code uses
(adrastea_models/src/kernels.rs:782-792, 849-863; the launch comments in
adrastea_kernels/cpp/matmul_nt_wmma_*.cu:5-7).  It needs a GPU and the cubins;
`available()` says whether both are there.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"

_modules: dict[str, object] = {}
_functions: dict[tuple[str, str], object] = {}


def available() -> bool:
    return torch.cuda.is_available() and (REF_DIR / "matmul.cubin").exists()


def _cu():
    from cuda.bindings import driver
    return driver


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1] if len(res) == 2 else res[1:]


def _function(cubin: str, name: str):
    key = (cubin, name)
    if key not in _functions:
        cu = _cu()
        torch.cuda.current_stream().synchronize()  # primary context is current after this
        if cubin not in _modules:
            data = (REF_DIR / f"{cubin}.cubin").read_bytes()
            _modules[cubin] = _check(cu.cuModuleLoadData(data))
        _functions[key] = _check(cu.cuModuleGetFunction(_modules[cubin], name.encode()))
    return _functions[key]


def _launch(fn, grid, block, smem, holders):
    cu = _cu()
    argv = (C.c_void_p * len(holders))(*[C.addressof(h) for h in holders])
    if smem > 48 * 1024:
        _check(cu.cuFuncSetAttribute(
            fn, cu.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem))
    stream = torch.cuda.current_stream().cuda_stream
    _check(cu.cuLaunchKernel(fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem,
                             stream, C.addressof(argv), 0))


def _cdiv(a, b):
    return (a + b - 1) // b


def matmul_f16(kernel: str, out_ptr: int, lhs_ptr: int, rhs_ptr: int, batches, m, k, n, strides,
               bias_ptr: int | None, beta: float, scale: float, store: int, load: int, mask: int):
    """kernel in {"matmul_f16", "matmul_f16_fast"} (matmul.cu:493-513)."""
    fn = _function("matmul", kernel)
    holders = [C.c_void_p(out_ptr), C.c_void_p(lhs_ptr), C.c_void_p(rhs_ptr), C.c_int(batches),
               C.c_int(m), C.c_int(k), C.c_int(n)]
    holders += [C.c_int(int(s)) for s in strides]
    holders += [C.c_void_p(bias_ptr or 0), C.c_float(beta), C.c_float(scale), C.c_uint(store),
                C.c_uint(load), C.c_uint(mask)]
    if kernel == "matmul_f16_fast":
        grid, block, smem = (_cdiv(n, 32), _cdiv(m, 16), batches), (32, 4, 1), 16 * 34 * 2 + 32 * 34 * 2
    else:
        grid, block, smem = (_cdiv(n, 16), _cdiv(m, 16), batches), (16, 16, 1), 0
    _launch(fn, grid, block, smem, holders)


def matmul_nt_fp16u8(out_ptr, lhs_ptr, rhs_ptr, scales_ptr, m, p, n, block_size, beta):
    """matmul_nt_fp16u8.cu:4-24; one thread per output."""
    fn = _function("matmul_nt_fp16u8", "matmul_nt_fp16u8")
    holders = [C.c_void_p(out_ptr), C.c_void_p(lhs_ptr), C.c_void_p(rhs_ptr),
               C.c_void_p(scales_ptr), C.c_int(m), C.c_int(p), C.c_int(n), C.c_int(block_size),
               C.c_float(beta)]
    _launch(fn, (_cdiv(n, 16), _cdiv(m, 16), 1), (16, 16, 1), 0, holders)


def matmul_nt_wmma_16x128x256_fp16u8(out_ptr, lhs_ptr, rhs_ptr, scales_ptr, m, p, n, block_size,
                                     beta):
    assert m % 16 == 0 and n % 128 == 0 and p % 256 == 0 and block_size % 4 == 0
    fn = _function("matmul_nt_wmma_16x128x256_fp16u8", "matmul_nt_wmma_16x128x256_fp16u8")
    holders = [C.c_void_p(out_ptr), C.c_void_p(lhs_ptr), C.c_void_p(rhs_ptr),
               C.c_void_p(scales_ptr), C.c_int(m), C.c_int(p), C.c_int(n), C.c_int(block_size),
               C.c_float(beta)]
    _launch(fn, ((m // 16) * (n // 128), 1, 1), (256, 1, 1), (16 + 128) * 272 * 2, holders)


def matmul_nt_wmma_16x128x256(out_ptr, lhs_ptr, rhs_ptr, m, p, n, beta):
    assert m % 16 == 0 and n % 128 == 0 and p % 256 == 0
    fn = _function("matmul_nt_wmma_16x128x256", "matmul_nt_wmma_16x128x256")
    holders = [C.c_void_p(out_ptr), C.c_void_p(lhs_ptr), C.c_void_p(rhs_ptr), C.c_int(m),
               C.c_int(p), C.c_int(n), C.c_float(beta)]
    _launch(fn, ((m // 16) * (n // 128), 1, 1), (256, 1, 1), (16 + 128) * 272 * 2, holders)


def matmul_nt_wmma_128x64x64(out_ptr, lhs_ptr, rhs_ptr, m, p, n, beta):
    assert m % 128 == 0 and n % 64 == 0 and p % 64 == 0
    fn = _function("matmul_nt_wmma_128x64x64", "matmul_nt_wmma_128x64x64")
    holders = [C.c_void_p(out_ptr), C.c_void_p(lhs_ptr), C.c_void_p(rhs_ptr), C.c_int(m),
               C.c_int(p), C.c_int(n), C.c_float(beta)]
    _launch(fn, ((m // 128) * (n // 64), 1, 1), (256, 1, 1), 128 * 64 * 4, holders)


class _TensorViewDesc(C.Structure):
    """Device-side TensorView<T> (compat.h:40-45): index 0 = innermost dimension."""
    _fields_ = [("ptr", C.c_void_p), ("dims", C.c_uint32), ("shape", C.c_uint32 * 7),
                ("strides", C.c_uint32 * 7)]


def _desc2d(ptr, rows, cols):
    d = _TensorViewDesc()
    d.ptr = ptr
    d.dims = 2
    d.shape[0], d.shape[1] = cols, rows
    d.strides[0], d.strides[1] = 1, cols
    return d


def quantize_absmax_uint8(q_ptr, scales_ptr, in_ptr, rows, k, block_size):
    fn = _function("quantize", "_Z21quantize_absmax_uint810TensorViewIhES_I6__halfES2_")
    groups = k // block_size
    holders = [_desc2d(q_ptr, rows, k), _desc2d(scales_ptr, rows, groups), _desc2d(in_ptr, rows, k)]
    _launch(fn, (groups, rows, 1), (min(block_size, 1024), 1, 1), 0, holders)


def dequantize_absmax_uint8(out_ptr, scales_ptr, q_ptr, rows, k, block_size):
    fn = _function("quantize", "_Z23dequantize_absmax_uint810TensorViewI6__halfES1_S_IhE")
    groups = k // block_size
    holders = [_desc2d(out_ptr, rows, k), _desc2d(scales_ptr, rows, groups), _desc2d(q_ptr, rows, k)]
    _launch(fn, (groups, rows, 1), (min(block_size, 1024), 1, 1), 0, holders)


def rms_norm(out_ptr, in_ptr, w_ptr, lx, ly, s_ox, s_oy, s_ix, s_iy, eps):
    """normalize.cu:7-16 with the launch of kernels.rs:686-704 (one block of 256 per row)."""
    fn = _function("normalize", "rms_norm")
    holders = [C.c_void_p(out_ptr), C.c_void_p(in_ptr), C.c_void_p(w_ptr)]
    holders += [C.c_int(int(v)) for v in (lx, ly, s_ox, s_oy, s_ix, s_iy)] + [C.c_float(eps)]
    _launch(fn, (ly, 1, 1), (256, 1, 1), 0, holders)


def layer_norm(out_ptr, in_ptr, w_ptr, b_ptr, lx, ly, s_ox, s_oy, s_ix, s_iy, eps):
    """normalize.cu:63-73 with the launch of kernels.rs:656-676 (one block of 256 per row)."""
    fn = _function("normalize", "layer_norm")
    holders = [C.c_void_p(out_ptr), C.c_void_p(in_ptr), C.c_void_p(w_ptr), C.c_void_p(b_ptr)]
    holders += [C.c_int(int(v)) for v in (lx, ly, s_ox, s_oy, s_ix, s_iy)] + [C.c_float(eps)]
    _launch(fn, (ly, 1, 1), (256, 1, 1), 0, holders)


def softmax_rows(out_ptr, in_ptr, heads, h, w, temp):
    """normalize.cu:150-154 with the launch of kernels.rs:895-913 (contiguous rows)."""
    fn = _function("normalize", "softmax_rows")
    holders = [C.c_void_p(out_ptr), C.c_void_p(in_ptr), C.c_int(h), C.c_int(w), C.c_float(temp)]
    _launch(fn, (h, heads, 1), (256, 1, 1), 0, holders)


def rotary(out_ptr, in_ptr, lx, ly, s_ox, s_oy, s_ix, s_iy, n_heads, pos_offset, theta):
    """rotary.cu:4-14 with the launch of kernels.rs:725-749."""
    fn = _function("rotary", "rotary")
    holders = [C.c_void_p(out_ptr), C.c_void_p(in_ptr)]
    holders += [C.c_int(int(v)) for v in (lx, ly, s_ox, s_oy, s_ix, s_iy, n_heads, pos_offset)]
    holders += [C.c_float(theta)]
    _launch(fn, (_cdiv(lx, 16), _cdiv(ly, 16), 1), (16, 16, 1), 0, holders)


def elementwise_binary_2d_f16(out_ptr, left_ptr, right_ptr, rows, cols, op):
    """elementwise.cu `elementwise_binary_2d_f16` with the launch of kernels.rs:636-648
    (contiguous [rows, cols] operands)."""
    fn = _function("elementwise", "elementwise_binary_2d_f16")
    holders = [_desc2d(out_ptr, rows, cols), _desc2d(left_ptr, rows, cols),
               _desc2d(right_ptr, rows, cols), C.c_uint(op)]
    _launch(fn, (_cdiv(cols, 16), _cdiv(rows, 16), 1), (16, 16, 1), 0, holders)


def embed_uint8(n_dim, n_ids, ids_ptr, out_ptr, table_ptr, scales_ptr, block_size):
    """embed_uint8.cu:3-9; the kernel has no call site in the reference: launched like the fp16
    `embed` kernel (kernels.rs:923-927), 1024 threads per block, one thread per token."""
    fn = _function("embed_uint8", "embed_uint8")
    holders = [C.c_int(n_dim), C.c_int(n_ids), C.c_void_p(ids_ptr), C.c_void_p(out_ptr),
               C.c_void_p(table_ptr), C.c_void_p(scales_ptr), C.c_int(block_size)]
    _launch(fn, (_cdiv(n_ids, 1024), 1, 1), (1024, 1, 1), 0, holders)
