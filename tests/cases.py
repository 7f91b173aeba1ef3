"""Seeded parity cases shared by the golden-vector generator, the CPU tests of
the oracle and the GPU parity tests.

Every case is small enough for the CPU oracle to finish in well under a
second.  A matmul case describes three storage buffers and the views on them
exactly as the reference's call sites build them (citations per case).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import numpy as np

ST_IDENTITY, ST_GELU_BIAS, ST_BETA_GELU_BIAS, ST_BETA_BIAS, ST_SCALE, ST_ADD, ST_QUICK_GELU = range(7)
LD_IDENTITY, LD_SCALE = 0, 1
MK_NONE, MK_CAUSAL = 0, 1


@dataclass
class MatmulCase:
    name: str
    batches: int
    m: int
    k: int
    n: int
    # (x, y, z) strides in elements and element offset, per operand
    out_strides: tuple
    lhs_strides: tuple
    rhs_strides: tuple
    out_size: int
    lhs_size: int
    rhs_size: int
    store: int = ST_IDENTITY
    load: int = LD_IDENTITY
    mask: int = MK_NONE
    beta: float = 0.0
    scale: float = 1.0
    std: float = 1.0
    seed: int = 0
    exact_vs_reference: bool = True  # no transcendental in the epilogue
    note: str = ""

    def strides9(self):
        return (*self.out_strides, *self.lhs_strides, *self.rhs_strides)

    def uses_bias(self):
        return self.store in (ST_BETA_GELU_BIAS, ST_BETA_BIAS, ST_QUICK_GELU)

    def inputs(self):
        """(out_init, lhs, rhs, bias) as flat float16 storage arrays."""
        rng = np.random.default_rng(1000 + self.seed)
        lhs = (rng.standard_normal(self.lhs_size) * self.std).astype(np.float16)
        rhs = (rng.standard_normal(self.rhs_size) * self.std).astype(np.float16)
        out = (rng.standard_normal(self.out_size) * 0.5).astype(np.float16)
        bias = (rng.standard_normal(self.n) * 0.5).astype(np.float16)
        return out, lhs, rhs, bias


def _rm(*dims):
    s, acc = [], 1
    for d in reversed(dims):
        s.append(acc)
        acc *= d
    return tuple(reversed(s))


def matmul_cases() -> list[MatmulCase]:
    cs: list[MatmulCase] = []
    i = 0

    def add(**kw):
        nonlocal i
        cs.append(MatmulCase(seed=i, **kw))
        i += 1

    # linear layer, weight [N,K] passed as permute([1,0]) (llama.rs:503-508): "rrc"
    m, k, n = 64, 256, 96
    add(name="linear_nt", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k, std=0.25)
    # all row-major "rrr" (main.rs:555-564) with tails in every dimension (k % 32 != 0 hits
    # the reference's scalar tail loop, matmul.cu:383-399)
    m, k, n = 33, 70, 45
    add(name="rrr_tails", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(1, n, 0), out_size=m * n, lhs_size=m * k, rhs_size=k * n, std=0.5)
    # the fp16 GEMM workload's distribution N(0, 0.02^2), NT, reduced size
    m, k, n = 64, 512, 128
    add(name="c1_small", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k, std=0.02)
    # attention scores q.k^T with Scale + Causal (llama.rs:535-550): q,k stored [S, H*hd]
    H, S, hd = 4, 37, 32
    D = H * hd
    add(name="qk_scale_causal", batches=H, m=S, k=hd, n=S, out_strides=(1, S, S * S),
        lhs_strides=(1, D, hd), rhs_strides=(D, 1, hd), out_size=H * S * S, lhs_size=S * D,
        rhs_size=S * D, store=ST_SCALE, mask=MK_CAUSAL, scale=1.0 / np.sqrt(hd), std=0.5)
    # CLIP scores: Scale, no mask, odd sequence length (clip.rs:368-377)
    H, S, hd = 3, 29, 64
    D = H * hd
    add(name="qk_scale_nomask", batches=H, m=S, k=hd, n=S, out_strides=(1, S, S * S),
        lhs_strides=(1, D, hd), rhs_strides=(D, 1, hd), out_size=H * S * S, lhs_size=S * D,
        rhs_size=S * D, store=ST_SCALE, scale=0.125, std=0.5)
    # probabilities . v into a strided view of [S, H, hd] (llama.rs:552-554)
    H, S, hd = 4, 37, 32
    D = H * hd
    add(name="pv_strided_out", batches=H, m=S, k=S, n=hd, out_strides=(1, D, hd),
        lhs_strides=(1, S, S * S), rhs_strides=(1, D, hd), out_size=S * D, lhs_size=H * S * S,
        rhs_size=S * D, std=0.3)
    # residual add in place (llama.rs:555-560)
    m, k, n = 40, 96, 80
    add(name="store_add", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k, store=ST_ADD, std=0.3)
    # BetaBias(0.0) and BetaBias(1.0) (clip.rs:350-366, 389-394)
    add(name="beta_bias_0", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k,
        store=ST_BETA_BIAS, beta=0.0, std=0.3)
    add(name="beta_bias_1", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k,
        store=ST_BETA_BIAS, beta=1.0, std=0.3)
    # QuickGeluBias (clip.rs:431-436), BetaGeluBias (whisper.rs:370-381)
    add(name="quick_gelu_bias", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0),
        lhs_strides=(1, k, 0), rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k,
        rhs_size=n * k, store=ST_QUICK_GELU, std=0.3, exact_vs_reference=False)
    add(name="beta_gelu_bias_0", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0),
        lhs_strides=(1, k, 0), rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k,
        rhs_size=n * k, store=ST_BETA_GELU_BIAS, beta=0.0, std=0.3, exact_vs_reference=False)
    add(name="beta_gelu_bias_half", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0),
        lhs_strides=(1, k, 0), rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k,
        rhs_size=n * k, store=ST_BETA_GELU_BIAS, beta=0.5, std=0.3, exact_vs_reference=False)
    # load Scale on both operands (whisper.rs:395-441), combined with a store Scale: the
    # host multiplies the two into one `scale` (kernels.rs:837-843)
    H, S, hd = 2, 24, 16
    D = H * hd
    add(name="load_scale", batches=H, m=S, k=hd, n=S, out_strides=(1, S, S * S),
        lhs_strides=(1, D, hd), rhs_strides=(D, 1, hd), out_size=H * S * S, lhs_size=S * D,
        rhs_size=S * D, load=LD_SCALE, scale=0.5, std=0.7)
    # batched lhs against one broadcast rhs (z-stride 0, kernels.rs:878-880)
    B, m, k, n = 3, 20, 48, 24
    add(name="rhs_broadcast", batches=B, m=m, k=k, n=n, out_strides=(1, n, m * n),
        lhs_strides=(1, k, m * k), rhs_strides=(k, 1, 0), out_size=B * m * n, lhs_size=B * m * k,
        rhs_size=n * k, std=0.4)
    # column-major lhs ("A transposed": stride_ly == 1)
    m, k, n = 24, 40, 56
    add(name="lhs_col_major", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0),
        lhs_strides=(m, 1, 0), rhs_strides=(1, n, 0), out_size=m * n, lhs_size=m * k,
        rhs_size=k * n, std=0.5)
    # column-major output
    add(name="out_col_major", batches=1, m=m, k=k, n=n, out_strides=(m, 1, 0),
        lhs_strides=(1, k, 0), rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k,
        rhs_size=n * k, std=0.5)
    # a 128-row / 256-column tile-aligned case for the tensor-core kernel
    m, k, n = 256, 320, 512
    add(name="tc_aligned", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k, std=0.1)
    # same with ragged m, n and k (k stays a multiple of 8 so rows are 16-byte aligned)
    m, k, n = 200, 328, 392
    add(name="tc_ragged", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k, std=0.1,
        store=ST_BETA_BIAS, beta=1.0)
    # m == 1 (a decode-time linear through the fp16 path)
    m, k, n = 1, 256, 192
    add(name="single_row", batches=1, m=m, k=k, n=n, out_strides=(1, n, 0), lhs_strides=(1, k, 0),
        rhs_strides=(k, 1, 0), out_size=m * n, lhs_size=m * k, rhs_size=n * k, std=0.3)
    return cs


@dataclass
class U8Case:
    name: str
    m: int
    p: int
    n: int
    block_size: int
    beta: float = 0.0
    zeros: bool = False
    seed: int = 0
    tiny_scales: bool = False  # include subnormal / tiny scales (the fp32 dequant path)

    def inputs(self):
        """(out_init, lhs, q, scales, zeros|None): config-2 distributions."""
        rng = np.random.default_rng(2000 + self.seed)
        lhs = rng.standard_normal((self.m, self.p)).astype(np.float16)
        q = rng.integers(0, 256, (self.n, self.p), dtype=np.uint8)
        g = self.p // self.block_size
        scales = rng.uniform(0.001, 0.01, (self.n, g)).astype(np.float16)
        if self.tiny_scales:
            flat = scales.reshape(-1)
            tiny = np.array([0x0001, 0x0003, 0x03FF, 0x0401, 0x07FF, 0x0801, 0x0000, 0x8403],
                            np.uint16).view(np.float16)
            flat[: tiny.size] = tiny
        zeros = rng.uniform(120, 136, (self.n, g)).astype(np.float16) if self.zeros else None
        out = (rng.standard_normal((self.m, self.n)) * 0.5).astype(np.float16)
        return out, lhs, q, scales, zeros


def u8_cases() -> list[U8Case]:
    cs = [
        U8Case("m1", 1, 512, 272, 128),
        U8Case("m1_beta", 1, 256, 130, 64, beta=0.5),
        U8Case("m2", 2, 512, 256, 128),
        U8Case("m4", 4, 512, 264, 128),
        U8Case("m4_bs32", 4, 256, 128, 32),
        U8Case("m8", 8, 512, 256, 128),
        U8Case("m16", 16, 512, 256, 128),
        U8Case("m16_wmma_shape", 16, 512, 256, 128, beta=1.0),
        U8Case("m13_ragged_n", 13, 384, 203, 64),
        U8Case("m1_zeros", 1, 512, 256, 128, zeros=True),
        U8Case("m16_zeros", 16, 512, 256, 128, zeros=True),
        U8Case("m5_zeros_bs256", 5, 512, 144, 256, zeros=True),
        U8Case("m4_tiny_scales", 4, 256, 64, 16, tiny_scales=True),
        U8Case("m40_multi_pass", 40, 256, 192, 128),
        U8Case("m3_p48", 3, 48, 40, 16),  # p not a multiple of 64
    ]
    for i, c in enumerate(cs):
        c.seed = i
    return cs


def digest(*arrays) -> str:
    h = hashlib.sha1()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


# ---------------------------------------------------------------------------
# Row ops (rms_norm, softmax_rows, rotary, elementwise binary): seeded inputs.
# ---------------------------------------------------------------------------
def rowop_cases():
    """name -> dict(kind=..., inputs and parameters).  Sizes cover a ragged tail of the
    256-thread loops, rows shorter than one pass, and large rotary positions."""
    rng = np.random.default_rng(4242)
    f16 = lambda a: np.ascontiguousarray(a, dtype=np.float16)
    out = {}
    for name, rows, lx in (("rms_4096", 5, 4096), ("rms_ragged", 3, 777), ("rms_short", 2, 96)):
        out[name] = dict(kind="rms", x=f16(rng.standard_normal((rows, lx)) * rng.uniform(0.1, 3.0, (rows, 1))),
                         w=f16(rng.uniform(0.5, 1.5, lx)), eps=1e-5)
    for name, heads, h, w, temp in (("softmax_257", 3, 7, 257, 1.0), ("softmax_1000_t", 2, 4, 1000, 0.7),
                                    ("softmax_causal", 2, 33, 33, 1.0)):
        x = rng.standard_normal((heads, h, w)) * 3.0
        if name == "softmax_causal":  # -inf above the diagonal, as the Causal mask stores it
            x[:, np.triu_indices(h, 1)[0], np.triu_indices(h, 1)[1]] = -np.inf
        out[name] = dict(kind="softmax", x=f16(x), temp=temp)
    for name, ly, lx, heads, pos in (("rotary_0", 9, 512, 4, 0), ("rotary_500", 4, 256, 2, 500),
                                     ("rotary_hd64", 17, 128, 2, 3)):
        out[name] = dict(kind="rotary", x=f16(rng.standard_normal((ly, lx))), n_heads=heads,
                         pos_offset=pos, theta=10000.0)
    for name, rows, cols, op in (("add_1000", 6, 1000, 1), ("silu_mul_1000", 6, 1000, 2),
                                 ("silu_mul_wide", 3, 4096, 2)):
        out[name] = dict(kind="binary", left=f16(rng.standard_normal((rows, cols)) * 2.5),
                         right=f16(rng.standard_normal((rows, cols))), op=op)
    return out
