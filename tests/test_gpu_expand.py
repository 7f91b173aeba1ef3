"""GPU parity of adr_matmul_nt_fp16u8_ws: the u8-weight product for long prefills that expands
panels of weight rows to fp16 in caller-provided scratch memory and multiplies them with the
fp16 tensor-core GEMM.  Same arithmetic as the prefill kernels (weights rounded to fp16,
matmul_nt_wmma_16x128x256_fp16u8.cu:5-7), so the same tolerance against the oracle."""
import numpy as np
import pytest
import torch

from adrastea_b200 import Kernel
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make(rng, m, p, n, bs, zp):
    x = rng.standard_normal((m, p)).astype(np.float16)
    q = rng.integers(0, 256, (n, p), dtype=np.uint8)
    s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
    z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
    out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
    return x, q, s, z, out0


@pytest.mark.parametrize("zp", [False, True])
def test_expansion_path_against_oracle(kernels, zp):
    """Enough rows for the expansion path; scratch sized for 256 weight rows, so the product
    runs as several panels with a ragged last one; beta on and off; twice, same bits."""
    rng = np.random.default_rng(31 + zp)
    for m, p, n, bs, beta in ((3072, 512, 520, 64, 0.0), (3200, 384, 776, 128, 0.5)):
        x, q, s, z, out0 = make(rng, m, p, n, bs, zp)
        want = oracle.matmul_nt_fp16u8(x, q, s, bs, beta, out0, z)
        ws = torch.empty(256 * p, dtype=torch.float16, device="cuda")
        xd, qd, sd, zd = dev(x), dev(q), dev(s), (dev(z) if zp else None)
        res = []
        for _ in range(2):
            o = dev(out0.copy())
            kernels.matmul_nt_fp16u8_ws(o, xd, qd, sd, bs, ws, beta, zd)
            kernels.device_status()
            res.append(o.cpu().numpy())
        assert kernels.last_kernel() == Kernel.F16Tc, "the scratch path did not run"
        assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))
        assert oracle.max_rel_err(res[0], want) <= TOL, (m, p, n)
        # the entry point without scratch computes the same product
        o = dev(out0.copy())
        kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs, beta, zd)
        assert oracle.max_rel_err(o.cpu().numpy(), res[0]) <= TOL


def test_expanded_panel_is_the_exact_dequantisation(kernels):
    """With an identity-like lhs (one 1.0 per row) the product reads back the expanded weights:
    they are the fp16-rounded dequantisation, bit for bit."""
    rng = np.random.default_rng(5)
    m, p, n, bs = 3072, 256, 264, 64
    _, q, s, z, _ = make(rng, m, p, n, bs, True)
    x = np.zeros((m, p), np.float16)
    x[np.arange(m), np.arange(m) % p] = 1.0
    ws = torch.empty(128 * p, dtype=torch.float16, device="cuda")
    o = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    kernels.matmul_nt_fp16u8_ws(o, dev(x), dev(q), dev(s), bs, ws, 0.0, dev(z))
    kernels.device_status()
    assert kernels.last_kernel() == Kernel.F16Tc
    w = oracle.dequantize(q, s, bs, z)          # [n, p] fp16
    want = w.T[np.arange(m) % p, :]                          # row i of out = column (i % p) of w
    assert np.array_equal(o.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_falls_back_without_usable_scratch(kernels):
    """Few rows, no scratch, or scratch too small for one tile of weight rows: the call gives
    exactly what adr_matmul_nt_fp16u8 gives."""
    rng = np.random.default_rng(9)
    for m, ws_rows in ((64, 256), (3072, 0), (3072, 64)):
        p, n, bs = 256, 136, 64
        x, q, s, _, out0 = make(rng, m, p, n, bs, False)
        xd, qd, sd = dev(x), dev(q), dev(s)
        a, b = dev(out0.copy()), dev(out0.copy())
        ws = torch.empty(max(ws_rows * p, 8), dtype=torch.float16, device="cuda")
        kernels.matmul_nt_fp16u8_ws(a, xd, qd, sd, bs, ws, 0.5)
        assert kernels.last_kernel() != Kernel.F16Tc
        kernels.matmul_nt_fp16u8(b, xd, qd, sd, bs, 0.5)
        kernels.device_status()
        assert np.array_equal(a.cpu().numpy().view(np.uint16), b.cpu().numpy().view(np.uint16))
