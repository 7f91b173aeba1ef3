"""GPU test of adr_matmul_nt_fp16u8_noalloc, the u8-weight product that takes its scratch from
an array built into the library instead of from the caller.  Collected last (file name), so it
also runs behind every other test's use of the library; it passes alone as well.

The reference result is the existing entry point adr_matmul_nt_fp16u8_ws given a workspace of
the built-in array's size: both then cut the weights into the same panels and launch the same
kernels, so the outputs agree bit for bit."""
import numpy as np
import pytest
import torch

from adrastea_b200 import AdrError, Kernel
from oracle import oracle

pytestmark = pytest.mark.gpu
BUILTIN_BYTES = 16 << 20
ERR_TOO_LARGE = 7


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def problem(rng, m, p, n, bs, zp):
    x = rng.standard_normal((m, p)).astype(np.float16)
    q = rng.integers(0, 256, (n, p), dtype=np.uint8)
    s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
    z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
    out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
    return x, q, s, z, out0


def test_two_calls_in_a_row_match_the_workspace_entry_point(kernels):
    """Two different products back to back over the same built-in array (the second finds the
    first one's panels in it): each equals the workspace entry point bit for bit and the oracle
    within the prefill tolerance; no device memory is taken or returned by the calls."""
    rng = np.random.default_rng(77)
    ws = torch.empty(BUILTIN_BYTES, dtype=torch.uint8, device="cuda")
    cases = [problem(rng, 3072, 512, 520, 64, False) + (64, 0.0),
             problem(rng, 3200, 4096, 2304, 128, True) + (128, 0.5)]  # 2048-row panels + a ragged one
    staged = [(dev(x), dev(q), dev(s), dev(z) if z is not None else None, out0, bs, beta)
              for x, q, s, z, out0, bs, beta in cases]
    want = []
    for xd, qd, sd, zd, out0, bs, beta in staged:
        o = dev(out0.copy())
        kernels.matmul_nt_fp16u8_ws(o, xd, qd, sd, bs, ws, beta, zd)
        assert kernels.last_kernel() == Kernel.F16Tc
        want.append(o.cpu().numpy())
    outs = [dev(c[4].copy()) for c in staged]
    # a first call so that the one-time look-up of the array (and lazy module loading) is done
    kernels.matmul_nt_fp16u8_noalloc(dev(staged[0][4].copy()), *staged[0][:3], staged[0][5],
                                     staged[0][6], staged[0][3])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for o, (xd, qd, sd, zd, _, bs, beta) in zip(outs, staged):
        kernels.matmul_nt_fp16u8_noalloc(o, xd, qd, sd, bs, beta, zd)
    kernels.device_status()
    assert torch.cuda.mem_get_info()[0] == free_before, "the calls changed the free device memory"
    assert kernels.last_kernel() == Kernel.F16Tc
    for o, w, (x, q, s, z, out0, bs, beta) in zip(outs, want, cases):
        got = o.cpu().numpy()
        assert np.array_equal(got.view(np.uint16), w.view(np.uint16))
        rows = slice(0, 96)  # the oracle on a slice of the rows keeps the test short
        ref = oracle.matmul_nt_fp16u8(x[rows], q, s, bs, beta, out0[rows], z)
        assert oracle.max_rel_err(got[rows], ref) <= 1e-2


def test_rows_too_long_for_the_array_are_refused(kernels):
    """More columns than 128 weight rows of the array can hold: a clear error and no launch."""
    p, n, bs = 65536 + 128, 8, 128
    x = torch.zeros((1, p), dtype=torch.float16, device="cuda")
    q = torch.zeros((n, p), dtype=torch.uint8, device="cuda")
    s = torch.ones((n, p // bs), dtype=torch.float16, device="cuda")
    o = torch.full((1, n), 3.0, dtype=torch.float16, device="cuda")
    launches = kernels.launch_count()
    with pytest.raises(AdrError) as e:
        kernels.matmul_nt_fp16u8_noalloc(o, x, q, s, bs)
    assert e.value.code == ERR_TOO_LARGE and "built-in scratch" in str(e.value)
    assert kernels.launch_count() == launches
    assert torch.all(o == 3.0)
