"""GPU parity tests: every call goes through the C ABI (libadrastea_b200.so)
and is compared with the CPU oracle, with the golden vectors and, when the
reference cubins travelled along, with the reference's own kernels run live.

Tolerances (the stated goal of this path): max relative error <= 1e-2 against the
fp32-accumulate ("ideal") oracle; u8 dequantisation bit-exact; the CUDA-core
fp16 kernel bit-exact against the reference kernels (it keeps their
arithmetic), up to 2 fp16 ulps where tanhf/expf sit in the epilogue.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from adrastea_b200 import (AdrError, Kernel, MatmulLoad, MatmulLoadOp, MatmulMask, MatmulOptions,
                           MatmulStore, MatmulTracer, TensorLayout, TensorView)
from oracle import oracle, refcubin

pytestmark = pytest.mark.gpu
TOL = 1e-2
GOLD = Path(__file__).resolve().parent / "golden"
CANARY = 64  # guard elements either side of every output buffer


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def options_of(c, bias_view):
    o = MatmulOptions.new()
    if c.load == cases.LD_SCALE:
        o = o.load(MatmulLoad.Scale(c.scale))
    st = {cases.ST_IDENTITY: MatmulStore.Identity(), cases.ST_ADD: MatmulStore.Add(),
          cases.ST_SCALE: MatmulStore.Scale(c.scale)}.get(c.store)
    if st is None:
        st = {cases.ST_BETA_BIAS: lambda: MatmulStore.BetaBias(c.beta, bias_view),
              cases.ST_BETA_GELU_BIAS: lambda: MatmulStore.BetaGeluBias(c.beta, bias_view),
              cases.ST_QUICK_GELU: lambda: MatmulStore.QuickGeluBias(bias_view)}[c.store]()
    o = o.store(st)
    if c.mask == cases.MK_CAUSAL:
        o = o.mask(MatmulMask.Causal)
    return o


def view_of(t, c, strides, dims3):
    if c.batches > 1:
        lay = TensorLayout.new(dims3, (strides[2] or 1, strides[1], strides[0]))
        if strides[2] == 0:  # broadcast operand: pass the 2-D view (z-stride becomes 0)
            lay = TensorLayout.new(dims3[1:], (strides[1], strides[0]))
    else:
        lay = TensorLayout.new(dims3[1:], (strides[1], strides[0]))
    return TensorView(t, lay, 0)


def run_case(kernels, c, slow):
    out0, lhs, rhs, bias = c.inputs()
    guard = np.full(CANARY, 123.0, np.float16)
    o = dev(np.concatenate([guard, out0, guard]))
    l, r, b = dev(lhs), dev(rhs), dev(bias)
    ov = view_of(o, c, c.out_strides, (c.batches, c.m, c.n))
    ov.offset = CANARY
    lv = view_of(l, c, c.lhs_strides, (c.batches, c.m, c.k))
    rv = view_of(r, c, c.rhs_strides, (c.batches, c.k, c.n))
    opts = options_of(c, TensorView.of(b))
    (kernels.matmul_f16_slow if slow else kernels.matmul_f16)(ov, lv, rv, opts)
    torch.cuda.synchronize()
    res = o.cpu().numpy()
    assert np.all(res[:CANARY] == guard) and np.all(res[-CANARY:] == guard), "wrote outside the output"
    return res[CANARY:-CANARY]


def oracle_out(c, ideal):
    out, lhs, rhs, bias = c.inputs()
    assert oracle.matmul_f16(out, lhs, rhs, c.batches, c.m, c.k, c.n, c.strides9(),
                             bias if c.uses_bias() else None, c.beta, c.scale, c.store, c.load,
                             c.mask, ideal=ideal) == 0
    return out


def ulp_diff(a, b):
    return a.view(np.uint16).astype(np.int32) - b.view(np.uint16).astype(np.int32)


@pytest.mark.parametrize("c", cases.matmul_cases(), ids=lambda c: c.name)
def test_matmul_f16_slow_is_bit_faithful(kernels, c):
    """The CUDA-core kernel keeps the reference's arithmetic: equal bits with the
    faithful oracle, with the golden vectors and with the live reference kernel."""
    got = run_case(kernels, c, slow=True)
    assert kernels.last_kernel() == Kernel.F16Simt
    want = oracle_out(c, ideal=False)
    d = ulp_diff(got, want)
    if c.exact_vs_reference:
        assert not d.any()
    else:
        assert np.abs(d).max() <= 2
    again = run_case(kernels, c, slow=True)
    assert np.array_equal(got.view(np.uint16), again.view(np.uint16)), "not deterministic"
    gold = GOLD / "reference_matmul_f16.npz"
    if gold.exists():
        ref = np.load(gold)[f"{c.name}/matmul_f16_fast"]
        assert np.abs(ulp_diff(got, ref)).max() <= (0 if c.exact_vs_reference else 1)


@pytest.mark.parametrize("c", cases.matmul_cases(), ids=lambda c: c.name)
def test_matmul_f16_against_ideal_oracle(kernels, c):
    """The dispatched kernel (tensor cores where the view allows) within 1e-2."""
    got = run_case(kernels, c, slow=False)
    want = oracle_out(c, ideal=True)
    err = oracle.max_rel_err(got, want)
    assert err <= TOL, (err, kernels.last_kernel())
    again = run_case(kernels, c, slow=False)
    assert np.array_equal(got.view(np.uint16), again.view(np.uint16)), "not deterministic"


@pytest.mark.parametrize("c", cases.matmul_cases(), ids=lambda c: c.name)
def test_tc_gather_kernel_takes_every_view(kernels, c):
    """The tensor-core kernel behind gathering loader warps accepts any strides and alignment:
    every case of the fp16 suite, forced through it, within 1e-2 of the ideal oracle."""
    try:
        kernels.force_kernel(Kernel.F16TcGather)
        got = run_case(kernels, c, slow=False)
        kernels.device_status()
        assert kernels.last_kernel() == Kernel.F16TcGather
        want = oracle_out(c, ideal=True)
        err = oracle.max_rel_err(got, want)
        assert err <= TOL, err
        again = run_case(kernels, c, slow=False)
        assert np.array_equal(got.view(np.uint16), again.view(np.uint16)), "not deterministic"
    finally:
        kernels.force_kernel(Kernel.Auto)


def test_unaligned_score_pitch_stays_on_tensor_cores(kernels):
    """The reference's own attention views at 257 tokens (clip.rs:374-388): scores and
    probabilities [H, 257, 257] contiguous, i.e. a 514-byte row pitch the copy engine cannot
    describe.  Both products are dispatched to the gathering tensor-core kernel, not to CUDA cores."""
    rng = np.random.default_rng(99)
    H, S, hd = 4, 257, 64
    D = H * hd
    q = (rng.standard_normal((S, D)) * 0.5).astype(np.float16)
    k = (rng.standard_normal((S, D)) * 0.5).astype(np.float16)
    v = (rng.standard_normal((S, D)) * 0.5).astype(np.float16)
    qd, kd, vd = dev(q), dev(k), dev(v)
    heads = TensorLayout.new((H, S, hd), (hd, D, 1))
    scores = torch.zeros((H, S, S), dtype=torch.float16, device="cuda")
    sv = TensorView.of(scores)
    kernels.matmul_f16(sv, TensorView(qd, heads), TensorView(kd, heads).permute([0, 2, 1]),
                       MatmulOptions.new().store(MatmulStore.Scale(0.125)))
    want_s = np.zeros(H * S * S, np.float16)
    oracle.matmul_f16(want_s, q.reshape(-1), k.reshape(-1), H, S, hd, S,
                      (1, S, S * S, 1, D, hd, D, 1, hd), scale=0.125, store=cases.ST_SCALE, ideal=True)
    assert oracle.max_rel_err(scores.cpu().numpy().reshape(-1), want_s) <= TOL
    kernels.softmax_rows_inplace(sv, 1.0)
    out = torch.zeros((S, D), dtype=torch.float16, device="cuda")
    kernels.matmul_f16(TensorView(out, heads), sv, TensorView(vd, heads))
    kernels.device_status()
    assert kernels.last_kernel() == Kernel.F16TcGather
    probs = scores.cpu().numpy()
    want_o = np.zeros(S * D, np.float16)
    oracle.matmul_f16(want_o, probs.reshape(-1), v.reshape(-1), H, S, S, hd,
                      (1, D, hd, 1, S, S * S, 1, D, hd), ideal=True)
    assert oracle.max_rel_err(out.cpu().numpy().reshape(-1), want_o) <= TOL


@pytest.mark.parametrize("c", cases.matmul_cases(), ids=lambda c: c.name)
def test_live_reference_kernels_agree_with_oracle(c):
    """Pins the oracle on this very GPU: matmul_f16 / matmul_f16_fast from the
    reference tree against orc_matmul_f16_ref."""
    if not refcubin.available():
        pytest.skip("reference cubins not present")
    want = oracle_out(c, ideal=False)
    for kern in ("matmul_f16", "matmul_f16_fast"):
        out0, lhs, rhs, bias = c.inputs()
        o, l, r, b = dev(out0), dev(lhs), dev(rhs), dev(bias)
        refcubin.matmul_f16(kern, o.data_ptr(), l.data_ptr(), r.data_ptr(), c.batches, c.m, c.k,
                            c.n, c.strides9(), b.data_ptr() if c.uses_bias() else None, c.beta,
                            c.scale, c.store, c.load, c.mask)
        torch.cuda.synchronize()
        d = ulp_diff(o.cpu().numpy(), want)
        assert np.abs(d).max() <= (0 if c.exact_vs_reference else 2), kern


def ksplit_takes(m, p, bs):
    """Shapes the cluster k-split kernel takes, and whether the dispatcher picks it."""
    ok = p % 128 == 0 and p >= 2048 and bs in (64, 128) and (p // bs) % 2 == 0
    if p <= 8192:
        return ok, ok and (m >= 5 or (m >= 4 and p == 8192))
    return ok, ok and (m >= 7 or (m >= 4 and p >= 16384))


def u8_kernels_for(c):
    ks = [Kernel.U8Simt]
    if c.m <= 4:
        ks.append(Kernel.U8Gemv)
    if c.p % 64 == 0:
        ks.append(Kernel.U8Mma)
        if c.m <= 16 and c.p % 128 == 0:
            ks.append(Kernel.U8Stream)
            if c.block_size in (64, 128) and c.n >= 16 and (c.p // c.block_size) % 2 == 0:
                ks.append(Kernel.U8Ring)
                if ksplit_takes(c.m, c.p, c.block_size)[0]:
                    ks.append(Kernel.U8KSplit)
    if c.p % 16 == 0:
        ks.append(Kernel.U8Tc)
    if c.p % 64 == 0 and c.block_size % 64 == 0:
        ks.append(Kernel.U8Ts)
    return ks


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("rows", [16, 32, 64])
def test_u8_stream_every_plan(kernels, split, rows):
    """Every cluster size (k-split) and rows-per-CTA choice of the streaming
    kernel gives the same answer within tolerance, deterministically, for
    ragged n, p not divisible by the split, both token blocks and zero points."""
    rng = np.random.default_rng(split * 10 + rows)
    try:
        kernels.force_kernel(Kernel.U8Stream)
        kernels.set_tunable("u8_split", split)
        kernels.set_tunable("u8_rows", rows)
        for m, p, n, bs, zp in ((1, 1024, 200, 128, False), (7, 1408, 333, 64, False),
                                (16, 1024, 128, 128, True), (9, 1152, 97, 32, False)):
            x = rng.standard_normal((m, p)).astype(np.float16)
            q = rng.integers(0, 256, (n, p), dtype=np.uint8)
            s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
            z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
            out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
            want = oracle.matmul_nt_fp16u8(x, q, s, bs, 0.5, out0, z)
            res = []
            for _ in range(2):
                o = dev(out0.copy())
                kernels.matmul_nt_fp16u8(o, dev(x), dev(q), dev(s), bs, 0.5, dev(z) if zp else None)
                kernels.device_status()
                res.append(o.cpu().numpy())
            assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))
            assert oracle.max_rel_err(res[0], want) <= TOL, (m, p, n)
    finally:
        kernels.set_tunable("u8_split", 0)
        kernels.set_tunable("u8_rows", 0)
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("pdl", [0, 1])
def test_u8_ring_kernel(kernels, pdl):
    """The persistent ring kernel: ragged n (partial last unit), k with a partial last stage,
    more units than SMs, both block sizes, both token blocks, zero points, beta; twice for
    determinism; then the dispatcher's choice and the fp16-rounded mode of the streaming
    kernel ("u8_exact") on the same inputs."""
    rng = np.random.default_rng(77 + pdl)
    try:
        kernels.set_tunable("pdl", pdl)
        for m, p, n, bs, zp in ((1, 1024, 200, 128, False), (7, 1280, 333, 64, False),
                                (16, 2048, 128, 128, True), (9, 1536, 97, 64, True),
                                (4, 4096, 3000, 128, False), (1, 11008, 64, 128, False),
                                # activations too large to stay resident: streamed through the ring
                                (16, 8192, 512, 64, False), (8, 11008, 256, 128, False),
                                (16, 11008, 272, 128, True), (12, 4224 + 4096, 300, 64, False)):
            x = rng.standard_normal((m, p)).astype(np.float16)
            q = rng.integers(0, 256, (n, p), dtype=np.uint8)
            s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
            z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
            out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
            want = oracle.matmul_nt_fp16u8(x, q, s, bs, 0.5, out0, z)
            xd, qd, sd, zd = dev(x), dev(q), dev(s), dev(z) if zp else None
            kernels.force_kernel(Kernel.U8Ring)
            res = []
            for _ in range(2):
                o = dev(out0.copy())
                kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs, 0.5, zd)
                kernels.device_status()
                res.append(o.cpu().numpy())
            assert kernels.last_kernel() == Kernel.U8Ring
            assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))
            assert oracle.max_rel_err(res[0], want) <= 2e-3, (m, p, n, oracle.max_rel_err(res[0], want))
            kernels.force_kernel(Kernel.Auto)
            o = dev(out0.copy())
            kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs, 0.5, zd)
            if ksplit_takes(m, p, bs)[1]:
                assert kernels.last_kernel() == Kernel.U8KSplit  # the cluster split takes these
                assert oracle.max_rel_err(o.cpu().numpy(), want) <= 2e-3
            else:
                assert kernels.last_kernel() == Kernel.U8Ring
                assert np.array_equal(o.cpu().numpy().view(np.uint16), res[0].view(np.uint16))
            kernels.set_tunable("u8_exact", 1)
            o = dev(out0.copy())
            kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs, 0.5, zd)
            assert kernels.last_kernel() == Kernel.U8Stream
            assert oracle.max_rel_err(o.cpu().numpy(), want) <= 2e-3
            kernels.set_tunable("u8_exact", 0)
            kernels.device_status()
    finally:
        kernels.set_tunable("pdl", 0)
        kernels.set_tunable("u8_exact", 0)
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("pdl", [0, 1])
def test_u8_cluster_ksplit_kernel(kernels, pdl):
    """The cluster k-split kernel: every cluster size (k = 2048 .. 8192 and beyond), ragged n, fewer
    units than clusters and many more, both block sizes, both token blocks, zero points, beta,
    several launches back to back (inbox slots and credits in rotation); thrice for determinism."""
    rng = np.random.default_rng(177 + pdl)
    try:
        kernels.set_tunable("pdl", pdl)
        kernels.force_kernel(Kernel.U8KSplit)
        for m, p, n, bs, zp in ((1, 4096, 200, 128, False), (7, 2048, 333, 64, False),
                                (16, 4096, 4096, 128, True), (9, 8192, 97, 64, True),
                                (4, 4096, 11008, 128, False), (16, 8192, 1000, 128, False),
                                (3, 3072, 16, 64, False), (16, 5120, 2500, 64, True),
                                (12, 7168, 640, 128, False),
                                # k that ends inside a CTA's slice; k beyond one cluster's reach
                                # (two and three launches over consecutive k ranges)
                                (6, 2304, 100, 128, False), (16, 11008, 272, 128, True),
                                (8, 11008, 256, 128, False), (12, 8320, 300, 64, False),
                                (5, 22016, 64, 64, False)):
            x = rng.standard_normal((m, p)).astype(np.float16)
            q = rng.integers(0, 256, (n, p), dtype=np.uint8)
            s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
            z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
            out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
            want = oracle.matmul_nt_fp16u8(x, q, s, bs, 0.5, out0, z)
            xd, qd, sd, zd = dev(x), dev(q), dev(s), dev(z) if zp else None
            res = []
            for _ in range(3):
                o = dev(out0.copy())
                kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs, 0.5, zd)
                kernels.device_status()
                res.append(o.cpu().numpy())
            assert kernels.last_kernel() == Kernel.U8KSplit
            assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))
            assert np.array_equal(res[0].view(np.uint16), res[2].view(np.uint16))
            assert oracle.max_rel_err(res[0], want) <= 2e-3, (m, p, n, oracle.max_rel_err(res[0], want))
        # shapes it does not take are refused, not mangled
        x = torch.zeros((1, 1024), dtype=torch.float16, device="cuda")
        q = torch.zeros((64, 1024), dtype=torch.uint8, device="cuda")
        s = torch.ones((64, 8), dtype=torch.float16, device="cuda")
        o = torch.zeros((1, 64), dtype=torch.float16, device="cuda")
        with pytest.raises(AdrError):
            kernels.matmul_nt_fp16u8(o, x, q, s, 128)
    finally:
        kernels.set_tunable("pdl", 0)
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("c", cases.u8_cases(), ids=lambda c: c.name)
def test_u8_matmul_all_kernels(kernels, c):
    out0, lhs, q, scales, zeros = c.inputs()
    want = oracle.matmul_nt_fp16u8(lhs, q, scales, c.block_size, c.beta, out0, zeros)
    l, qq, s = dev(lhs), dev(q), dev(scales)
    z = dev(zeros) if zeros is not None else None
    try:
        for k in u8_kernels_for(c) + [Kernel.Auto]:
            kernels.force_kernel(k)
            res = []
            for _ in range(2):
                o = dev(out0.copy())
                kernels.matmul_nt_fp16u8(o, l, qq, s, c.block_size, c.beta, z)
                torch.cuda.synchronize()
                res.append(o.cpu().numpy())
            assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16)), f"{k!r} not deterministic"
            err = oracle.max_rel_err(res[0], want)
            assert err <= TOL, (k, err)
    finally:
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("c", cases.u8_cases(), ids=lambda c: c.name)
def test_u8_dequantisation_is_bit_exact(kernels, c):
    """The in-register dequantisation every u8 kernel uses, dumped through
    adr_dequantize_absmax_uint8, equals fp16((q - zero) * s) bit for bit."""
    _, _, q, scales, zeros = c.inputs()
    want = oracle.dequantize(q, scales, c.block_size, zeros)
    w = torch.empty((c.n, c.p), dtype=torch.float16, device="cuda")
    kernels.dequantize_absmax_uint8(w, dev(scales), dev(q), dev(zeros) if zeros is not None else None)
    torch.cuda.synchronize()
    assert np.array_equal(w.cpu().numpy().view(np.uint16), want.view(np.uint16))
    if zeros is None and refcubin.available():
        r = torch.empty_like(w)
        sd, qd = dev(scales), dev(q)  # keep the device buffers alive across the launch
        refcubin.dequantize_absmax_uint8(r.data_ptr(), sd.data_ptr(), qd.data_ptr(), c.n, c.p, c.block_size)
        torch.cuda.synchronize()
        assert torch.equal(w.view(torch.int16), r.view(torch.int16))


def test_dequantisation_every_code_and_many_scales(kernels):
    """All 256 codes against a sweep of scale bit patterns, including subnormal,
    tiny, large and negative scales (fast and fp32 paths of the dequantiser)."""
    sb = np.concatenate([np.arange(0, 0x0C00, 7), np.arange(0x0C00, 0x7C00, 97), [0x7BFF, 0x8001, 0x9234, 0xB000]]).astype(np.uint16)
    n = sb.size
    q = np.tile(np.arange(256, dtype=np.uint8), (n, 1))
    scales = np.repeat(sb.view(np.float16)[:, None], 256 // 16, axis=1)
    want = oracle.dequantize(q, scales, 16)
    w = torch.empty((n, 256), dtype=torch.float16, device="cuda")
    kernels.dequantize_absmax_uint8(w, dev(scales), dev(q))
    torch.cuda.synchronize()
    assert np.array_equal(w.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_quantizer_matches_oracle_and_reference(kernels):
    rng = np.random.default_rng(11)
    for rows, k, bs in ((24, 512, 128), (8, 256, 32), (5, 512, 256)):
        x = (rng.standard_normal((rows, k)) * rng.uniform(0.01, 2.0, (rows, 1))).astype(np.float16)
        x[1, :bs] = 0
        q = torch.zeros((rows, k), dtype=torch.uint8, device="cuda")
        s = torch.zeros((rows, k // bs), dtype=torch.float16, device="cuda")
        kernels.quantize_absmax_uint8(q, s, dev(x))
        torch.cuda.synchronize()
        wq, ws = oracle.quantize(x, bs)
        assert np.array_equal(s.cpu().numpy().view(np.uint16), ws.view(np.uint16))
        assert np.array_equal(q.cpu().numpy(), wq)
        if refcubin.available():
            rq, rs = torch.zeros_like(q), torch.zeros_like(s)
            xd = dev(x)
            refcubin.quantize_absmax_uint8(rq.data_ptr(), rs.data_ptr(), xd.data_ptr(), rows, k, bs)
            torch.cuda.synchronize()
            assert torch.equal(rq, q) and torch.equal(rs.view(torch.int16), s.view(torch.int16))


def test_matmul_nt_f16(kernels):
    rng = np.random.default_rng(12)
    for m, p, n, beta in ((128, 192, 128, 0.0), (256, 128, 64, 0.5), (16, 256, 128, 1.0), (7, 40, 13, 0.25)):
        lhs = (rng.standard_normal((m, p)) * 0.3).astype(np.float16)
        rhs = (rng.standard_normal((n, p)) * 0.3).astype(np.float16)
        out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
        o = dev(out0.copy())
        kernels.matmul_nt_f16(o, dev(lhs), dev(rhs), beta)
        torch.cuda.synchronize()
        want = oracle.matmul_nt_f16(lhs, rhs, beta, out0)
        assert oracle.max_rel_err(o.cpu().numpy(), want) <= TOL


def test_error_codes_instead_of_traps(kernels):
    t = torch.zeros(16, 16, dtype=torch.float16, device="cuda")
    v = TensorView.of(t)
    with pytest.raises(AdrError) as e:  # GELU_BIAS has no device code in the reference (it traps)
        kernels.matmul_f16(v, v, v, MatmulOptions.new().store(MatmulStore.GeluBias(TensorView.of(t[0]))))
    assert e.value.code == 3
    with pytest.raises(AssertionError):  # shape mismatch: the reference panics
        kernels.matmul_f16(v, v, TensorView.of(t[:8]))
    q = torch.zeros(16, 48, dtype=torch.uint8, device="cuda")
    s = torch.zeros(16, 2, dtype=torch.float16, device="cuda")
    x = torch.zeros(1, 48, dtype=torch.float16, device="cuda")
    o = torch.zeros(1, 16, dtype=torch.float16, device="cuda")
    with pytest.raises(AdrError) as e:  # block size 24 is not a multiple of 16
        kernels.matmul_nt_fp16u8(o, x, q, s, 24)
    assert e.value.code == 2
    # the context is still usable afterwards
    kernels.matmul_f16(v, v, v)
    torch.cuda.synchronize()


def test_tracer_records_distinct_layouts(kernels):
    tr = MatmulTracer(kernels)
    a = TensorView.of(torch.zeros(8, 32, dtype=torch.float16, device="cuda"))
    w = TensorView.of(torch.zeros(16, 32, dtype=torch.float16, device="cuda"))
    o = TensorView.of(torch.zeros(8, 16, dtype=torch.float16, device="cuda"))
    kernels.trace_enable(True)
    for _ in range(3):
        tr.matmul_f16(o, a, w.permute([1, 0]))
    assert len(tr.shapes()) == 1
    dump = kernels.trace_dump()
    assert any(d["m"] == 8 and d["k"] == 32 and d["n"] == 16 and d["rhs_strides"] == [32, 1, 0] for d in dump)
    kernels.trace_enable(False)


# ------------------------------------------------------------ full workload sizes
def test_config1_full_size(kernels):
    """C[64,4096] = A[64,4096] . W[4096,4096], N(0, 0.02^2), both W layouts."""
    rng = np.random.default_rng(100)
    m = 64
    k = n = 4096
    a = (rng.standard_normal((m, k)) * 0.02).astype(np.float16)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float16)  # W[K,N] row-major ("rrr")
    want = np.zeros(m * n, np.float16)
    oracle.matmul_f16(want, a.reshape(-1), w.reshape(-1), 1, m, k, n, (1, n, 0, 1, k, 0, 1, n, 0), ideal=True)
    ad, wd = dev(a), dev(w)
    o = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    kernels.matmul_f16(TensorView.of(o), TensorView.of(ad), TensorView.of(wd))
    torch.cuda.synchronize()
    assert oracle.max_rel_err(o.cpu().numpy().reshape(-1), want) <= TOL
    wt = dev(np.ascontiguousarray(w.T))  # the reference's storage: [N,K], passed permuted ("rrc")
    o2 = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    kernels.matmul_f16(TensorView.of(o2), TensorView.of(ad), TensorView.of(wt).permute([1, 0]))
    torch.cuda.synchronize()
    assert oracle.max_rel_err(o2.cpu().numpy().reshape(-1), want) <= TOL


@pytest.mark.parametrize("m", [1, 4, 16])
@pytest.mark.parametrize("n", [4096, 11008])
def test_config2_full_size(kernels, m, n):
    """u8 decode shapes at full size: every kernel against the oracle on a
    random subset of output columns (a column depends on one weight row only),
    and the kernels against each other on all columns."""
    p, bs = 4096, 128
    rng = np.random.default_rng(200 + m + n)
    x = rng.standard_normal((m, p)).astype(np.float16)
    q = rng.integers(0, 256, (n, p), dtype=np.uint8)
    s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
    z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16)
    cols = np.sort(rng.choice(n, 96, replace=False))
    xd, qd, sd, zd = dev(x), dev(q), dev(s), dev(z)
    try:
        for zeros_np, zeros_d in ((None, None), (z, zd)):
            want = oracle.matmul_nt_fp16u8(x, q[cols], s[cols], bs, zeros=None if zeros_np is None else zeros_np[cols])
            outs = {}
            for kern in [Kernel.U8Mma, Kernel.U8Stream, Kernel.U8Ring] + ([Kernel.U8Gemv] if m <= 4 else []) + [Kernel.Auto]:
                kernels.force_kernel(kern)
                o = torch.zeros(m, n, dtype=torch.float16, device="cuda")
                kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs, 0.0, zeros_d)
                torch.cuda.synchronize()
                outs[kern] = o.cpu().numpy()
                assert oracle.max_rel_err(outs[kern][:, cols], want) <= TOL, kern
            base = outs[Kernel.U8Mma]
            for kern, o in outs.items():
                assert oracle.max_rel_err(o, base) <= TOL, kern
    finally:
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("split", [2, 4, 8])
@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_tc_gemm_every_tile_and_split(kernels, bn, split):
    """Every N-tile and cluster k-split of the tensor-core kernel against the ideal
    oracle, with ragged m/n/k, a fused op that reads the output, and a batch."""
    rng = np.random.default_rng(bn + split)
    try:
        kernels.force_kernel(Kernel.F16Tc)
        kernels.set_tunable("tc_bn", bn)
        kernels.set_tunable("tc_split", split)
        for (b, m, k, n, store, beta) in ((1, 70, 1096, 300, cases.ST_ADD, 0.0), (3, 130, 1024, 72, cases.ST_BETA_BIAS, 0.5)):
            lhs = (rng.standard_normal(b * m * k) * 0.1).astype(np.float16)
            rhs = (rng.standard_normal(b * n * k) * 0.1).astype(np.float16)
            out0 = (rng.standard_normal(b * m * n) * 0.5).astype(np.float16)
            bias = (rng.standard_normal(n) * 0.5).astype(np.float16)
            strides = (1, n, m * n, 1, k, m * k, k, 1, n * k)
            want = out0.copy()
            assert oracle.matmul_f16(want, lhs, rhs, b, m, k, n, strides, bias, beta, 1.0, store, 0, 0, ideal=True) == 0
            o, l, r, bd = dev(out0.copy()), dev(lhs), dev(rhs), dev(bias)
            shp = (lambda *d: d if b > 1 else d[1:])
            ov = TensorView(o, TensorLayout.row_major(shp(b, m, n)))
            lv = TensorView(l, TensorLayout.row_major(shp(b, m, k)))
            rv = TensorView(r, TensorLayout.row_major(shp(b, n, k))).permute([0, 2, 1] if b > 1 else [1, 0])
            st = MatmulStore.Add() if store == cases.ST_ADD else MatmulStore.BetaBias(beta, TensorView.of(bd))
            kernels.matmul_f16(ov, lv, rv, MatmulOptions.new().store(st))
            kernels.device_status()
            assert kernels.last_kernel() == Kernel.F16Tc
            assert oracle.max_rel_err(o.cpu().numpy(), want) <= TOL, (b, m, k, n)
    finally:
        kernels.set_tunable("tc_bn", 0)
        kernels.set_tunable("tc_split", 0)
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("split", [0, 2])
@pytest.mark.parametrize("bn", [64, 128, 256])
def test_tc_gemm_n_contiguous_rhs(kernels, bn, split):
    """rhs stored [K, N] row-major ("rrr", the fp16 GEMM workload as worded) and the
    probabilities . values product with a 16-byte-aligned score pitch (k = 257)."""
    rng = np.random.default_rng(7 * bn + split)
    try:
        kernels.force_kernel(Kernel.F16Tc)
        kernels.set_tunable("tc_bn", bn)
        kernels.set_tunable("tc_split", split)
        # plain NN with ragged m, k, n
        m, k, n = 200, 328, 392
        a = (rng.standard_normal((m, k)) * 0.1).astype(np.float16)
        w = (rng.standard_normal((k, n)) * 0.1).astype(np.float16)
        want = np.zeros(m * n, np.float16)
        oracle.matmul_f16(want, a.reshape(-1), w.reshape(-1), 1, m, k, n, (1, n, 0, 1, k, 0, 1, n, 0), ideal=True)
        o = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        kernels.matmul_f16(TensorView.of(o), TensorView.of(dev(a)), TensorView.of(dev(w)))
        kernels.device_status()
        assert kernels.last_kernel() == Kernel.F16Tc
        assert oracle.max_rel_err(o.cpu().numpy().reshape(-1), want) <= TOL
        # P.V: lhs [H, S, S] with row pitch 264 (S = 257), rhs a [S, H*hd] buffer viewed [H, S, hd],
        # out a strided view of [S, H, hd] (llama.rs:552-554, clip.rs:378-388)
        H, S, hd, pitch = 3, 257, 64, 264
        D = H * hd
        pbuf = np.zeros(H * S * pitch, np.float16)
        pv = pbuf.reshape(H, S, pitch)
        pv[:, :, :S] = rng.uniform(0, 2.0 / S, (H, S, S)).astype(np.float16)
        pv[:, :, S:] = np.float16(7.0)  # padding columns must never be read
        v = (rng.standard_normal(S * D) * 0.5).astype(np.float16)
        want = np.zeros(S * D, np.float16)
        strides = (1, D, hd, 1, pitch, S * pitch, 1, D, hd)
        oracle.matmul_f16(want, pbuf, v, H, S, S, hd, strides, ideal=True)
        o, pd, vd = dev(np.zeros(S * D, np.float16)), dev(pbuf), dev(v)
        ov = TensorView(o, TensorLayout.new((H, S, hd), (hd, D, 1)))
        lv = TensorView(pd, TensorLayout.new((H, S, S), (S * pitch, pitch, 1)))
        rv = TensorView(vd, TensorLayout.new((H, S, hd), (hd, D, 1)))
        kernels.matmul_f16(ov, lv, rv)
        kernels.device_status()
        assert kernels.last_kernel() == Kernel.F16Tc
        assert oracle.max_rel_err(o.cpu().numpy(), want) <= TOL
    finally:
        kernels.set_tunable("tc_bn", 0)
        kernels.set_tunable("tc_split", 0)
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("zp", [False, True])
def test_u8_prefill_tensor_core_kernel(kernels, zp):
    """m > 32 takes a dequantising tensor-core kernel: the one that dequantises into tensor
    memory when p and the block size are multiples of 64, else the one that stages the
    dequantised operand in shared memory; both forced in turn on the shapes they take.  Ragged
    m/n, several k-steps and tiles per CTA, both tile widths, beta, zero points; against the
    ideal oracle (fp16-rounded weights, exact products)."""
    rng = np.random.default_rng(31 + zp)
    try:
        for m, p, n, bs, beta in ((130, 1088, 300, 64, 0.5), (512, 512, 1024, 128, 0.0),
                                  (40, 256, 192, 128, 1.0), (300, 4096, 260, 128, 0.5),
                                  (700, 832, 520, 64, 0.0), (33, 1040, 100, 16, 0.5)):
            x = rng.standard_normal((m, p)).astype(np.float16)
            q = rng.integers(0, 256, (n, p), dtype=np.uint8)
            s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
            z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
            out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
            want = oracle.matmul_nt_fp16u8(x, q, s, bs, beta, out0, z)
            takes_ts = p % 64 == 0 and bs % 64 == 0
            for kern in ([Kernel.Auto, Kernel.U8Ts, Kernel.U8Tc] if takes_ts else [Kernel.Auto, Kernel.U8Tc]):
                kernels.force_kernel(kern)
                res = []
                for _ in range(2):
                    o = dev(out0.copy())
                    kernels.matmul_nt_fp16u8(o, dev(x), dev(q), dev(s), bs, beta, dev(z) if zp else None)
                    kernels.device_status()
                    res.append(o.cpu().numpy())
                expect = kern if kern != Kernel.Auto else (Kernel.U8Ts if takes_ts else Kernel.U8Tc)
                assert kernels.last_kernel() == expect
                assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))
                assert oracle.max_rel_err(res[0], want) <= TOL, (kern, m, p, n)
    finally:
        kernels.force_kernel(Kernel.Auto)


@pytest.mark.parametrize("zp", [False, True])
def test_u8_prefill_cluster_split(kernels, zp):
    """With too few tiles for the GPU the tensor-memory prefill kernel runs a tile on a cluster
    of two or four CTAs, each with a share of the k-steps, and sums the partial accumulators
    through distributed shared memory before the one rounding.  Forced here to 1, 2 and 4 on
    ragged m and n (n not a multiple of 4 takes the scalar stores), both tile widths, beta and
    zero points; each against the ideal oracle, repeatable bit for bit."""
    rng = np.random.default_rng(77 + zp)
    try:
        kernels.force_kernel(Kernel.U8Ts)
        for m, p, n, bs, beta in ((64, 2048, 256, 128, 0.0), (200, 4096, 301, 64, 0.5),
                                  (512, 2112, 384, 64, 1.0), (33, 1024, 130, 128, 0.5)):
            x = rng.standard_normal((m, p)).astype(np.float16)
            q = rng.integers(0, 256, (n, p), dtype=np.uint8)
            s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
            z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
            out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
            want = oracle.matmul_nt_fp16u8(x, q, s, bs, beta, out0, z)
            for bt in (0, 128, 256):
                for split in (1, 2, 3, 4):
                    if (p // 64) // split < 8:
                        continue
                    kernels.set_tunable("ts_bt", bt)
                    kernels.set_tunable("ts_split", split)
                    res = []
                    for _ in range(2):
                        o = dev(out0.copy())
                        kernels.matmul_nt_fp16u8(o, dev(x), dev(q), dev(s), bs, beta, dev(z) if zp else None)
                        kernels.device_status()
                        res.append(o.cpu().numpy())
                    assert kernels.last_kernel() == Kernel.U8Ts
                    assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))
                    assert oracle.max_rel_err(res[0], want) <= TOL, (m, p, n, bt, split)
        # more than one wave of tiles with a small last wave (150 tiles on 148 SMs): the full
        # waves run as the persistent kernel, the last two tiles on clusters
        kernels.set_tunable("ts_bt", 0)
        kernels.set_tunable("ts_split", 0)
        m, p, n, bs, beta = 768, 1024, 6400, 128, 0.5
        x = rng.standard_normal((m, p)).astype(np.float16)
        q = rng.integers(0, 256, (n, p), dtype=np.uint8)
        s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
        z = rng.uniform(120, 136, (n, p // bs)).astype(np.float16) if zp else None
        out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
        want = oracle.matmul_nt_fp16u8(x, q, s, bs, beta, out0, z)
        o = dev(out0.copy())
        kernels.matmul_nt_fp16u8(o, dev(x), dev(q), dev(s), bs, beta, dev(z) if zp else None)
        kernels.device_status()
        assert oracle.max_rel_err(o.cpu().numpy(), want) <= TOL
    finally:
        kernels.set_tunable("ts_bt", 0)
        kernels.set_tunable("ts_split", 0)
        kernels.force_kernel(Kernel.Auto)


def fp16_spacing(v):
    """Distance between neighbouring fp16 values at magnitude |v| (normal range)."""
    v = np.maximum(np.abs(v.astype(np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(v)) - 10)


@pytest.mark.parametrize("kernel", [Kernel.U8Ring, Kernel.U8Stream, Kernel.U8KSplit, Kernel.Auto])
def test_u8_decode_kernels_follow_the_unrounded_reference_form(kernels, kernel):
    """The decode kernels claim the arithmetic of matmul_nt_fp16u8.cu:13-23 (weights not rounded
    to fp16).  Held to it here: against the oracle's faithful restatement of that kernel and,
    when the reference cubins travelled along, against the kernel itself run live.  The only
    difference left is the order of the fp32 additions (sequential over k there, per scale
    group here), about 1e-6 relative on a sum before the final rounding to fp16, so almost
    every output has the same bits and none is more than one fp16 step away (steps measured
    at max(|ref|, rms/4), since a sum that cancels to nearly zero has no meaningful ulp)."""
    rng = np.random.default_rng(2024)
    worst, same, total = 0.0, 0, 0
    try:
        kernels.force_kernel(kernel)
        for m in (1, 4, 16):
            for bs in (64, 128):
                p, n = 4096, 512
                x = rng.standard_normal((m, p)).astype(np.float16)
                q = rng.integers(0, 256, (n, p), dtype=np.uint8)
                s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
                want = oracle.matmul_nt_fp16u8(x, q, s, bs, faithful=True)
                xd, qd, sd = dev(x), dev(q), dev(s)
                o = torch.zeros((m, n), dtype=torch.float16, device="cuda")
                kernels.matmul_nt_fp16u8(o, xd, qd, sd, bs)
                kernels.device_status()
                got = o.cpu().numpy()
                refs = [want]
                if refcubin.available():
                    r = torch.zeros_like(o)
                    refcubin.matmul_nt_fp16u8(r.data_ptr(), xd.data_ptr(), qd.data_ptr(), sd.data_ptr(),
                                              m, p, n, bs, 0.0)
                    torch.cuda.synchronize()
                    refs.append(r.cpu().numpy())
                for ref in refs:
                    rf = ref.astype(np.float64)
                    unit = fp16_spacing(np.maximum(np.abs(rf), np.sqrt(np.mean(rf ** 2)) / 4))
                    steps = np.abs(got.astype(np.float64) - rf) / unit
                    worst = max(worst, float(steps.max()))
                    same += int(np.count_nonzero(got.view(np.uint16) == ref.view(np.uint16)))
                    total += got.size
    finally:
        kernels.force_kernel(Kernel.Auto)
    assert worst <= 1.0, worst
    assert same / total >= 0.97, same / total


def test_matmul_f16_second_batch_dimension(kernels):
    """adr_matmul_f16_b2 on the [B, H, S, hd] views of [B, S, H*hd] storage that a batched attention
    block multiplies: the same bits as one matmul_f16 call per outer index; operands whose two
    batch dimensions fold go out as one launch; a rank-3 operand is broadcast over the outer one."""
    B, H, S, hd = 3, 4, 72, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((B, S, H * hd), device="cuda", generator=g).half()
    k = torch.randn((B, S, H * hd), device="cuda", generator=g).half()
    lay4 = TensorLayout.new((B, H, S, hd), (S * H * hd, hd, H * hd, 1))
    qv, kv = TensorView(q, lay4), TensorView(k, lay4)
    opts = MatmulOptions.new().store(MatmulStore.Scale(0.125)).mask(MatmulMask.Causal)
    out = torch.zeros((B, H, S, S), dtype=torch.float16, device="cuda")
    n0 = kernels.launch_count()
    kernels.matmul_f16_b2(TensorView.of(out), qv, kv.permute([0, 1, 3, 2]), opts)
    assert kernels.launch_count() - n0 == B  # the outer stride of q and k does not fold
    want = torch.zeros_like(out)
    lay3 = TensorLayout.new((H, S, hd), (hd, H * hd, 1))
    for b in range(B):
        kernels.matmul_f16(TensorView.of(want[b]), TensorView(q[b], lay3),
                           TensorView(k[b], lay3).permute([0, 2, 1]), opts)
    kernels.device_status()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    ref = torch.einsum("bhsd,bhtd->bhst", q.view(B, S, H, hd).permute(0, 2, 1, 3).float(),
                       k.view(B, S, H, hd).permute(0, 2, 1, 3).float()) * 0.125
    mask = torch.ones((S, S), dtype=torch.bool, device="cuda").tril()
    got = out.float()
    assert torch.all(torch.isinf(got[..., ~mask]) & (got[..., ~mask] < 0))
    err = (got[..., mask] - ref[..., mask]).abs().max() / ref[..., mask].abs().max()
    assert err.item() <= TOL
    # contiguous [B, H, S, hd] operands fold into one launch; the rhs is a rank-3 view shared by all b
    a = torch.randn((B, H, S, hd), device="cuda", generator=g).half()
    w = torch.randn((H, hd, 48), device="cuda", generator=g).half()
    o2 = torch.zeros((B, H, S, 48), dtype=torch.float16, device="cuda")
    n0 = kernels.launch_count()
    kernels.matmul_f16_b2(TensorView.of(o2), TensorView.of(a), TensorView.of(w))
    assert kernels.launch_count() - n0 == B  # the broadcast operand's strides (z != 0, w == 0) do not fold
    w4 = w.unsqueeze(0).expand(B, H, hd, 48).contiguous()
    o3 = torch.zeros_like(o2)
    n0 = kernels.launch_count()
    kernels.matmul_f16_b2(TensorView.of(o3), TensorView.of(a), TensorView.of(w4))
    assert kernels.launch_count() - n0 == 1
    kernels.device_status()
    assert torch.equal(o2.view(torch.int16), o3.view(torch.int16))
    ref2 = torch.einsum("bhsd,hdn->bhsn", a.float(), w.float())
    assert ((o2.float() - ref2).abs().max() / ref2.abs().max()).item() <= TOL


@pytest.mark.parametrize("pdl", [0, 1])
def test_u8_grouped_products_equal_separate_calls(kernels, pdl):
    """adr_matmul_nt_fp16u8_grouped: q/k/v-like and gate/up-like groups over the same activations
    give the bits of separate calls of the persistent kernel (ragged n, zero points, beta, more
    than four matrices, both token blocks); a shape the grouped form does not take still works."""
    rng = np.random.default_rng(311 + pdl)
    try:
        kernels.set_tunable("pdl", pdl)
        for m, p, ns, bs, zp, beta in ((1, 4096, (4096, 4096, 4096), 128, False, 0.0),
                                       (4, 4096, (11008, 11008), 128, False, 0.5),
                                       (16, 2048, (200, 1000, 48, 333, 640), 64, True, 0.5),
                                       (3, 1280, (64, 4000), 64, False, 0.0),
                                       (16, 11008, (256, 272), 128, False, 0.0)):  # activations too large: separate calls
            x = dev(rng.standard_normal((m, p)).astype(np.float16))
            qs = [dev(rng.integers(0, 256, (n, p), dtype=np.uint8)) for n in ns]
            ss = [dev(rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)) for n in ns]
            zs = [dev(rng.uniform(120, 136, (n, p // bs)).astype(np.float16)) for n in ns] if zp else None
            o0 = [(rng.standard_normal((m, n)) * 0.5).astype(np.float16) for n in ns]
            want = []
            kernels.force_kernel(Kernel.U8Ring)
            for i, n in enumerate(ns):
                o = dev(o0[i].copy())
                kernels.matmul_nt_fp16u8(o, x, qs[i], ss[i], bs, beta, zs[i] if zp else None)
                want.append(o)
            kernels.force_kernel(Kernel.Auto)
            outs = [dev(a.copy()) for a in o0]
            n0 = kernels.launch_count()
            kernels.matmul_nt_fp16u8_grouped(outs, x, qs, ss, bs, beta, zs)
            launches = kernels.launch_count() - n0
            kernels.device_status()
            if p <= 4096:
                assert launches == (len(ns) + 3) // 4  # four matrices per launch, a lone last one by itself
                for i, (got, ref) in enumerate(zip(outs, want)):
                    if len(ns) % 4 == 1 and i == len(ns) - 1:  # served by a separate call: any decode kernel
                        w = oracle.matmul_nt_fp16u8(x.cpu().numpy(), qs[i].cpu().numpy(), ss[i].cpu().numpy(),
                                                    bs, beta, o0[i], zs[i].cpu().numpy() if zp else None)
                        assert oracle.max_rel_err(got.cpu().numpy(), w) <= 2e-3
                    else:
                        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), (m, p, ns, i)
            else:
                assert launches >= len(ns)
                for got, q, s_, a0 in zip(outs, qs, ss, o0):
                    w = oracle.matmul_nt_fp16u8(x.cpu().numpy(), q.cpu().numpy(), s_.cpu().numpy(), bs, beta, a0)
                    assert oracle.max_rel_err(got.cpu().numpy(), w) <= 2e-3
    finally:
        kernels.set_tunable("pdl", 0)
        kernels.force_kernel(Kernel.Auto)
