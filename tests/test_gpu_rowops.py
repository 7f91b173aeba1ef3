"""GPU parity of the row ops (rms_norm, softmax_rows, rotary, elementwise binary and the two
decode forms), called through the C ABI.

Three checks per reference-derived kernel: the same bits as the reference's own kernel run
live (oracle/_ref cubins), the same bits as the committed golden vectors those kernels
produced, and agreement with the CPU oracle to one unit in the last place of the fp16 result
(the oracle uses libm where the device uses its own expf/powf/sinf/cosf/rsqrt)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from oracle import oracle, refcubin

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden" / "reference_rowops.npz"
CASES = cases.rowop_cases()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ulp_diff(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 units in the last place between finite values (0 where both are
    the same non-finite pattern)."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    d = np.abs(key(np.ascontiguousarray(a)) - key(np.ascontiguousarray(b)))
    same = a.view(np.uint16) == b.view(np.uint16)
    return np.where(same, 0, d)


def run_ours(kernels, c):
    from adrastea_b200 import BinaryOp, TensorView
    if c["kind"] == "rms":
        x, w = dev(c["x"]), dev(c["w"])
        o = torch.zeros_like(x)
        kernels.rms_norm(TensorView.of(o), TensorView.of(x), TensorView.of(w), c["eps"])
    elif c["kind"] == "softmax":
        o = dev(c["x"])
        kernels.softmax_rows_inplace(TensorView.of(o), c["temp"])
    elif c["kind"] == "rotary":
        o = dev(c["x"])
        kernels.rotary_inplace(TensorView.of(o), c["n_heads"], c["pos_offset"], c["theta"])
    else:
        o, r = dev(c["left"]), dev(c["right"])
        kernels.elementwise_binary_2d_f16_inplace(TensorView.of(o), TensorView.of(r), BinaryOp(c["op"]))
    torch.cuda.synchronize()
    kernels.device_status()
    return o.cpu().numpy()


def run_oracle(c):
    if c["kind"] == "rms":
        return oracle.rms_norm(c["x"], c["w"], c["eps"])
    if c["kind"] == "softmax":
        return oracle.softmax_rows(c["x"], temp=c["temp"])
    if c["kind"] == "rotary":
        return oracle.rotary(c["x"], c["n_heads"], c["pos_offset"], c["theta"])
    return oracle.elementwise_binary(c["left"], c["right"], c["op"])


def run_reference(c):
    if c["kind"] == "rms":
        x, w = dev(c["x"]), dev(c["w"])
        o = torch.zeros_like(x)
        ly, lx = c["x"].shape
        refcubin.rms_norm(o.data_ptr(), x.data_ptr(), w.data_ptr(), lx, ly, 1, lx, 1, lx, c["eps"])
    elif c["kind"] == "softmax":
        x = dev(c["x"])
        o = torch.zeros_like(x)
        heads, h, w_ = c["x"].shape
        refcubin.softmax_rows(o.data_ptr(), x.data_ptr(), heads, h, w_, c["temp"])
    elif c["kind"] == "rotary":
        x = dev(c["x"])
        o = torch.zeros_like(x)
        ly, lx = c["x"].shape
        refcubin.rotary(o.data_ptr(), x.data_ptr(), lx, ly, 1, lx, 1, lx, c["n_heads"],
                        c["pos_offset"], c["theta"])
    else:
        l, r = dev(c["left"]), dev(c["right"])
        o = torch.zeros_like(l)
        rows, cols = c["left"].shape
        refcubin.elementwise_binary_2d_f16(o.data_ptr(), l.data_ptr(), r.data_ptr(), rows, cols, c["op"])
    torch.cuda.synchronize()
    return o.cpu().numpy()


@pytest.mark.parametrize("name", list(CASES), ids=list(CASES))
def test_rowop_against_oracle(kernels, name):
    c = CASES[name]
    got, want = run_ours(kernels, c), run_oracle(c)
    d = ulp_diff(got, want)
    if c["kind"] == "binary" and c["op"] == 1:
        assert d.max() == 0
    else:
        assert d.max() <= 1 and (d != 0).mean() < 0.02, (int(d.max()), float((d != 0).mean()))


@pytest.mark.parametrize("name", list(CASES), ids=list(CASES))
def test_rowop_same_bits_as_live_reference_kernel(kernels, name):
    if not refcubin.available():
        pytest.skip("reference cubins not built")
    c = CASES[name]
    got, ref = run_ours(kernels, c), run_reference(c)
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16)), int(ulp_diff(got, ref).max())


@pytest.mark.parametrize("name", list(CASES), ids=list(CASES))
def test_rowop_same_bits_as_golden(kernels, name):
    if not GOLD.exists():
        pytest.skip("reference_rowops.npz not generated yet")
    g = np.load(GOLD)
    c = CASES[name]
    ins = [c[k] for k in ("x", "w", "left", "right") if k in c]
    assert bytes(g[name + "/digest"]).decode() == cases.digest(*ins), "input generator drifted"
    got = run_ours(kernels, c)
    assert np.array_equal(got.view(np.uint16), g[name + "/out"].view(np.uint16))


def test_softmax_padded_rows_and_strided_rms(kernels):
    """Extensions over the reference launch: padded softmax rows keep their pad columns;
    rms_norm with row strides on both sides."""
    from adrastea_b200 import TensorLayout, TensorView
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((4, 9, 40)) * 2).astype(np.float16)
    o = dev(x)
    view = TensorView(o, TensorLayout.new((4, 9, 33), (9 * 40, 40, 1)))
    kernels.softmax_rows_inplace(view, 1.0)
    got = o.cpu().numpy()
    want = oracle.softmax_rows(x, w=33)
    assert ulp_diff(got[:, :, :33], want[:, :, :33]).max() <= 1
    assert np.array_equal(got[:, :, 33:].view(np.uint16), x[:, :, 33:].view(np.uint16))
    xs = (rng.standard_normal((6, 300))).astype(np.float16)
    w = rng.uniform(0.5, 1.5, 256).astype(np.float16)
    xi, oo = dev(xs), torch.zeros((6, 320), dtype=torch.float16, device="cuda")
    kernels.rms_norm(TensorView(oo, TensorLayout.new((6, 256), (320, 1))),
                     TensorView(xi, TensorLayout.new((6, 256), (300, 1))), TensorView.of(dev(w)), 1e-6)
    want = oracle.rms_norm(xs[:, :256], w, 1e-6)
    assert ulp_diff(oo.cpu().numpy()[:, :256], want).max() <= 1
    assert float(oo[:, 256:].abs().max()) == 0.0
    kernels.device_status()


@pytest.mark.parametrize("B,H,hd,S,pos", [(3, 4, 128, 64, 0), (2, 2, 128, 640, 517), (5, 3, 64, 40, 39),
                                          (1, 2, 256, 24, 10), (16, 16, 128, 64, 50), (8, 16, 128, 72, 70),
                                          (4, 16, 64, 200, 133), (3, 2, 128, 16, 2), (2, 3, 96, 40, 17)])
def test_decode_rope_append_and_attention(kernels, B, H, hd, S, pos):
    """Covers every cluster size of the wide attention kernel (B*H >= 256, 128, 64, fewer),
    fewer positions than CTAs in a cluster, and a head size only the general kernel takes."""
    from adrastea_b200 import TensorView
    rng = np.random.default_rng(B * 1000 + pos)
    width = H * hd
    f16 = lambda a: np.ascontiguousarray(a, dtype=np.float16)
    # q, k, v as three column blocks of one [B, 3*width] buffer (row stride 3*width)
    qkv = f16(rng.standard_normal((B, 3 * width)))
    kc = f16(rng.standard_normal((B, S, width)) * 0.7)
    vc = f16(rng.standard_normal((B, S, width)))
    d_qkv, d_kc, d_vc = dev(qkv), dev(kc), dev(vc)
    pos_dev = torch.tensor([pos], dtype=torch.int32, device="cuda")
    tv = lambda i: TensorView.of(d_qkv[:, i * width:(i + 1) * width])
    kernels.decode_rope_append(tv(0), tv(1), tv(2), d_kc, d_vc, H, pos_dev, 10000.0)
    torch.cuda.synchronize()
    q_rot = oracle.rotary(qkv[:, :width], H, pos, 10000.0, same_pos=True)
    k_rot = oracle.rotary(qkv[:, width:2 * width], H, pos, 10000.0, same_pos=True)
    got = d_qkv.cpu().numpy()
    assert ulp_diff(got[:, :width], q_rot).max() <= 1
    assert np.array_equal(got[:, width:], qkv[:, width:])  # k and v inputs untouched
    kc2, vc2 = d_kc.cpu().numpy(), d_vc.cpu().numpy()
    assert ulp_diff(kc2[:, pos], k_rot).max() <= 1
    assert np.array_equal(vc2[:, pos], qkv[:, 2 * width:])
    keep = np.arange(S) != pos
    assert np.array_equal(kc2[:, keep], kc[:, keep]) and np.array_equal(vc2[:, keep], vc[:, keep])
    # attention over the cache as the device left it
    out = torch.zeros((B, width), dtype=torch.float16, device="cuda")
    scale = 1.0 / np.sqrt(hd)
    kernels.decode_attention(TensorView.of(out), tv(0), d_kc, d_vc, H, pos_dev, scale)
    torch.cuda.synchronize()
    kernels.device_status()
    want = oracle.decode_attention(got[:, :width], kc2, vc2, H, pos, scale)
    assert oracle.max_rel_err(out.cpu().numpy(), want) <= 2e-3
    again = torch.zeros_like(out)
    kernels.decode_attention(TensorView.of(again), tv(0), d_kc, d_vc, H, pos_dev, scale)
    assert torch.equal(out, again), "not deterministic"


@pytest.mark.parametrize("rows,heads,hd,pos", [(40, 64, 128, 7), (5, 6, 32, 2000), (130, 8, 64, 0), (3, 4, 256, 511)])
def test_rotary_many_heads_same_bits(kernels, rows, heads, hd, pos):
    """From four heads on (contiguous columns) the rotation computes cos, sin and the power once
    per (row, pair of a head) and applies them to every head.  Same bits as the kernel that
    computes them per element (reached here through two-head column slices), as the reference
    kernel run live, and within two units in the last place of the CPU oracle (libm against the
    device's functions; where the two products nearly cancel the second unit shows)."""
    from adrastea_b200 import TensorView
    rng = np.random.default_rng(rows + heads + hd)
    x = rng.standard_normal((rows, heads * hd)).astype(np.float16)
    got = dev(x.copy())
    kernels.rotary_inplace(TensorView.of(got), heads, pos, 10000.0)
    kernels.device_status()
    per_pair = dev(x.copy())
    for h0 in range(0, heads, 2):
        kernels.rotary_inplace(TensorView.of(per_pair[:, h0 * hd:(h0 + 2) * hd]), 2, pos, 10000.0)
    assert torch.equal(got.view(torch.int16), per_pair.view(torch.int16))
    assert ulp_diff(got.cpu().numpy(), oracle.rotary(x, heads, pos, 10000.0)).max() <= 2
    if refcubin.available():
        xd, r = dev(x), torch.zeros_like(got)
        lx = heads * hd
        refcubin.rotary(r.data_ptr(), xd.data_ptr(), lx, rows, 1, lx, 1, lx, heads, pos, 10000.0)
        torch.cuda.synchronize()
        assert torch.equal(r.view(torch.int16), got.view(torch.int16))


def test_rowop_argument_errors(kernels):
    from adrastea_b200 import AdrError, TensorLayout, TensorView
    x = torch.zeros((4, 30), dtype=torch.float16, device="cuda")
    with pytest.raises(AdrError):  # 30 columns over 4 heads: odd head_dim 7.5
        kernels.rotary_inplace(TensorView.of(x), 4, 0, 10000.0)
    with pytest.raises(AdrError):  # temperature must be positive
        kernels.softmax_rows_inplace(TensorView.of(x), 0.0)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc = torch.zeros((4, 12, 30), dtype=torch.float16, device="cuda")
    with pytest.raises(AdrError):  # head_dim 15 is not a multiple of 8
        kernels.decode_attention(TensorView.of(x), TensorView.of(x), kc, kc, 2, pos, 1.0)


@pytest.mark.parametrize("m,p,n,bs", [(1, 4096, 512, 128), (5, 2048, 300, 64), (16, 4096, 256, 128),
                                      (8, 1024, 64, 128)])
def test_rms_norm_fused_into_the_decode_gemv(kernels, m, p, n, bs):
    """adr_rms_norm_matmul_nt_fp16u8 gives the bits of adr_rms_norm followed by
    adr_matmul_nt_fp16u8 (it replays the reference's reduction order inside the GEMV kernel)."""
    from adrastea_b200 import Kernel, TensorView
    rng = np.random.default_rng(m * 7 + n)
    x = dev((rng.standard_normal((m, p)) * rng.uniform(0.2, 3.0, (m, 1))).astype(np.float16))
    w = dev(rng.uniform(0.5, 1.5, p).astype(np.float16))
    q = dev(rng.integers(0, 256, (n, p), dtype=np.uint8))
    s = dev(rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16))
    out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
    xn = torch.zeros_like(x)
    kernels.rms_norm(TensorView.of(xn), TensorView.of(x), TensorView.of(w), 1e-5)
    two = dev(out0.copy())
    kernels.force_kernel(Kernel.U8Ring)  # the fused form lives in the ring kernel: same bits as its plain form
    try:
        kernels.matmul_nt_fp16u8(two, xn, q, s, bs, 0.5)
    finally:
        kernels.force_kernel(Kernel.Auto)
    assert kernels.last_kernel() == Kernel.U8Ring
    one = dev(out0.copy())
    kernels.rms_norm_matmul_nt_fp16u8(one, x, w, 1e-5, q, s, bs, 0.5)
    torch.cuda.synchronize()
    kernels.device_status()
    assert torch.equal(one.view(torch.int16), two.view(torch.int16))


def test_embed_uint8_same_bits_as_reference_and_oracle(kernels):
    rng = np.random.default_rng(31)
    vocab, d, bs = 500, 256, 64
    table = rng.integers(0, 256, (vocab, d), dtype=np.uint8)
    scales = rng.uniform(0.001, 0.01, (vocab, d // bs)).astype(np.float16)
    ids = rng.integers(0, vocab, 37).astype(np.int16)
    want = oracle.embed_uint8(ids, table, scales, bs)
    t, s, i = dev(table), dev(scales), dev(ids)
    out = torch.zeros((37, d), dtype=torch.float16, device="cuda")
    kernels.embed_uint8(out, i, t, s, bs)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    if refcubin.available():
        ref = torch.zeros_like(out)
        refcubin.embed_uint8(d, 37, i.data_ptr(), ref.data_ptr(), t.data_ptr(), s.data_ptr(), bs)
        torch.cuda.synchronize()
        assert torch.equal(ref.view(torch.int16), out.view(torch.int16))
    kernels.device_status()


@pytest.mark.parametrize("rows,lx", [(5, 1024), (3, 1000), (2, 4100), (4, 64), (1, 8192),
                                     (1030, 1024), (2051, 1000), (1025, 64)])  # many rows: four rows per CTA
def test_layer_norm_same_bits_as_reference(kernels, rows, lx):
    """adr_layer_norm against the reference kernel run live (same bits: it keeps the kernel's
    summation order) and against the CPU oracle (one fp16 step: libm division and square root
    against the device's)."""
    from adrastea_b200 import TensorView
    rng = np.random.default_rng(rows * 100 + lx)
    x = (rng.standard_normal((rows, lx)) * rng.uniform(0.2, 3.0, (rows, 1)) + rng.uniform(-1, 1, (rows, 1))).astype(np.float16)
    w = rng.uniform(0.5, 1.5, lx).astype(np.float16)
    b = rng.uniform(-0.5, 0.5, lx).astype(np.float16)
    xd, wd, bd = dev(x), dev(w), dev(b)
    o = torch.zeros_like(xd)
    kernels.layer_norm(TensorView.of(o), TensorView.of(xd), TensorView.of(wd), TensorView.of(bd), 1e-5)
    kernels.device_status()
    got = o.cpu().numpy()
    want = oracle.layer_norm(x, w, b, 1e-5)
    assert ulp_diff(got, want).max() <= 1
    if refcubin.available():
        r = torch.zeros_like(xd)
        refcubin.layer_norm(r.data_ptr(), xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), lx, rows, 1, lx, 1, lx, 1e-5)
        torch.cuda.synchronize()
        assert torch.equal(r.view(torch.int16), o.view(torch.int16))


@pytest.mark.parametrize("m,p,n,bs,zp", [(1, 4096, 11008, 128, False), (4, 4096, 1000, 64, False),
                                          (16, 2048, 333, 128, True), (7, 1280, 4000, 64, True),
                                          (2, 4096, 16, 128, False)])
def test_silu_mul_fused_into_the_gate_and_up_products(kernels, m, p, n, bs, zp):
    """adr_silu_mul_matmul_nt_fp16u8 gives the bits of two adr_matmul_nt_fp16u8 calls (persistent
    kernel) followed by the SiluMul elementwise kernel; the two matrices are the halves of one
    [2n, p] matrix, as a harness that fuses gate and up at load time holds them."""
    from adrastea_b200 import BinaryOp, Kernel, TensorView
    rng = np.random.default_rng(m * 11 + n)
    x = dev(rng.standard_normal((m, p)).astype(np.float16))
    q = dev(rng.integers(0, 256, (2 * n, p), dtype=np.uint8))
    s = dev(rng.uniform(0.001, 0.01, (2 * n, p // bs)).astype(np.float16))
    z = dev(rng.uniform(120, 136, (2 * n, p // bs)).astype(np.float16)) if zp else None
    g = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    u = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    kernels.force_kernel(Kernel.U8Ring)
    try:
        kernels.matmul_nt_fp16u8(g, x, q[:n], s[:n], bs, 0.0, z[:n] if zp else None)
        kernels.matmul_nt_fp16u8(u, x, q[n:], s[n:], bs, 0.0, z[n:] if zp else None)
    finally:
        kernels.force_kernel(Kernel.Auto)
    want = torch.zeros_like(g)
    kernels.elementwise_binary_2d_f16(TensorView.of(want), TensorView.of(g), TensorView.of(u), BinaryOp.SiluMul)
    for pdl in (0, 1):
        kernels.set_tunable("pdl", pdl)
        try:
            for _ in range(2):
                got = torch.full((m, n), 7.0, dtype=torch.float16, device="cuda")
                n0 = kernels.launch_count()
                kernels.silu_mul_matmul_nt_fp16u8(got, x, q[:n], s[:n], q[n:], s[n:], bs,
                                                  z[:n] if zp else None, z[n:] if zp else None)
                assert kernels.launch_count() - n0 == 1
                kernels.device_status()
                assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (m, p, n, pdl)
        finally:
            kernels.set_tunable("pdl", 0)


@pytest.mark.parametrize("m,p,width,heads,bs,with_norm", [(1, 4096, 4096, 32, 128, False), (4, 4096, 4096, 32, 128, True),
                                                          (2, 1024, 512, 4, 64, True), (16, 2048, 256, 2, 128, False),
                                                          (3, 1280, 192, 3, 64, False)])
def test_qkv_product_with_rotary_and_cache_append_fused(kernels, m, p, width, heads, bs, with_norm):
    """adr_qkv_rope_append_matmul_nt_fp16u8 gives the bits of (adr_rms_norm +) adr_matmul_nt_fp16u8
    (persistent kernel) followed by adr_decode_rope_append: rotated q, and the rows of the key and
    value caches at the position; every other cache row stays untouched."""
    from adrastea_b200 import Kernel, TensorView
    rng = np.random.default_rng(m * 13 + width)
    S, pos_val, theta, eps = 24, 17, 10000.0, 1e-5
    x = dev((rng.standard_normal((m, p)) * rng.uniform(0.5, 2.0, (m, 1))).astype(np.float16))
    nw = dev(rng.uniform(0.5, 1.5, p).astype(np.float16))
    q = dev(rng.integers(0, 256, (3 * width, p), dtype=np.uint8))
    s = dev(rng.uniform(0.001, 0.01, (3 * width, p // bs)).astype(np.float16))
    pos = torch.tensor([pos_val], dtype=torch.int32, device="cuda")
    fill = 0.25
    # the separate kernels
    xin = x
    if with_norm:
        xin = torch.zeros_like(x)
        kernels.rms_norm(TensorView.of(xin), TensorView.of(x), TensorView.of(nw), eps)
    qkv = torch.zeros((m, 3 * width), dtype=torch.float16, device="cuda")
    kernels.force_kernel(Kernel.U8Ring)
    try:
        kernels.matmul_nt_fp16u8(qkv, xin, q, s, bs)
    finally:
        kernels.force_kernel(Kernel.Auto)
    kc = torch.full((m, S, width), fill, dtype=torch.float16, device="cuda")
    vc = torch.full((m, S, width), fill, dtype=torch.float16, device="cuda")
    qv, kv, vv = (TensorView.of(qkv[:, i * width:(i + 1) * width]) for i in range(3))
    kernels.decode_rope_append(qv, kv, vv, kc, vc, heads, pos, theta)
    kernels.device_status()
    for pdl in (0, 1):
        kernels.set_tunable("pdl", pdl)
        try:
            out = torch.full((m, 3 * width), 9.0, dtype=torch.float16, device="cuda")
            kc2 = torch.full((m, S, width), fill, dtype=torch.float16, device="cuda")
            vc2 = torch.full((m, S, width), fill, dtype=torch.float16, device="cuda")
            n0 = kernels.launch_count()
            kernels.qkv_rope_append_matmul_nt_fp16u8(out[:, :width], x, q, s, bs, heads, kc2, vc2, pos, theta,
                                                     nw if with_norm else None, eps)
            assert kernels.launch_count() - n0 == 1
            kernels.device_status()
            assert torch.equal(out[:, :width].contiguous().view(torch.int16),
                               qkv[:, :width].contiguous().view(torch.int16)), (m, p, width, pdl)
            assert torch.all(out[:, width:] == 9.0)
            assert torch.equal(kc2.view(torch.int16), kc.view(torch.int16))
            assert torch.equal(vc2.view(torch.int16), vc.view(torch.int16))
        finally:
            kernels.set_tunable("pdl", 0)
    # a position outside the cache writes nothing
    bad = torch.tensor([S], dtype=torch.int32, device="cuda")
    out = torch.full((m, 3 * width), 9.0, dtype=torch.float16, device="cuda")
    kc2 = torch.full((m, S, width), fill, dtype=torch.float16, device="cuda")
    vc2 = kc2.clone()
    kernels.qkv_rope_append_matmul_nt_fp16u8(out[:, :width], x, q, s, bs, heads, kc2, vc2, bad, theta)
    kernels.device_status()
    assert torch.all(out == 9.0) and torch.all(kc2 == fill) and torch.all(vc2 == fill)
