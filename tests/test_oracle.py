"""The CPU oracle against independent numpy restatements and against the
golden vectors produced by the reference's own kernels (tests/golden/).
No GPU needed."""
from pathlib import Path

import numpy as np
import pytest

import cases
from oracle import oracle

GOLD = Path(__file__).resolve().parent / "golden"
F16 = np.float16


# ---------------------------------------------------------------- fp16 basics
def test_f16_to_f32_exhaustive():
    lib = oracle.lib()
    allh = np.arange(65536, dtype=np.uint16)
    want = allh.view(F16).astype(np.float32)
    got = np.array([lib.orc_f16_to_f32(int(h)) for h in allh], np.float32)
    nan = np.isnan(want)  # NaN payloads may be quieted on the way through a float return
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])


def test_f32_and_f64_to_f16_round_to_nearest_even():
    lib = oracle.lib()
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000),
                        [0.0, -0.0, 65504.0, 65520.0, 65519.99, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                         np.inf, -np.inf, 6.1e-5, 6.0975e-5]])
    f32 = x.astype(np.float32)
    got = np.array([lib.orc_f32_to_f16(float(v)) for v in f32], np.uint16)
    assert np.array_equal(got, f32.astype(F16).view(np.uint16))
    got = np.array([lib.orc_f64_to_f16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, x.astype(F16).view(np.uint16))


def test_half_mul_and_add_round_once():
    lib = oracle.lib()
    rng = np.random.default_rng(2)
    a = (rng.standard_normal(5000) * 10.0 ** rng.integers(-4, 3, 5000)).astype(F16)
    b = (rng.standard_normal(5000) * 10.0 ** rng.integers(-4, 3, 5000)).astype(F16)
    mul = np.array([lib.orc_hmul(int(x), int(y)) for x, y in zip(a.view(np.uint16), b.view(np.uint16))], np.uint16)
    add = np.array([lib.orc_hadd(int(x), int(y)) for x, y in zip(a.view(np.uint16), b.view(np.uint16))], np.uint16)
    assert np.array_equal(mul, (a.astype(np.float64) * b.astype(np.float64)).astype(F16).view(np.uint16))
    assert np.array_equal(add, (a.astype(np.float64) + b.astype(np.float64)).astype(F16).view(np.uint16))


# ------------------------------------------------- independent restatements
def _views(c, out, lhs, rhs):
    es = 2
    ast = np.lib.stride_tricks.as_strided
    L = ast(lhs, (c.batches, c.m, c.k), (c.lhs_strides[2] * es, c.lhs_strides[1] * es, c.lhs_strides[0] * es))
    R = ast(rhs, (c.batches, c.k, c.n), (c.rhs_strides[2] * es, c.rhs_strides[1] * es, c.rhs_strides[0] * es))
    O = ast(out, (c.batches, c.m, c.n), (c.out_strides[2] * es, c.out_strides[1] * es, c.out_strides[0] * es))
    return O, L, R


def _py_epilogue(c, acc32, old, bias):
    """numpy restatement of the store functors (matmul.cu:45-176, 444-491)."""
    hs = acc32.astype(F16)
    if c.store == cases.ST_IDENTITY:
        return hs
    if c.store == cases.ST_SCALE:
        return (hs.astype(np.float64) * np.float64(F16(c.scale))).astype(F16)
    if c.store == cases.ST_ADD:
        return (hs.astype(np.float64) + old.astype(np.float64)).astype(F16)
    t = hs.astype(np.float32) + bias.astype(np.float32)[None, None, :]
    if c.store == cases.ST_BETA_GELU_BIAS:
        t = (np.float32(0.5) * t * (np.float32(1) + np.tanh(np.float32(0.7978845608028654) * (t + np.float32(0.044715) * t * t * t)))).astype(np.float32)
    if c.store == cases.ST_QUICK_GELU:
        return (t * (np.float32(1) / (np.float32(1) + np.exp(-np.float32(1.702) * t)))).astype(F16)
    # beta * old + t with a single rounding
    return (np.float64(np.float32(c.beta)) * old.astype(np.float64) + t.astype(np.float64)).astype(np.float32).astype(F16)


def _run_oracle(c, ideal):
    out, lhs, rhs, bias = c.inputs()
    rc = oracle.matmul_f16(out, lhs, rhs, c.batches, c.m, c.k, c.n, c.strides9(),
                           bias if c.uses_bias() else None, c.beta, c.scale, c.store, c.load,
                           c.mask, ideal=ideal)
    assert rc == 0
    return out


@pytest.mark.parametrize("c", cases.matmul_cases(), ids=lambda c: c.name)
def test_ideal_oracle_against_numpy_float64(c):
    out0, lhs, rhs, bias = c.inputs()
    got = _run_oracle(c, ideal=True)
    O0, L, R = _views(c, out0.copy(), lhs, rhs)
    L64, R64 = L.astype(np.float64), R.astype(np.float64)
    if c.load == cases.LD_SCALE:
        hsc = np.float64(F16(c.scale))
        L64 = (L64 * hsc).astype(F16).astype(np.float64)
        R64 = (R64 * hsc).astype(F16).astype(np.float64)
    acc = np.einsum("bmk,bkn->bmn", L64, R64).astype(np.float32)
    want = _py_epilogue(c, acc, O0.copy(), bias)
    if c.mask == cases.MK_CAUSAL:
        y, x = np.meshgrid(np.arange(c.m), np.arange(c.n), indexing="ij")
        want = np.where((x > y)[None], F16(-np.inf), want)
    G, _, _ = _views(c, got, lhs, rhs)
    # summation order in double differs from einsum's: allow a handful of 1-ulp flips
    diff = G.view(np.uint16).astype(np.int32) - want.view(np.uint16).astype(np.int32)
    assert np.abs(diff).max() <= (1 if c.exact_vs_reference else 2)
    assert (diff != 0).mean() < 0.01
    # elements of the storage outside the view are untouched
    untouched = np.ones(out0.size, bool)
    idx = (np.arange(c.batches)[:, None, None] * c.out_strides[2] + np.arange(c.m)[None, :, None] * c.out_strides[1]
           + np.arange(c.n)[None, None, :] * c.out_strides[0])
    untouched[idx.reshape(-1)] = False
    assert np.array_equal(got[untouched].view(np.uint16), out0[untouched].view(np.uint16))


def test_faithful_oracle_against_scalar_python_loop():
    """fp16-rounded products summed sequentially in fp32 (matmul.cu:214-218)."""
    rng = np.random.default_rng(3)
    m, k, n = 5, 37, 7
    lhs = rng.standard_normal(m * k).astype(F16)
    rhs = rng.standard_normal(k * n).astype(F16)
    out = np.zeros(m * n, F16)
    assert oracle.matmul_f16(out, lhs, rhs, 1, m, k, n, (1, n, 0, 1, k, 0, 1, n, 0)) == 0
    want = np.zeros((m, n), F16)
    for y in range(m):
        for x in range(n):
            s = np.float32(0)
            for i in range(k):
                s = np.float32(s + np.float32(F16(lhs[y * k + i] * rhs[i * n + x])))
            want[y, x] = F16(s)
    assert np.array_equal(out.view(np.uint16), want.reshape(-1).view(np.uint16))


def test_unsupported_store_op_is_reported():
    z = np.zeros(4, F16)
    assert oracle.matmul_f16(z, z, z, 1, 2, 2, 2, (1, 2, 0, 1, 2, 0, 1, 2, 0), store=cases.ST_GELU_BIAS) == 3


@pytest.mark.parametrize("c", cases.u8_cases(), ids=lambda c: c.name)
def test_u8_oracle_against_numpy(c):
    out0, lhs, q, scales, zeros = c.inputs()
    g = np.repeat(scales.astype(np.float32), c.block_size, axis=1)
    z = np.float32(127.5) if zeros is None else np.repeat(zeros.astype(np.float32), c.block_size, axis=1)
    w = ((q.astype(np.float32) - z).astype(np.float32) * g).astype(np.float32).astype(F16)
    got_w = oracle.dequantize(q, scales, c.block_size, zeros)
    assert np.array_equal(got_w.view(np.uint16), w.view(np.uint16))
    acc = lhs.astype(np.float64) @ w.astype(np.float64).T
    want = (np.float64(np.float32(c.beta)) * out0.astype(np.float64) + acc.astype(np.float32).astype(np.float64)).astype(np.float32).astype(F16)
    got = oracle.matmul_nt_fp16u8(lhs, q, scales, c.block_size, c.beta, out0, zeros)
    fin = np.isfinite(want.astype(np.float32))
    assert np.array_equal(np.isfinite(got.astype(np.float32)), fin)
    diff = got.view(np.uint16).astype(np.int32)[fin] - want.view(np.uint16).astype(np.int32)[fin]
    assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 0.01


def test_quantize_roundtrip_and_layout():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((6, 256)) * 0.3).astype(F16)
    q, s = oracle.quantize(x, 64)
    assert q.shape == (6, 256) and s.shape == (6, 4)
    absmax = np.abs(x.astype(np.float32)).reshape(6, 4, 64).max(-1)
    assert np.array_equal(s.view(np.uint16), (absmax / np.float32(127.5)).astype(F16).view(np.uint16))
    back = oracle.dequantize(q, s, 64).astype(np.float32)
    step = np.repeat(s.astype(np.float32), 64, axis=1)
    assert np.all(np.abs(back - x.astype(np.float32)) <= step * 0.51 + 1e-3 * np.abs(x.astype(np.float32)))
    # an all-zero group quantises to code 0 with scale 0 (0/0 -> NaN -> 0)
    x[2, 64:128] = 0
    q, s = oracle.quantize(x, 64)
    assert s[2, 1] == 0 and np.all(q[2, 64:128] == 0)


def test_sgemm_against_numpy_all_layouts():
    rng = np.random.default_rng(6)
    m, k, n = 9, 130, 70
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    for aa in (a, np.asfortranarray(a)):
        for bb in (b, np.asfortranarray(b)):
            got = oracle.sgemm(aa, bb)
            assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    got = oracle.sgemm(a, b, c0.copy(), alpha=0.5, beta=2.0)
    assert np.allclose(got, 0.5 * want + 2.0 * c0, rtol=1e-4, atol=1e-4)
    big = rng.standard_normal((64, k)).astype(np.float32)
    assert np.allclose(oracle.sgemm(big, b), big.astype(np.float64) @ b, rtol=1e-4, atol=1e-4)


# ------------------------------------------------ golden vectors (reference)
def _gold(name):
    p = GOLD / name
    if not p.exists():
        pytest.skip(f"{name} not generated yet (tests/golden/make_golden.py needs a GPU)")
    return np.load(p)


@pytest.mark.parametrize("c", cases.matmul_cases(), ids=lambda c: c.name)
def test_faithful_oracle_matches_reference_kernels(c):
    """orc_matmul_f16_ref against matmul_f16 and matmul_f16_fast run on a B200."""
    g = _gold("reference_matmul_f16.npz")
    out0, lhs, rhs, bias = c.inputs()
    assert bytes(g[c.name + "/digest"]).decode() == cases.digest(out0, lhs, rhs, bias), "input generator drifted"
    got = _run_oracle(c, ideal=False)
    for kern in ("matmul_f16", "matmul_f16_fast"):
        ref = g[f"{c.name}/{kern}"]
        if c.exact_vs_reference:
            assert np.array_equal(got.view(np.uint16), ref.view(np.uint16)), kern
        else:  # tanhf / expf differ by an ulp between libm and the device
            d = got.view(np.uint16).astype(np.int32) - ref.view(np.uint16).astype(np.int32)
            assert np.abs(d).max() <= 2 and (d != 0).mean() < 0.02, kern


@pytest.mark.parametrize("c", [c for c in cases.u8_cases() if not c.zeros], ids=lambda c: c.name)
def test_u8_oracle_matches_reference_kernels(c):
    g = _gold("reference_u8.npz")
    out0, lhs, q, scales, _ = c.inputs()
    assert bytes(g[c.name + "/digest"]).decode() == cases.digest(out0, lhs, q, scales)
    # dequantize_absmax_uint8: bit-exact
    assert np.array_equal(oracle.dequantize(q, scales, c.block_size).view(np.uint16),
                          g[c.name + "/dequantize"].view(np.uint16))
    # matmul_nt_fp16u8: the faithful restatement, bit-exact up to fma contraction in double
    faithful = oracle.matmul_nt_fp16u8(lhs, q, scales, c.block_size, c.beta, out0, faithful=True)
    ref = g[c.name + "/matmul_nt_fp16u8"]
    fin = np.isfinite(ref.astype(np.float32))
    d = faithful.view(np.uint16).astype(np.int32)[fin] - ref.view(np.uint16).astype(np.int32)[fin]
    assert np.abs(d).max() <= 1 and (d != 0).mean() < 0.005
    # the WMMA kernel (tensor cores) against the ideal form: north-star tolerance 1e-2
    key = c.name + "/wmma_fp16u8"
    if key in g:
        ideal = oracle.matmul_nt_fp16u8(lhs, q, scales, c.block_size, c.beta, out0)
        assert oracle.max_rel_err(g[key], ideal) <= 1e-2


def test_quantizer_and_nt_oracles_match_reference_kernels():
    g = _gold("reference_quantize.npz")
    for name, bs in (("q_128", 128), ("q_32", 32), ("q_256", 256)):
        q, s = oracle.quantize(g[name + "/x"], bs)
        assert np.array_equal(s.view(np.uint16), g[name + "/scales"].view(np.uint16)), name
        assert np.array_equal(q, g[name + "/q"]), name
    for name in ("nt_128x64x64", "nt_128x64x64_beta", "nt_16x128x256", "nt_16x128x256_beta"):
        want = oracle.matmul_nt_f16(g[name + "/lhs"], g[name + "/rhs"], float(g[name + "/beta"]), g[name + "/out0"])
        assert oracle.max_rel_err(g[name + "/out"], want) <= 1e-2, name


@pytest.mark.parametrize("name", list(cases.rowop_cases()), ids=list(cases.rowop_cases()))
def test_rowop_oracle_matches_reference_kernels(name):
    """orc_rms_norm / orc_softmax_rows / orc_rotary / orc_elementwise_binary_2d_f16 against
    the reference's normalize.cu, rotary.cu and elementwise.cu kernels run on a B200: equal
    to one unit in the last place (libm here, device intrinsics there), Add bit-exact."""
    g = _gold("reference_rowops.npz")
    c = cases.rowop_cases()[name]
    ins = [c[k] for k in ("x", "w", "left", "right") if k in c]
    assert bytes(g[name + "/digest"]).decode() == cases.digest(*ins), "input generator drifted"
    if c["kind"] == "rms":
        got = oracle.rms_norm(c["x"], c["w"], c["eps"])
    elif c["kind"] == "softmax":
        got = oracle.softmax_rows(c["x"], temp=c["temp"])
    elif c["kind"] == "rotary":
        got = oracle.rotary(c["x"], c["n_heads"], c["pos_offset"], c["theta"])
    else:
        got = oracle.elementwise_binary(c["left"], c["right"], c["op"])
    ref = g[name + "/out"]
    same = got.view(np.uint16) == ref.view(np.uint16)
    d = np.abs(got.astype(np.float32) - ref.astype(np.float32))
    ulp = np.spacing(np.abs(ref).astype(np.float16)).astype(np.float32)
    ok = same | (d <= ulp)
    assert ok.all()
    if c["kind"] == "binary" and c["op"] == 1:
        assert same.all()
    else:
        assert (~same).mean() < 0.02


def test_decode_attention_oracle_against_numpy():
    """orc_decode_attention against a float64 numpy softmax attention (tolerance: the fp16
    rounding points of the chain)."""
    rng = np.random.default_rng(9)
    B, H, hd, S, pos = 2, 3, 32, 24, 17
    q = rng.standard_normal((B, H * hd)).astype(np.float16)
    kc = rng.standard_normal((B, S, H * hd)).astype(np.float16)
    vc = rng.standard_normal((B, S, H * hd)).astype(np.float16)
    got = oracle.decode_attention(q, kc, vc, H, pos, 1 / np.sqrt(hd)).astype(np.float64)
    qh = q.astype(np.float64).reshape(B, H, hd)
    kh = kc.astype(np.float64).reshape(B, S, H, hd)[:, :pos + 1]
    vh = vc.astype(np.float64).reshape(B, S, H, hd)[:, :pos + 1]
    sc = np.einsum("bhd,bthd->bht", qh, kh) / np.sqrt(hd)
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bht,bthd->bhd", p, vh).reshape(B, H * hd)
    assert np.abs(got - want).max() / np.abs(want).max() < 5e-3


def test_layer_norm_oracle_against_float64():
    """The layer_norm restatement (normalize.cu:60-145) against the formula in float64: the
    fp32 reductions cost at most one fp16 step on the output."""
    rng = np.random.default_rng(12)
    x = (rng.standard_normal((6, 1024)) * 2 + 0.3).astype(np.float16)
    w = rng.uniform(0.5, 1.5, 1024).astype(np.float16)
    b = rng.uniform(-0.5, 0.5, 1024).astype(np.float16)
    got = oracle.layer_norm(x, w, b, 1e-5).astype(np.float64)
    xf = x.astype(np.float64)
    mean = xf.mean(-1, keepdims=True)
    var = ((xf - mean) ** 2).mean(-1, keepdims=True)
    want = (xf - mean) / np.sqrt(var + 1e-5) * w.astype(np.float64) + b.astype(np.float64)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 0.25)) < 2e-3
