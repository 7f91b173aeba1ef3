"""The fused attention kernel (adr_attention_f16) against the reference's three-call chain run
through this library (matmul Scale [+ Causal] -> softmax_rows -> matmul) and against an fp32
PyTorch restatement with the chain's rounding points.  Tolerance 1e-2 (max error relative to
the largest output), the bar of the fp16 tensor-core path."""
import math

import pytest
import torch

from adrastea_b200 import MatmulMask, MatmulOptions, MatmulStore, TensorLayout, TensorView

pytestmark = pytest.mark.gpu


def torch_ref(q, k, v, scale, causal):
    """q, k, v: [..., S, hd] fp16 -> fp32 math with the chain's fp16 rounding points."""
    sc = (q.float() @ k.float().transpose(-1, -2)).half() * torch.tensor(scale).half()
    if causal:
        sq, sk = sc.shape[-2:]
        sc = sc.masked_fill(torch.triu(torch.ones(sq, sk, dtype=torch.bool, device=q.device), 1), float("-inf"))
    p = torch.softmax(sc.float(), -1).half().float()
    return (p @ v.float()).half()


def rel(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.mark.parametrize("hd,H,sq,sk,causal", [
    (64, 3, 257, 257, False),     # CLIP: odd length, three key blocks, the last of one key
    (64, 2, 128, 128, False),
    (64, 2, 40, 300, False),      # fewer queries than keys
    (128, 4, 512, 512, True),     # LLaMA prefill
    (128, 2, 130, 130, True),     # ragged causal
    (128, 1, 17, 17, True),
    (64, 2, 200, 200, True),
    (128, 2, 1, 96, False),       # a single query row
    (64, 2, 258, 258, True),      # two rows past two query tiles: the row kernel, causal
    (128, 2, 130, 200, False),    # two rows past a tile, more keys than queries
    (64, 2, 260, 260, True),      # four rows past two tiles: a third tile
    (128, 1, 129, 129, True),     # one row past a tile, head_dim 128
    (64, 3, 129, 129, False),     # one row past a tile, head_dim 64
])
def test_attention_contiguous_heads(kernels, hd, H, sq, sk, causal):
    torch.manual_seed(hd + sq + sk)
    q = torch.randn((H, sq, hd), device="cuda").half()
    k = torch.randn((H, sk, hd), device="cuda").half()
    v = torch.randn((H, sk, hd), device="cuda").half()
    out = torch.full((H, sq, hd), float("nan"), dtype=torch.float16, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    mask = MatmulMask.Causal if causal else MatmulMask.None_
    kernels.attention_f16(TensorView.of(out), TensorView.of(q), TensorView.of(k), TensorView.of(v), scale, mask)
    kernels.device_status()
    want = torch_ref(q, k, v, scale, causal)
    assert torch.isfinite(out).all()
    assert rel(out, want) < 1e-2, rel(out, want)
    # the three-call chain through this library
    spad = (sk + 7) // 8 * 8
    scores = torch.zeros((H, sq, spad), dtype=torch.float16, device="cuda")
    sv = TensorView(scores, TensorLayout.new((H, sq, sk), (sq * spad, spad, 1)))
    chain = torch.zeros_like(out)
    opts = MatmulOptions.new().store(MatmulStore.Scale(scale))
    if causal:
        opts = opts.mask(MatmulMask.Causal)
    kernels.matmul_f16(sv, TensorView.of(q), TensorView.of(k).permute([0, 2, 1]), opts)
    kernels.softmax_rows_inplace(sv, 1.0)
    kernels.matmul_f16(TensorView.of(chain), sv, TensorView.of(v))
    kernels.device_status()
    assert rel(out, chain) < 1e-2, rel(out, chain)
    # deterministic
    out2 = torch.zeros_like(out)
    kernels.attention_f16(TensorView.of(out2), TensorView.of(q), TensorView.of(k), TensorView.of(v), scale, mask)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_attention_reference_views(kernels):
    """The reference's own layouts: q, k, v and out are [B, S, H, hd] activations viewed as
    [B, H, S, hd] (clip.rs:368-388) - two batch dimensions, strided rows, strided output."""
    torch.manual_seed(3)
    B, S, H, hd = 3, 257, 16, 64
    d = H * hd
    qkv = [torch.randn((B, S, d), device="cuda").half() for _ in range(3)]
    out = torch.zeros((B, S, d), dtype=torch.float16, device="cuda")
    lay = TensorLayout.new((B, H, S, hd), (S * d, hd, d, 1))
    views = [TensorView(t, lay) for t in qkv]
    scale = 1.0 / math.sqrt(hd)
    kernels.attention_f16(TensorView(out, lay), views[0], views[1], views[2], scale)
    kernels.device_status()
    hv = lambda t: t.view(B, S, H, hd).permute(0, 2, 1, 3)
    want = torch_ref(hv(qkv[0]), hv(qkv[1]), hv(qkv[2]), scale, False).permute(0, 2, 1, 3).reshape(B, S, d)
    assert rel(out, want) < 1e-2, rel(out, want)


def test_attention_rejects_what_it_cannot_take(kernels):
    from adrastea_b200 import AdrError
    q = torch.zeros((2, 16, 80), dtype=torch.float16, device="cuda")
    with pytest.raises(AdrError) as e:  # head_dim 80
        kernels.attention_f16(TensorView.of(q), TensorView.of(q), TensorView.of(q), TensorView.of(q), 1.0)
    assert e.value.code == 2
    base = torch.zeros((16 * 68,), dtype=torch.float16, device="cuda")
    odd = TensorView(base, TensorLayout.new((16, 64), (68, 1)))  # row pitch 136 bytes: not 16-byte rows
    with pytest.raises(AdrError) as e:
        kernels.attention_f16(odd, odd, odd, odd, 1.0)
    assert e.value.code == 2
