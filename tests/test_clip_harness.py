"""The CLIP image-encoder harness (adrastea_b200/clip.py) at toy dimensions against a plain
PyTorch fp32 restatement with the same glue and the same fp16 rounding points."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_forward(model, pixels):
    sh, B = model.shape, model.B
    S, H, d = sh.tokens, sh.heads, sh.hidden
    hd = d // H
    ln = lambda x: torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), eps=sh.eps).half()
    lin = lambda x, l: x.float() @ l.w.float().t()
    quick_gelu = lambda t: t * torch.sigmoid(1.702 * t)
    emb = torch.nn.functional.conv2d(pixels, model.patch_w, stride=sh.patch).flatten(2).transpose(1, 2)
    x = torch.cat([model.cls.expand(B, 1, d), emb], dim=1) + model.pos
    h = ln(x).reshape(B * S, d)
    for blk in model.blocks:
        n1 = ln(h)
        q, k, v = [(lin(n1, blk[n]).half().float() + blk[n].b.float()).half() for n in ("q", "k", "v")]
        hv = lambda t: t.view(B, S, H, hd).permute(0, 2, 1, 3).float()
        sc = ((hv(q) @ hv(k).transpose(-1, -2)).half() * torch.tensor(1 / math.sqrt(hd)).half())
        p = torch.softmax(sc.float(), -1).half().float()
        att = (p @ hv(v)).half().permute(0, 2, 1, 3).reshape(B * S, d)
        h = (lin(att, blk["o"]).half().float() + blk["o"].b.float() + h.float()).half()
        n2 = ln(h)
        mid = quick_gelu(lin(n2, blk["fc1"]).half().float() + blk["fc1"].b.float()).half()
        h = (lin(mid, blk["fc2"]).half().float() + blk["fc2"].b.float() + h.float()).half()
    return h.view(B, S, d)


def test_clip_encoder_matches_pytorch(kernels):
    from adrastea_b200 import Kernel
    from adrastea_b200.clip import ClipVisionShape, ClipVisionU
    shape = ClipVisionShape(hidden=128, heads=2, mlp=256, layers=2, patch=14, image=56)
    assert shape.tokens == 17
    model = ClipVisionU(kernels, shape, batch=3, seed=1)
    for blk in model.blocks:  # larger weights than N(0, 0.02^2) so that every term matters
        for lin in blk.values():
            lin.w.mul_(4.0)
    px = torch.randn((3, 3, 56, 56), device="cuda").half()
    got = model.forward(px).clone()
    assert kernels.last_kernel() == Kernel.F16Tc
    kernels.device_status()
    want = ref_forward(model, px)
    rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert rel < 2e-2, rel
