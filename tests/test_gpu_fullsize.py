"""One full-size layer of each model workload against an fp32 PyTorch restatement on the GPU:
LLaMA-7B dimensions (hidden 4096, 32 heads x 128, FFN 11008, KV cache) and CLIP ViT-L/14
dimensions (hidden 1024, 16 heads x 64, MLP 4096, 257 tokens, scores at the reference's
natural pitch of 257 elements as well as the padded 264).  The toy-size harness tests cover
the control flow; these cover the real shapes (odd sequence length, unaligned pitch, the
dispatcher's choices at D = 4096 / F = 11008)."""
import pytest
import torch

from test_clip_harness import ref_forward as clip_ref
from test_llama_harness import ref_forward as llama_ref

pytestmark = pytest.mark.gpu


def test_llama_7b_layer_prefill_and_decode(kernels):
    from adrastea_b200.llama import LlamaShape, LlamaU8
    torch.manual_seed(1)
    shape = LlamaShape(dim=4096, n_heads=32, ffn=11008, n_layers=1, vocab=32000, block=128)
    B, S0, steps = 1, 64, 2
    model = LlamaU8(kernels, shape, max_batch=B, max_seq=S0 + steps, seed=5)
    model.embed.mul_(0.5)
    # the seeded scales ~U(0.001, 0.01) give weights of std 0.4, which at these widths overflow
    # fp16 activations after one FFN; a tenth of that keeps every tensor finite
    for ly in model.layers:
        for lin in (ly.wqkv, ly.wo, ly.wgu, ly.down):  # q/k/v and gate/up are views of these
            lin.w.scales.mul_(0.1)
    model.lm_head.scales.mul_(0.1)
    toks = torch.randint(0, shape.vocab, (B, S0), device="cuda")
    model.prefill(toks)
    hist = toks
    want = llama_ref(model, kernels, hist)
    assert torch.isfinite(want).all() and torch.isfinite(model.logits).all()
    rel = ((model.logits.float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert rel < 3e-2, rel
    for _ in range(steps):
        hist = torch.cat([hist, model.tokens[:, None]], dim=1)
        model.decode_step()
        want = llama_ref(model, kernels, hist)
        rel = ((model.logits.float() - want.float()).abs().max() / want.float().abs().max()).item()
        assert rel < 3e-2, rel
    kernels.device_status()


@pytest.mark.parametrize("pitch", [257, 264])
def test_clip_l14_block(kernels, pitch):
    from adrastea_b200.clip import ClipVisionShape, ClipVisionU
    shape = ClipVisionShape(hidden=1024, heads=16, mlp=4096, layers=1, patch=14, image=224)
    assert shape.tokens == 257
    model = ClipVisionU(kernels, shape, batch=2, seed=2, score_pitch=pitch)
    for blk in model.blocks:  # larger weights than N(0, 0.02^2) so that every term matters
        for lin in blk.values():
            lin.w.mul_(2.0)
    px = torch.randn((2, 3, 224, 224), device="cuda").half()
    got = model.forward(px).clone()
    kernels.device_status()
    want = clip_ref(model, px)
    rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert rel < 2e-2, rel
