"""The LLaMA-shape harness (adrastea_b200/llama.py) at toy dimensions against a plain
PyTorch fp32 restatement that uses the same glue formulas and dequantised weights."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_forward(model, kernels, tokens_hist):
    """Full-prefix recomputation (what the reference does, llama.rs:426-427) in fp32 matmuls
    on the dequantised weights; returns the logits of the last position per sequence."""
    from adrastea_b200.llama import rms_norm, rotary
    sh = model.shape
    B, S = tokens_hist.shape
    H, hd = sh.n_heads, sh.head_dim

    def deq(w):
        # (q - 127.5) * scale in fp32, not rounded to fp16: the arithmetic of
        # matmul_nt_fp16u8.cu:13-23, which the decode kernels follow
        return (w.q.float() - 127.5) * w.scales.float().repeat_interleave(w.block, dim=1)

    def lin(x, w):
        return (x.float() @ deq(w).t()).half()

    h = model.embed[tokens_hist.reshape(-1)].clone()
    pos = torch.arange(S, device=h.device).repeat(B)
    for ly in model.layers:
        x = rms_norm(h, ly.attn_norm, sh.norm_eps)
        q = rotary(lin(x, ly.wq.w), pos, H, sh.theta).view(B, S, H, hd).permute(0, 2, 1, 3).float()
        k = rotary(lin(x, ly.wk.w), pos, H, sh.theta).view(B, S, H, hd).permute(0, 2, 1, 3).float()
        v = lin(x, ly.wv.w).view(B, S, H, hd).permute(0, 2, 1, 3).float()
        sc = ((q @ k.transpose(-1, -2)).half() * torch.tensor(1.0 / math.sqrt(hd)).half()).float()
        sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=h.device), 1), float("-inf"))
        p = torch.softmax(sc, -1).half().float()
        att = (p @ v).half().permute(0, 2, 1, 3).reshape(B * S, H * hd)
        h = (lin(att, ly.wo.w) + h)
        x = rms_norm(h, ly.ffn_norm, sh.norm_eps)
        g = torch.nn.functional.silu(lin(x, ly.gate.w).float()).half() * lin(x, ly.up.w)
        h = (lin(g, ly.down.w) + h)
    last = rms_norm(h.view(B, S, -1)[:, -1].contiguous(), model.out_norm, sh.norm_eps)
    return lin(last, model.lm_head)


@pytest.mark.parametrize("graph,expand", [(False, False), (True, False), (False, True)])
def test_prefill_and_decode_match_full_recomputation(kernels, graph, expand):
    from adrastea_b200.llama import LlamaShape, LlamaU8
    torch.manual_seed(0)
    shape = LlamaShape(dim=256, n_heads=4, ffn=512, n_layers=2, vocab=512, block=64)
    B, S0, steps = 2, 12, 3
    model = LlamaU8(kernels, shape, max_batch=B, max_seq=S0 + steps, seed=3)
    if expand:  # prefill through the fp16 expansion of the weights + tensor-core GEMM
        model.PREFILL_DEQUANT_ROWS = 8
    model.embed.mul_(0.5)
    toks = torch.randint(0, shape.vocab, (B, S0), device="cuda")
    model.prefill(toks)
    hist = toks
    want = ref_forward(model, kernels, hist)
    assert torch.equal(model.tokens, torch.argmax(want.float(), -1))
    rel = ((model.logits.float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert rel < 3e-2, rel
    if graph:
        pos0, tok0 = model.pos.clone(), model.tokens.clone()
        model.capture()
        model.pos.copy_(pos0)
        model.tokens.copy_(tok0)
    for _ in range(steps):
        hist = torch.cat([hist, model.tokens[:, None]], dim=1)
        model.decode_step()
        want = ref_forward(model, kernels, hist)
        rel = ((model.logits.float() - want.float()).abs().max() / want.float().abs().max()).item()
        assert rel < 3e-2, rel
        assert torch.equal(model.next_tokens, torch.argmax(want.float(), -1))
    kernels.device_status()
