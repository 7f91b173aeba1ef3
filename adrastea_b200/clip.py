"""CLIP ViT image-encoder harness: the second caller of the matmul path.

Restates the call sequence of the reference's `ClipAttention::forward`,
`ClipMLP::forward` and `ClipVisionTransformer` (adrastea_models/src/clip.rs:342-486,
754-817) around this library's kernels: layer norms through `adr_layer_norm`, q/k/v
projections with `BetaBias(0.0)`, the attention chain (scores `q.k^T` with
`Scale(1/sqrt(hd))`, row softmax, probabilities . v) through the fused
`adr_attention_f16` (or, with `fused_attention=False`, as the reference's three calls),
the output projection and fc2 with `BetaBias(1.0)` (the residual), fc1 with
`QuickGeluBias`.  The patch embedding is harness glue done with a PyTorch op.

The reference encodes one image at a time ([257, 1024]); the CLIP workload here is a
batch of 64, which this harness runs as [B*257, 1024] linears and B*heads batched
attention products.  Activations are kept token-major so that the per-head operands are
strided views (no copies); the score tensor has a row pitch that is a multiple of 8
elements (264 for 257 tokens) so that both attention products take the tensor-core path
(a 514-byte pitch cannot be described to TMA).  Weights are seeded N(0, 0.02^2).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .kernels import GpuKernels, MatmulOptions, MatmulStore
from .tensor import TensorLayout, TensorView


@dataclass(frozen=True)
class ClipVisionShape:
    hidden: int = 1024
    heads: int = 16
    mlp: int = 4096
    layers: int = 24
    patch: int = 14
    image: int = 224
    eps: float = 1e-5

    @property
    def tokens(self) -> int:
        return (self.image // self.patch) ** 2 + 1


VIT_L_14 = ClipVisionShape()


class _Linear:
    def __init__(self, n, k, gen, device):
        self.w = (torch.randn((n, k), device=device, generator=gen) * 0.02).half()
        self.b = (torch.randn((n,), device=device, generator=gen) * 0.02).half()


class ClipVisionU:
    def __init__(self, kernels: GpuKernels, shape: ClipVisionShape = VIT_L_14, batch: int = 64,
                 seed: int = 0, device="cuda", score_pitch: int | None = None,
                 fused_attention: bool = True):
        self.k, self.shape, self.B = kernels, shape, batch
        self.fused_attention = fused_attention and (shape.hidden // shape.heads) in (64, 128)
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device).manual_seed(4242 + seed)
        d, f = shape.hidden, shape.mlp
        L = lambda n, k: _Linear(n, k, gen, self.device)
        self.blocks = [dict(q=L(d, d), k=L(d, d), v=L(d, d), o=L(d, d), fc1=L(f, d), fc2=L(d, f))
                       for _ in range(shape.layers)]
        # q, k and v of a block share their input: their weights and biases are kept side by side
        # ([3d, d] and [3d]; the per-projection tensors are views of them), so that with fused
        # attention the three products run as one GEMM (1548 tiles instead of 3 x 516: the last,
        # partly filled wave of tiles is paid once) whose [S*B, 3d] output the attention kernel
        # reads through strided views.  Each output element is the same dot product as before.
        self.qkv_lin = []
        for blk in self.blocks:
            fused = _Linear.__new__(_Linear)
            fused.w = torch.cat([blk[n].w for n in "qkv"], dim=0)
            fused.b = torch.cat([blk[n].b for n in "qkv"], dim=0)
            for i, n in enumerate("qkv"):
                blk[n].w = fused.w[i * d:(i + 1) * d]
                blk[n].b = fused.b[i * d:(i + 1) * d]
            self.qkv_lin.append(fused)
        self.patch_w = (torch.randn((d, 3, shape.patch, shape.patch), device=self.device, generator=gen) * 0.02).half()
        self.cls = (torch.randn((d,), device=self.device, generator=gen) * 0.02).half()
        self.pos = (torch.randn((shape.tokens, d), device=self.device, generator=gen) * 0.02).half()
        S, H, hd, B = shape.tokens, shape.heads, shape.hidden // shape.heads, batch
        # distance between score rows in elements: padded to a multiple of 8 by default;
        # `score_pitch=S` gives the reference's own contiguous [heads, S, S] scores (clip.rs:374-388)
        self.Sp = score_pitch or (S + 7) // 8 * 8
        assert self.Sp >= S
        f16 = dict(dtype=torch.float16, device=self.device)
        z = lambda *s: torch.zeros(s, **f16)
        # activations are token-major, [S*B, d] (row = token * B + image): the [B*H, S, hd]
        # operand of the batched attention products is then a plain strided view
        # (z = image*H + head -> stride hd, token -> stride B*d) and no re-layout is needed
        self.h, self.att = z(S * B, d), z(S * B, d)
        self.fused_qkv = self.fused_attention
        if self.fused_qkv:
            self.qkv = z(S * B, 3 * d)
            self.q, self.kx, self.v = (self.qkv[:, i * d:(i + 1) * d] for i in range(3))
        else:
            self.q, self.kx, self.v = (z(S * B, d) for _ in range(3))
        # raw scores keep -inf in the pad columns (the GEMM writes only the first S of each
        # row), so a softmax over whole padded rows leaves exact zeros there
        self.scores = torch.full((B * H, S, self.Sp), float("-inf"), **f16)
        self.probs = z(B * H, S, self.Sp)
        self.mid = z(S * B, f)
        self.n1 = z(S * B, d)
        # layer-norm scale and shift (the seeded workload uses gamma = 1, beta = 0)
        self.ln_w = torch.ones(d, **f16)
        self.ln_b = torch.zeros(d, **f16)
        if self.fused_qkv:
            # [image, head, token, hd] views: rows of the fused projection are 3d apart
            pitch = self.q.stride(0)
            heads_in = TensorLayout.new((B, H, S, hd), (pitch, hd, B * pitch, 1))
            heads = TensorLayout.new((B, H, S, hd), (d, hd, B * d, 1))
        else:
            heads_in = heads = TensorLayout.new((B * H, S, hd), (hd, B * d, 1))
        self.qv, self.kv, self.vv = (TensorView(t, heads_in) for t in (self.q, self.kx, self.v))
        self.ov = TensorView(self.att, heads)
        sl = TensorLayout.new((B * H, S, S), (S * self.Sp, self.Sp, 1))
        self.sv, self.pv = TensorView(self.scores, sl), TensorView(self.probs, sl)

    def _linear(self, out, x, lin, store):
        self.k.matmul_f16(TensorView.of(out), TensorView.of(x), TensorView.of(lin.w).permute([1, 0]),
                          MatmulOptions.new().store(store))

    def _ln(self, out, x):
        """layer_norm (clip.rs:431-442 / kernels.rs:652-678) of the rows of x into out."""
        self.k.layer_norm(TensorView.of(out), TensorView.of(x), TensorView.of(self.ln_w),
                          TensorView.of(self.ln_b), self.shape.eps)
        return out

    def _attention(self, hd):
        scale = 1.0 / math.sqrt(hd)
        if self.fused_attention:
            self.k.attention_f16(self.ov, self.qv, self.kv, self.vv, scale)
            return
        self.k.matmul_f16(self.sv, self.qv, self.kv.permute([0, 2, 1]),
                          MatmulOptions.new().store(MatmulStore.Scale(scale)))
        if self.Sp == self.shape.tokens:
            self.k.softmax_rows_inplace(self.sv, 1.0)
            probs = self.sv
        else:
            # padded rows: the pad columns hold -inf, a softmax over whole rows leaves zeros there
            torch.softmax(self.scores, dim=-1, out=self.probs)
            probs = self.pv
        self.k.matmul_f16(self.ov, probs, self.vv)

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels: [B, 3, image, image] fp16 -> final hidden state [B, tokens, hidden]."""
        sh, B = self.shape, self.B
        S, H, d = sh.tokens, sh.heads, sh.hidden
        hd = d // H
        emb = torch.nn.functional.conv2d(pixels, self.patch_w, stride=sh.patch)  # clip.rs:767-779
        emb = emb.flatten(2).permute(2, 0, 1)                                     # [256, B, d]
        x = torch.cat([self.cls.expand(1, B, d), emb], dim=0) + self.pos[:, None, :]
        self._ln(self.h, x.reshape(S * B, d).contiguous())                          # pre-layernorm
        for li, blk in enumerate(self.blocks):
            n1 = self._ln(self.n1, self.h)
            if self.fused_qkv:
                fused = self.qkv_lin[li]
                self._linear(self.qkv, n1, fused, MatmulStore.BetaBias(0.0, TensorView.of(fused.b)))
            else:
                self._linear(self.q, n1, blk["q"], MatmulStore.BetaBias(0.0, TensorView.of(blk["q"].b)))
                self._linear(self.kx, n1, blk["k"], MatmulStore.BetaBias(0.0, TensorView.of(blk["k"].b)))
                self._linear(self.v, n1, blk["v"], MatmulStore.BetaBias(0.0, TensorView.of(blk["v"].b)))
            self._attention(hd)
            self._linear(self.h, self.att, blk["o"], MatmulStore.BetaBias(1.0, TensorView.of(blk["o"].b)))
            n2 = self._ln(self.n1, self.h)
            self._linear(self.mid, n2, blk["fc1"], MatmulStore.QuickGeluBias(TensorView.of(blk["fc1"].b)))
            self._linear(self.h, self.mid, blk["fc2"], MatmulStore.BetaBias(1.0, TensorView.of(blk["fc2"].b)))
        return self.h.view(S, B, d).transpose(0, 1)

    def flops(self) -> float:
        sh, B = self.shape, self.B
        S, d, f, H = sh.tokens, sh.hidden, sh.mlp, sh.heads
        per_layer = 2 * B * S * (4 * d * d + 2 * d * f) + 4 * B * H * S * S * (d // H)
        return float(sh.layers * per_layer)


def main():
    """python -m adrastea_b200.clip [--batch 64]: one JSON line with the forward time."""
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    kern = GpuKernels(0)
    model = ClipVisionU(kern, VIT_L_14, args.batch)
    px = torch.randn((args.batch, 3, 224, 224), device="cuda").half()
    model.forward(px)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        model.forward(px)
    e1.record()
    torch.cuda.synchronize()
    kern.device_status()
    ms = e0.elapsed_time(e1) / args.iters
    print(json.dumps({"model": "CLIP ViT-L/14 image encoder, fp16", "batch": args.batch,
                      "ms_per_forward": ms, "images_per_s": args.batch / (ms * 1e-3),
                      "matmul_tflops": model.flops() / (ms * 1e-3) / 1e12}))


if __name__ == "__main__":
    main()
