"""LLaMA-shape decoder harness with u8 weights: the caller of the matmul path.

Restates the call sequence of the reference's `LlamaContext::process_layer` /
`decode` (adrastea_models/src/llama.rs:456-589) around this library's kernels:
every linear layer goes through `adr_matmul_nt_fp16u8`, prefill attention through
`adr_matmul_f16` with the reference's views (q.k^T with `Scale` and the causal
mask, `softmax_rows`, probabilities . v into a strided output view), and
`rms_norm`, `rotary` and `SiluMul` through the library's restatements of the
reference kernels (normalize.cu:7-58, rotary.cu:4-29, elementwise.cu:28-33).
Embedding lookup and argmax are PyTorch ops.

Differences from the reference, which re-runs the whole prefix for every token
(llama.rs:426-427): a KV cache ([B, S, heads*head_dim] per layer) with the two
decode kernels that serve it (`decode_rope_append`, `decode_attention`), batches of
sequences, q/k/v and gate/up stored as one matrix each (one GEMV instead of three
or two; the separate matrices remain available as row slices), tensor parallelism
(adrastea_b200/tp.py) and CUDA-graph capture of the decode step are harness glue
that the LLaMA-7B and 65B-shape decode workloads need.  Weights are seeded random u8 codes with
the config-2 distributions; there are no checkpoints in this environment.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .kernels import BinaryOp, GpuKernels, MatmulMask, MatmulOptions, MatmulStore
from .tensor import TensorLayout, TensorView
from .tp import ColumnParallelU8Linear, RowParallelU8Linear, TPContext, U8Weight


@dataclass(frozen=True)
class LlamaShape:
    dim: int
    n_heads: int
    ffn: int
    n_layers: int
    vocab: int = 32000
    block: int = 128
    norm_eps: float = 1e-5
    theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


LLAMA_7B = LlamaShape(4096, 32, 11008, 32)
LLAMA_65B = LlamaShape(8192, 64, 22016, 80, block=64)  # block 64: 22016/8 = 2752 = 43 * 64


def _rand_u8(n, k, block, gen, device) -> U8Weight:
    q = torch.randint(0, 256, (n, k), dtype=torch.uint8, device=device, generator=gen)
    s = (torch.rand((n, k // block), device=device, generator=gen) * 0.009 + 0.001).half()
    return U8Weight(q, s, block)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """normalize.cu:7-58: weights * fp16(x * rsqrt(mean(x^2) + eps)), statistics in fp32."""
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return w * (xf * inv).half()


def rotary(x: torch.Tensor, pos: torch.Tensor, n_heads: int, theta: float) -> torch.Tensor:
    """rotary.cu:4-29: interleaved pairs (2i, 2i+1) of every head rotated by
    pos / theta^(2i / head_dim).  x: [rows, n_heads*head_dim], pos: [rows] (int)."""
    rows, width = x.shape
    hd = width // n_heads
    c = torch.arange(0, hd, 2, device=x.device, dtype=torch.float32)
    # theta^(c/hd) as exp(c/hd * ln theta): no host scalar becomes a device tensor here, so the
    # function can run under CUDA-graph capture
    ang = pos.float()[:, None] / torch.exp(c / hd * math.log(theta))[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    xv = x.float().view(rows, n_heads, hd // 2, 2)
    re, im = xv[..., 0], xv[..., 1]
    out = torch.stack((re * cos - im * sin, re * sin + im * cos), dim=-1)
    return out.view(rows, width).half()


def _rows(w: U8Weight, lo: int, hi: int) -> U8Weight:
    """Rows [lo, hi) of a quantised matrix as a view (no copy)."""
    return U8Weight(w.q[lo:hi], w.scales[lo:hi], w.block, None if w.zeros is None else w.zeros[lo:hi])


class LlamaU8Layer:
    def __init__(self, kernels: GpuKernels, shape: LlamaShape, tp: TPContext, gen, device):
        t = tp.world
        d, f, bs = shape.dim, shape.ffn, shape.block
        assert d % t == 0 and f % t == 0 and shape.n_heads % t == 0
        dl, fl = d // t, f // t
        # shards are generated directly (seeded per rank); no full matrix is ever materialised.
        # q, k, v share one [3*dl, d] storage and gate, up one [2*fl, d] storage.
        col = lambda w: ColumnParallelU8Linear(kernels, w, tp, True)
        row = lambda n, k: RowParallelU8Linear(kernels, _rand_u8(n, k // t, bs, gen, device), tp, True)
        qkv = _rand_u8(3 * dl, d, bs, gen, device)
        self.wqkv = col(qkv)
        self.wq, self.wk, self.wv = (col(_rows(qkv, i * dl, (i + 1) * dl)) for i in range(3))
        self.wo = row(d, d)
        gu = _rand_u8(2 * fl, d, bs, gen, device)
        self.wgu = col(gu)
        self.gate, self.up = col(_rows(gu, 0, fl)), col(_rows(gu, fl, 2 * fl))
        self.down = row(d, f)
        self.attn_norm = torch.ones(d, dtype=torch.float16, device=device)
        self.ffn_norm = torch.ones(d, dtype=torch.float16, device=device)

    def linears(self):
        return (self.wq, self.wk, self.wv, self.wo, self.gate, self.up, self.down)

    def weight_bytes(self) -> int:
        return sum(l.w.nbytes() for l in self.linears())


class LlamaU8:
    """Decoder stack with a KV cache.  `tp.world` ranks each hold 1/world of every
    sharded matrix and of the heads; embeddings, norms and the output head are replicated."""

    def __init__(self, kernels: GpuKernels, shape: LlamaShape, tp: TPContext | None = None,
                 max_batch: int = 16, max_seq: int = 640, n_layers: int | None = None,
                 seed: int = 0, device: str | torch.device = "cuda"):
        self.k, self.shape = kernels, shape
        self.tp = tp or TPContext()
        self.device = torch.device(device)
        self.B, self.S = max_batch, (max_seq + 7) // 8 * 8  # score rows stay 16-byte aligned
        self.L = n_layers or shape.n_layers
        gen = torch.Generator(device=self.device).manual_seed(1000 * seed + self.tp.rank)
        self.layers = [LlamaU8Layer(kernels, shape, self.tp, gen, self.device) for _ in range(self.L)]
        rep = torch.Generator(device=self.device).manual_seed(777 + seed)  # same on every rank
        self.embed = (torch.randn((shape.vocab, shape.dim), device=self.device, generator=rep)).half()
        self.out_norm = torch.ones(shape.dim, dtype=torch.float16, device=self.device)
        self.lm_head = _rand_u8(shape.vocab, shape.dim, shape.block, rep, self.device)
        self.Hl = shape.n_heads // self.tp.world
        hd = shape.head_dim
        dl = self.Hl * hd
        f16 = dict(dtype=torch.float16, device=self.device)
        self.k_cache = torch.zeros((self.L, self.B, self.S, dl), **f16)
        self.v_cache = torch.zeros((self.L, self.B, self.S, dl), **f16)
        # decode-step buffers (fixed addresses, so the step can be captured in a CUDA graph)
        B, d, fl = self.B, shape.dim, shape.ffn // self.tp.world
        self.dl, self.fl = dl, fl
        self.h = torch.zeros((B, d), **f16)
        self.x = torch.zeros((B, d), **f16)
        self.qkv = torch.zeros((B, 3 * dl), **f16)
        self.att = torch.zeros((B, dl), **f16)
        self.gu = torch.zeros((B, 2 * fl), **f16)
        self.g = torch.zeros((B, fl), **f16)
        self.partial = torch.zeros((B, d), **f16)
        self.logits = torch.zeros((B, shape.vocab), **f16)
        self.pos = torch.zeros((1,), dtype=torch.int32, device=self.device)
        self.tokens = torch.zeros((B,), dtype=torch.int64, device=self.device)
        self.next_tokens = torch.zeros((B,), dtype=torch.int64, device=self.device)
        # prefill attention in one launch (adr_attention_f16) instead of the reference's
        # matmul(Scale, Causal) -> softmax_rows -> matmul chain per sequence
        self.fused_attention = hd in (64, 128) and dl % 8 == 0  # what adr_attention_f16 takes
        self._graph = None
        self._deq = None  # fp16 scratch for one expanded weight matrix (prefill)
        # rms_norm inside the decode GEMV (adr_rms_norm_matmul_nt_fp16u8).  Same bits, one launch
        # fewer per norm, but measured no faster (2.31 against 2.28 ms per step at batch 1, 4.49
        # against 4.30 at batch 16: every CTA normalises the rows for itself before its first MMA,
        # while the separate kernel overlaps the GEMV's prologue), so it is off by default.
        self.fuse_norm = False
        # gate/up products + SiluMul in one launch of the decode kernel
        # (adr_silu_mul_matmul_nt_fp16u8: same bits as the three kernels, one launch instead of two
        # and no [tokens, 2 * ffn] round trip); used for decode batches the kernel takes
        self.fuse_silu = True
        # q/k/v product + rotary + cache append (+ rms_norm with fuse_norm) in one launch of the
        # decode kernel (adr_qkv_rope_append_matmul_nt_fp16u8: same bits as the separate kernels).
        # One or two launches fewer per layer, but measured slower (2.18 -> 2.25 ms per step at
        # batch 1, 2.90 -> 3.25 at batch 4): the kernel's form with fused ops is slower than the
        # plain one by more than the small kernels cost when they overlap their neighbours under
        # programmatic dependent launch.  Off by default.
        self.fuse_rope = False

    # ------------------------------------------------------------------ sizes
    def weight_bytes_per_token(self) -> int:
        """u8 weights + scales this rank streams per decode step (all layers + output head)."""
        return sum(l.weight_bytes() for l in self.layers) + self.lm_head.nbytes()

    # ----------------------------------------------------------- decode step
    def _norm(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor):
        self.k.rms_norm(TensorView.of(out), TensorView.of(x), TensorView.of(w), self.shape.norm_eps)

    def _norm_linear(self, out: torch.Tensor, h: torch.Tensor, norm_w: torch.Tensor, w: U8Weight):
        """out = rms_norm(h) . deq(w)^T in one launch where the decode kernel takes the shape
        (same bits as the two kernels), else rms_norm into self.x followed by the product."""
        if self.fuse_norm:
            from .kernels import AdrError
            try:
                self.k.rms_norm_matmul_nt_fp16u8(out, h, norm_w, self.shape.norm_eps, w.q, w.scales,
                                                 w.block, 0.0, w.zeros)
                return
            except AdrError as e:
                if e.code != 2:  # anything but "shape not taken"
                    raise
        self._norm(self.x, h, norm_w)
        self.k.matmul_nt_fp16u8(out, self.x, w.q, w.scales, w.block, 0.0, w.zeros)

    def _norm_qkv_rope(self, ly, li: int) -> bool:
        """q (rotated) into self.qkv[:, :dl], k (rotated) and v into the caches of layer li, from
        rms_norm(self.h), in one launch; False if the decode kernel does not take the shape."""
        from .kernels import AdrError
        w = ly.wqkv.w
        src = self.h
        if not self.fuse_norm:
            self._norm(self.x, self.h, ly.attn_norm)
            src = self.x
        try:
            self.k.qkv_rope_append_matmul_nt_fp16u8(
                self.qkv[:, :self.dl], src, w.q, w.scales, w.block, self.Hl, self.k_cache[li],
                self.v_cache[li], self.pos, self.shape.theta,
                ly.attn_norm if self.fuse_norm else None, self.shape.norm_eps, w.zeros)
            return True
        except AdrError as e:
            if e.code != 2:  # anything but "shape not taken"
                raise
            return False

    def _norm_gate_up_silu(self, ly) -> bool:
        """self.g = SiluMul(gate, up) of rms_norm(self.h) in two launches (norm, fused product);
        False if the decode kernel does not take the shape."""
        from .kernels import AdrError
        w, fl = ly.wgu.w, self.fl
        self._norm(self.x, self.h, ly.ffn_norm)
        try:
            self.k.silu_mul_matmul_nt_fp16u8(
                self.g, self.x, w.q[:fl], w.scales[:fl], w.q[fl:], w.scales[fl:], w.block,
                w.zeros[:fl] if w.zeros is not None else None,
                w.zeros[fl:] if w.zeros is not None else None)
            return True
        except AdrError as e:
            if e.code != 2:  # anything but "shape not taken"
                raise
            return False

    def _silu_mul(self, out: torch.Tensor, gu: torch.Tensor):
        """out = SiluMul(gate, up), the two halves of the fused gate/up product."""
        fl = self.fl
        self.k.elementwise_binary_2d_f16(TensorView.of(out), TensorView.of(gu[:, :fl]),
                                         TensorView.of(gu[:, fl:]), BinaryOp.SiluMul)

    def _decode_step_body(self):
        sh, dl = self.shape, self.dl
        torch.index_select(self.embed, 0, self.tokens, out=self.h)
        qv, kv, vv = (TensorView.of(self.qkv[:, i * dl:(i + 1) * dl]) for i in range(3))
        scale = 1.0 / math.sqrt(sh.head_dim)
        for li, ly in enumerate(self.layers):
            if not (self.fuse_rope and self.h.shape[0] <= 4 and self._norm_qkv_rope(ly, li)):
                self._norm_linear(self.qkv, self.h, ly.attn_norm, ly.wqkv.w)
                self.k.decode_rope_append(qv, kv, vv, self.k_cache[li], self.v_cache[li], self.Hl,
                                          self.pos, sh.theta)
            self.k.decode_attention(TensorView.of(self.att), qv, self.k_cache[li], self.v_cache[li],
                                    self.Hl, self.pos, scale)
            ly.wo(self.h, self.att, self.partial, residual=True)       # store = Add, llama.rs:555-560
            # (from five tokens on the cluster kernel + the elementwise kernel are as fast or faster)
            if not (self.fuse_silu and self.h.shape[0] <= 4 and self._norm_gate_up_silu(ly)):
                self._norm_linear(self.gu, self.h, ly.ffn_norm, ly.wgu.w)
                self._silu_mul(self.g, self.gu)
            ly.down(self.h, self.g, self.partial, residual=True)       # llama.rs:584-589
        self._norm_linear(self.logits, self.h, self.out_norm, self.lm_head)
        torch.argmax(self.logits, dim=-1, out=self.next_tokens)

    def capture(self):
        """Capture one decode step (fixed shapes, position and tokens in device memory)."""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._decode_step_body()  # warm-up outside capture (allocator, descriptor cache)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._decode_step_body()

    def decode_step(self):
        """Consumes self.tokens at position self.pos, leaves the argmax in self.next_tokens."""
        if self._graph is not None:
            self._graph.replay()
        else:
            self._decode_step_body()
        self.tokens.copy_(self.next_tokens)
        self.pos.add_(1)

    # ------------------------------------------------------------- prefill
    # ------------------------------------------------------------- prefill
    PREFILL_DEQUANT_ROWS = 4096

    def _prefill_linear(self, lin, out: torch.Tensor, x: torch.Tensor, part: torch.Tensor | None = None,
                        residual: bool = False):
        """A linear layer over many rows.  Up to PREFILL_DEQUANT_ROWS rows go through
        `adr_matmul_nt_fp16u8` (the kernel that dequantises into tensor memory).  From there on
        the u8 matrix is first expanded to fp16 in a scratch buffer (`adr_dequantize_absmax_uint8`:
        the same fp16-rounded weights) and multiplied by the fp16 tensor-core GEMM: with that
        many rows the fp16 GEMM's higher rate outweighs one extra pass over the matrix."""
        w = lin.w
        rows = x.shape[0]
        row_split = isinstance(lin, RowParallelU8Linear)
        if rows < self.PREFILL_DEQUANT_ROWS or w.zeros is not None:
            return lin(out, x, part, residual=residual) if row_split else lin(out, x)
        need = w.n * w.k
        if self._deq is None or self._deq.numel() < need:
            self._deq = torch.empty(need, dtype=torch.float16, device=self.device)
        wf = self._deq[:need].view(w.n, w.k)
        self.k.dequantize_absmax_uint8(wf, w.scales, w.q)
        wv = TensorView.of(wf).permute([1, 0])
        if not row_split:
            self.k.matmul_f16(TensorView.of(out), TensorView.of(x), wv)
            return out
        if self.tp.world == 1:
            opts = MatmulOptions.new().store(MatmulStore.Add()) if residual else MatmulOptions.new()
            self.k.matmul_f16(TensorView.of(out), TensorView.of(x), wv, opts)
            return out
        buf = part if part is not None else torch.zeros_like(out)
        self.k.matmul_f16(TensorView.of(buf), TensorView.of(x), wv)
        self.tp.all_reduce(buf)
        if residual:
            out.add_(buf)
        else:
            out.copy_(buf)
        return out

    def prefill(self, tokens: torch.Tensor):
        """tokens: [B, S0] int64.  Fills the cache for positions [0, S0) and leaves the
        last-position argmax in self.tokens, self.pos = S0."""
        sh, tp = self.shape, self.tp
        B, S0 = tokens.shape
        assert B == self.B and S0 <= self.S
        hd, Hl, d, dl, fl = sh.head_dim, self.Hl, sh.dim, self.dl, self.fl
        f16 = dict(dtype=torch.float16, device=self.device)
        h = self.embed[tokens.reshape(-1)].clone()                       # [B*S0, d]
        # zero-filled like the reference's Tensor::new_gpu: the u8 kernels always read `out`
        # (beta * old, even for beta = 0), so stale NaNs in a fresh buffer would propagate
        x, part = torch.zeros((B * S0, d), **f16), torch.zeros((B * S0, d), **f16)
        qkv, att = torch.zeros((B * S0, 3 * dl), **f16), torch.zeros((B * S0, dl), **f16)
        gu, g = torch.zeros((B * S0, 2 * fl), **f16), torch.zeros((B * S0, fl), **f16)
        Sp = (S0 + 7) // 8 * 8
        scores = torch.zeros((Hl, S0, Sp), **f16)
        sv = TensorView(scores, TensorLayout.new((Hl, S0, S0), (S0 * Sp, Sp, 1)))
        scale = 1.0 / math.sqrt(hd)
        for li, ly in enumerate(self.layers):
            self._norm(x, h, ly.attn_norm)
            self._prefill_linear(ly.wqkv, qkv, x)
            for b in range(B):  # one sequence at a time, with the reference's views (llama.rs:503-554)
                rows = qkv[b * S0:(b + 1) * S0]
                q_b, k_b, v_b = (rows[:, i * dl:(i + 1) * dl] for i in range(3))
                # q and k lie side by side in the projection's rows and a head is rotated by its
                # own pair index and the row's position only: one launch over 2 * Hl heads gives
                # the bits of the reference's two (llama.rs:509-532)
                self.k.rotary_inplace(TensorView.of(rows[:, :2 * dl]), 2 * Hl, 0, sh.theta)
                if self.fused_attention:
                    continue
                head = lambda t, order: TensorView(t, TensorLayout.new((S0, Hl, hd), (t.stride(0), hd, 1))).permute(order)
                self.k.matmul_f16(sv, head(q_b, [1, 0, 2]), head(k_b, [1, 2, 0]),
                                  MatmulOptions.new().store(MatmulStore.Scale(scale)).mask(MatmulMask.Causal))
                self.k.softmax_rows_inplace(sv, 1.0)
                self.k.matmul_f16(head(att[b * S0:(b + 1) * S0], [1, 0, 2]), sv, head(v_b, [1, 0, 2]))
            if self.fused_attention:
                # all sequences and heads at once: [B, heads, S0, hd] views of the [B*S0, 3*dl]
                # projections and of the [B*S0, dl] output
                hv = lambda t: TensorView(t, TensorLayout.new((B, Hl, S0, hd), (S0 * t.stride(0), hd, t.stride(0), 1)))
                self.k.attention_f16(hv(att), hv(qkv[:, :dl]), hv(qkv[:, dl:2 * dl]), hv(qkv[:, 2 * dl:]),
                                     scale, MatmulMask.Causal)
            # the strided row copies go through 16-byte elements: PyTorch's copy of a strided fp16
            # view moves one element per thread step (78 us for 67 MB; 8x fewer elements this way)
            wide = torch.complex128 if dl % 8 == 0 else torch.float16
            self.k_cache[li][:, :S0].view(wide).copy_(qkv[:, dl:2 * dl].view(wide).view(B, S0, -1))
            self.v_cache[li][:, :S0].view(wide).copy_(qkv[:, 2 * dl:].view(wide).view(B, S0, -1))
            self._prefill_linear(ly.wo, h, att, part, residual=True)
            self._norm(x, h, ly.ffn_norm)
            self._prefill_linear(ly.wgu, gu, x)
            self._silu_mul(g, gu)
            self._prefill_linear(ly.down, h, g, part, residual=True)
        last = h.view(B, S0, d)[:, -1].contiguous()
        self._norm(self.x, last, self.out_norm)
        self.k.matmul_nt_fp16u8(self.logits, self.x, self.lm_head.q, self.lm_head.scales, self.lm_head.block)
        self.tokens.copy_(torch.argmax(self.logits, dim=-1))
        self.pos.fill_(S0)


def main():
    """python -m adrastea_b200.llama --shape 7b --batch 16 --prefill 512 --decode 128
    (under torchrun for tensor parallelism).  Prints one JSON line with decode tokens/s,
    timed with CUDA events around the captured decode steps, max over ranks."""
    import argparse
    import json
    import os

    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="7b", choices=["7b", "65b"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prefill", type=int, default=512)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="use only the first N layers (0 = all)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--nccl", action="store_true", help="tensor parallel: NCCL all-reduce in decode too (no graph)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    kern = GpuKernels(local)
    kern.set_tunable("pdl", 0 if args.no_pdl else 1)
    shape = LLAMA_7B if args.shape == "7b" else LLAMA_65B
    tp = TPContext()
    if world > 1 and not args.nccl:
        # decode-size all-reduces go through the library's one-shot kernel over peer memory, which
        # (unlike an NCCL call here) can be captured with the step; prefill-size ones stay on NCCL
        from .tp import PeerAllReduce
        tp.peer_ar = PeerAllReduce(kern, tp, args.batch * shape.dim, torch.device("cuda", local))
    model = LlamaU8(kern, shape, tp, max_batch=args.batch,
                    max_seq=args.prefill + args.decode, n_layers=args.layers or None,
                    device=torch.device("cuda", local))
    toks = torch.randint(0, shape.vocab, (args.batch, args.prefill), device=model.device)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    e[0].record()
    model.prefill(toks)
    e[1].record()
    if not args.no_graph and not (world > 1 and args.nccl):
        pos0, tok0 = model.pos.clone(), model.tokens.clone()
        model.capture()
        model.pos.copy_(pos0)
        model.tokens.copy_(tok0)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e[2].record()
    for _ in range(args.decode):
        model.decode_step()
    e[3].record()
    torch.cuda.synchronize()
    ms_pre, ms_dec = e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3])
    if world > 1:
        t = torch.tensor([ms_pre, ms_dec], device=model.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_pre, ms_dec = t.tolist()
    kern.device_status()
    if int(os.environ.get("RANK", "0")) == 0:
        wb = model.weight_bytes_per_token()
        print(json.dumps({
            "model": f"llama-{args.shape}-shape u8", "layers": model.L, "tp": world, "batch": args.batch,
            "prefill_tokens": args.batch * args.prefill, "prefill_ms": ms_pre,
            "prefill_tok_s": args.batch * args.prefill / (ms_pre * 1e-3),
            "decode_steps": args.decode, "decode_ms_per_step": ms_dec / args.decode,
            "decode_tok_s": args.batch * args.decode / (ms_dec * 1e-3),
            "weight_bytes_per_step_per_gpu": wb,
            "weight_stream_gbs_per_gpu": wb * args.decode / (ms_dec * 1e-3) / 1e9,
            "graph": not args.no_graph}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
