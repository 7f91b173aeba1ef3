"""Tensor-parallel sharding of the u8 linear layers (one process per GPU).

The reference has no multi-GPU path ("bring back multi-gpu and quantization",
adrastea_models/src/llama.rs:28-29); this is the Megatron-style split of a 65B-shape
model over 2, 4 or 8 GPUs, around the reference's weight layout (`[N, K]` u8 codes, fp16
scales `[N, K/block]`, adrastea_kernels/cpp/quantize.cu:3-56):

  column split (q, k, v, gate, up): rank r keeps rows [r*N/t, (r+1)*N/t) of the
      `[N, K]` storage and of the scales: independent GEMVs, no exchange;
  row split (o, down): rank r keeps columns [r*K/t, (r+1)*K/t) of every row (a
      contiguous `[N, K/t]` copy made once at load time) and the matching scale
      groups; each rank produces a partial `[M, N]` and one all-reduce (sum) over
      NCCL completes it.  The quantisation block must divide K/t.

The sharding functions are pure slicing and run anywhere; `RowParallelU8Linear` and
`ColumnParallelU8Linear` launch the library's kernels and need a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class U8Weight:
    """One quantised matrix in the reference's layout."""
    q: torch.Tensor        # uint8 [N, K]
    scales: torch.Tensor   # float16 [N, K // block]
    block: int
    zeros: torch.Tensor | None = None

    @property
    def n(self) -> int:
        return self.q.shape[0]

    @property
    def k(self) -> int:
        return self.q.shape[1]

    def nbytes(self) -> int:
        b = self.q.numel() + 2 * self.scales.numel()
        if self.zeros is not None:
            b += 2 * self.zeros.numel()
        return b


def shard_column(w: U8Weight, rank: int, world: int) -> U8Weight:
    """Rows [rank*N/world, (rank+1)*N/world) of codes and scales (output features)."""
    if w.n % world != 0:
        raise ValueError(f"N={w.n} is not divisible by the tensor-parallel size {world}")
    lo, hi = rank * w.n // world, (rank + 1) * w.n // world
    z = None if w.zeros is None else w.zeros[lo:hi].contiguous()
    return U8Weight(w.q[lo:hi].contiguous(), w.scales[lo:hi].contiguous(), w.block, z)


def shard_row(w: U8Weight, rank: int, world: int) -> U8Weight:
    """Columns [rank*K/world, (rank+1)*K/world) of every row (input features), with the
    scale groups that cover them.  A group may not straddle two ranks."""
    if w.k % world != 0:
        raise ValueError(f"K={w.k} is not divisible by the tensor-parallel size {world}")
    kk = w.k // world
    if kk % w.block != 0:
        raise ValueError(f"the quantisation block {w.block} does not divide K/world = {kk}: "
                         "groups would straddle ranks (use a smaller block for this matrix)")
    g = kk // w.block
    z = None if w.zeros is None else w.zeros[:, rank * g:(rank + 1) * g].contiguous()
    return U8Weight(w.q[:, rank * kk:(rank + 1) * kk].contiguous(),
                    w.scales[:, rank * g:(rank + 1) * g].contiguous(), w.block, z)


class TPContext:
    """Rank, world size and the process group; world 1 needs no process group."""

    def __init__(self, group=None):
        if dist.is_available() and dist.is_initialized():
            self.group = group
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.group, self.rank, self.world = None, 0, 1
        self.peer_ar = None  # a PeerAllReduce replaces the NCCL call in RowParallelU8Linear

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t


class PeerAllReduce:
    """Two symmetric fp16 buffers per rank, peer-mapped on every GPU of the group, and the
    library's one-shot all-reduce kernel over them (csrc/allreduce.cu).  Row-split products are
    written into `buffer(i)` and reduced with `all_reduce(i, out)`; the two buffers are used
    alternately.  Unlike an NCCL call the kernel can be captured in a CUDA graph."""

    BLOCKS = 64
    MAX_CTAS = 512

    def __init__(self, kernels, tp: "TPContext", max_elems: int, device):
        import torch.distributed._symmetric_memory as symm
        assert tp.world > 1
        self.kernels, self.tp = kernels, tp
        self.max_elems = max_elems
        group = tp.group if tp.group is not None else dist.group.WORLD
        self.bufs, self.buf_ptrs = [], []
        for _ in range(2):
            t = symm.empty(max_elems, dtype=torch.float16, device=device)
            t.zero_()  # the u8 kernels read their output buffer (beta * old) even for beta = 0
            h = symm.rendezvous(t, group)
            self.bufs.append(t)
            self.buf_ptrs.append([int(p) for p in h.buffer_ptrs])
        flags = symm.empty(self.BLOCKS * tp.world, dtype=torch.int32, device=device)
        flags.zero_()
        fh = symm.rendezvous(flags, group)
        self.flags, self.flag_ptrs = flags, [int(p) for p in fh.buffer_ptrs]
        self.epochs = torch.zeros(self.BLOCKS, dtype=torch.int32, device=device)
        self._handles = fh  # keeps the mappings alive
        self._next = 0
        # for the GEMV with the all-reduce fused in: two inboxes of `world` slots, flags and epochs
        # per CTA of the decode kernel
        self.inboxes, self.inbox_ptrs = [], []
        for _ in range(2):
            t = symm.empty(tp.world * max_elems, dtype=torch.float16, device=device)
            t.zero_()
            h = symm.rendezvous(t, group)
            self.inboxes.append(t)
            self.inbox_ptrs.append([int(p) for p in h.buffer_ptrs])
        fflags = symm.empty(self.MAX_CTAS * tp.world, dtype=torch.int32, device=device)
        fflags.zero_()
        ffh = symm.rendezvous(fflags, group)
        self.fused_flags, self.fused_flag_ptrs = fflags, [int(p) for p in ffh.buffer_ptrs]
        self.fused_epochs = torch.zeros(self.MAX_CTAS, dtype=torch.int32, device=device)
        self._handles2 = ffh
        # RowParallelU8Linear uses the fused kernel when this is set.  Off by default: at 2 GPUs the
        # GEMV followed by the one-shot all-reduce kernel measured faster (1.71 ms against 1.88 ms
        # per 8-layer step of the 65B shape): the flag round trip sits at the tail of every GEMV
        # CTA instead of overlapping the next launch's prologue.
        self.fused = False
        torch.cuda.synchronize(device)
        dist.barrier(group=tp.group)  # every rank's flags are zero before anyone signals

    def next_buffer(self) -> int:
        """Index of the buffer the next row-split product must write (they alternate)."""
        i = self._next
        self._next ^= 1
        return i

    def buffer(self, i: int, rows: int, cols: int) -> torch.Tensor:
        return self.bufs[i][: rows * cols].view(rows, cols)

    def all_reduce(self, i: int, out: torch.Tensor, residual: bool = False):
        self.kernels.allreduce_oneshot(out, self.buf_ptrs[i], self.flag_ptrs, self.epochs,
                                       self.BLOCKS, self.tp.rank, self.tp.world, out.numel(), residual)


class ColumnParallelU8Linear:
    """y[:, shard] = x . deq(W[shard rows])^T; the output stays sharded along N."""

    def __init__(self, kernels, w_full_or_shard: U8Weight, tp: TPContext, already_sharded=False):
        self.kernels, self.tp = kernels, tp
        self.w = w_full_or_shard if already_sharded else shard_column(w_full_or_shard, tp.rank, tp.world)

    def __call__(self, out: torch.Tensor, x: torch.Tensor, beta: float = 0.0) -> torch.Tensor:
        self.kernels.matmul_nt_fp16u8(out, x, self.w.q, self.w.scales, self.w.block, beta, self.w.zeros)
        return out


class RowParallelU8Linear:
    """y = all_reduce_sum_r( x[:, shard_r] . deq(W[:, shard_r])^T ).

    `beta` (accumulate into `out`, e.g. the residual) is applied after the reduction on
    the reduced value, so the residual is added exactly once."""

    def __init__(self, kernels, w_full_or_shard: U8Weight, tp: TPContext, already_sharded=False):
        self.kernels, self.tp = kernels, tp
        self.w = w_full_or_shard if already_sharded else shard_row(w_full_or_shard, tp.rank, tp.world)

    def __call__(self, out: torch.Tensor, x_shard: torch.Tensor, partial: torch.Tensor | None = None,
                 residual: bool = False) -> torch.Tensor:
        if self.tp.world == 1 and not residual:
            self.kernels.matmul_nt_fp16u8(out, x_shard, self.w.q, self.w.scales, self.w.block, 0.0, self.w.zeros)
            return out
        if self.tp.world == 1:
            self.kernels.matmul_nt_fp16u8(out, x_shard, self.w.q, self.w.scales, self.w.block, 1.0, self.w.zeros)
            return out
        if self.tp.peer_ar is not None and out.numel() <= self.tp.peer_ar.max_elems:
            ar = self.tp.peer_ar
            i = ar.next_buffer()
            if ar.fused and out.shape[0] <= 16 and out.is_contiguous():
                from .kernels import AdrError
                try:
                    self.kernels.matmul_nt_fp16u8_allreduce(
                        out, x_shard, self.w.q, self.w.scales, self.w.block, residual,
                        ar.inbox_ptrs[i], ar.fused_flag_ptrs, ar.fused_epochs, ar.MAX_CTAS,
                        self.tp.rank, self.tp.world, self.w.zeros)
                    return out
                except AdrError as e:
                    if e.code != 2:  # ADR_ERR_SHAPE: a shape the decode kernel does not take
                        raise
            buf = ar.buffer(i, out.shape[0], out.shape[1])
            self.kernels.matmul_nt_fp16u8(buf, x_shard, self.w.q, self.w.scales, self.w.block, 0.0, self.w.zeros)
            ar.all_reduce(i, out, residual)
            return out
        buf = partial if partial is not None else torch.zeros_like(out)
        self.kernels.matmul_nt_fp16u8(buf, x_shard, self.w.q, self.w.scales, self.w.block, 0.0, self.w.zeros)
        self.tp.all_reduce(buf)
        if residual:
            out.add_(buf)
        else:
            out.copy_(buf)
        return out
