"""Child of tests/test_gpu_peer_allreduce.py: one rank of a 2..4-GPU group.  Checks the one-shot
all-reduce over peer memory (adr_allreduce_oneshot) against NCCL, eagerly and replayed from a CUDA
graph, then a row-parallel u8 linear through it against the single-GPU product."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from adrastea_b200 import GpuKernels  # noqa: E402
from adrastea_b200.tp import PeerAllReduce, RowParallelU8Linear, TPContext, U8Weight  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    k = GpuKernels(local)
    tp = TPContext()
    M, N = 16, 2048
    ar = PeerAllReduce(k, tp, M * N, dev)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    shared = torch.Generator(device=dev).manual_seed(55)  # the residual is replicated on all ranks
    for it in range(6):
        x = torch.randn((M, N), device=dev, generator=gen).half()
        res = torch.randn((M, N), device=dev, generator=shared).half()
        i = ar.next_buffer()
        ar.buffer(i, M, N).copy_(x)
        out = res.clone()
        ar.all_reduce(i, out, residual=(it % 2 == 1))
        ref = x.float().clone()
        dist.all_reduce(ref)
        if it % 2 == 1:
            ref += res.float()
        assert (out.float() - ref).abs().max().item() < 2e-2, it
        # every rank holds the same bits
        bits = out.view(torch.int16).to(torch.int32)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "ranks disagree"
    # replayed from a graph: an even number of all-reduces per replay keeps the buffers alternating
    outs = torch.zeros((M, N), device=dev, dtype=torch.float16)
    srcs = [torch.randn((M, N), device=dev, generator=gen).half() for _ in range(2)]

    def step():
        for j in range(2):
            i = ar.next_buffer()
            ar.buffer(i, M, N).copy_(srcs[j])
            ar.all_reduce(i, outs, residual=False)

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    ref = srcs[1].float().clone()
    dist.all_reduce(ref)
    assert (outs.float() - ref).abs().max().item() < 2e-2
    # a row-parallel u8 linear through the peer all-reduce against the unsplit product
    full = torch.Generator(device=dev).manual_seed(7)  # same on every rank
    n, kk, bs = 512, 1024, 64
    q = torch.randint(0, 256, (n, kk), dtype=torch.uint8, device=dev, generator=full)
    sc = (torch.rand((n, kk // bs), device=dev, generator=full) * 0.009 + 0.001).half()
    x = torch.randn((M, kk), device=dev, generator=full).half()
    want = torch.zeros((M, n), device=dev, dtype=torch.float16)
    k.matmul_nt_fp16u8(want, x, q, sc, bs)
    tp.peer_ar = PeerAllReduce(k, tp, M * n, dev)
    lin = RowParallelU8Linear(k, U8Weight(q, sc, bs), tp)
    shard = x[:, rank * kk // world:(rank + 1) * kk // world].contiguous()
    scale = want.float().abs().max()
    for fused in (False, True):  # GEMV + all-reduce kernel, then the all-reduce inside the GEMV kernel
        tp.peer_ar.fused = fused
        got = torch.zeros((M, n), device=dev, dtype=torch.float16)
        lin(got, shard)
        torch.cuda.synchronize()
        rel = ((got.float() - want.float()).abs().max() / scale).item()
        assert rel < 5e-3, (fused, rel)
        # with the residual, four calls in a row (the inboxes alternate), replayed from a graph
        acc = torch.zeros((M, n), device=dev, dtype=torch.float16)

        def four():
            for _ in range(4):
                lin(acc, shard, residual=True)

        four()
        torch.cuda.synchronize()
        rel = ((acc.float() - 4 * want.float()).abs().max() / (4 * scale)).item()
        assert rel < 5e-3, (fused, "residual", rel)
        dist.barrier()
        gg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gg):
            four()
        acc.zero_()
        gg.replay()
        gg.replay()
        torch.cuda.synchronize()
        rel = ((acc.float() - 8 * want.float()).abs().max() / (8 * scale)).item()
        assert rel < 5e-3, (fused, "graph", rel)
        bits = acc.view(torch.int16).to(torch.int32)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "ranks disagree"
        k.device_status()
    k.device_status()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("peer all-reduce ok")


if __name__ == "__main__":
    main()
