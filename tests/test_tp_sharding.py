"""Tensor-parallel sharding logic (adrastea_b200/tp.py) on CPU: pure slicing checks and a
world-size-2 gloo run in which each rank computes its shard with the oracle and the
all-reduce completes the row-split product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from adrastea_b200.tp import TPContext, U8Weight, shard_column, shard_row
from oracle import oracle


def make_weight(n, k, bs, seed=0):
    rng = np.random.default_rng(seed)
    q = torch.from_numpy(rng.integers(0, 256, (n, k), dtype=np.uint8))
    s = torch.from_numpy(rng.uniform(0.001, 0.01, (n, k // bs)).astype(np.float16))
    return U8Weight(q, s, bs)


def test_column_and_row_shards_tile_the_matrix():
    w = make_weight(48, 256, 32)
    cols = [shard_column(w, r, 4) for r in range(4)]
    assert torch.equal(torch.cat([c.q for c in cols], 0), w.q)
    assert torch.equal(torch.cat([c.scales for c in cols], 0), w.scales)
    rows = [shard_row(w, r, 4) for r in range(4)]
    assert torch.equal(torch.cat([c.q for c in rows], 1), w.q)
    assert torch.equal(torch.cat([c.scales for c in rows], 1), w.scales)
    assert all(c.q.is_contiguous() and c.scales.is_contiguous() for c in cols + rows)


def test_group_straddling_a_rank_is_refused():
    # FFN 22016 over 8 ranks is 2752 columns per rank: 128 does not divide it, 64 does
    w = make_weight(8, 22016, 128)
    with pytest.raises(ValueError):
        shard_row(w, 0, 8)
    assert shard_row(make_weight(8, 22016, 64), 3, 8).q.shape == (8, 2752)
    with pytest.raises(ValueError):
        shard_column(make_weight(10, 64, 32), 0, 4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = TPContext()
        assert (tp.rank, tp.world) == (rank, world)
        m, d, f, bs = 3, 128, 256, 32
        rng = np.random.default_rng(5)
        x = rng.standard_normal((m, d)).astype(np.float16)
        up, down = make_weight(f, d, bs, 1), make_weight(d, f, bs, 2)
        # column-split up-projection: this rank's slice of the hidden activation
        ups = shard_column(up, rank, world)
        hid = oracle.matmul_nt_fp16u8(x, ups.q.numpy(), ups.scales.numpy(), bs)           # [m, f/world]
        # row-split down-projection: partial sums, then the all-reduce
        dws = shard_row(down, rank, world)
        part = oracle.matmul_nt_fp16u8(hid, dws.q.numpy(), dws.scales.numpy(), bs)        # [m, d]
        t = torch.from_numpy(part.astype(np.float32))
        tp.all_reduce(t)
        if rank == 0:
            full_hid = oracle.matmul_nt_fp16u8(x, up.q.numpy(), up.scales.numpy(), bs)
            want = oracle.matmul_nt_fp16u8(full_hid, down.q.numpy(), down.scales.numpy(), bs)
            err = oracle.max_rel_err(t.numpy().astype(np.float16), want)
            with open(out_path, "w") as fh:
                fh.write(repr(err))
    finally:
        dist.destroy_process_group()


def test_row_split_allreduce_world2_gloo(tmp_path):
    out = tmp_path / "err.txt"
    mp.spawn(_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert float(out.read_text()) <= 1e-2


def _failing_worker(rank, world, port, out_path):
    """Rank 1 leaves before the collective; rank 0's all-reduce must end with an error
    within the process-group timeout instead of hanging."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(0)
    try:
        TPContext().all_reduce(torch.ones(4))
        result = "no error"
    except Exception as e:  # noqa: BLE001
        result = "error: " + type(e).__name__
    with open(out_path, "w") as fh:
        fh.write(result)
    os._exit(0)


def test_peer_that_never_joins_surfaces_as_an_error(tmp_path):
    out = tmp_path / "res.txt"
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, p, str(out)))
             for p in [_free_port()] for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(60)
        assert not pr.is_alive()
    assert out.read_text().startswith("error")
