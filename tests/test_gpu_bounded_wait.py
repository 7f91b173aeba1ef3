"""A bounded wait that runs out, on one GPU, without faulting anything.

The peer all-reduce waits for flags that the other ranks store.  Here world = 2 is claimed but
the "peer" is a second set of ordinary local buffers that nothing ever signals, and the wait
limit is shortened with the tunable "wait_ms": the kernel must give up, finish, set the
context's status word (adr_device_status returns ADR_ERR_DEVICE exactly once), and leave the
context usable for the next, ordinary call.
"""
import numpy as np
import pytest
import torch

from adrastea_b200 import AdrError
from oracle import oracle

pytestmark = pytest.mark.gpu
ADR_ERR_DEVICE = 5


def check_plain_matmul(kernels):
    rng = np.random.default_rng(5)
    m, p, n, bs = 4, 1024, 256, 128
    x = rng.standard_normal((m, p)).astype(np.float16)
    q = rng.integers(0, 256, (n, p), dtype=np.uint8)
    s = rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)
    o = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    kernels.matmul_nt_fp16u8(o, torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda(),
                             torch.from_numpy(s).cuda(), bs)
    kernels.device_status()
    assert oracle.max_rel_err(o.cpu().numpy(), oracle.matmul_nt_fp16u8(x, q, s, bs)) <= 1e-2


def test_allreduce_wait_runs_out_and_the_context_survives(kernels):
    blocks, count = 8, 4096
    bufs = [torch.ones(count, dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(blocks * 2, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = torch.zeros(blocks, dtype=torch.int32, device="cuda")
    out = torch.zeros(count, dtype=torch.float16, device="cuda")
    try:
        kernels.set_tunable("wait_ms", 20)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        kernels.allreduce_oneshot(out, [b.data_ptr() for b in bufs], [f.data_ptr() for f in flags],
                                  epochs, blocks, 0, 2, count, False)
        t1.record()
        with pytest.raises(AdrError) as err:
            kernels.device_status()
        assert err.value.code == ADR_ERR_DEVICE
        assert t0.elapsed_time(t1) < 1000.0  # gave up after about 20 ms, not after a second
        kernels.device_status()              # the flag was cleared: fine again
        # the kernel still completed: it wrote its sum (of whatever the buffers held)
        assert torch.all(out == 2.0)
        assert torch.all(epochs == 1)
        # a second call times out the same way and is reported again
        kernels.allreduce_oneshot(out, [b.data_ptr() for b in bufs], [f.data_ptr() for f in flags],
                                  epochs, blocks, 0, 2, count, False)
        with pytest.raises(AdrError):
            kernels.device_status()
        kernels.device_status()
    finally:
        kernels.set_tunable("wait_ms", 0)
    check_plain_matmul(kernels)


def test_fused_gemv_allreduce_wait_runs_out(kernels):
    """The same for the GEMV with the all-reduce fused in: rank 0 of a claimed world of 2 whose
    peer inbox and flags are local buffers that nobody signals."""
    rng = np.random.default_rng(6)
    m, p, n, bs, max_ctas = 4, 1024, 512, 128, 512
    x = torch.from_numpy(rng.standard_normal((m, p)).astype(np.float16)).cuda()
    q = torch.from_numpy(rng.integers(0, 256, (n, p), dtype=np.uint8)).cuda()
    s = torch.from_numpy(rng.uniform(0.001, 0.01, (n, p // bs)).astype(np.float16)).cuda()
    inboxes = [torch.zeros(2 * m * n, dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(max_ctas * 2, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = torch.zeros(max_ctas, dtype=torch.int32, device="cuda")
    out = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    try:
        kernels.set_tunable("wait_ms", 20)
        kernels.matmul_nt_fp16u8_allreduce(out, x, q, s, bs, False, [b.data_ptr() for b in inboxes],
                                           [f.data_ptr() for f in flags], epochs, max_ctas, 0, 2)
        with pytest.raises(AdrError) as err:
            kernels.device_status()
        assert err.value.code == ADR_ERR_DEVICE
        kernels.device_status()
    finally:
        kernels.set_tunable("wait_ms", 0)
    check_plain_matmul(kernels)
