#!/usr/bin/env python
"""Benchmark of the adrastea matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at N=1 (the u8 decode configuration, configs[1] of the workload list): the u8-weight decode GEMV/GEMM,
M in {1, 4, 16}, K = 4096, N in {4096, 11008}, block size 128, reference
layout (zero point 127.5).  One step = for every M, one pass over LAYERS
distinct weight sets of 4 x [4096,4096] + 2 x [11008,4096] (the decode-time
linears of a LLaMA-7B block that have K = 4096), 1.26 GB of distinct u8
weights per M, far beyond the 126 MB L2, so every launch streams from HBM.
The metric is algorithmic bytes per second; the roofline is HBM bandwidth.

One JSON line is printed by rank 0.  `value` is timed with CUDA events on the
launching stream with all inputs resident in HBM; `e2e` is the same work
through the public API with the activations starting in pinned host memory
and the results read back to the host inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

NCU_TRAFFIC_RATIO = 17.08 / 17.06  # measured DRAM bytes / algorithmic bytes of the decode kernel
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

K = 4096
NS = (4096, 4096, 4096, 4096, 11008, 11008)
MS = (1, 4, 16)
BS = 128
LAYERS = 8
FALLBACK_HBM_GBS = 6650.0


def gemv_bytes(m, n, k=K, bs=BS):
    """Algorithmic bytes of one u8 GEMV launch: weights + scales + activations + output."""
    return n * k + 2 * n * (k // bs) + 2 * m * k + 2 * m * n


def step_bytes():
    return sum(LAYERS * sum(gemv_bytes(m, n) for n in NS) for m in MS)


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str | None):
        self.uuid = uuid
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            cmd = ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"]
            if self.uuid:
                cmd += ["-i", self.uuid]
            self.proc = subprocess.Popen(cmd, stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [l.split(",") for l in Path(self.path).read_text().splitlines() if l.strip()]
            os.unlink(self.path)
            sm = [float(r[0]) for r in rows if r[0].strip().replace(".", "").isdigit()]
            mx = [float(r[1]) for r in rows if r[1].strip().replace(".", "").isdigit()]
            reasons = set()
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            for r in rows:
                for name, v in zip(names, r[4:8]):
                    if v.strip().lower().startswith("active"):
                        reasons.add(name)
            if sm:
                out["sm_mhz"] = float(np.median(sm))
                out["samples"] = len(sm)
            if mx:
                out["sm_max_mhz"] = max(mx)
            out["reasons"] = sorted(reasons)
        except Exception:
            pass
        return out


# ----------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's host matmul
# (matrixmultiply::sgemm call convention, f32, all host threads) on a bounded
# sample of the same workload.
# ----------------------------------------------------------------------------
def cpu_sample(seconds: float = 10.0):
    from oracle import oracle
    rng = np.random.default_rng(7)
    mats = []
    for n in (4096, 11008):
        q = rng.integers(0, 256, (n, K), dtype=np.uint8)
        s = rng.uniform(0.001, 0.01, (n, K // BS)).astype(np.float16)
        w32 = oracle.dequantize(q, s, BS).astype(np.float32)  # [n, K], as the host path would hold it
        mats.append((n, w32))
    xs = {m: rng.standard_normal((m, K)).astype(np.float32) for m in MS}
    # C[m,n] = X[m,K] . W[n,K]^T : B = W^T has row stride 1, column stride K
    def one_pass():
        b = 0
        for m in MS:
            for n, w in mats:
                oracle.sgemm(xs[m], w.T)
                b += gemv_bytes(m, n)
        return b
    one_pass()  # warm-up
    t0 = time.perf_counter()
    total = 0
    passes = 0
    while True:
        total += one_pass()
        passes += 1
        if time.perf_counter() - t0 >= seconds:
            break
    dt = time.perf_counter() - t0
    return {"value": total / dt / 1e9, "unit": "GB/s", "cores": oracle.lib().orc_num_threads(),
            "kind": "port",
            "sample": f"{passes} passes over M in {list(MS)} x N in [4096, 11008], K=4096, f32 sgemm "
                      f"on weights dequantised once outside the timed region ({dt:.1f} s)"}, dt / passes


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_budget = max(2.0, min(20.0, 1.0 * (args.steps + args.warmup)))
    base, per_pass = cpu_sample(t_budget)
    line = {
        "impl": "reference", "metric": "u8_decode_gemv_hbm_gbs", "value": base["value"],
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_pass * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(), "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference has no host matmul for this path except matrixmultiply::sgemm (f32); "
                "timed: the oracle's port of that call convention on all host cores; one 'step' here "
                "is one pass over the bounded sample, not the full GPU step",
    }
    print(json.dumps(line))


def workload_config():
    return {"workload": "configs[1]: u8 decode GEMV, M in {1,4,16}, K=4096, N in {4096,11008}, "
                        "block 128, zero point 127.5",
            "layers_per_step": LAYERS, "distinct_weight_bytes_per_m": LAYERS * sum(n * K for n in NS),
            "l2_policy": "inputs larger than L2: 1.26 GB of distinct weights between reuses"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from adrastea_b200 import GpuKernels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    kern = GpuKernels(local)
    # The weights of this workload are never written after set-up, so the decode kernel may
    # prefetch them while the previous launch is still running (programmatic dependent launch).
    kern.set_tunable("pdl", 0 if args.no_pdl else 1)
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    weights = []
    for _ in range(LAYERS):
        layer = []
        for n in NS:
            q = torch.randint(0, 256, (n, K), dtype=torch.uint8, device="cuda", generator=gen)
            s = (torch.rand((n, K // BS), device="cuda", generator=gen) * 0.009 + 0.001).half()
            layer.append((n, q, s))
        weights.append(layer)
    xs_host = {m: torch.randn((m, K), dtype=torch.float16).pin_memory() for m in MS}
    xs = {m: xs_host[m].cuda() for m in MS}
    outs = {(m, n): torch.zeros((m, n), dtype=torch.float16, device="cuda") for m in MS for n in (4096, 11008)}
    outs_host = {key: torch.zeros(v.shape, dtype=torch.float16).pin_memory() for key, v in outs.items()}
    stream = torch.cuda.current_stream()

    def step():
        for m in MS:
            x = xs[m]
            for layer in weights:
                for n, q, s in layer:
                    kern.matmul_nt_fp16u8(outs[(m, n)], x, q, s, BS)

    def step_e2e():
        for m in MS:
            xs[m].copy_(xs_host[m], non_blocking=True)
            x = xs[m]
            for layer in weights:
                for n, q, s in layer:
                    kern.matmul_nt_fp16u8(outs[(m, n)], x, q, s, BS)
            for n in (4096, 11008):
                outs_host[(m, n)].copy_(outs[(m, n)], non_blocking=True)
        stream.synchronize()  # the caller reads the result on the host every step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # The step is launch-bound when driven from Python (about 14 us per call), so the
    # launches of one step are captured once into a CUDA graph and replayed.
    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    eager_step = step
    step = graph.replay
    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        step()
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid)
    if rank == 0:
        sampler.start()
    launches0 = kern.launch_count()
    ms = timed(step, args.steps)
    launches = kern.launch_count() - launches0
    if launches == 0:  # graph replays do not pass through the library's counter
        eager_step()
        launches = (kern.launch_count() - launches0) * args.steps
    # per-M breakdown (untimed for the headline; each is its own event pair)
    per_m = {}
    for m in MS:
        def one_m(m=m):
            for layer in weights:
                for n, q, s in layer:
                    kern.matmul_nt_fp16u8(outs[(m, n)], xs[m], q, s, BS)
        gm = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gm):
            one_m()
        t = timed(gm.replay, args.steps)
        b = LAYERS * sum(gemv_bytes(m, n) for n in NS)
        per_m[f"M={m}"] = round(b * args.steps / (t * 1e-3) / 1e9, 1)
    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else {}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    bytes_step = step_bytes()
    value = world * bytes_step * args.steps / (ms * 1e-3) / 1e9
    e2e_value = world * bytes_step * args.steps / (ms_e2e * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = value / world
    h2d = sum(m * K * 2 for m in MS)
    d2h = sum(m * n * 2 for m in MS for n in (4096, 11008))
    line = {
        "metric": "u8_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak,
                     # DRAM bytes per launch: the ncu capture of one [4096,4096], M=1 launch read
                     # 17.08 MB for 17.06 MB algorithmic (profiles/u8_ring_kernel_4096x4096.md);
                     # traffic grows in proportion to the weights, so the average launch of the
                     # step is scaled by that ratio
                     "traffic": bytes_step / max(launches / args.steps, 1) * NCU_TRAFFIC_RATIO,
                     "traffic_unit": "bytes per launch (ncu capture of a 17.06 MB launch, scaled)",
                     "peak_kind": f"of {peak_kind}",
                     "kernel": "u8_ring_kernel", "per_m_gbs": per_m,
                     "bytes_per_launch_avg": bytes_step / max(launches / args.steps, 1)},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        base, _ = cpu_sample(10.0)
        line["cpu_baseline"] = base
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_ours_tp(args):
    """N > 1: configs[4] of the workload list, the LLaMA-65B-shape decode linears (hidden 8192, FFN 22016,
    block 64), batch 16, tensor-parallel over the N ranks: column-split q/k/v/gate/up, row-split
    o/down, one NCCL all-reduce of [16, 8192] fp16 after each row-split product.  One step =
    TP_LAYERS distinct layers (6.5 GB of u8 weights in total, sharded N ways, so every launch
    streams from HBM).  Strong scaling: the model is fixed, the shards shrink with N.  The
    metric is the same as at N = 1: algorithmic bytes of all ranks per second."""
    import torch
    import torch.distributed as dist

    from adrastea_b200 import GpuKernels
    from adrastea_b200.llama import LLAMA_65B, LlamaU8Layer
    from adrastea_b200.tp import TPContext

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    def note(msg):
        if os.environ.get("ADR_BENCH_VERBOSE"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    note("process group up")
    tp = TPContext()
    kern = GpuKernels(local)
    kern.set_tunable("pdl", 0 if args.no_pdl else 1)
    sh, M, TP_LAYERS = LLAMA_65B, 16, 8
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    layers = [LlamaU8Layer(kern, sh, tp, gen, dev) for _ in range(TP_LAYERS)]
    d, dl, fl = sh.dim, sh.dim // world, sh.ffn // world
    f16 = dict(dtype=torch.float16, device=dev)
    x_host = torch.randn((M, d), dtype=torch.float16).pin_memory()
    x = x_host.to(dev)
    h = torch.zeros((M, d), **f16)
    qkv, att = torch.zeros((M, 3 * dl), **f16), torch.randn((M, dl), **f16)
    gu, g = torch.zeros((M, 2 * fl), **f16), torch.randn((M, fl), **f16)
    part = torch.zeros((M, d), **f16)
    h_host = torch.zeros((M, d), dtype=torch.float16).pin_memory()
    stream = torch.cuda.current_stream()
    use_peer = not args.nccl
    if use_peer:
        # peer-mapped symmetric buffers; if any rank cannot set them up, every rank falls back to
        # the NCCL form (the ranks agree through a MIN all-reduce of a success flag)
        from adrastea_b200.tp import PeerAllReduce
        okf = torch.ones(1, device=dev)
        try:
            tp.peer_ar = PeerAllReduce(kern, tp, M * d, dev)
            tp.peer_ar.fused = args.fused_ar
        except Exception as e:  # noqa: BLE001 - reported, then the slower path is used
            note(f"symmetric memory unavailable: {e!r}")
            okf.zero_()
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        if float(okf.item()) < 1.0:
            tp.peer_ar = None
            use_peer = False
        note("symmetric buffers mapped" if use_peer else "falling back to NCCL all-reduce")

    # q/k/v and gate/up are one matrix each (adrastea_b200/llama.py); `att` and `g` stand in for
    # the attention output and the SiluMul output, which are not part of this workload.
    # Default: the row-split products are reduced by the library's one-shot all-reduce over peer
    # memory, and the whole step is ONE CUDA graph.  --nccl: the step is cut at every all-reduce,
    # the kernels between two collectives are captured as one graph each and the NCCL calls stay
    # eager between the replays (capturing them hung in this environment).
    def seg_attn(ly):
        ly.wqkv(qkv, x)
        if use_peer:
            ly.wo(h, att, residual=True)
        else:
            ly.wo.kernels.matmul_nt_fp16u8(part, att, ly.wo.w.q, ly.wo.w.scales, ly.wo.w.block)

    def seg_ffn(ly):
        if not use_peer:
            h.copy_(part)  # the reduced o-projection
        ly.wgu(gu, x)
        if use_peer:
            ly.down(h, g, residual=True)
        else:
            ly.down.kernels.matmul_nt_fp16u8(part, g, ly.down.w.q, ly.down.w.scales, ly.down.w.block)

    segments = []
    for ly in layers:
        segments.append(lambda ly=ly: seg_attn(ly))
        segments.append(lambda ly=ly: seg_ffn(ly))
    replay = list(segments)

    def step():
        for seg in replay:
            seg()
            if not use_peer:
                tp.all_reduce(part)
        if not use_peer:
            h.copy_(part)

    def act_bytes(ly):
        b = 0
        for lin in ly.linears():
            b += 2 * M * lin.w.k + 2 * M * lin.w.n
        return b

    bytes_rank = sum(ly.weight_bytes() + act_bytes(ly) for ly in layers)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    note("weights ready")
    step()
    torch.cuda.synchronize()
    note("first eager step done")
    launches0 = kern.launch_count()
    step()
    launches_per_step = kern.launch_count() - launches0
    torch.cuda.synchronize()
    note("second eager step done")
    graph = None
    if not args.no_graph:
        if use_peer:
            whole = torch.cuda.CUDAGraph()
            with torch.cuda.graph(whole):
                step()
            replay = [whole.replay]
            graph = [whole]
        else:
            graphs = []
            for seg in segments:
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph):
                    seg()
                graphs.append(gph)
            replay = [gph.replay for gph in graphs]
            graph = graphs
    note("segments captured" if graph else "eager segments")
    run = step
    note(f"graph={'yes' if graph is not None else 'no'}")
    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    note("warm-up done")
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid)
    if rank == 0:
        sampler.start()
    ms = timed(run, args.steps)
    note(f"timed {ms:.2f} ms")

    def run_e2e():
        x.copy_(x_host, non_blocking=True)
        run()
        h_host.copy_(h, non_blocking=True)
        stream.synchronize()

    run_e2e()
    ms_e2e = timed(run_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    tb = torch.tensor([float(bytes_rank)], device=dev, dtype=torch.float64)
    dist.all_reduce(tb)
    total_bytes = float(tb.item())
    if rank == 0:
        peak, peak_kind = measured_peak()
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        line = {
            "metric": "u8_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "configs[4]: LLaMA-65B-shape decode linears, M=16, hidden 8192, FFN 22016, "
                                   "block 64, tensor-parallel: column-split qkv and gate/up, row-split o/down, "
                                   + ("one-shot all-reduce over peer memory after o and down, one CUDA graph per step"
                                      if use_peer else "NCCL all-reduce after o and down (eager, between graph segments)"),
                       "layers_per_step": TP_LAYERS, "tp": world,
                       "weight_bytes_per_step_all_ranks": int(total_bytes),
                       "all_reduces_per_step": 2 * TP_LAYERS, "all_reduce_bytes": M * d * 2,
                       "cuda_graph": graph is not None,
                       "l2_policy": "inputs larger than L2: each rank streams its own "
                                    f"{bytes_rank / 1e9:.2f} GB of distinct weights per step"},
            "e2e": {"value": total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": M * d * 2, "d2h_bytes_per_step": M * d * 2,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches_per_step * args.steps),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                         "kernel": "u8_ring_kernel" + (" with the all-reduce fused in" if use_peer and args.fused_ar
                                                     else " + allreduce_oneshot_kernel" if use_peer else " + ncclAllReduce")},
            "clocks": clocks,
        }
        print(json.dumps(line))
    dist.destroy_process_group()


def run_profile_case(args):
    """Small, self-terminating cases for `ncu` captures (a few hundred MB on the device).

    u8 : the decode kernel over 12 distinct [--n,4096] u8 weights (201 MB at n = 4096, larger
         than L2), two passes, m = --m.
    f16: the tensor-core GEMM, [m,4096] x [4096,4096]^T over 6 distinct weights, m = --m.
    attn: the decode-attention kernel, batch --m, 32 heads x 128, 600 of 640 cached positions.
    """
    import torch

    from adrastea_b200 import GpuKernels, TensorView
    torch.cuda.set_device(0)
    kern = GpuKernels(0)
    m = args.m
    if args.profile_case == "u8":
        ws = [(torch.randint(0, 256, (args.n, K), dtype=torch.uint8, device="cuda"),
               (torch.rand((args.n, K // BS), device="cuda") * 0.009 + 0.001).half()) for _ in range(12)]
        x = torch.randn((m, K), dtype=torch.float16, device="cuda")
        o = torch.zeros((m, args.n), dtype=torch.float16, device="cuda")
        for _ in range(2):
            for q, s in ws:
                kern.matmul_nt_fp16u8(o, x, q, s, BS)
    elif args.profile_case == "attn":
        # decode attention at the LLaMA-7B shape: batch --m sequences, 32 heads of 128, 600 cached
        # positions of 640 (K and V caches of 84 MB each at batch 16)
        B, H, hd, S = m, 32, 128, 640
        kc = torch.randn((B, S, H * hd), device="cuda").half()
        vc = torch.randn((B, S, H * hd), device="cuda").half()
        q = torch.randn((B, H * hd), device="cuda").half()
        o = torch.zeros((B, H * hd), dtype=torch.float16, device="cuda")
        pos = torch.tensor([599], dtype=torch.int32, device="cuda")
        for _ in range(4):
            kern.decode_attention(TensorView.of(o), TensorView.of(q), kc, vc, H, pos, 1.0 / 128 ** 0.5)
    else:
        ws = [(torch.randn(4096, K, device="cuda") * 0.02).half() for _ in range(6)]
        a = (torch.randn(m, K, device="cuda") * 0.02).half()
        o = torch.zeros((m, 4096), dtype=torch.float16, device="cuda")
        for _ in range(2):
            for w in ws:
                kern.matmul_f16(TensorView.of(o), TensorView.of(a), TensorView.of(w).permute([1, 0]))
    torch.cuda.synchronize()
    kern.device_status()
    print(json.dumps({"profile_case": args.profile_case, "m": m, "kernel": kern.last_kernel().name}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream-ordered launches")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: do not capture the step in a CUDA graph")
    ap.add_argument("--fused-ar", action="store_true",
                    help="N > 1: all-reduce inside the row-split GEMV kernel instead of a kernel of its own")
    ap.add_argument("--nccl", action="store_true",
                    help="N > 1: reduce the row-split products with NCCL instead of the library's peer-memory kernel")
    ap.add_argument("--profile-case", default=None, choices=["u8", "f16", "attn"],
                    help="run a small fixed case of one kernel family and exit (for ncu captures)")
    ap.add_argument("--m", type=int, default=1, help="rows of the activation in --profile-case")
    ap.add_argument("--n", type=int, default=4096, help="weight rows in --profile-case u8")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    elif int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_ours_tp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
