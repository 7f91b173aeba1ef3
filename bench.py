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
and the results read back to the host inside the timed region.  The timed
loop of --steps steps is repeated --repeats times; the line carries the
median and the spread.

The headline metric has three parts (u8 GB/s, fp16 GEMM TFLOP/s, LLaMA-7B
decode tokens/s).  `value` is the first; the others are measured in the same
process with CUDA events and reported under `extra` (skipped by --no-extra).

N > 1 (under torchrun) is a DIFFERENT workload: the LLaMA-65B-shape decode
linears, tensor-parallel, strong scaling; its tp = 1 point is in the N = 1
line's `extra.tp1_65b`.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

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
FALLBACK_TFLOPS = 1590.0


def ncu_traffic_ratio():
    """DRAM bytes / algorithmic bytes of the decode kernel from the committed summary of an ncu
    capture (a small case; traffic grows in proportion to the weights), or None."""
    f = ROOT / "profiles" / "dram_traffic.json"
    try:
        d = json.loads(f.read_text())["u8_decode"]
        return float(d["dram_bytes"]) / float(d["algorithmic_bytes"]), d.get("kernel")
    except Exception:
        return None, None


def gemv_bytes(m, n, k=K, bs=BS):
    """Algorithmic bytes of one u8 GEMV launch: weights + scales + activations + output."""
    return n * k + 2 * n * (k // bs) + 2 * m * k + 2 * m * n


def step_bytes():
    return sum(LAYERS * sum(gemv_bytes(m, n) for n in NS) for m in MS)


def measured_peak(key="hbm_gbs"):
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())[key]), "measured"
        except Exception:
            pass
    return (FALLBACK_HBM_GBS if key == "hbm_gbs" else FALLBACK_TFLOPS), "fallback"


def spread(ms_list):
    a = sorted(ms_list)
    return {"n": len(a), "median_ms": float(np.median(a)), "min_ms": a[0], "max_ms": a[-1]}


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
def host_threads():
    """All the host threads this process may use (launchers such as torchrun export
    OMP_NUM_THREADS=1 to every rank, which would pin the CPU arm to one core)."""
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_sample(seconds: float = 10.0):
    from oracle import oracle
    cores = oracle.lib().orc_set_num_threads(host_threads())
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
    return {"value": total / dt / 1e9, "unit": "GB/s", "cores": cores,
            "kind": "port",
            "sample": f"{passes} passes over M in {list(MS)} x N in [4096, 11008], K=4096, f32 sgemm "
                      f"on weights dequantised once outside the timed region ({dt:.1f} s)"}, dt / passes


TP_M, TP_LAYERS, TP_DIM, TP_FFN, TP_BLOCK = 16, 8, 8192, 22016, 64


def tp_shard_shapes(world):
    """[n, k] of the four products of one 65B-shape layer on one rank of `world`."""
    dl, fl = TP_DIM // world, TP_FFN // world
    return [(3 * dl, TP_DIM), (TP_DIM, dl), (2 * fl, TP_DIM), (TP_DIM, fl)]


def tp_workload(world, how):
    return ("configs[4]: LLaMA-65B-shape decode linears, M=16, hidden 8192, FFN 22016, "
            "block 64, tensor-parallel: column-split qkv and gate/up, row-split o/down, " + how)


def cpu_sample_tp(world, seconds):
    """The N > 1 workload on the host: the f32 sgemm over the shard shapes of all `world` ranks of
    one layer (the same products the GPUs run, done one after another), on a bounded sample."""
    from oracle import oracle
    cores = oracle.lib().orc_set_num_threads(host_threads())
    rng = np.random.default_rng(11)
    shapes = tp_shard_shapes(world)
    # one f32 matrix per distinct shard shape, reused for every rank's shard (values do not matter
    # for the timing; distinct buffers per rank would need 6.5 GB x 4 bytes of host memory)
    mats = [(n, k, rng.standard_normal((n, k), dtype=np.float32)) for n, k in shapes]
    xs = {k: rng.standard_normal((TP_M, k), dtype=np.float32) for _, k in shapes}

    def one_layer():
        b = 0
        for _ in range(world):
            for n, k, w in mats:
                oracle.sgemm(xs[k], w.T)
                b += gemv_bytes(TP_M, n, k, TP_BLOCK)
        return b
    one_layer()
    t0 = time.perf_counter()
    total, passes = 0, 0
    while True:
        total += one_layer()
        passes += 1
        if time.perf_counter() - t0 >= seconds:
            break
    dt = time.perf_counter() - t0
    return {"value": total / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{passes} passes over one 65B-shape layer (all {world} ranks' shards, M=16), f32 sgemm "
                      f"on f32 weights ({dt:.1f} s)"}, dt / passes


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    t_budget = max(2.0, min(20.0, 1.0 * (args.steps + args.warmup)))
    if world > 1:
        base, per_pass = cpu_sample_tp(world, t_budget)
        config = tp_config(world)
        scaling = "strong"
    else:
        base, per_pass = cpu_sample(t_budget)
        config = workload_config()
        scaling = "weak"
    line = {
        "impl": "reference", "metric": "u8_decode_gemv_hbm_gbs", "value": base["value"],
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_pass * 1e3, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config, "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference has no host matmul for this path except matrixmultiply::sgemm (f32); "
                "timed: the oracle's port of that call convention on all host cores; one 'step' here "
                "is one pass over the bounded sample, not the full GPU step",
    }
    print(json.dumps(line))


def tp_rank_bytes(world):
    """Algorithmic bytes one rank moves per step: the four fused products of TP_LAYERS layers."""
    return TP_LAYERS * sum(gemv_bytes(TP_M, n, k, TP_BLOCK) for n, k in tp_shard_shapes(world))


def tp_config(world, use_peer=True):
    """The N > 1 workload description; identical in both arms (nothing measured in it)."""
    how = ("one-shot all-reduce over peer memory after o and down, one CUDA graph per step"
           if use_peer else "NCCL all-reduce after o and down (eager, between graph segments)")
    return {"workload": tp_workload(world, how), "layers_per_step": TP_LAYERS, "tp": world,
            "weight_bytes_per_step_all_ranks": world * tp_rank_bytes(world),
            "all_reduces_per_step": 2 * TP_LAYERS, "all_reduce_bytes": TP_M * TP_DIM * 2,
            "l2_policy": "inputs larger than L2: each rank streams its own shard of 6.5 GB of distinct "
                         "weights per step"}


def workload_config():
    return {"workload": "configs[1]: u8 decode GEMV, M in {1,4,16}, K=4096, N in {4096,11008}, "
                        "block 128, zero point 127.5",
            "layers_per_step": LAYERS, "distinct_weight_bytes_per_m": LAYERS * sum(n * K for n in NS),
            "l2_policy": "inputs larger than L2: 1.26 GB of distinct weights between reuses"}


def make_timer(stream_fn, world=1):
    """CUDA-event timing of `steps` calls of fn on the launching stream, bracketed by a barrier
    and a device synchronisation on both sides; max over ranks when there are several."""
    import torch
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        stream = stream_fn()
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
    return timed


def graphed(fn):
    """Run fn once eagerly, then capture it into a CUDA graph; returns the replay callable."""
    import torch
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g.replay, g


def decode_weights(kern, gen, with_zeros):
    import torch
    weights = []
    for _ in range(LAYERS):
        layer = []
        for n in NS:
            q = torch.randint(0, 256, (n, K), dtype=torch.uint8, device="cuda", generator=gen)
            s = (torch.rand((n, K // BS), device="cuda", generator=gen) * 0.009 + 0.001).half()
            z = ((torch.rand((n, K // BS), device="cuda", generator=gen) * 16 + 120).half()
                 if with_zeros else None)
            layer.append((n, q, s, z))
        weights.append(layer)
    return weights


# ------------------------------------------------------------------ extras
def extra_fp16_gemm(kern, timed, args):
    """fp16 tensor-core GEMM at the reference's own bench shape (2048 x 4096 x 4096, rhs stored
    [N,K] ("rrc") and [K,N] ("rrr"); adrastea/src/main.rs:555-594), a large prefill shape, and
    the 64 x 4096 x 4096 case of configs[0] against the HBM roof."""
    import torch
    from adrastea_b200 import TensorView
    peak, kind = measured_peak("bf16_tflops")
    hbm, _ = measured_peak("hbm_gbs")
    out = {"peak_tflops": peak, "peak_kind": f"of {kind} (cuBLAS bf16 burst)"}
    reps = max(3, args.repeats // 2)

    def case(m, k, n, layout, nw, iters):
        a = (torch.randn(m, k, device="cuda") * 0.02).half()
        ws = [(torch.randn((n, k) if layout == "rrc" else (k, n), device="cuda") * 0.02).half()
              for _ in range(nw)]
        o = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        views = [TensorView.of(w).permute([1, 0]) if layout == "rrc" else TensorView.of(w) for w in ws]

        def body():
            for v in views:
                kern.matmul_f16(TensorView.of(o), TensorView.of(a), v)
        replay, g = graphed(body)
        for _ in range(2):
            replay()
        ms = float(np.median([timed(replay, iters) for _ in range(reps)])) / (iters * nw)
        return ms
    for name, (m, k, n, layout, nw, iters) in {
            "2048x4096x4096_rrc": (2048, 4096, 4096, "rrc", 6, 10),
            "2048x4096x4096_rrr": (2048, 4096, 4096, "rrr", 6, 10),
            "16384x8192x8192_rrc": (16384, 8192, 8192, "rrc", 2, 3)}.items():
        ms = case(m, k, n, layout, nw, iters)
        tf = 2.0 * m * k * n / (ms * 1e-3) / 1e12
        out[name] = {"us": ms * 1e3, "tflops": tf, "frac_of_peak": tf / peak}
    for layout in ("rrc", "rrr"):
        ms = case(64, 4096, 4096, layout, 8, 10)  # 8 distinct weights = 268 MB between reuses
        by = 2 * (64 * 4096 + 4096 * 4096 + 64 * 4096)
        out[f"config1_64x4096x4096_{layout}"] = {"us": ms * 1e3, "gbs": by / (ms * 1e-3) / 1e9,
                                                 "frac_of_hbm": by / (ms * 1e-3) / 1e9 / hbm,
                                                 "tflops": 2.0 * 64 * 4096 * 4096 / (ms * 1e-3) / 1e12}
    return out


def extra_u8_prefill(kern, timed, args):
    """u8-weight prefill GEMM (m > 32: weights dequantised into tensor memory) on LLaMA-7B
    projection shapes at 2048 and 512 tokens, against the measured bf16 peak.  At 512 tokens a
    problem has fewer tiles than the GPU has SMs and a thread-block cluster shares each tile's
    k-steps.  Distinct weights per launch (more than L2 between reuses)."""
    import torch
    peak, kind = measured_peak("bf16_tflops")
    out = {"peak_tflops": peak, "peak_kind": f"of {kind} (cuBLAS bf16 burst)"}
    gen = torch.Generator(device="cuda").manual_seed(7)
    reps = max(3, args.repeats // 2)
    for m, n, k, nw in ((2048, 4096, 4096, 12), (2048, 11008, 4096, 6), (512, 4096, 4096, 12),
                        (512, 12288, 4096, 6), (512, 4096, 11008, 6), (64, 4096, 4096, 12)):
        ws = [(torch.randint(0, 256, (n, k), dtype=torch.uint8, device="cuda", generator=gen),
               (torch.rand((n, k // BS), device="cuda", generator=gen) * 0.009 + 0.001).half())
              for _ in range(nw)]
        x = (torch.randn((m, k), device="cuda", generator=gen) * 0.5).half()
        o = torch.zeros((m, n), dtype=torch.float16, device="cuda")

        def body(ws=ws, x=x, o=o):
            for q, sc in ws:
                kern.matmul_nt_fp16u8(o, x, q, sc, BS)
        replay, g = graphed(body)
        # the section before this one ends under the power cap; a pause and a few untimed
        # replays keep its tail out of the first case
        torch.cuda.synchronize()
        time.sleep(0.3)
        for _ in range(4):
            replay()
        ms = float(np.median([timed(replay, 5) for _ in range(reps)])) / (5 * nw)
        tf = 2.0 * m * k * n / (ms * 1e-3) / 1e12
        out[f"{m}x{n}x{k}"] = {"us": ms * 1e3, "tflops": tf, "frac_of_peak": tf / peak,
                               "kernel": kern.last_kernel().name}
        del ws
    return out


def extra_zero_points(kern, timed, args, xs, outs):
    """The headline decode mix with fp16 zero points ~U(120,136) (configs[1] as worded)."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(99)
    weights = decode_weights(kern, gen, True)

    def step():
        for m in MS:
            for layer in weights:
                for n, q, s, z in layer:
                    kern.matmul_nt_fp16u8(outs[(m, n)], xs[m], q, s, BS, 0.0, z)
    replay, g = graphed(step)
    for _ in range(3):
        replay()
    ms = float(np.median([timed(replay, args.steps) for _ in range(args.repeats)])) / args.steps
    by = sum(LAYERS * sum(gemv_bytes(m, n) + 2 * n * (K // BS) for n in NS) for m in MS)
    hbm, _ = measured_peak()
    return {"ms_per_step": ms, "gbs": by / (ms * 1e-3) / 1e9, "frac_of_hbm": by / (ms * 1e-3) / 1e9 / hbm,
            "bytes_per_step": by}


def extra_grouped(kern, timed, args, weights, xs, outs_by):
    """The same decode mix through adr_matmul_nt_fp16u8_grouped: per layer the four [4096,4096]
    products as one launch and the two [11008,4096] products as another (they share their
    activations in this workload, as q/k/v and gate/up do in a decoder layer).  Its own line:
    the headline stays the per-launch figure."""
    import torch
    per_m = {}
    total_ms = 0.0
    for m in MS:
        groups = []
        for layer in weights:
            by_n = {}
            for n, q, s, _ in layer:
                by_n.setdefault(n, []).append((q, s))
            for n, lst in by_n.items():
                o = [torch.zeros((m, n), dtype=torch.float16, device="cuda") for _ in lst]
                groups.append((o, [q for q, _ in lst], [s for _, s in lst]))

        def run(groups=groups, m=m):
            for o, qs, ss in groups:
                kern.matmul_nt_fp16u8_grouped(o, xs[m], qs, ss, BS)
        rm, gm = graphed(run)
        t = float(np.median([timed(rm, args.steps) for _ in range(max(3, args.repeats // 2))]))
        b = LAYERS * sum(gemv_bytes(m, n) for n in NS)
        per_m[f"M={m}"] = round(b * args.steps / (t * 1e-3) / 1e9, 1)
        total_ms += t / args.steps
        del gm
    hbm, _ = measured_peak()
    gbs = step_bytes() / (total_ms * 1e-3) / 1e9
    return {"ms_per_step": total_ms, "gbs": gbs, "frac_of_hbm": gbs / hbm, "per_m_gbs": per_m,
            "launches_per_step": 2 * LAYERS * len(MS),
            "what": "adr_matmul_nt_fp16u8_grouped: 2 launches per layer instead of 6"}


def extra_llama7b(kern, batch, prefill=512, decode=128):
    """LLaMA-7B shape, u8 weights, KV cache: `decode` graph-replayed steps after a `prefill`-token
    prefill; tokens/s and the fraction of the weight-stream ceiling (all weights once per step at
    the measured HBM peak)."""
    import torch
    from adrastea_b200.llama import LLAMA_7B, LlamaU8
    model = LlamaU8(kern, LLAMA_7B, max_batch=batch, max_seq=prefill + decode)
    toks = torch.randint(0, LLAMA_7B.vocab, (batch, prefill), device="cuda")
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    model.prefill(toks)  # warm-up (descriptor cache, allocator)
    torch.cuda.synchronize()
    e[0].record()
    model.prefill(toks)
    e[1].record()
    pos0, tok0 = model.pos.clone(), model.tokens.clone()
    model.capture()
    model.pos.copy_(pos0)
    model.tokens.copy_(tok0)
    torch.cuda.synchronize()
    e[2].record()
    for _ in range(decode):
        model.decode_step()
    e[3].record()
    torch.cuda.synchronize()
    kern.device_status()
    ms_pre, ms_dec = e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3]) / decode
    wb = model.weight_bytes_per_token()
    hbm, _ = measured_peak()
    ceiling = batch / (wb / (hbm * 1e9))
    tok_s = batch / (ms_dec * 1e-3)
    # the KV cache read by a step: keys and values of every layer over the context so far
    # (its mean over the timed steps); at batch 16 it is two thirds of the weights' bytes
    kv = 2 * LLAMA_7B.n_layers * batch * (prefill + decode / 2.0) * LLAMA_7B.dim * 2
    del model
    torch.cuda.empty_cache()
    return {"decode_ms_per_step": ms_dec, "decode_tok_s": tok_s, "weight_bytes_per_step": wb,
            "weight_stream_ceiling_tok_s": ceiling, "frac_of_ceiling": tok_s / ceiling,
            "kv_cache_bytes_per_step": kv,
            "frac_of_hbm_weights_and_kv": (wb + kv) / (ms_dec * 1e-3) / 1e9 / hbm,
            "prefill_tokens": batch * prefill, "prefill_ms": ms_pre,
            "prefill_tok_s": batch * prefill / (ms_pre * 1e-3)}


def extra_clip(kern, batch=64, iters=3):
    """CLIP ViT-L/14 image encoder forward, fp16, random weights (configs[2])."""
    import torch
    from adrastea_b200.clip import VIT_L_14, ClipVisionU
    model = ClipVisionU(kern, VIT_L_14, batch)
    px = torch.randn((batch, 3, 224, 224), device="cuda").half()
    model.forward(px)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        model.forward(px)
    e1.record()
    torch.cuda.synchronize()
    kern.device_status()
    ms = e0.elapsed_time(e1) / iters
    peak, _ = measured_peak("bf16_tflops")
    tf = model.flops() / (ms * 1e-3) / 1e12
    del model
    torch.cuda.empty_cache()
    return {"batch": batch, "ms_per_forward": ms, "images_per_s": batch / (ms * 1e-3),
            "matmul_tflops": tf, "frac_of_peak": tf / peak}


def extra_tp1_65b(kern, timed, args):
    """The N > 1 workload (8 layers of the 65B-shape decode linears, M = 16) on ONE GPU, tp = 1:
    the base point of the strong-scaling curve (efficiency at N = this / (N x ms_per_step))."""
    import torch
    from adrastea_b200.llama import LLAMA_65B, LlamaU8Layer
    from adrastea_b200.tp import TPContext
    tp = TPContext()
    gen = torch.Generator(device="cuda").manual_seed(4321)
    layers = [LlamaU8Layer(kern, LLAMA_65B, tp, gen, torch.device("cuda")) for _ in range(TP_LAYERS)]
    f16 = dict(dtype=torch.float16, device="cuda")
    d, f, M = TP_DIM, TP_FFN, TP_M
    x, h = torch.randn((M, d), **f16), torch.zeros((M, d), **f16)
    qkv, att = torch.zeros((M, 3 * d), **f16), torch.randn((M, d), **f16)
    gu, g = torch.zeros((M, 2 * f), **f16), torch.randn((M, f), **f16)

    def step():
        h.copy_(x)
        for ly in layers:
            ly.wqkv(qkv, x)
            ly.wo(h, att, residual=True)
            ly.wgu(gu, x)
            ly.down(h, g, residual=True)
    replay, gr = graphed(step)
    for _ in range(3):
        replay()
    ms = float(np.median([timed(replay, args.steps) for _ in range(max(3, args.repeats // 2))])) / args.steps
    by = tp_rank_bytes(1)
    hbm, _ = measured_peak()
    kern.device_status()
    del layers
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "gbs": by / (ms * 1e-3) / 1e9, "frac_of_hbm": by / (ms * 1e-3) / 1e9 / hbm,
            "bytes_per_step": by, "workload": tp_workload(1, "no exchange at tp = 1")}


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
    weights = decode_weights(kern, gen, False)
    # Activations and outputs of the three batch sizes live in one staging buffer each (host pinned
    # and device), so that the end-to-end step moves them with one copy per direction.
    x_all_host = torch.randn((sum(MS), K), dtype=torch.float16).pin_memory()
    x_all = x_all_host.cuda()
    xs, row = {}, 0
    for m in MS:
        xs[m] = x_all[row:row + m]
        row += m
    o_elems = sum(m * n for m in MS for n in (4096, 11008))
    o_all = torch.zeros((o_elems,), dtype=torch.float16, device="cuda")
    o_all_host = torch.zeros((o_elems,), dtype=torch.float16).pin_memory()
    outs, off = {}, 0
    for m in MS:
        for n in (4096, 11008):
            outs[(m, n)] = o_all[off:off + m * n].view(m, n)
            off += m * n

    def step():
        for m in MS:
            x = xs[m]
            for layer in weights:
                for n, q, s, _ in layer:
                    kern.matmul_nt_fp16u8(outs[(m, n)], x, q, s, BS)

    # The step is launch-bound when driven from Python (about 14 us per call), so the
    # launches of one step are captured once into a CUDA graph and replayed.
    launches0 = kern.launch_count()
    step()
    launches_per_step = kern.launch_count() - launches0
    kernel_name = kern.last_kernel().name
    replay, graph = graphed(step)
    stream_fn = torch.cuda.current_stream
    timed = make_timer(stream_fn, world)

    def step_e2e():
        x_all.copy_(x_all_host, non_blocking=True)
        replay()
        o_all_host.copy_(o_all, non_blocking=True)
        stream_fn().synchronize()  # the caller reads the result on the host every step

    for _ in range(max(args.warmup, 3)):
        replay()
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid)
    if rank == 0:
        sampler.start()
    ms_runs = [timed(replay, args.steps) for _ in range(args.repeats)]
    ms = float(np.median(ms_runs))
    # per-M breakdown (each its own graph and event pair)
    per_m, per_m_kernel = {}, {}
    for m in MS:
        def one_m(m=m):
            for layer in weights:
                for n, q, s, _ in layer:
                    kern.matmul_nt_fp16u8(outs[(m, n)], xs[m], q, s, BS)
        rm, gm = graphed(one_m)
        per_m_kernel[f"M={m}"] = kern.last_kernel().name
        t = float(np.median([timed(rm, args.steps) for _ in range(max(3, args.repeats // 2))]))
        b = LAYERS * sum(gemv_bytes(m, n) for n in NS)
        per_m[f"M={m}"] = round(b * args.steps / (t * 1e-3) / 1e9, 1)
    for _ in range(2):
        step_e2e()
    e2e_runs = [timed(step_e2e, args.steps) for _ in range(max(3, args.repeats // 2))]
    ms_e2e = float(np.median(e2e_runs))
    kern.device_status()
    extra = {}
    if rank == 0 and world == 1 and not args.no_extra:
        for name, fn in (("fp16_gemm", lambda: extra_fp16_gemm(kern, timed, args)),
                         ("u8_prefill", lambda: extra_u8_prefill(kern, timed, args)),
                         ("u8_zero_points", lambda: extra_zero_points(kern, timed, args, xs, outs)),
                         ("u8_grouped", lambda: extra_grouped(kern, timed, args, weights, xs, outs)),
                         ("llama7b_decode_b1", lambda: extra_llama7b(kern, 1)),
                         ("llama7b_decode_b16", lambda: extra_llama7b(kern, 16)),
                         ("clip_vit_l14_b64", lambda: extra_clip(kern, 64)),
                         ("tp1_65b", lambda: extra_tp1_65b(kern, timed, args))):
            try:
                extra[name] = fn()
            except Exception as e:  # noqa: BLE001 - reported in the line; the headline stands
                extra[name] = {"error": repr(e)}
                torch.cuda.empty_cache()
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
    ratio, ratio_kernel = ncu_traffic_ratio()
    line = {
        "metric": "u8_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "repeats": spread([t / args.steps for t in ms_runs]),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps, "repeats": spread([t / args.steps for t in e2e_runs])},
        "gpu_launches": int(launches_per_step * args.steps),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak,
                     # DRAM bytes per launch: an ncu capture of one small launch of the same kernel
                     # gives measured / algorithmic bytes; traffic grows in proportion to the
                     # weights, so the average launch of the step is scaled by that ratio
                     "traffic": (bytes_step / max(launches_per_step, 1) * ratio) if ratio else None,
                     "traffic_unit": "bytes per launch (ncu capture of a small launch, scaled)",
                     "traffic_kernel": ratio_kernel,
                     "peak_kind": f"of {peak_kind}",
                     "kernel": "+".join(sorted(set(per_m_kernel.values()))) or kernel_name,
                     "per_m_gbs": per_m, "per_m_kernel": per_m_kernel,
                     "bytes_per_launch_avg": bytes_step / max(launches_per_step, 1)},
        "clocks": clocks,
        "note": "N = 1 runs configs[1] (weak scaling: every rank its own copy); N > 1 runs configs[4] "
                "(65B-shape, tensor-parallel, strong scaling), whose tp = 1 point is extra.tp1_65b",
    }
    if extra:
        line["extra"] = extra
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
    sh, M = LLAMA_65B, TP_M
    assert (sh.dim, sh.ffn, sh.block) == (TP_DIM, TP_FFN, TP_BLOCK)
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
        if use_peer:
            h.copy_(x)  # the residual stream starts from the step's input (it would otherwise grow without bound)
        for seg in replay:
            seg()
            if not use_peer:
                tp.all_reduce(part)
        if not use_peer:
            h.copy_(part)

    bytes_rank = tp_rank_bytes(world)
    timed = make_timer(torch.cuda.current_stream, world)

    def tp_check():
        """Outside the timed region: one row-split product reduced by the path under test against
        an fp32 sum of the ranks' partial products gathered with NCCL, and the same bits on every
        rank (MIN and MAX over ranks of the raw fp16 patterns agree)."""
        ly = layers[0]
        shared = torch.Generator(device=dev).manual_seed(99)  # the residual is replicated
        h0 = torch.randn((M, d), device=dev, generator=shared).half()
        got = h0.clone()
        if use_peer:
            ly.wo(got, att, residual=True)
        else:
            ly.wo(got, att, torch.zeros_like(got), residual=True)
        w = ly.wo.w
        deq = (w.q.float() - 127.5) * w.scales.float().repeat_interleave(w.block, dim=1)
        want = att.float() @ deq.t()
        dist.all_reduce(want)
        want += h0.float()
        max_rel = float(((got.float() - want).abs().max() / want.abs().max()).item())
        bits = got.view(torch.int16).to(torch.int32)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool(torch.equal(lo, hi))
        kern.device_status()
        return {"max_rel": max_rel, "same_bits": same, "tolerance": 1e-2,
                "what": "layer 0 o-projection + all-reduce + residual vs fp32 sum over ranks (NCCL)"}

    note("weights ready")
    check = tp_check()
    note(f"tp_check {check}")
    if check["max_rel"] > check["tolerance"] or not check["same_bits"]:
        if rank == 0:
            print(json.dumps({"metric": "u8_decode_gemv_hbm_gbs", "n_gpus": world, "tp_check": check,
                              "error": "tensor-parallel result check failed; nothing timed"}))
        dist.destroy_process_group()
        sys.exit(1)
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
    kern.device_status()  # no bounded wait ran out during warm-up
    note("warm-up done")
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid)
    if rank == 0:
        sampler.start()
    ms_runs = [timed(run, args.steps) for _ in range(args.repeats)]
    ms = float(np.median(ms_runs))
    note(f"timed {ms:.2f} ms")

    def run_e2e():
        x.copy_(x_host, non_blocking=True)
        run()
        h_host.copy_(h, non_blocking=True)
        stream.synchronize()

    run_e2e()
    e2e_runs = [timed(run_e2e, args.steps) for _ in range(max(3, args.repeats // 2))]
    ms_e2e = float(np.median(e2e_runs))
    kern.device_status()
    check_after = tp_check()
    clocks = sampler.stop() if rank == 0 else {}
    total_bytes = float(world * bytes_rank)
    if rank == 0:
        peak, peak_kind = measured_peak()
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        line = {
            "metric": "u8_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": tp_config(world, use_peer), "cuda_graph": graph is not None,
            "repeats": spread([t / args.steps for t in ms_runs]),
            "tp_check": check, "tp_check_after_timing": check_after,
            "e2e": {"value": total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": M * d * 2, "d2h_bytes_per_step": M * d * 2,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches_per_step * args.steps),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                         "kernel": "u8_ksplit_kernel (k = 8192) / u8_ring_kernel" + (" with the all-reduce fused in" if use_peer and args.fused_ar
                                                     else " + allreduce_oneshot_kernel" if use_peer else " + ncclAllReduce")},
            "clocks": clocks,
            "note": "N > 1 is configs[4] (strong scaling); its tp = 1 point is extra.tp1_65b of the N = 1 line, "
                    "which itself runs configs[1]",
        }
        print(json.dumps(line))
    dist.destroy_process_group()


def run_profile_case(args):
    """Small, self-terminating cases for `ncu` captures (a few hundred MB on the device).

    u8 : the decode kernel over 12 distinct [--n,4096] u8 weights (201 MB at n = 4096, larger
         than L2), two passes, m = --m (m > 32 reaches the prefill kernel).
    fattn: the fused attention kernel, 1024 heads of 257 x 64 (the CLIP encoder's shape at batch
         64) when --m is 64, else --m heads of 512 x 128 with the causal mask (LLaMA prefill).
    f16: the tensor-core GEMM, [m,4096] x [4096,4096]^T over 6 distinct weights, m = --m.
    attn: the decode-attention kernel, batch --m, 32 heads x 128, 600 of 640 cached positions.
    """
    import torch

    from adrastea_b200 import GpuKernels, Kernel, TensorView
    torch.cuda.set_device(0)
    kern = GpuKernels(0)
    if args.kernel:
        kern.force_kernel(Kernel[args.kernel])
    m = args.m
    if args.profile_case == "u8":
        ws = [(torch.randint(0, 256, (args.n, K), dtype=torch.uint8, device="cuda"),
               (torch.rand((args.n, K // BS), device="cuda") * 0.009 + 0.001).half()) for _ in range(12)]
        x = torch.randn((m, K), dtype=torch.float16, device="cuda")
        o = torch.zeros((m, args.n), dtype=torch.float16, device="cuda")
        for _ in range(2):
            for q, s in ws:
                kern.matmul_nt_fp16u8(o, x, q, s, BS)
    elif args.profile_case == "fattn":
        import math
        if m == 64:
            B, S, H, hd = 64, 257, 16, 64
            t = [torch.randn((S * B, H * hd), device="cuda").half() for _ in range(4)]
            from adrastea_b200 import TensorLayout
            lay = TensorLayout.new((B * H, S, hd), (hd, B * H * hd, 1))
            v = [TensorView(x, lay) for x in t]
            for _ in range(3):
                kern.attention_f16(v[3], v[0], v[1], v[2], 1.0 / math.sqrt(hd))
        else:
            H, S, hd = m, 512, 128
            t = [torch.randn((H, S, hd), device="cuda").half() for _ in range(4)]
            from adrastea_b200 import MatmulMask
            for _ in range(3):
                kern.attention_f16(TensorView.of(t[3]), TensorView.of(t[0]), TensorView.of(t[1]),
                                   TensorView.of(t[2]), 1.0 / math.sqrt(hd), MatmulMask.Causal)
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
    ap.add_argument("--repeats", type=int, default=10, help="repetitions of the timed loop (median reported)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the fp16 / zero-point / model extras")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream-ordered launches")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: do not capture the step in a CUDA graph")
    ap.add_argument("--fused-ar", action="store_true",
                    help="N > 1: all-reduce inside the row-split GEMV kernel instead of a kernel of its own")
    ap.add_argument("--nccl", action="store_true",
                    help="N > 1: reduce the row-split products with NCCL instead of the library's peer-memory kernel")
    ap.add_argument("--profile-case", default=None, choices=["u8", "f16", "attn", "fattn"],
                    help="run a small fixed case of one kernel family and exit (for ncu captures)")
    ap.add_argument("--kernel", default=None, help="--profile-case: pin a kernel family by name, e.g. U8Ring")
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
