"""Generate the golden vectors of tests/golden/ by running the REFERENCE's own
device kernels (oracle/_ref/*.cubin, compiled unmodified from the reference
tree by oracle/Makefile) on the seeded cases of tests/cases.py.

Needs a GPU.  Run from the repository root:

    python tests/golden/make_golden.py [output_dir]

It writes reference_matmul_f16.npz, reference_u8.npz, reference_quantize.npz and
reference_rowops.npz (`--only rowops` writes just the last).  Inputs of the first
two are not stored; each entry carries a SHA-1 of the regenerated inputs so that
a drifting generator is caught.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import cases  # noqa: E402
from oracle import refcubin  # noqa: E402


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rowops(outdir: Path):
    """rms_norm, softmax_rows, rotary and elementwise_binary_2d_f16 of the reference
    (normalize.cu, rotary.cu, elementwise.cu) on tests/cases.rowop_cases()."""
    store = {}
    for name, c in cases.rowop_cases().items():
        if c["kind"] == "rms":
            x, w = dev(c["x"]), dev(c["w"])
            o = torch.zeros_like(x)
            ly, lx = c["x"].shape
            refcubin.rms_norm(o.data_ptr(), x.data_ptr(), w.data_ptr(), lx, ly, 1, lx, 1, lx, c["eps"])
        elif c["kind"] == "softmax":
            x = dev(c["x"])
            o = torch.zeros_like(x)
            heads, h, w_ = c["x"].shape
            refcubin.softmax_rows(o.data_ptr(), x.data_ptr(), heads, h, w_, c["temp"])
        elif c["kind"] == "rotary":
            x = dev(c["x"])
            o = torch.zeros_like(x)
            ly, lx = c["x"].shape
            refcubin.rotary(o.data_ptr(), x.data_ptr(), lx, ly, 1, lx, 1, lx, c["n_heads"],
                            c["pos_offset"], c["theta"])
        else:
            l, r = dev(c["left"]), dev(c["right"])
            o = torch.zeros_like(l)
            rows, cols = c["left"].shape
            refcubin.elementwise_binary_2d_f16(o.data_ptr(), l.data_ptr(), r.data_ptr(), rows, cols, c["op"])
        torch.cuda.synchronize()
        ins = [c[k] for k in ("x", "w", "left", "right") if k in c]
        store[name + "/digest"] = np.frombuffer(cases.digest(*ins).encode(), np.uint8)
        store[name + "/out"] = o.cpu().numpy()
    np.savez_compressed(outdir / "reference_rowops.npz", **store)
    print("row-op golden vectors written to", outdir)


def main(outdir: Path, only: str | None = None):
    assert refcubin.available(), "needs a GPU and oracle/_ref/*.cubin"
    outdir.mkdir(parents=True, exist_ok=True)
    rowops(outdir)
    if only == "rowops":
        return

    # ---- matmul_f16 (slow) and matmul_f16_fast ----
    store = {}
    for c in cases.matmul_cases():
        out0, lhs, rhs, bias = c.inputs()
        store[c.name + "/digest"] = np.frombuffer(cases.digest(out0, lhs, rhs, bias).encode(), np.uint8)
        for kern in ("matmul_f16", "matmul_f16_fast"):
            o, l, r, b = dev(out0.copy()), dev(lhs), dev(rhs), dev(bias)
            refcubin.matmul_f16(kern, o.data_ptr(), l.data_ptr(), r.data_ptr(), c.batches, c.m,
                                c.k, c.n, c.strides9(), b.data_ptr() if c.uses_bias() else None,
                                c.beta, c.scale, c.store, c.load, c.mask)
            torch.cuda.synchronize()
            store[f"{c.name}/{kern}"] = o.cpu().numpy()
    np.savez_compressed(outdir / "reference_matmul_f16.npz", **store)

    # ---- u8 kernels ----
    store = {}
    for c in cases.u8_cases():
        if c.zeros:
            continue  # the reference has no zero-point tensor
        out0, lhs, q, scales, _ = c.inputs()
        store[c.name + "/digest"] = np.frombuffer(cases.digest(out0, lhs, q, scales).encode(), np.uint8)
        o, l, qq, s = dev(out0.copy()), dev(lhs), dev(q), dev(scales)
        refcubin.matmul_nt_fp16u8(o.data_ptr(), l.data_ptr(), qq.data_ptr(), s.data_ptr(), c.m,
                                  c.p, c.n, c.block_size, c.beta)
        torch.cuda.synchronize()
        store[c.name + "/matmul_nt_fp16u8"] = o.cpu().numpy()
        if c.m % 16 == 0 and c.n % 128 == 0 and c.p % 256 == 0:
            o = dev(out0.copy())
            refcubin.matmul_nt_wmma_16x128x256_fp16u8(o.data_ptr(), l.data_ptr(), qq.data_ptr(),
                                                      s.data_ptr(), c.m, c.p, c.n, c.block_size,
                                                      c.beta)
            torch.cuda.synchronize()
            store[c.name + "/wmma_fp16u8"] = o.cpu().numpy()
        w = torch.empty((c.n, c.p), dtype=torch.float16, device="cuda")
        refcubin.dequantize_absmax_uint8(w.data_ptr(), s.data_ptr(), qq.data_ptr(), c.n, c.p,
                                         c.block_size)
        torch.cuda.synchronize()
        store[c.name + "/dequantize"] = w.cpu().numpy()
    np.savez_compressed(outdir / "reference_u8.npz", **store)

    # ---- quantiser and the fp16 WMMA kernels ----
    store = {}
    rng = np.random.default_rng(77)
    for name, rows, k, bs in (("q_128", 24, 512, 128), ("q_32", 8, 256, 32), ("q_256", 5, 512, 256)):
        x = (rng.standard_normal((rows, k)) * rng.uniform(0.01, 2.0, (rows, 1))).astype(np.float16)
        if name == "q_32":
            x[3, 64:96] = 0  # an all-zero group: scale 0, 0/0 in the code
        xd = dev(x)
        q = torch.zeros((rows, k), dtype=torch.uint8, device="cuda")
        s = torch.zeros((rows, k // bs), dtype=torch.float16, device="cuda")
        refcubin.quantize_absmax_uint8(q.data_ptr(), s.data_ptr(), xd.data_ptr(), rows, k, bs)
        torch.cuda.synchronize()
        store[name + "/x"] = x
        store[name + "/q"] = q.cpu().numpy()
        store[name + "/scales"] = s.cpu().numpy()
    for name, m, p, n, beta in (("nt_128x64x64", 128, 192, 128, 0.0), ("nt_128x64x64_beta", 256, 128, 64, 0.5),
                                ("nt_16x128x256", 32, 512, 256, 0.0), ("nt_16x128x256_beta", 16, 256, 128, 1.0)):
        lhs = (rng.standard_normal((m, p)) * 0.3).astype(np.float16)
        rhs = (rng.standard_normal((n, p)) * 0.3).astype(np.float16)
        out0 = (rng.standard_normal((m, n)) * 0.5).astype(np.float16)
        o, l, r = dev(out0.copy()), dev(lhs), dev(rhs)
        fn = refcubin.matmul_nt_wmma_128x64x64 if "128x64" in name else refcubin.matmul_nt_wmma_16x128x256
        fn(o.data_ptr(), l.data_ptr(), r.data_ptr(), m, p, n, beta)
        torch.cuda.synchronize()
        store[name + "/lhs"], store[name + "/rhs"], store[name + "/out0"] = lhs, rhs, out0
        store[name + "/out"] = o.cpu().numpy()
        store[name + "/beta"] = np.float32(beta)
    np.savez_compressed(outdir / "reference_quantize.npz", **store)
    print("golden vectors written to", outdir)


if __name__ == "__main__":
    argv = [a for a in sys.argv[1:] if a != "--only" and a != "rowops"]
    main(Path(argv[0]) if argv else ROOT / "tests" / "golden",
         "rowops" if "--only" in sys.argv else None)
