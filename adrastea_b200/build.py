"""Build recipe of the CUDA library (nvcc, sm_100a only, in-tree output).

The shared object is written next to this file so that it travels with the
source tree; nothing is cached outside the repository.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libadrastea_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "adrastea_b200.h"]


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + _headers()
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into libadrastea_b200.so (sm_100a).

    Each source becomes an object file under csrc/build/ (compiled in parallel, reused while
    neither the source nor any header is newer), then everything is linked into the library.
    """
    if not force and not _stale():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor
    obj_dir = CSRC / "build"
    obj_dir.mkdir(exist_ok=True)
    hdr_time = max(h.stat().st_mtime for h in _headers())
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src: Path):
        obj = obj_dir / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_time):
            return obj, ""
        cmd = [_nvcc(), *compile_flags, "-c", "-o", str(obj), str(src)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n" + res.stdout + res.stderr)
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    if verbose:
        for _, log in results:
            if log:
                print(log)
    # drop objects whose source is gone
    keep = {o for o, _ in results}
    for o in obj_dir.glob("*.o"):
        if o not in keep:
            o.unlink()
    tmp = LIB_PATH.with_suffix(".so.tmp")  # linked aside, then moved into place in one step
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(tmp), *map(str, sorted(keep))]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + res.stdout + res.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
