"""Builds librichkv.so (the CUDA kernels + C ABI + host control plane) in-tree for sm_100a.

    python -m richengine_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. Objects are rebuilt only when a source or
header is newer. The CUDA runtime is linked statically and the driver API is
resolved at run time, so the library loads on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
OBJ = PACKAGE / "build"
LIBRARY = PACKAGE / "librichkv.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++20",
    "-Xcompiler", "-fPIC,-Wall", "--expt-relaxed-constexpr",
    # bit-exact quantisation: IEEE division/sqrt, no flush-to-zero, and no
    # fused multiply-add contraction across the (x*range)/amax recipe
    "--prec-div=true", "--prec-sqrt=true", "--ftz=false", "--fmad=true",
    f"-I{ROOT / 'include'}",
    *os.environ.get("RICHKV_NVCC_FLAGS", "").split(),
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted((CSRC / "host").glob("*.cpp"))


def _newest_header() -> float:
    headers = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list((ROOT / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    header_time = _newest_header()
    jobs = []
    objects = []
    for source in sources():
        obj = OBJ / (source.stem + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(source.stat().st_mtime, header_time)
        if stale:
            command = [nvcc, *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
            if source.suffix == ".cpp":
                command[1:1] = ["-x", "cu"]
            jobs.append(command)

    def run(command):
        if verbose:
            print(" ".join(command), flush=True)
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(command)}\n{done.stdout}\n{done.stderr}")
        if verbose and done.stderr.strip():
            print(done.stderr)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(run, jobs))
    if jobs or not LIBRARY.exists():
        run([nvcc, "-shared", "-cudart", "static", "-o", str(LIBRARY), *map(str, objects),
             "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"])
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
