"""Compile the CUDA library in-tree for sm_100a.

``python -m riftco_transformer_b200.build`` (or ``build_library()``) runs nvcc
on every ``csrc/*.cu`` and links ``riftco_transformer_b200/lib/libriftco_b200.so``.
nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libriftco_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


def _run(cmd: list[str], verbose: bool) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted((ROOT / "include").glob("*.h"))
    newest_header = max(h.stat().st_mtime for h in headers)
    OBJ.mkdir(parents=True, exist_ok=True)
    # B2_NVCC_EXTRA: extra nvcc flags (space separated), e.g. a -D switch for an instrumented build.
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else []) + os.environ.get("B2_NVCC_EXTRA", "").split()

    def compile_one(src: Path) -> tuple[Path, bool]:
        obj = OBJ / (src.stem + ".o")
        stale = (force or ptxas_info or not obj.exists()
                 or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header))
        if stale:
            out = _run([_nvcc(), *flags, "-c", str(src), "-o", str(obj)], verbose)
            if ptxas_info:
                print(out)
        return obj, stale

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        results = list(pool.map(compile_one, sources))
    objects = [o for o, _ in results]
    if any(stale for _, stale in results) or not LIB.exists():
        _run([_nvcc(), "-shared", "-o", str(LIB), *map(str, objects),
              "-gencode", "arch=compute_100a,code=sm_100a", "-lcuda"], verbose)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
