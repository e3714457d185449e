"""Build the CPU checkers (test infrastructure, never the product path).

Two shared libraries come out of this script:

* ``oracle/_build/libriftco_oracle.so`` - the plain C restatement in
  ``riftco_oracle.c`` (gcc, ``-ffp-contract=off``, OpenMP). Always built.
* ``oracle/_ref/libriftco_ref.so`` - the reference project's own CPU sources,
  compiled where they lie in a checkout of quangng2000/riftco-transformer
  together with ``ref_bridge.cpp``. Built only when such a checkout is
  present; only the binary is kept, no reference source is copied.

The reference sources compiled are the ones its own build lists for the core
library without accelerators (CMakeLists.txt:87-104,
cmake/RiftcoTransformerBackends.cmake:1-14 plus the three accelerator stubs):
backend registry and dispatchers, the CPU adapter, the reference loops,
quantisation and tensor storage. They need nothing but g++ (C++20) and libm.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD_DIR = HERE / "_build"
REF_DIR = HERE / "_ref"
ORACLE_LIB = BUILD_DIR / "libriftco_oracle.so"
REF_LIB = REF_DIR / "libriftco_ref.so"
REF_B200_LIB = REF_DIR / "libriftco_ref_b200.so"

DEFAULT_REFERENCE_DIR = "/root/reference"

# Paths inside the reference checkout.
REFERENCE_SOURCES = [
    "src/core/backend/adapters/cpu/adapter.cpp",
    "src/core/backend/adapters/cuda/stub.cpp",
    "src/core/backend/adapters/metal/stub.cpp",
    "src/core/backend/adapters/tpu/stub.cpp",
    "src/core/backend/attention/dispatch.cpp",
    "src/core/backend/attention/reference/flash_causal.cpp",
    "src/core/backend/attention/reference/materialized_causal.cpp",
    "src/core/backend/attention/reference/paged_decode.cpp",
    "src/core/backend/nn/dispatch.cpp",
    "src/core/backend/nn/quantized_linear/dispatch.cpp",
    "src/core/backend/nn/quantized_linear/reference/operations.cpp",
    "src/core/backend/nn/reference/operations.cpp",
    "src/core/backend/optim/adam/dispatch.cpp",
    "src/core/backend/optim/adam/reference/update.cpp",
    "src/core/backend/registry.cpp",
    "src/core/quantization/nf4.cpp",
    "src/core/quantization/quantized_weight.cpp",
    "src/core/tensor/detail/validation.cpp",
    "src/core/tensor/elementwise.cpp",
    "src/core/tensor/indexing.cpp",
    "src/core/tensor/layout.cpp",
    "src/core/tensor/layout_ops.cpp",
    "src/core/tensor/matmul.cpp",
    "src/core/tensor/reductions.cpp",
    "src/core/tensor/softmax.cpp",
    "src/core/tensor/storage.cpp",
]

# -O2 is the reference's own release level; -ffp-contract=off keeps every
# multiply and add separately rounded on any host ISA.
CXXFLAGS = ["-std=c++20", "-O2", "-ffp-contract=off", "-fPIC", "-pthread"]


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(
            "command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr
        )


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.stat().st_mtime <= t for s in sources)


def build_oracle(force: bool = False) -> Path:
    """Compile the C restatement; returns the library path."""
    sources = [HERE / "riftco_oracle.c", HERE / "riftco_oracle.h"]
    if not force and _newer(ORACLE_LIB, sources):
        return ORACLE_LIB
    BUILD_DIR.mkdir(exist_ok=True)
    _run([
        "gcc", "-std=c11", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC",
        "-shared", "-o", str(ORACLE_LIB), str(HERE / "riftco_oracle.c"), "-lm",
    ])
    return ORACLE_LIB


def reference_dir() -> Path | None:
    root = Path(os.environ.get("RIFTCO_REFERENCE_DIR", DEFAULT_REFERENCE_DIR))
    probe = root / "src/core/backend/nn/quantized_linear/reference/operations.cpp"
    return root if probe.exists() else None


def build_reference(force: bool = False) -> Path | None:
    """Compile the reference's own CPU core + bridge; None without a checkout."""
    root = reference_dir()
    if root is None:
        return REF_LIB if REF_LIB.exists() else None
    bridge = HERE / "ref_bridge.cpp"
    sources = [root / s for s in REFERENCE_SOURCES] + [bridge]
    if not force and _newer(REF_LIB, sources):
        return REF_LIB
    REF_DIR.mkdir(exist_ok=True)
    obj_dir = REF_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    includes = ["-I", str(root / "include"), "-I", str(root / "src")]

    def compile_one(src: Path) -> Path:
        tag = hashlib.sha1(str(src).encode()).hexdigest()[:12]
        obj = obj_dir / f"{src.stem}-{tag}.o"
        if force or not obj.exists() or obj.stat().st_mtime < src.stat().st_mtime:
            _run(["g++", *CXXFLAGS, *includes, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objects = list(pool.map(compile_one, sources))
    _run([
        "g++", "-shared", "-pthread", "-o", str(REF_LIB), *map(str, objects),
        "-Wl,--no-undefined",
    ])
    return REF_LIB


def build_reference_with_b200_adapter(force: bool = False) -> Path | None:
    """The reference's core with its CUDA seam defined by
    riftco_transformer_b200/adapter/cuda_b200_adapter.cpp instead of adapters/cuda/stub.cpp,
    linked against the product library: lets the tests drive the reference's own
    dispatch layer on ExecutionBackend::Cuda. None without a checkout or without
    the product library."""
    root = reference_dir()
    product = HERE.parent / "riftco_transformer_b200" / "lib" / "libriftco_b200.so"
    if root is None or not product.exists():
        return REF_B200_LIB if REF_B200_LIB.exists() else None
    if build_reference(force) is None:
        return None
    adapter = HERE.parent / "riftco_transformer_b200" / "adapter" / "cuda_b200_adapter.cpp"
    stub = root / "src/core/backend/adapters/cuda/stub.cpp"
    sources = [root / s for s in REFERENCE_SOURCES if (root / s) != stub] + [HERE / "ref_bridge.cpp"]
    if not force and _newer(REF_B200_LIB, sources + [adapter, product]):
        return REF_B200_LIB
    obj_dir = REF_DIR / "obj"
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    includes = ["-I", str(root / "include"), "-I", str(root / "src"), "-I", str(HERE.parent / "include"),
                "-I", str(cuda / "include")]
    adapter_obj = obj_dir / "cuda_b200_adapter.o"
    _run(["g++", *CXXFLAGS, *includes, "-c", str(adapter), "-o", str(adapter_obj)])
    objects = []
    for src in sources:   # compiled by build_reference() above
        tag = hashlib.sha1(str(src).encode()).hexdigest()[:12]
        objects.append(obj_dir / f"{src.stem}-{tag}.o")
    _run([
        "g++", "-shared", "-pthread", "-o", str(REF_B200_LIB), *map(str, objects), str(adapter_obj),
        "-L", str(product.parent), "-lriftco_b200", "-L", str(cuda / "lib64"), "-lcudart",
        "-Wl,-rpath,$ORIGIN/../../riftco_transformer_b200/lib", "-Wl,-rpath," + str(cuda / "lib64"),
        "-Wl,--no-undefined",
    ])
    return REF_B200_LIB


def main() -> None:
    force = "--force" in sys.argv
    print("oracle:", build_oracle(force))
    print("reference:", build_reference(force))
    print("reference + B200 adapter:", build_reference_with_b200_adapter(force))


if __name__ == "__main__":
    main()
