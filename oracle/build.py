"""Build the CPU checkers (test infrastructure, never the product path).

Two shared libraries come out of this script:

* ``oracle/_build/libriftco_oracle.so`` - the plain C restatement in
  ``riftco_oracle.c`` (gcc, ``-ffp-contract=off``, OpenMP). Always built.
* ``oracle/_ref/libriftco_ref.so`` - the reference project's own CPU sources,
  compiled where they lie in a checkout of quangng2000/riftco-transformer
  together with ``ref_bridge.cpp``. Built only when such a checkout is
  present; only the binary is kept, no reference source is copied.

The reference sources compiled are the ones its own build lists for the CPU
library (CMakeLists.txt:87-135, cmake/RiftcoTransformerBackends.cmake:1-14) plus
the three accelerator stubs and, for the canonical packed-model-state stream,
the translation units of its C API (CMakeLists.txt:363-377) with the symbolic
compiler, lowering, analysis and programmed-model sources those link against.
They need nothing but g++ (C++20), pthreads and libm: no cmake, no generated
code, no external library. The checkout is found through the
RIFTCO_REFERENCE_DIR environment variable, else as a directory named
``reference`` beside this repository.
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
ORACLE_SAN_LIB = BUILD_DIR / "libriftco_oracle_san.so"
REF_LIB = REF_DIR / "libriftco_ref.so"
REF_B200_LIB = REF_DIR / "libriftco_ref_b200.so"

# Paths inside the reference checkout: the CPU library ...
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
    "src/artifacts/state.cpp",
    "src/core/autograd/checkpoint.cpp",
    "src/core/autograd/custom_gradient.cpp",
    "src/core/autograd/graph.cpp",
    "src/core/autograd/operations.cpp",
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
    "src/data/token_batch.cpp",
    "src/data/tokenizer.cpp",
    "src/model/causal_self_attention.cpp",
    "src/model/decoder_only_transformer.cpp",
    "src/model/feed_forward.cpp",
    "src/model/grouped_query_attention.cpp",
    "src/model/llama_mistral_transformer.cpp",
    "src/model/rotary_embedding.cpp",
    "src/model/swiglu.cpp",
    "src/model/transformer_block.cpp",
    "src/optim/adam.cpp",
    "src/nn/activations.cpp",
    "src/nn/embedding.cpp",
    "src/nn/initialization.cpp",
    "src/nn/layer_norm.cpp",
    "src/nn/linear.cpp",
    "src/nn/low_rank_adapter.cpp",
    "src/nn/loss.cpp",
    "src/nn/module.cpp",
    "src/nn/parameter.cpp",
    "src/nn/quantized_linear.cpp",
    "src/nn/rms_norm.cpp",
    "src/stages/serving/config.cpp",
    "src/stages/serving/cache/contiguous_kv_cache.cpp",
    "src/stages/serving/cache/page_storage.cpp",
    "src/stages/serving/cache/page_table_cache.cpp",
    "src/stages/serving/cache/paged_kv_cache.cpp",
    "src/stages/serving/cache/validation.cpp",
    "src/stages/serving/generation.cpp",
    "src/stages/serving/stack.cpp",
]
# ... and its C API with what that links against (every .cpp of these directories).
REFERENCE_SOURCE_DIRS = ["src/c_api", "src/programmed", "src/compiler/cajal", "src/lowering", "src/analysis"]


def reference_sources(root: Path) -> list[Path]:
    extra = sorted(p for d in REFERENCE_SOURCE_DIRS for p in (root / d).glob("*.cpp"))
    return [root / s for s in REFERENCE_SOURCES] + extra


# -O2 is the reference's own release level; -ffp-contract=off keeps every
# multiply and add separately rounded on any host ISA.
CXXFLAGS = ["-std=c++20", "-O2", "-ffp-contract=off", "-fPIC", "-pthread", "-DRIFTCO_TRANSFORMER_C_EXPORTS"]


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


def build_oracle(force: bool = False, sanitize: bool = False) -> Path:
    """Compile the C restatement; returns the library path. `sanitize` builds a second library
    with AddressSanitizer and UndefinedBehaviorSanitizer (single-threaded, -O1), which
    tests/test_oracle_sanitized_cpu.py runs the golden-vector tests against."""
    sources = [HERE / "riftco_oracle.c", HERE / "riftco_oracle.h"]
    target = ORACLE_SAN_LIB if sanitize else ORACLE_LIB
    if not force and _newer(target, sources):
        return target
    BUILD_DIR.mkdir(exist_ok=True)
    if sanitize:
        flags = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
                 "-fno-sanitize-recover=undefined"]
    else:
        flags = ["-O2", "-fopenmp"]
    _run([
        "gcc", "-std=c11", *flags, "-ffp-contract=off", "-fPIC",
        "-shared", "-o", str(target), str(HERE / "riftco_oracle.c"), "-lm",
    ])
    return target


def reference_dir() -> Path | None:
    where = os.environ.get("RIFTCO_REFERENCE_DIR")
    root = Path(where) if where else HERE.parent.parent / "reference"
    probe = root / "src/core/backend/nn/quantized_linear/reference/operations.cpp"
    return root if probe.exists() else None


def build_reference(force: bool = False) -> Path | None:
    """Compile the reference's own CPU core + bridge; None without a checkout."""
    root = reference_dir()
    if root is None:
        return REF_LIB if REF_LIB.exists() else None
    bridge = HERE / "ref_bridge.cpp"
    sources = reference_sources(root) + [bridge]
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
    sources = [s for s in reference_sources(root) if s != stub] + [HERE / "ref_bridge.cpp"]
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


REF_CONFORMANCE = REF_DIR / "quantized_linear_backend_tests"


def build_reference_conformance_tests(force: bool = False) -> Path | None:
    """The reference's own accelerator conformance executable for the packed-NF4 linear
    (tests/core/backend/test_quantized_linear_backend.cpp, target quantized_linear_backend_tests of
    tests/CMakeLists.txt:549-563), compiled where it lies with RIFTCO_TRANSFORMER_TEST_REQUIRE_CUDA=1
    and linked against the reference core that carries this repo's adapter: run on a B200 it fails
    unless the CUDA backend is available and matches the CPU oracle on the reference's fixtures.
    None without a checkout or without the adapter build."""
    root = reference_dir()
    lib = build_reference_with_b200_adapter(force)
    if root is None or lib is None:
        return REF_CONFORMANCE if REF_CONFORMANCE.exists() else None
    source = root / "tests/core/backend/test_quantized_linear_backend.cpp"
    if not force and _newer(REF_CONFORMANCE, [source, lib]):
        return REF_CONFORMANCE
    includes = ["-I", str(root / "include"), "-I", str(root / "src")]
    _run([
        "g++", *CXXFLAGS, *includes, "-DRIFTCO_TRANSFORMER_TEST_REQUIRE_CUDA=1", str(source),
        "-o", str(REF_CONFORMANCE), "-pthread", "-L", str(REF_DIR), "-lriftco_ref_b200",
        "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../riftco_transformer_b200/lib",
    ])
    return REF_CONFORMANCE


def main() -> None:
    force = "--force" in sys.argv
    print("oracle:", build_oracle(force))
    print("reference:", build_reference(force))
    print("reference + B200 adapter:", build_reference_with_b200_adapter(force))
    print("reference conformance executable:", build_reference_conformance_tests(force))


if __name__ == "__main__":
    main()
