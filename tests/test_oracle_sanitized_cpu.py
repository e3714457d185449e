"""The C restatement under AddressSanitizer and UndefinedBehaviorSanitizer: the golden-vector
tests (edge layouts, odd tails, 33-block double quantisation, paged attention with poison) run in
a child interpreter that loads the sanitised build of oracle/riftco_oracle.c. A checker that reads
or writes out of bounds would otherwise be able to agree with itself."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _runtime(name: str) -> str | None:
    try:
        path = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True, timeout=30).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        return None
    return path if os.path.isabs(path) and os.path.exists(path) else None


def test_golden_vectors_under_asan_and_ubsan():
    asan = _runtime("libasan.so")
    if asan is None:
        pytest.skip("no AddressSanitizer runtime next to gcc")
    env = dict(os.environ, RIFTCO_ORACLE_SANITIZE="1", LD_PRELOAD=asan,
               ASAN_OPTIONS="detect_leaks=0:halt_on_error=1:abort_on_error=0",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1", OMP_NUM_THREADS="1")
    proc = subprocess.run([sys.executable, "-m", "pytest", str(ROOT / "tests" / "test_oracle_golden.py"), "-x", "-q",
                           "-p", "no:cacheprovider"], env=env, capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    tail = proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.returncode == 0, tail
    assert "AddressSanitizer" not in tail and "runtime error" not in tail, tail
