"""Runs the small-batch cases of the decode-batch linear with B2_DECODE_IMPL=tmem (set by the
caller), i.e. on the fp16 form of the persistent tensor-core kernel, against the oracle at the
decode tolerance of 2e-3. Started by tests/test_gpu_decode_linear.py."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main() -> None:
    assert os.environ.get("B2_DECODE_IMPL") == "tmem"
    import oracle
    import riftco_transformer_b200 as b2
    from decode_linear_cases import CASES, SMALL_ROW_CASES, run_case
    assert b2.is_available(), b2.unavailability_reason()
    port = oracle.port()
    for case in SMALL_ROW_CASES:
        run_case(b2, port, case, 2e-3)
    for case in CASES[:3]:
        run_case(b2, port, case, 1e-2)
    print("decode linear worker ok")


if __name__ == "__main__":
    main()
