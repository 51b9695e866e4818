#!/usr/bin/env python3
"""`python ops/benchmark_gemm.py ...` -- isolated GEMM timing on the production shapes.

Thin entry point kept at the path users of the original project expect; the implementation is
`warpstate_ai_b200.bench.gemm_bench`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from warpstate_ai_b200.bench.gemm_bench import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
