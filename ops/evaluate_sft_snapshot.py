#!/usr/bin/env python3
"""`python ops/evaluate_sft_snapshot.py ...` -- full-hold-out evaluation of a sealed snapshot.

Thin entry point kept at the path users of the original project expect; the implementation is
`warpstate_ai_b200.train.evaluate_snapshot`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from warpstate_ai_b200.train.evaluate_snapshot import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
