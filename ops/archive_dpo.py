#!/usr/bin/env python3
"""`python ops/archive_dpo.py ...` -- seal / verify the archive of a completed DPO run.

Thin entry point kept at the path users of the original project expect; the implementation is
`warpstate_ai_b200.orchestration.archive_dpo`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from warpstate_ai_b200.orchestration.archive_dpo import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
