#!/usr/bin/env python3
"""`python ops/dpo_handoff.py ...` -- guardian for the SFT -> DPO hand-off; adds `--stage dpo`.

Thin entry point kept at the path users of the original project expect; the implementation is
`warpstate_ai_b200.orchestration.handoff`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from warpstate_ai_b200.orchestration.handoff import main  # noqa: E402

if __name__ == "__main__":
    argv = sys.argv[1:]
    if "--stage" not in argv:
        argv = ['--stage', 'dpo'] + argv
    sys.exit(main(argv))
