#!/usr/bin/env python3
"""WarpState base-model probe (snapshot capture + interactive / one-shot generation).

Same command line as the reference's chat.py (plus ``--device cuda``); the implementation lives
in `warpstate_ai_b200.serve.chat`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from warpstate_ai_b200.serve.chat import (FORMAT, capture_latest, generate, load_model, main, reply,  # noqa: E402,F401
                                          resolve_snapshot)
from warpstate_ai_b200.serve.sampling import banned_ngram_tokens, sample_token  # noqa: E402,F401

if __name__ == "__main__":
    main()
