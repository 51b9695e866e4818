#!/usr/bin/env python3
"""WarpState assistant-only SFT entry point.

    torchrun --standalone --nproc-per-node N posttrain.py --config plan.json --work-dir ... \
        --data-dir ... --weights model.pt --tokenizer tokenizer.model

Same command line and file formats as the reference's posttrain.py; the implementation lives in
`warpstate_ai_b200.train.sft`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from warpstate_ai_b200.data.sft import collate, encode_messages, update_indices  # noqa: E402,F401
from warpstate_ai_b200.train.sft import (DEFAULTS, FORMAT, evaluate, learning_rate, load_plan, main,  # noqa: E402,F401
                                         shared_pipeline_lock, source_identity, token_weighted_loss, train,
                                         training_update, validate_paths, validate_resume)
from warpstate_ai_b200.utils.io import atomic_json, digest  # noqa: E402,F401

if __name__ == "__main__":
    main()
