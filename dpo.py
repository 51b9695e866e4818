#!/usr/bin/env python3
"""WarpState DPO entry point.

    torchrun --standalone --nproc-per-node N dpo.py --config plan.json --work-dir ... --data-dir ... \
        --weights sft-model.pt --tokenizer tokenizer.model --reference-cache-dir ...

Same command line and file formats as the reference's dpo.py; the implementation lives in
`warpstate_ai_b200.train.dpo`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from warpstate_ai_b200.data.dpo import collate_pairs, encode_pair, load_data  # noqa: E402,F401
from warpstate_ai_b200.train.dpo import (DEFAULTS, FORMAT, evaluate, learning_rate, load_model, load_plan,  # noqa: E402,F401
                                         main, preference_metrics, prepare_reference, train, training_update,
                                         validate_cache)

if __name__ == "__main__":
    main()
