#!/usr/bin/env python3
"""WarpState pretraining entry point (corpus preparation + training).

    python run_40b.py --from-scratch --work-dir work --config configs/warpstate_2b.json ...
    torchrun --standalone --nproc-per-node 8 run_40b.py --stage train ...

Same command line as the reference's runner; the implementation lives in
`warpstate_ai_b200.train.pretrain`.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from warpstate_ai_b200.data.prepare import check_manifest, data_signature, is_holdout, prepare  # noqa: E402,F401
from warpstate_ai_b200.data.tokens import batches, update_slices  # noqa: E402,F401
from warpstate_ai_b200.train.pretrain import arguments, configure_memory, main, preflight, train  # noqa: E402,F401
from warpstate_ai_b200.train.signature import check_resume_signature, train_signature  # noqa: E402,F401
from warpstate_ai_b200.utils.io import digest, process_lock  # noqa: E402,F401

if __name__ == "__main__":
    main()
