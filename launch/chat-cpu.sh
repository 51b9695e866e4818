#!/usr/bin/env bash
# CPU-only chat: leaves every GPU to the training job.
set -euo pipefail
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
export CUDA_VISIBLE_DEVICES=""
export OMP_NUM_THREADS=16 MKL_NUM_THREADS=16
cd "$WARPSTATE_REPO"
exec "$WARPSTATE_PYTHON" -B -u chat.py "$@"
