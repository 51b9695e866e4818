#!/usr/bin/env bash
# Tokenise the pretraining corpus on the CPU at low priority (no GPU is touched).
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
export CUDA_VISIBLE_DEVICES=""
export OMP_NUM_THREADS=1 OPENBLAS_NUM_THREADS=1 MKL_NUM_THREADS=1
export HF_HUB_DOWNLOAD_TIMEOUT=120 HF_HUB_ETAG_TIMEOUT=30
cd "$WARPSTATE_REPO"
exec /usr/bin/nice -n 10 "$WARPSTATE_PYTHON" -u -m warpstate_ai_b200.data.prepare_entry \
  --no-bootstrap --stage prepare --work-dir "$WARPSTATE_WORK" \
  --train-tokens "${WARPSTATE_TRAIN_TOKENS:-40000000000}" --val-tokens 1048576 --workers "${WARPSTATE_PREPARE_WORKERS:-16}" "$@"
