#!/usr/bin/env bash
# A GPU shared with other jobs: small micro-batch, activation recomputation, 40 GiB cap.
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
export CUDA_VISIBLE_DEVICES="${CUDA_VISIBLE_DEVICES-0}"
cd "$WARPSTATE_REPO"
exec "$WARPSTATE_PYTHON" -u -m warpstate_ai_b200.orchestration.launcher \
  --processes 1 --work-dir "$WARPSTATE_WORK" -- \
  --no-bootstrap --stage train --reconfigure \
  --seq-len 2048 --micro-batch 2 --grad-accum 32 --activation-checkpointing \
  --vram-limit-gib 40 --vram-headroom-gib 3 \
  --workers 2 --eval-batches 8 --eval-micro-batch 1 --eval-every 100 --save-every 100 \
  "$@"
