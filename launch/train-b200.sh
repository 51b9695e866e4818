#!/usr/bin/env bash
# One B200: micro-batch 16 x accumulation 4 x 2048 tokens = 131072 tokens per update, activations
# kept (no recomputation), asynchronous checkpoints, 150 GiB allocator cap.
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
export CUDA_VISIBLE_DEVICES="${CUDA_VISIBLE_DEVICES-0}"
cd "$WARPSTATE_REPO"
exec "$WARPSTATE_PYTHON" -u -m warpstate_ai_b200.orchestration.launcher \
  --processes 1 --work-dir "$WARPSTATE_WORK" -- \
  --no-bootstrap --stage train --reconfigure \
  --seq-len 2048 --micro-batch 16 --grad-accum 4 \
  --no-activation-checkpointing --async-checkpoint \
  --vram-limit-gib 150 --vram-headroom-gib 3 \
  --workers 4 --eval-batches 8 --eval-micro-batch 1 --eval-every 100 --save-every 50 \
  "$@"
