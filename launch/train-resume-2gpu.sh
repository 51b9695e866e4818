#!/usr/bin/env bash
# Resume an existing run on two GPUs (micro-batch 4 x accumulation 8 x 2 ranks keeps the 131072-token
# update of the one-GPU preset; --reconfigure accepts the world-size change, reference
# run_40b.py:544-555).  Refuses to start without a full checkpoint.
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
export CUDA_VISIBLE_DEVICES="${CUDA_VISIBLE_DEVICES-0,1}"
cd "$WARPSTATE_REPO"
if [[ ! -s "$WARPSTATE_WORK/run/latest.pt" ]]; then
  printf '%s\n' "Resume requires the verified full checkpoint at $WARPSTATE_WORK/run/latest.pt." >&2
  exit 1
fi
exec "$WARPSTATE_PYTHON" -u -m warpstate_ai_b200.orchestration.launcher \
  --processes 2 --work-dir "$WARPSTATE_WORK" -- \
  --no-bootstrap --stage train --reconfigure \
  --seq-len 2048 --micro-batch 4 --grad-accum 8 \
  --no-activation-checkpointing --bf16-residuals --async-checkpoint \
  --vram-limit-gib 88 --vram-headroom-gib 3 \
  --workers 4 --eval-batches 8 --eval-micro-batch 1 --eval-every 100 --save-every 100 \
  "$@"
