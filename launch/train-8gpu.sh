#!/usr/bin/env bash
# One HGX node, 8 x B200, replicated data parallel: micro-batch 8 x accumulation 1 per GPU keeps the
# 131072-token update; gradients are reduced by the in-kernel all-reduce over NVLink, and with
# WARPSTATE_SHARD_OPTIMIZER=1 AdamW state is sharded and the update broadcasts its own weights.
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
cd "$WARPSTATE_REPO"
extra=()
if [[ "${WARPSTATE_SHARD_OPTIMIZER:-0}" == 1 ]]; then extra+=(--shard-optimizer); fi
exec "$WARPSTATE_PYTHON" -u -m warpstate_ai_b200.orchestration.launcher \
  --processes "${WARPSTATE_PROCESSES:-8}" --work-dir "$WARPSTATE_WORK" -- \
  --no-bootstrap --stage train --reconfigure \
  --seq-len 2048 --micro-batch 8 --grad-accum 1 \
  --no-activation-checkpointing --async-checkpoint --grad-sync fused \
  --vram-limit-gib 150 --vram-headroom-gib 3 \
  --workers 4 --eval-batches 8 --eval-micro-batch 1 --eval-every 100 --save-every 100 \
  "${extra[@]}" "$@"
