#!/usr/bin/env bash
# Guardian that waits for the pretraining job to finish, seals its archive and starts SFT.
set -euo pipefail
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
cd "$WARPSTATE_REPO"
exec "$WARPSTATE_PYTHON" -B -m warpstate_ai_b200.orchestration.handoff --stage sft \
  --config "${WARPSTATE_POSTTRAIN_PLAN:-$WARPSTATE_REPO/configs/posttrain_plan.json}" "$@"
