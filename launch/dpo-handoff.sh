#!/usr/bin/env bash
# Guardian that waits for SFT to finish, seals the SFT archive and starts DPO.
set -euo pipefail
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
cd "$WARPSTATE_REPO"
exec "$WARPSTATE_PYTHON" -B -m warpstate_ai_b200.orchestration.handoff --stage dpo \
  --config "${WARPSTATE_DPO_PLAN:-$WARPSTATE_REPO/configs/dpo_plan.json}" "$@"
