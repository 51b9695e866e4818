#!/usr/bin/env bash
# Chat with a sealed post-training (SFT / DPO) snapshot.
set -euo pipefail
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
cd "$WARPSTATE_REPO"
exec "$WARPSTATE_PYTHON" -B -m warpstate_ai_b200.serve.posttrain_chat "$@"
