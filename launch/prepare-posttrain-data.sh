#!/usr/bin/env bash
# Render and tokenise the SFT / DPO datasets (CPU only).
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
export CUDA_VISIBLE_DEVICES=""
cd "$WARPSTATE_REPO"
exec /usr/bin/nice -n 10 "$WARPSTATE_PYTHON" -u prepare_posttrain_data.py "$@"
