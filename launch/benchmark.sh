#!/usr/bin/env bash
# Disposable update benchmark (never writes a checkpoint).  WARPSTATE_BENCH_PROCESSES ranks on
# WARPSTATE_BENCH_DEVICES; arguments go to warpstate_ai_b200.bench.train_bench.
set -euo pipefail
ulimit -c 0
source "$(dirname "${BASH_SOURCE[0]}")/env.sh"
cd "$WARPSTATE_REPO"
processes="${WARPSTATE_BENCH_PROCESSES:-1}"
if [[ -n "${WARPSTATE_BENCH_DEVICES:-}" ]]; then export CUDA_VISIBLE_DEVICES="$WARPSTATE_BENCH_DEVICES"; fi
if [[ "$processes" == 1 ]]; then
  exec "$WARPSTATE_PYTHON" -u -m warpstate_ai_b200.bench.train_bench "$@"
else
  exec "$WARPSTATE_PYTHON" -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nnodes 1 \
    --nproc-per-node "$processes" --log-dir "$WARPSTATE_WORK/logs/torchrun-benchmark" \
    -m warpstate_ai_b200.bench.train_bench "$@"
fi
