#!/usr/bin/env bash
# Source before training, benchmarking or data preparation.  Everything the jobs write goes below
# $WARPSTATE_WORKSPACE (default: the directory above this repository), never to $HOME.
export WARPSTATE_REPO="${WARPSTATE_REPO:-$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)}"
export WARPSTATE_WORKSPACE="${WARPSTATE_WORKSPACE:-$(dirname "$WARPSTATE_REPO")}"
export WARPSTATE_WORK="${WARPSTATE_WORK:-$WARPSTATE_REPO/work}"
export WARPSTATE_PYTHON="${WARPSTATE_PYTHON:-python3}"
export TMPDIR="$WARPSTATE_WORKSPACE/tmp"
export XDG_CACHE_HOME="$WARPSTATE_WORKSPACE/.cache"
export HF_HOME="$WARPSTATE_WORK/hf-cache"
export HF_DATASETS_CACHE="$HF_HOME/datasets"
export TORCH_HOME="$XDG_CACHE_HOME/torch"
export CUDA_CACHE_PATH="$XDG_CACHE_HOME/cuda"
export PYTHONDONTWRITEBYTECODE=1
export PYTHONPATH="$WARPSTATE_REPO${PYTHONPATH:+:$PYTHONPATH}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-4}"
export MKL_NUM_THREADS="${MKL_NUM_THREADS:-4}"
export OPENBLAS_NUM_THREADS=1
# Reproducible cuBLAS workspaces for the few library GEMMs outside the kernel library.
export CUBLAS_WORKSPACE_CONFIG=:4096:8
# One rendezvous address for every torchrun on this node.
export MASTER_ADDR=127.0.0.1
mkdir -p "$TMPDIR" "$XDG_CACHE_HOME" "$CUDA_CACHE_PATH" "$WARPSTATE_WORK/logs" "$WARPSTATE_WORK/control"
