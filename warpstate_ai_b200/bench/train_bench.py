"""Disposable full-model update benchmark with per-update records, profiling and stall diagnosis.

Loads a training checkpoint (model + optimizer) or builds a random-init model of a named
configuration, runs ``--warmup-updates`` untimed and ``--measured-updates`` timed optimizer
updates of ``--global-tokens-per-update`` tokens through the same `Trainer` the pretraining CLI
uses, and writes into ``--output-dir``:

* ``rank-<r>.jsonl``   one record per measured update: seconds (host wall clock around a device
  synchronisation), tokens/s, loss, gradient norm, peak allocated / reserved bytes;
* ``summary.json``     geometry, precision, identity of checkpoint and data, and per-update
  elapsed time as the MAX over ranks (the number that decides throughput);
* with ``--profile``:  for the last measured update a chrome trace, a per-kernel TSV, and a
  summary with name-based categories, the summed device time and the union of busy intervals
  (overlapping streams are not counted twice);
* with ``--diagnose-stalls``: host wall time per stage (stage / forward+backward / gradient sync /
  optimizer / read-back) and a traceback dump every 10 s while an update is in flight.

    torchrun --standalone --nproc-per-node 2 -m warpstate_ai_b200.bench.train_bench --micro-batch 8 \
        --global-tokens-per-update 131072 --output-dir bench-out

Same outputs and flags as the reference's ops/benchmark_training.py:28-593.  The flags that select between
its execution adapters (compiled cores, loss and activation variants, compiled autograd and its overlap
scheduler, BLAS preference, CUDA-graph replay counting) are accepted and recorded in ``summary.json`` under
``reference_execution_flags``; there is one execution path here, so they change nothing that runs.
"""
from __future__ import annotations

import argparse
import contextlib
import faulthandler
import hashlib
import json
import os
import sys
import time
from pathlib import Path

import torch


def arguments(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--checkpoint", type=Path, help="warpstate-server-v1 training checkpoint; random init if omitted")
    p.add_argument("--model", choices=["2b", "smoke"], default="2b", help="configuration when no checkpoint is given")
    p.add_argument("--data", type=Path, help="uint16 token file; synthetic uniform tokens if omitted")
    p.add_argument("--output-dir", type=Path, required=True)
    p.add_argument("--micro-batch", type=int, required=True)
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--global-tokens-per-update", type=int, default=131072)
    p.add_argument("--activation-checkpointing", action=argparse.BooleanOptionalAction, default=False)
    p.add_argument("--warmup-updates", type=int, default=1)
    p.add_argument("--measured-updates", type=int, default=2)
    p.add_argument("--profile", action="store_true", help="profile the last measured update (adds overhead)")
    p.add_argument("--diagnose-stalls", action="store_true")
    p.add_argument("--optimizer-state", choices=["resume", "fresh"], default="resume")
    p.add_argument("--vram-limit-gib", type=float)
    p.add_argument("--threads", type=int, default=4)
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--grad-sync", choices=["auto", "fused", "nccl"], default="auto")
    p.add_argument("--shard-optimizer", action="store_true")
    p.add_argument("--shard-params", choices=["off", "stream", "resident"], default="off")
    p.add_argument("--bf16-residuals", action="store_true", help="BF16 residual stream (FP32 by default)")
    p.add_argument("--loss-chunk-size", type=int, default=1024, help="rows per block of the host (CPU) loss head")
    p.add_argument("--ddp-bucket-cap-mb", type=float, default=0.0,
                   help="largest gradient range reduced by one launch, in MiB of FP32 gradients; 0 = one bucket per core")
    from ..train.flags import REFERENCE_EXECUTION_FLAGS, Flag
    compat = p.add_argument_group("reference execution experiments", "accepted and recorded; no effect on what runs here")
    one_path = "no tracing compiler: every core is one autograd node over hand-written kernels"
    for flag in (*[f for f in REFERENCE_EXECUTION_FLAGS if f.name not in ("--compile", "--compile-core")],
                 Flag("--compile-cores", "toggle", False, native=one_path),
                 Flag("--fused-rms-norm", "toggle", False, native="RMSNorm is one kernel with the depth modulation folded in"),
                 Flag("--blas-backend", str, None, choices=("default", "cublas", "cublaslt"),
                      native="GEMMs are this library's tcgen05 kernels, not a BLAS call"),
                 Flag("--cudagraph-diagnostics", "switch", native="training launches no CUDA graph; decode counts its own "
                                                                  "(serve/graph_stats.py)")):
        flag.add_to(compat)
        INERT.append(flag)
    a = p.parse_args(argv)
    if a.loss_chunk_size < 1 or a.ddp_bucket_cap_mb < 0 or a.overlap_memory_budget < 0:
        p.error("--loss-chunk-size must be positive; --ddp-bucket-cap-mb and --overlap-memory-budget must not be negative")
    return a


INERT: list = []            # the reference-execution flags of the last `arguments` call


def inert_settings(a) -> dict:
    """Reference-execution flags that were given a non-default value, for the record."""
    return {flag.name: str(getattr(a, flag.dest)) if isinstance(getattr(a, flag.dest), Path) else getattr(a, flag.dest)
            for flag in INERT if getattr(a, flag.dest) != (False if flag.kind == "switch" else flag.default)}


def file_identity(path: Path | None):
    if path is None:
        return None
    info = path.stat()
    return {"path": str(path), "bytes": info.st_size, "mtime_ns": info.st_mtime_ns}


def source_hash(path) -> str:
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


# --------------------------------------------------------------------------------- profile export
def kernel_category(name: str) -> str:
    from .profile_step import category
    return category(name)


def cuda_activity_summary(trace_events) -> dict:
    """Per-kernel totals, category shares and the union of busy intervals of a chrome trace."""
    kernels, intervals, annotations = {}, [], 0
    for event in trace_events:
        if event.get("ph") != "X":
            continue
        if event.get("cat") == "gpu_user_annotation":
            annotations += 1
        if event.get("cat") not in ("kernel", "gpu_memcpy", "gpu_memset"):
            continue
        device = event.get("args", {}).get("device", event.get("pid"))
        row = kernels.setdefault((event["name"], device), {"name": event["name"], "device_index": device,
                                                           "category": kernel_category(event["name"]), "count": 0,
                                                           "self_cuda_us": 0.0})
        row["count"] += 1
        row["self_cuda_us"] += event["dur"]
        intervals.append((event["ts"], event["ts"] + event["dur"]))
    rows = sorted(kernels.values(), key=lambda r: -r["self_cuda_us"])
    total = sum(r["self_cuda_us"] for r in rows)
    categories = {}
    for r in rows:
        c = categories.setdefault(r["category"], {"self_cuda_us": 0.0, "count": 0})
        c["self_cuda_us"] += r["self_cuda_us"]
        c["count"] += r["count"]
    for c in categories.values():
        c["fraction_of_summed_cuda_time"] = c["self_cuda_us"] / total if total else 0.0
    busy, end = 0.0, None
    for begin, stop in sorted(intervals):
        busy += max(0.0, stop - max(begin, end if end is not None else begin))
        end = max(end if end is not None else stop, stop)
    return {"kernels": rows, "kernel_name_count": len(rows), "categories": categories, "summed_cuda_event_us": total,
            "cuda_event_union_us": busy, "excluded_gpu_annotation_ranges": annotations}


def export_profile(profiler, output_dir: Path, rank: int, update: int, elapsed: float) -> dict:
    prefix = f"profile-rank-{rank}"
    trace = output_dir / f"{prefix}-trace.json"
    profiler.export_chrome_trace(str(trace))
    activity = cuda_activity_summary(json.loads(trace.read_text()).get("traceEvents", []))
    summary = {"rank": rank, "update": update, "profiled_update_seconds": elapsed, "trace": str(trace),
               "aggregation_source_sha256": source_hash(__file__), **activity,
               "limitations": ["Profiling adds overhead; use unprofiled runs for throughput.",
                               "Kernels on different streams overlap; summed category time is not wall time.",
                               "Categories are name-based; raw kernel names are kept."]}
    (output_dir / f"{prefix}-summary.json").write_text(json.dumps(summary, indent=2) + "\n")
    lines = ["self_cuda_ms\tcount\tcategory\tkernel"]
    lines += [f"{r['self_cuda_us'] / 1000:.3f}\t{r['count']}\t{r['category']}\t{r['name']}" for r in activity["kernels"]]
    (output_dir / f"{prefix}-kernels.tsv").write_text("\n".join(lines) + "\n")
    return {"summary": str(output_dir / f"{prefix}-summary.json"), "trace": str(trace),
            **{k: v for k, v in activity.items() if k != "kernels"}}


# --------------------------------------------------------------------------------- stall diagnosis
class StageTimers:
    """Host wall time per named stage (includes implicit waits; never synchronises the device)."""

    def __init__(self, enabled: bool):
        self.enabled = enabled
        self.totals: dict[str, float] = {}

    @contextlib.contextmanager
    def mark(self, name: str):
        if not self.enabled:
            yield
            return
        with torch.profiler.record_function(f"warpstate::{name}"):
            begin = time.perf_counter()
            try:
                yield
            finally:
                self.totals[name] = self.totals.get(name, 0.0) + time.perf_counter() - begin


@contextlib.contextmanager
def stalled_update_tracebacks(enabled: bool, seconds: int = 10):
    if not enabled:
        yield
        return
    faulthandler.dump_traceback_later(seconds, repeat=True)
    try:
        yield
    finally:
        faulthandler.cancel_dump_traceback_later()


def timed_update(trainer, data, cursor, tokens, micro_batch, seq_len, lr, batcher, timers: StageTimers):
    """`Trainer.pretrain_update` unrolled so that each stage can be timed on the host."""
    from ..data.tokens import update_slices
    slices = list(update_slices(tokens, micro_batch * seq_len, trainer.world_size, trainer.rank))
    with timers.mark("begin"):
        trainer.begin_update()
    for index, (offset, valid) in enumerate(slices):
        with timers.mark("stage_batch"):
            handle = batcher.stage(data, cursor + offset, valid)
            x, y = batcher.take(handle)

        def loss_fn(x=x, y=y, valid=valid):
            _, loss = trainer.model(x, y, return_logits=False)
            return loss, valid * trainer.world_size / tokens, valid / tokens

        with timers.mark("forward_backward"):
            trainer.micro_step(loss_fn, last=index == len(slices) - 1)
        batcher.release(handle)
    with timers.mark("sync_clip_step"):
        stats = trainer.finish_update(lr)
    with timers.mark("read_back"):
        loss, norm, coef = trainer.read_update_scalars(stats)
    return loss, norm, coef


# --------------------------------------------------------------------------------- the benchmark
def benchmark(a) -> dict:
    import torch.distributed as dist
    from .. import WarpStateConfig, WarpStateLM, warpstate_2b, warpstate_smoke
    from ..data.tokens import HostBatcher, SyntheticTokens
    from ..train.engine import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.set_num_threads(a.threads)
    torch.manual_seed(a.seed)
    if a.device == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        if a.vram_limit_gib:
            total = torch.cuda.get_device_properties(device).total_memory
            torch.cuda.set_per_process_memory_fraction(min(1.0, a.vram_limit_gib * 2 ** 30 / total), device)
    else:
        device = torch.device("cpu")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if a.device == "cuda" else "gloo",
                                **({"device_id": device} if a.device == "cuda" else {}))
    per_update = a.micro_batch * a.seq_len * world
    if a.global_tokens_per_update % per_update:
        raise SystemExit(f"--global-tokens-per-update must be a multiple of micro_batch*seq_len*world = {per_update}")
    checkpoint = None
    if a.checkpoint is not None:
        checkpoint = torch.load(a.checkpoint, map_location="cpu", weights_only=False, mmap=True)
        cfg = WarpStateConfig(**checkpoint["config"])
    else:
        cfg = warpstate_2b() if a.model == "2b" else warpstate_smoke()
    cfg.gradient_checkpointing = a.activation_checkpointing
    cap = int(a.ddp_bucket_cap_mb * 2 ** 20)
    if a.profile:
        # kernels launched as programmatic dependents wait for their predecessor inside the kernel, which a
        # profiler books as their own time: the profiled run uses plain launches
        os.environ.setdefault("WS_TRAIN_PDL", "0")
    with torch.device(device):
        model = WarpStateLM(cfg)
    if checkpoint is not None:
        model.load_state_dict(checkpoint["model"])
    model.loss_chunk_size = a.loss_chunk_size
    model.bf16_residuals = bool(a.bf16_residuals)
    model.train()
    sync = None
    if world > 1:
        from ..parallel.grad_sync import make_grad_sync
        sync = make_grad_sync(device, world, rank, None,
                              kind={"auto": "auto", "fused": "fused", "nccl": "collective"}[a.grad_sync], bucket_cap_bytes=cap)
    trainer = Trainer(model, device=device, rank=rank, world_size=world, grad_sync=sync,
                      shard_optimizer=a.shard_optimizer,
                      shard_params=None if a.shard_params == "off" else a.shard_params, bucket_cap_bytes=cap)
    if checkpoint is not None and a.optimizer_state == "resume":
        trainer.optimizer.load_state_dict(checkpoint["optimizer"])
    del checkpoint
    tokens = a.global_tokens_per_update
    total_updates = a.warmup_updates + a.measured_updates
    if a.data is not None:
        import numpy as np
        data = np.memmap(a.data, dtype=np.uint16, mode="r")
    else:
        data = SyntheticTokens(tokens * total_updates + 1, cfg.vocab_size, seed=a.seed)
    batcher = HostBatcher(a.micro_batch, a.seq_len, device)
    out = a.output_dir
    out.mkdir(parents=True, exist_ok=True)
    timers = StageTimers(a.diagnose_stalls)
    records, profile_report = [], None
    log = (out / f"rank-{rank}.jsonl").open("w")

    def synchronize():
        if device.type == "cuda":
            torch.cuda.synchronize(device)

    cursor = 0
    for update in range(total_updates):
        measured = update >= a.warmup_updates
        profiled = a.profile and update == total_updates - 1
        if device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(device)
        if world > 1:
            dist.barrier()
        synchronize()
        timers.totals = {}
        profiler = None
        if profiled:
            activities = [torch.profiler.ProfilerActivity.CPU]
            if device.type == "cuda":
                activities.append(torch.profiler.ProfilerActivity.CUDA)
            profiler = torch.profiler.profile(activities=activities)
            profiler.__enter__()
        begin = time.perf_counter()
        with stalled_update_tracebacks(a.diagnose_stalls and measured):
            loss, norm, coef = timed_update(trainer, data, cursor, tokens, a.micro_batch, a.seq_len, 1.5e-4, batcher, timers)
            synchronize()
        elapsed = time.perf_counter() - begin
        if profiler is not None:
            profiler.__exit__(None, None, None)
            profile_report = export_profile(profiler, out, rank, update, elapsed)
        cursor += tokens
        slowest = torch.tensor([elapsed], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        record = {"update": update, "measured": measured, "profiled": profiled, "seconds": elapsed,
                  "slowest_rank_seconds": float(slowest), "tokens": tokens, "tokens_per_second": tokens / float(slowest),
                  "loss": loss, "grad_norm": norm, "clip_coef": coef}
        if device.type == "cuda":
            record.update(peak_allocated_bytes=torch.cuda.max_memory_allocated(device),
                          peak_reserved_bytes=torch.cuda.max_memory_reserved(device))
        if a.diagnose_stalls:
            record["host_stage_seconds"] = dict(timers.totals)
        log.write(json.dumps(record) + "\n")
        log.flush()
        if measured:
            records.append(record)
        if rank == 0:
            print(json.dumps(record), flush=True)
    log.close()
    clean = [r for r in records if not r["profiled"]] or records
    summary = {"format": "warpstate-training-benchmark-v1", "world_size": world, "device": str(device),
               "model": {"parameters": model.num_parameters(), "config": vars(cfg).copy()},
               "geometry": {"micro_batch": a.micro_batch, "seq_len": a.seq_len, "global_tokens_per_update": tokens,
                            "grad_accum": tokens // per_update},
               "precision": {"compute": "bf16" if device.type == "cuda" else "fp32", "master": "fp32", "grads": "fp32",
                             "residual_stream": "bf16" if a.bf16_residuals else "fp32"},
               "bucket_cap_mb": a.ddp_bucket_cap_mb, "reference_execution_flags": inert_settings(a),
               "grad_sync": getattr(sync, "kind", "none"), "optimizer": "sharded" if a.shard_optimizer and world > 1 else "replicated",
               "checkpoint": file_identity(a.checkpoint), "data": file_identity(a.data) or "synthetic",
               "optimizer_state": a.optimizer_state if a.checkpoint else "fresh",
               "warmup_updates": a.warmup_updates, "measured_updates": a.measured_updates,
               "updates": records,
               "mean_tokens_per_second": sum(r["tokens_per_second"] for r in clean) / max(1, len(clean)),
               "profile": profile_report, "torch": torch.__version__, "source_sha256": source_hash(__file__)}
    if rank == 0:
        (out / "summary.json").write_text(json.dumps(summary, indent=2, default=str) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return summary


def main(argv=None) -> int:
    a = arguments(argv)
    if a.warmup_updates < 0 or a.measured_updates < 1:
        raise SystemExit("need at least one measured update")
    summary = benchmark(a)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"mean_tokens_per_second": summary["mean_tokens_per_second"],
                          "summary": str(a.output_dir / "summary.json")}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
