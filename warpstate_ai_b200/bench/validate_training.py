"""Production-shaped training validation: the fused sm_100a path against the plain-PyTorch definition.

A model with the production attention and FFN dimensions (d_model 2048, 32 heads of 64, FFN 7168, chunk 128,
sequence 2048) but few cores is trained for three accumulated updates -- two full ones and a final one with
nine valid tokens, so that most ranks and micro-batches of the last update are empty -- by five arms:

* ``exact``      the PyTorch definition of the model in FP32 (no autocast, kernels disabled): the ground truth;
* ``stock``      the same definition under BF16 autocast: the role the reference's compiled baseline plays in its
                 harness, and the yardstick for what BF16 arithmetic alone costs against ``exact``;
* ``fused``      the hand-written kernel path, everything else identical;
* ``partial``    the fused arm stopped after two updates and saved (model, optimizer, RNG);
* ``resumed``    a fresh process state loaded from that checkpoint, running the third update.

Judged per tensor against ``exact``: gradients of the first update and AdamW moments by relative L2 and relative
max, parameters after the last update by the share of elements further than the declared absolute bound, losses
by absolute gap.  A tensor passes when it is inside the declared table (the reference's,
ops/validate_backward_layout_training.py:35-44, which compares two BF16 arms that differ only in a store layout)
or when the fused arm is no further from ``exact`` than ``stock`` is, with the declared margin: two independent
BF16 evaluations of this model differ by about one percent in their gradients, and AdamW turns a sign change of a
near-zero gradient into a parameter difference of a whole learning rate, so "not less accurate than PyTorch's own
BF16 path" is the criterion a correct kernel path can meet and a wrong one cannot.  ``resumed`` against ``fused``
must be byte-identical.  World size 1, or 2 under ``torch.distributed.run`` (each arm then synchronises gradients
its own way: NCCL all-reduce for the PyTorch arms, the in-kernel reduction for the fused arms).

    python -m warpstate_ai_b200.bench.validate_training --output-dir work/validation/run1 [--cores 1]

Writes ``report.json`` into the fresh output directory and exits non-zero when a criterion is missed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

TOLERANCES = {
    "gradient_relative_l2": 0.005, "gradient_relative_max": 0.01, "gradient_absolute": 1e-8,
    "parameter_absolute": 2e-5,
    "moment_relative_l2": 0.005, "moment_relative_max": 0.01, "moment_absolute": 1e-8,
    "loss_absolute": 2e-4,
    # the yardstick rule: fused-vs-exact may be at most this multiple of stock-vs-exact (plus the slack below)
    "stock_margin": 1.5, "parameter_share_slack": 1e-3,
    "sparse_loss_relative": 0.005,      # the nine-token update: relative, as reference test_residual_execution.py:72
}
SEQ_LEN = 2048            # overridden by --seq-len for quick checks of the harness
ACCUMULATION = 3          # no-sync first micro-batch, no-sync accumulation, final synchronised micro-batch
UPDATES = 3


def fixture_config(cores: int, vocab: int, shape: str = "production"):
    """``production``: the trained model's layer shape.  ``small``: 2 heads of 64, FFN 256 -- for checking the
    harness itself in seconds (still a shape the kernels accept)."""
    from ..config import WarpStateConfig
    d, heads, ffn = (2048, 32, 7168) if shape == "production" else (128, 2, 256)
    return WarpStateConfig(vocab_size=vocab, d_model=d, n_heads=heads, n_cores=cores, logical_depth=cores,
                           ffn_hidden=ffn, chunk_size=128, gradient_checkpointing=False, parallel_memory=True,
                           loss_chunk_size=512)


def update_tokens(update: int, micro_tokens: int, world: int) -> int:
    """Two full accumulated updates, then nine valid global tokens."""
    return micro_tokens * ACCUMULATION * world if update < UPDATES - 1 else 9


def compare(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    a, e = actual.detach().double().cpu().reshape(-1), expected.detach().double().cpu().reshape(-1)
    difference = a - e
    scale_l2, scale_max = float(e.norm()), float(e.abs().max())
    return {"bitwise_equal": bool(torch.equal(actual.detach().cpu(), expected.detach().cpu())),
            "finite": bool(torch.isfinite(a).all() and torch.isfinite(e).all()),
            "absolute_max": float(difference.abs().max()),
            "share_beyond_parameter_bound": float((difference.abs() > TOLERANCES["parameter_absolute"]).double().mean()),
            "relative_l2": float(difference.norm()) / scale_l2 if scale_l2 > 0 else float(difference.norm()),
            "relative_max": float(difference.abs().max()) / scale_max if scale_max > 0 else float(difference.abs().max())}


def within(result: dict, kind: str, yardstick: dict | None = None) -> bool:
    """``result``: fused against exact.  ``yardstick``: stock (PyTorch BF16) against exact, same tensor."""
    if not result["finite"]:
        return False
    margin = TOLERANCES["stock_margin"]
    if kind == "parameter":
        if result["absolute_max"] <= TOLERANCES["parameter_absolute"]:
            return True
        return (yardstick is not None and result["absolute_max"] <= result["adam_travel"]
                and result["share_beyond_parameter_bound"]
                <= margin * yardstick["share_beyond_parameter_bound"] + TOLERANCES["parameter_share_slack"])
    if (result["absolute_max"] <= TOLERANCES[f"{kind}_absolute"]
            or (result["relative_l2"] <= TOLERANCES[f"{kind}_relative_l2"]
                and result["relative_max"] <= TOLERANCES[f"{kind}_relative_max"])):
        return True
    return (yardstick is not None and result["relative_l2"] <= margin * yardstick["relative_l2"]
            and result["relative_max"] <= margin * yardstick["relative_max"])


class Arm:
    """One way of running the fixture; records the first update's gradients and every update's loss."""

    def __init__(self, name: str, a, rank: int, world: int, device, fused_kernels: bool, bf16: bool = True):
        from .. import WarpStateLM
        from ..ops import fused
        from ..parallel.grad_sync import CollectiveGradSync, FusedGradSync
        from ..train.engine import Trainer
        self.name, self.a, self.rank, self.world, self.device, self.fused_kernels = name, a, rank, world, device, fused_kernels
        torch.manual_seed(a.seed)
        with torch.device(device):
            self.model = WarpStateLM(fixture_config(a.cores, a.vocab, a.shape))
        self.model.train()
        sync = None
        if world > 1:
            sync = (FusedGradSync(device, world, rank) if fused_kernels and device.type == "cuda"
                    else CollectiveGradSync(device, world, rank))
        self._switch = fused.disabled if not fused_kernels else None
        self.trainer = Trainer(self.model, device=device, rank=rank, world_size=world, lr=a.lr, weight_decay=0.1,
                               grad_sync=sync, bf16_autocast=bf16)
        self.first_gradients = None
        self.losses: list[float] = []
        original = self.trainer.optimizer.step

        def recording_step(lr=None, stats=None):
            if self.first_gradients is None:
                self.first_gradients = self.trainer.arena.grad.detach().clone()
            return original(lr=lr, stats=stats)

        self.trainer.optimizer.step = recording_step

    def run(self, updates) -> None:
        import contextlib
        from ..data.tokens import SyntheticTokens
        a = self.a
        micro_tokens = a.micro_batch * SEQ_LEN
        data = SyntheticTokens(micro_tokens * ACCUMULATION * self.world * UPDATES + 64, a.vocab, seed=a.seed + 1)
        cursor = sum(update_tokens(u, micro_tokens, self.world) for u in range(min(updates, default=0)))
        for update in updates:
            target = update_tokens(update, micro_tokens, self.world)
            with (self._switch() if self._switch is not None else contextlib.nullcontext()):
                result = self.trainer.pretrain_update(data, cursor, target, a.micro_batch, SEQ_LEN, a.lr)
            self.losses.append(result.loss)
            cursor += target

    def tensors(self) -> dict:
        state = self.trainer.optimizer.state_dict()["state"]
        names = [name for name, _ in self.trainer.arena.order]
        out = {"parameter": {n: p.detach().clone() for n, p in self.trainer.arena.named_master()}}
        out["moment"] = {f"{names[i]}.{k}": s[k] for i, s in state.items() for k in ("exp_avg", "exp_avg_sq")}
        arena = self.trainer.arena
        out["gradient"] = {s.name: arena.view(self.first_gradients, s).clone() for s in arena.slots}
        return out

    def checkpoint(self) -> dict:
        from ..ckpt.formats import capture_rng
        return {"model": {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()},
                "optimizer": self.trainer.optimizer.state_dict(), "rng": capture_rng(self.device)}

    def restore(self, checkpoint: dict) -> None:
        from ..ckpt.formats import restore_rng
        self.trainer.load_model_state_dict(checkpoint["model"])
        self.trainer.optimizer.load_state_dict(checkpoint["optimizer"])
        restore_rng(checkpoint["rng"], self.device)


def judge(actual: dict, stock: dict, exact: dict, kinds, adam_travel: float) -> tuple[dict, list]:
    table, failures = {}, []
    for kind in kinds:
        for name, tensor in actual[kind].items():
            result = compare(tensor, exact[kind][name])
            yardstick = compare(stock[kind][name], exact[kind][name])
            result["adam_travel"] = adam_travel
            result["stock_vs_exact"] = {k: yardstick[k] for k in ("absolute_max", "relative_l2", "relative_max",
                                                                 "share_beyond_parameter_bound")}
            result["within_tolerance"] = within(result, kind, yardstick)
            table[f"{kind}:{name}"] = result
            if not result["within_tolerance"]:
                failures.append(f"{kind}:{name}")
    return table, failures


def main(argv=None) -> int:
    global SEQ_LEN
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--output-dir", type=Path, required=True, help="fresh directory for report.json")
    p.add_argument("--cores", type=int, default=1, help="distinct cores (= logical layers) of the fixture")
    p.add_argument("--micro-batch", type=int, default=2)
    p.add_argument("--vocab", type=int, default=512, help="small on purpose: repeated embedding rows in every batch")
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--seed", type=int, default=41619)
    p.add_argument("--shape", choices=["production", "small"], default="production")
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    a = p.parse_args(argv)
    SEQ_LEN = a.seq_len
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    if a.cores < 1 or a.micro_batch < 1 or world not in (1, 2):
        p.error("need --cores >= 1, --micro-batch >= 1 and one or two ranks")
    device = torch.device("cuda", local) if a.device == "cuda" else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", **({"device_id": device} if device.type == "cuda" else {}))
    if rank == 0:
        a.output_dir.mkdir(parents=True, exist_ok=False)

    def finished(arm: Arm, updates) -> Arm:
        arm.run(updates)
        if device.type == "cuda":
            from ..ops.gemm import check_device_errors
            check_device_errors()
        return arm

    everything = range(UPDATES)
    exact = finished(Arm("exact", a, rank, world, device, fused_kernels=False, bf16=False), everything)
    truth, exact_losses = exact.tensors(), exact.losses
    del exact
    stock = finished(Arm("stock", a, rank, world, device, fused_kernels=False), everything)
    yardstick, stock_losses = stock.tensors(), stock.losses
    del stock
    fused = finished(Arm("fused", a, rank, world, device, fused_kernels=True), everything)
    mine = fused.tensors()
    # AdamW moves a parameter by at most about one learning rate per update; two runs can differ by twice that
    table, failures = judge(mine, yardstick, truth, ("gradient", "moment", "parameter"), 2.1 * a.lr * UPDATES)
    loss_gaps = [abs(x - y) for x, y in zip(fused.losses, exact_losses)]
    stock_gaps = [abs(x - y) for x, y in zip(stock_losses, exact_losses)]
    for update, (gap, stock_gap, loss) in enumerate(zip(loss_gaps, stock_gaps, exact_losses)):
        bound = TOLERANCES["loss_absolute"] if update < UPDATES - 1 else TOLERANCES["sparse_loss_relative"] * abs(loss)
        if gap > max(bound, TOLERANCES["stock_margin"] * stock_gap):
            failures.append(f"loss:{update}")
    fused_losses = fused.losses
    del fused
    partial = finished(Arm("partial", a, rank, world, device, fused_kernels=True), range(UPDATES - 1))
    saved = partial.checkpoint()
    del partial
    resumed = Arm("resumed", a, rank, world, device, fused_kernels=True)
    resumed.restore(saved)
    finished(resumed, range(UPDATES - 1, UPDATES))
    again = resumed.tensors()
    continuation = {f"{kind}:{name}": bool(torch.equal(tensor.cpu(), mine[kind][name].cpu()))
                    for kind in ("moment", "parameter") for name, tensor in again[kind].items()}
    if not all(continuation.values()) or resumed.losses[-1] != fused_losses[-1]:
        failures.append("resumed state is not byte-identical to the uninterrupted run")
    report = {"format": "warpstate-training-validation-v1", "tolerances": TOLERANCES, "world_size": world, "rank": rank,
              "fixture": {"cores": a.cores, "micro_batch": a.micro_batch, "seq_len": SEQ_LEN, "vocab": a.vocab,
                          "accumulation": ACCUMULATION, "updates": UPDATES, "lr": a.lr, "seed": a.seed,
                          "device": str(device), "torch": torch.__version__},
              "losses": {"exact": exact_losses, "stock": stock_losses, "fused": fused_losses, "absolute_gaps": loss_gaps,
                         "stock_absolute_gaps": stock_gaps},
              "fused_vs_exact": table,
              "worst": {kind: max((r[metric] for k, r in table.items() if k.startswith(kind)), default=0.0)
                        for kind, metric in (("gradient", "relative_l2"), ("moment", "relative_l2"),
                                              ("parameter", "share_beyond_parameter_bound"))},
              "worst_stock": {kind: max((r["stock_vs_exact"][metric] for k, r in table.items() if k.startswith(kind)), default=0.0)
                              for kind, metric in (("gradient", "relative_l2"), ("moment", "relative_l2"),
                                                   ("parameter", "share_beyond_parameter_bound"))},
              "resumed_byte_identical": all(continuation.values()), "failures": failures, "passed": not failures}
    if world > 1:
        import torch.distributed as dist
        verdicts = [None] * world
        dist.all_gather_object(verdicts, not failures)
        report["passed_on_every_rank"] = all(verdicts)
    if rank == 0:
        (a.output_dir / "report.json").write_text(json.dumps(report, indent=2, allow_nan=False) + "\n")
        print(json.dumps({"passed": report["passed"], "worst": report["worst"], "worst_stock": report["worst_stock"],
                          "loss_gaps": loss_gaps, "stock_loss_gaps": stock_gaps,
                          "resumed_byte_identical": report["resumed_byte_identical"], "failures": failures[:8]}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if not failures else 1


if __name__ == "__main__":
    sys.exit(main())
