"""Checkpoint writer: immutability of a pending snapshot, atomic publication, back-pressure,
sticky errors, context-manager behaviour, and two-rank fault injection over gloo.

Scenarios follow the reference's (test_checkpoint_writer.py:50-258,
test_distributed_checkpoint_writer.py:18-196): failures are injected on the host (a save
function that raises, a snapshot that raises, a state factory that raises); both ranks must
raise, none may hang, and an exceptional exit must not issue a collective.
"""
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import pytest
import torch

from warpstate_ai_b200.ckpt import writer as W

ROOT = Path(__file__).resolve().parents[1]


def make_state():
    weight = torch.arange(6, dtype=torch.float32)
    return {"model": {"w": weight, "tied": weight}, "optimizer": {"state": {0: {"exp_avg": torch.ones(3)}}},
            "step": 3, "tokens_seen": 96, "meta": {"history": [1, 2]}}


def test_snapshot_is_frozen_and_keeps_aliasing():
    state = make_state()
    snap = W.snapshot_to_cpu(state)
    state["model"]["w"].add_(100)
    state["meta"]["history"].append(3)
    state["optimizer"]["state"][0]["exp_avg"].zero_()
    assert torch.equal(snap["model"]["w"], torch.arange(6, dtype=torch.float32))
    assert snap["model"]["w"] is snap["model"]["tied"]
    assert snap["meta"]["history"] == [1, 2]
    assert torch.equal(snap["optimizer"]["state"][0]["exp_avg"], torch.ones(3))


def test_pending_save_sees_the_state_at_submit_time(tmp_path):
    release = threading.Event()
    seen = {}

    def slow_save(path, snap):
        assert release.wait(10)
        seen["w"] = snap["model"]["w"].clone()
        W.atomic_torch_save(path, snap)

    state = make_state()
    with W.AsyncCheckpointWriter(tmp_path / "latest.pt", save_fn=slow_save) as writer:
        writer.submit(state)
        state["model"]["w"].mul_(0)
        release.set()
    assert torch.equal(seen["w"], torch.arange(6, dtype=torch.float32))
    assert torch.equal(torch.load(tmp_path / "latest.pt")["model"]["w"], torch.arange(6, dtype=torch.float32))


def test_failed_serialization_keeps_the_old_file_and_leaves_no_partial(tmp_path, monkeypatch):
    path = tmp_path / "latest.pt"
    W.atomic_torch_save(path, {"step": 1})

    def broken(obj, handle, *a, **k):
        handle.write(b"partial")
        raise OSError("disk full")

    monkeypatch.setattr(torch, "save", broken)
    with pytest.raises(OSError):
        W.atomic_torch_save(path, {"step": 2})
    monkeypatch.undo()
    assert torch.load(path)["step"] == 1
    assert sorted(p.name for p in tmp_path.iterdir()) == ["latest.pt"]


def test_second_submit_waits_for_the_first_write(tmp_path):
    release = threading.Event()
    order = []

    def slow_save(path, snap):
        order.append(("write-begin", snap["step"]))
        assert release.wait(10)
        order.append(("write-end", snap["step"]))

    writer = W.AsyncCheckpointWriter(tmp_path / "latest.pt", save_fn=slow_save)
    writer.submit({"step": 1, "tokens_seen": 1})
    done = threading.Event()

    def second():
        writer.submit({"step": 2, "tokens_seen": 2})
        order.append(("second-staged", 2))
        done.set()

    t = threading.Thread(target=second)
    t.start()
    time.sleep(0.3)
    assert not done.is_set()  # still blocked behind write 1: no second snapshot allocated yet
    release.set()
    t.join(10)
    writer.close()
    assert order.index(("write-end", 1)) < order.index(("second-staged", 2))


def test_background_failure_is_sticky(tmp_path):
    def failing(path, snap):
        raise OSError("injected")

    writer = W.AsyncCheckpointWriter(tmp_path / "latest.pt", save_fn=failing)
    writer.submit({"step": 1})
    with pytest.raises(OSError):
        writer.flush()
    for call in (writer.check, writer.flush, lambda: writer.submit({"step": 2}), writer.close):
        with pytest.raises(OSError):
            call()


@pytest.mark.parametrize("exceptional", [False, True])
def test_context_exit_joins_pending_write(tmp_path, exceptional):
    path = tmp_path / "latest.pt"
    try:
        with W.AsyncCheckpointWriter(path) as writer:
            writer.submit({"step": 7, "tokens_seen": 70})
            if exceptional:
                raise KeyError("training failed")
    except KeyError:
        assert exceptional
    assert torch.load(path)["step"] == 7


def test_training_exception_survives_a_failing_cleanup(tmp_path):
    def failing(path, snap):
        raise OSError("injected write failure")

    with pytest.raises(ValueError) as info:
        with W.AsyncCheckpointWriter(tmp_path / "latest.pt", save_fn=failing) as writer:
            writer.submit({"step": 1})
            raise ValueError("training failed")
    assert any("Checkpoint cleanup also failed" in note for note in getattr(info.value, "__notes__", []))


# --------------------------------------------------------------------------- two ranks over gloo
def _worker(rank: int, directory: str, scenario: str) -> None:
    from datetime import timedelta

    import torch.distributed as dist
    directory = Path(directory)
    report = {"rank": rank, "writes": 0, "raised": None, "factory_calls": 0}
    original_save = W.atomic_torch_save
    original_snapshot = W.snapshot_to_cpu

    def save(path, state):
        report["writes"] += 1
        if scenario in {"check", "submit", "flush", "close"}:
            raise OSError("injected checkpoint disk failure")
        original_save(path, state)

    def snapshot(state):
        if scenario == "snapshot":
            raise MemoryError("injected CPU snapshot failure")
        return original_snapshot(state)

    W.atomic_torch_save = save
    W.snapshot_to_cpu = snapshot
    dist.init_process_group("gloo", init_method=(directory / "rendezvous").as_uri(), rank=rank, world_size=2,
                            timeout=timedelta(seconds=15))
    try:
        if scenario == "exceptional":
            try:
                with W.DistributedCheckpointWriter(directory / "latest.pt", rank=rank, distributed=True) as writer:
                    writer.submit({"step": 1, "tokens_seen": 1} if rank == 0 else None)

                    def forbidden(*a, **k):
                        raise AssertionError("exceptional exit attempted a collective")

                    dist.broadcast_object_list = forbidden
                    dist.broadcast = forbidden
                    raise KeyError("rank-local training failure")
            except KeyError:
                report["raised"] = "KeyError"
        else:
            try:
                with W.DistributedCheckpointWriter(directory / "latest.pt", rank=rank, distributed=True) as writer:
                    state = {"weight": torch.tensor([1.0, 2.0]), "step": 1, "tokens_seen": 2}

                    def factory():
                        report["factory_calls"] += 1
                        assert rank == 0
                        if scenario == "factory":
                            raise ValueError("injected checkpoint construction failure")
                        return state

                    if scenario in {"factory", "normal_factory"}:
                        writer.submit(state_factory=factory)
                    else:
                        writer.submit(state if rank == 0 else None)
                    if scenario in {"check", "submit", "flush", "close"}:
                        if rank == 0:
                            writer._writer._idle.wait(10)  # the injected disk error has happened
                        dist.barrier()
                        if scenario == "check":
                            writer.check()
                        elif scenario == "submit":
                            writer.submit(state if rank == 0 else None)
                        elif scenario == "flush":
                            writer.flush()
            except BaseException as error:  # noqa: BLE001
                report["raised"] = f"{type(error).__name__}: {error}"
    finally:
        (directory / f"report-{rank}.json").write_text(json.dumps(report))
        dist.destroy_process_group()


def _spawn(tmp_path, scenario):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(ROOT))
    procs = [subprocess.Popen([sys.executable, __file__, str(rank), str(tmp_path), scenario], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outs = [p.communicate(timeout=60)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    return [json.loads((tmp_path / f"report-{r}.json").read_text()) for r in range(2)]


@pytest.mark.parametrize("scenario", ["check", "submit", "flush", "close", "snapshot", "factory"])
def test_rank_zero_failure_reaches_both_ranks(tmp_path, scenario):
    reports = _spawn(tmp_path, scenario)
    assert reports[0]["raised"] and reports[1]["raised"], reports
    assert "injected" in reports[0]["raised"] and "injected" in reports[1]["raised"]
    assert reports[1]["writes"] == 0 and reports[1]["factory_calls"] == 0


@pytest.mark.parametrize("scenario", ["normal", "normal_factory"])
def test_normal_exit_publishes_one_checkpoint(tmp_path, scenario):
    reports = _spawn(tmp_path, scenario)
    assert reports[0]["raised"] is None and reports[1]["raised"] is None
    assert reports[0]["writes"] == 1 and reports[1]["writes"] == 0
    assert torch.equal(torch.load(tmp_path / "latest.pt")["weight"], torch.tensor([1.0, 2.0]))


def test_exceptional_exit_issues_no_collective(tmp_path):
    reports = _spawn(tmp_path, "exceptional")
    assert [r["raised"] for r in reports] == ["KeyError", "KeyError"]
    assert torch.load(tmp_path / "latest.pt")["step"] == 1


if __name__ == "__main__":
    _worker(int(sys.argv[1]), sys.argv[2], sys.argv[3])
