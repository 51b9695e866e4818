"""Supervise a (torchrun) training job so that a stop request gives the workers time to finish
the current update and save, and escalates only when they do not.

Protocol (reference ops/launch_training.py:67-159): SIGTERM / SIGINT / SIGUSR1 to the supervisor
touches a *stop file* (workers poll ``WARPSTATE_STOP_FILE``; a signal cannot reach them because
torchrun gives each worker its own session); after ``grace_seconds`` the launcher gets SIGTERM;
after a further ``terminate_seconds`` every recorded descendant is SIGKILLed.  Descendants are
tracked by (pid, start time) pairs read from ``/proc`` so that a recycled PID is never
signalled.  Lock file descriptors can be passed down to the child so that exclusion outlives the
supervisor.
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

from ..utils.io import process_lock

PACKAGE = Path(__file__).resolve().parents[2]


def workspace_root() -> Path:
    return Path(os.environ.get("WARPSTATE_WORKSPACE", "/workspace/WarpState")).resolve()


def workspace_path(value) -> Path:
    path = Path(value).expanduser().resolve()
    if not path.is_relative_to(workspace_root()):
        raise ValueError(f"Created paths must stay inside {workspace_root()}: {path}")
    return path


def process_info(pid: int):
    """(parent pid, start time in clock ticks) or None; the start time disambiguates PID reuse."""
    try:
        fields = Path(f"/proc/{pid}/stat").read_text().rsplit(")", 1)[1].split()
        return int(fields[1]), int(fields[19])
    except (OSError, ValueError, IndexError):
        return None


class ProcessTree:
    """Remembers every descendant ever seen under a root process."""

    def __init__(self, root_pid: int):
        self.root = root_pid
        info = process_info(root_pid)
        self.root_started = info[1] if info else None
        self.known: dict[int, int] = {}

    @staticmethod
    def _snapshot() -> dict[int, tuple[int, int]]:
        table = {}
        for entry in Path("/proc").iterdir():
            if entry.name.isdigit():
                info = process_info(int(entry.name))
                if info is not None:
                    table[int(entry.name)] = info
        return table

    def scan(self) -> None:
        table = self._snapshot()
        alive = set()
        if table.get(self.root, (None, None))[1] == self.root_started:
            alive.add(self.root)
        alive.update(pid for pid, started in self.known.items() if table.get(pid, (None, None))[1] == started)
        frontier = set(alive)
        while frontier:
            frontier = {pid for pid, (ppid, _) in table.items() if ppid in frontier} - alive
            alive |= frontier
        for pid in alive - {self.root}:
            self.known[pid] = table[pid][1]

    def kill_all(self) -> None:
        for pid, started in self.known.items():
            info = process_info(pid)
            if info is not None and info[1] == started:
                try:
                    os.kill(pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass


def supervise(command, stop_path, environment, *, grace_seconds: float = 820, terminate_seconds: float = 45,
              pass_fds=(), poll_seconds: float = 0.2, scan_seconds: float = 2.0) -> int:
    stop_path = workspace_path(stop_path)
    state = {"stopped_at": None}
    previous = {}

    def request_stop(signum, frame):
        if state["stopped_at"] is None:
            state["stopped_at"] = time.monotonic()
        os.close(os.open(stop_path, os.O_CREAT | os.O_WRONLY, 0o600))

    for sig in (signal.SIGTERM, signal.SIGINT, signal.SIGUSR1):
        previous[sig] = signal.signal(sig, request_stop)
    child = None
    tree = None
    try:
        if state["stopped_at"] is not None or stop_path.exists():
            return 0
        child = subprocess.Popen(command, env=environment, start_new_session=True, pass_fds=pass_fds)
        tree = ProcessTree(child.pid)
        print(f"Training launcher started PID {child.pid}; stop requests use {stop_path}", flush=True)
        last_scan = 0.0
        announced = False
        terminated_at = None
        while child.poll() is None:
            now = time.monotonic()
            if now - last_scan >= scan_seconds:
                tree.scan()
                last_scan = now
            stopped_at = state["stopped_at"]
            if stopped_at is not None:
                if not announced:
                    print("Stop requested; waiting for the current update and checkpoint.", flush=True)
                    announced = True
                if terminated_at is None and now - stopped_at >= grace_seconds:
                    tree.scan()
                    print("Graceful-stop deadline exceeded; asking torchrun to terminate its workers.", flush=True)
                    try:
                        child.send_signal(signal.SIGTERM)
                    except ProcessLookupError:
                        pass
                    terminated_at = now
                elif terminated_at is not None and now - terminated_at >= terminate_seconds:
                    tree.scan()
                    print("Termination deadline exceeded; killing remaining training processes.", flush=True)
                    tree.kill_all()
                    child.kill()
                    child.wait(timeout=5)
                    break
            try:
                child.wait(timeout=poll_seconds)
            except subprocess.TimeoutExpired:
                pass
        return child.returncode
    finally:
        if child is not None and tree is not None:
            tree.scan()
            if child.poll() is None:
                tree.kill_all()
                child.kill()
                child.wait(timeout=5)
            tree.kill_all()
        for sig, handler in previous.items():
            signal.signal(sig, handler)


def training_environment(work: Path) -> dict:
    root = workspace_root()
    cache = workspace_path(root / ".cache")
    hf = workspace_path(work / "hf-cache")
    locations = {"TMPDIR": root / "tmp", "XDG_CACHE_HOME": cache, "PIP_CACHE_DIR": cache / "pip",
                 "TORCH_HOME": cache / "torch", "CUDA_CACHE_PATH": cache / "cuda",
                 "TORCH_EXTENSIONS_DIR": cache / "torch-extensions", "HF_HOME": hf, "HF_DATASETS_CACHE": hf / "datasets"}
    environment = os.environ.copy()
    for key, value in locations.items():
        path = workspace_path(value)
        path.mkdir(parents=True, exist_ok=True)
        environment[key] = str(path)
    environment["PYTHONDONTWRITEBYTECODE"] = "1"
    environment["WARPSTATE_STOP_FILE"] = str(workspace_path(work / "control/training-stop-request"))
    return environment


def build_command(processes: int, runner: Path, work: Path, logs: Path, extra) -> list[str]:
    command = [sys.executable]
    if processes > 1:
        command += ["-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes", "1",
                    "--nproc-per-node", str(processes), "--log-dir", str(logs)]
    return command + [str(runner), "--work-dir", str(work), *extra]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--processes", type=int, default=8)
    parser.add_argument("--work-dir", type=Path, default=PACKAGE / "work")
    parser.add_argument("--runner", type=Path, default=PACKAGE / "run_40b.py")
    parser.add_argument("--grace-seconds", type=float, default=820)
    parser.add_argument("--terminate-seconds", type=float, default=45)
    parser.add_argument("runner_args", nargs=argparse.REMAINDER)
    args = parser.parse_args(argv)
    if args.processes < 1:
        parser.error("--processes must be positive")
    extra = args.runner_args[1:] if args.runner_args[:1] == ["--"] else args.runner_args
    if any(v == "--work-dir" or v.startswith("--work-dir=") for v in extra):
        parser.error("Pass --work-dir to the launcher, before the -- separator")
    try:
        work = workspace_path(args.work_dir)
        control = workspace_path(work / "control")
        logs = workspace_path(work / "logs/torchrun-training")
        stop_path = workspace_path(control / "training-stop-request")
        lock_path = workspace_path(control / "training-launcher.lock")
    except ValueError as error:
        parser.error(str(error))
    control.mkdir(parents=True, exist_ok=True)
    with process_lock(lock_path):
        stop_path.unlink(missing_ok=True)
        logs.mkdir(parents=True, exist_ok=True)
        result = supervise(build_command(args.processes, args.runner, work, logs, extra), stop_path,
                           training_environment(work), grace_seconds=args.grace_seconds,
                           terminate_seconds=args.terminate_seconds)
    return 128 - result if result < 0 else result


if __name__ == "__main__":
    sys.exit(main())
