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


class Supervisor:
    """Runs one child command and walks it through the stop protocol.

    Phases: ``running`` -> (stop signal) ``draining``: the stop file exists, workers finish their update and
    save -> (grace period over) ``terminating``: the child got SIGTERM -> (second deadline over) ``killing``:
    every descendant ever seen is SIGKILLed.  Each phase has one entry action and one deadline."""

    SIGNALS = (signal.SIGTERM, signal.SIGINT, signal.SIGUSR1)

    def __init__(self, stop_path: Path, grace_seconds: float, terminate_seconds: float):
        self.stop_path = stop_path
        self.deadlines = {"draining": grace_seconds, "terminating": terminate_seconds}
        self.phase = "running"
        self.phase_began = None
        self.stop_seen_at = None         # set by the signal handler; the loop does the phase change
        self.child = None
        self.tree = None

    # ---- signal side: only record and touch the file (async-signal-simple)
    def _on_signal(self, signum, frame) -> None:
        if self.stop_seen_at is None:
            self.stop_seen_at = time.monotonic()
        os.close(os.open(self.stop_path, os.O_WRONLY | os.O_CREAT, 0o600))

    def _enter(self, phase: str, now: float) -> None:
        self.phase, self.phase_began = phase, now
        self.tree.scan()
        if phase == "draining":
            print("Stop requested: letting the workers finish their update and checkpoint.", flush=True)
        elif phase == "terminating":
            print("The grace period is over: sending SIGTERM to the launcher process.", flush=True)
            with _ignore_missing():
                self.child.send_signal(signal.SIGTERM)
        elif phase == "killing":
            print("The termination deadline is over: killing every process of the job.", flush=True)
            self.tree.kill_all()
            self.child.kill()

    def _advance(self, now: float) -> None:
        if self.phase == "running" and self.stop_seen_at is not None:
            self._enter("draining", self.stop_seen_at)
        following = {"draining": "terminating", "terminating": "killing"}.get(self.phase)
        if following and now - self.phase_began >= self.deadlines[self.phase]:
            self._enter(following, now)

    def run(self, command, environment, pass_fds=(), poll_seconds: float = 0.2, scan_seconds: float = 2.0) -> int:
        saved = {sig: signal.signal(sig, self._on_signal) for sig in self.SIGNALS}
        try:
            if self.stop_seen_at is not None or self.stop_path.exists():
                return 0                                   # a stop request was already pending: start nothing
            self.child = subprocess.Popen(command, env=environment, start_new_session=True, pass_fds=pass_fds)
            self.tree = ProcessTree(self.child.pid)
            print(f"Started PID {self.child.pid}; a stop request creates {self.stop_path}", flush=True)
            next_scan = 0.0
            while self.child.poll() is None and self.phase != "killing":
                now = time.monotonic()
                if now >= next_scan:
                    self.tree.scan()
                    next_scan = now + scan_seconds
                self._advance(now)
                with _ignore_timeout():
                    self.child.wait(timeout=poll_seconds)
            if self.phase == "killing":
                self.child.wait(timeout=5)
            return self.child.returncode
        finally:
            if self.child is not None:
                self.tree.scan()
                if self.child.poll() is None:
                    self.tree.kill_all()
                    self.child.kill()
                    self.child.wait(timeout=5)
                self.tree.kill_all()                       # orphans of a child that exited on its own
            for sig, handler in saved.items():
                signal.signal(sig, handler)


class _ignore_missing:
    def __enter__(self):
        return self

    def __exit__(self, kind, value, trace):
        return kind is not None and issubclass(kind, ProcessLookupError)


class _ignore_timeout:
    def __enter__(self):
        return self

    def __exit__(self, kind, value, trace):
        return kind is not None and issubclass(kind, subprocess.TimeoutExpired)


def supervise(command, stop_path, environment, *, grace_seconds: float = 820, terminate_seconds: float = 45,
              pass_fds=(), poll_seconds: float = 0.2, scan_seconds: float = 2.0) -> int:
    """Run ``command`` under the stop protocol; returns its exit status (negative: killed by that signal)."""
    supervisor = Supervisor(workspace_path(stop_path), grace_seconds, terminate_seconds)
    return supervisor.run(command, environment, pass_fds, poll_seconds, scan_seconds)


# every tool that caches on disk is pointed inside the workspace (the reference's list, reference
# ops/launch_training.py:140-160; the compiler caches matter to the bootstrap and to the PyTorch yardstick arms)
CACHE_VARIABLES = {"XDG_CACHE_HOME": "", "UV_CACHE_DIR": "uv", "PIP_CACHE_DIR": "pip", "TORCH_HOME": "torch",
                   "CUDA_CACHE_PATH": "cuda", "TRITON_CACHE_DIR": "triton", "TORCHINDUCTOR_CACHE_DIR": "torchinductor",
                   "TORCH_EXTENSIONS_DIR": "torch-extensions"}


def training_environment(work: Path) -> dict:
    """The child's environment: every cache and temporary directory inside the workspace, no bytecode files,
    and the stop file the workers poll."""
    root = workspace_root()
    places = {"TMPDIR": root / "tmp", "HF_HOME": work / "hf-cache", "HF_DATASETS_CACHE": work / "hf-cache/datasets",
              "HF_XET_CACHE": work / "hf-cache/xet"}
    places.update({name: root / ".cache" / sub for name, sub in CACHE_VARIABLES.items()})
    environment = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    for name, place in places.items():
        place = workspace_path(place)
        place.mkdir(parents=True, exist_ok=True)
        environment[name] = str(place)
    environment["WARPSTATE_STOP_FILE"] = str(workspace_path(work / "control/training-stop-request"))
    return environment


def build_command(processes: int, runner: Path, work: Path, logs: Path, extra) -> list[str]:
    """One interpreter for a single process, otherwise a standalone ``torch.distributed.run`` on the loopback."""
    prefix = [sys.executable]
    if processes > 1:
        prefix += ["-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes", "1",
                   "--nproc-per-node", str(processes), "--log-dir", str(logs)]
    return [*prefix, str(runner), "--work-dir", str(work), *extra]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--processes", type=int, default=8, help="worker processes (one per GPU)")
    parser.add_argument("--work-dir", type=Path, default=PACKAGE / "work")
    parser.add_argument("--runner", type=Path, default=PACKAGE / "run_40b.py")
    parser.add_argument("--grace-seconds", type=float, default=820, help="time the workers get to stop by themselves")
    parser.add_argument("--terminate-seconds", type=float, default=45, help="time between SIGTERM and SIGKILL")
    parser.add_argument("runner_args", nargs=argparse.REMAINDER, help="after --: arguments of the runner")
    args = parser.parse_args(argv)
    if args.processes < 1:
        parser.error("--processes must be at least 1")
    forwarded = args.runner_args[1:] if args.runner_args[:1] == ["--"] else args.runner_args
    if any(item.split("=", 1)[0] == "--work-dir" for item in forwarded):
        parser.error("--work-dir belongs to the launcher (before the -- separator), which passes it on")
    try:
        work = workspace_path(args.work_dir)
        control, logs = workspace_path(work / "control"), workspace_path(work / "logs/torchrun-training")
    except ValueError as problem:
        parser.error(str(problem))
    control.mkdir(parents=True, exist_ok=True)
    stop_file = control / "training-stop-request"
    with process_lock(control / "training-launcher.lock"):
        stop_file.unlink(missing_ok=True)
        logs.mkdir(parents=True, exist_ok=True)
        status = supervise(build_command(args.processes, args.runner, work, logs, forwarded), stop_file,
                           training_environment(work), grace_seconds=args.grace_seconds,
                           terminate_seconds=args.terminate_seconds)
    return 128 - status if status < 0 else status


if __name__ == "__main__":
    sys.exit(main())
