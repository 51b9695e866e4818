"""Resumable, verified transfer of large artifacts (checkpoints, archives) between hosts.

Both ends of a transfer are *endpoints* that run the same stdlib-only agent
(``transfer_agent.py``): the local one as ``python -c <agent>``, the remote one as
``ssh ... python3 -c <agent>``.  A chunk moves by piping the source endpoint's ``read`` into the
destination endpoint's ``write``; no chunk is ever buffered in this process, the receiver
verifies each chunk's SHA-256 before writing its receipt, up to ``--connections`` chunks are in
flight on independent connections, a failed chunk is retried with back-off, and the file
appears under its final name only after a full-file hash (never replacing an existing file).
Re-running the same command resumes: receipted chunks are re-hashed at the receiver and skipped.

    python -m warpstate_ai_b200.orchestration.transfer SRC DST --host user@box \
        --key KEY --known-hosts FILE [--pull] [--connections 8] [--chunk-mib 256]

Same behaviour and on-disk receiver layout as the reference's ops/transfer_artifacts.py:369-660
(which embeds two copies of the agent as function source instead of one shared file).
"""
from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import json
import os
import re
import shlex
import subprocess
import sys
import threading
import time
from pathlib import Path

from . import transfer_agent as agent

AGENT_SOURCE = Path(agent.__file__).read_text()
MIB = 1 << 20


class Endpoint:
    """One side of a transfer: a command prefix that runs the agent with given arguments."""

    def __init__(self, prefix: list[str] | None = None, python: str | None = None, env: dict | None = None):
        self.prefix = list(prefix or [])
        self.python = python or (sys.executable if not prefix else "python3")
        self.env = env

    def command(self, *arguments) -> list[str]:
        words = [self.python, "-c", AGENT_SOURCE, *(str(a) for a in arguments)]
        if not self.prefix:
            return words
        exports = "" if not self.env else " ".join(f"{k}={shlex.quote(v)}" for k, v in self.env.items()) + " "
        return self.prefix + [exports + shlex.join(words)]

    def popen(self, arguments, **kwargs) -> subprocess.Popen:
        environment = None if self.prefix or not self.env else dict(os.environ, **self.env)
        return subprocess.Popen(self.command(*arguments), env=environment, **kwargs)

    def call(self, arguments, payload: bytes | None = None) -> dict:
        process = self.popen(arguments, stdin=subprocess.PIPE if payload is not None else subprocess.DEVNULL,
                             stdout=subprocess.PIPE, stderr=subprocess.PIPE)
        out, err = process.communicate(payload)
        if process.returncode:
            raise RuntimeError(f"endpoint failed ({process.returncode}): {err.decode(errors='replace').strip()[-400:]}")
        return json.loads(out)


def ssh_prefix(host: str, port: int, key: Path, known_hosts: Path, compress: bool = False) -> list[str]:
    """A locked-down ssh invocation: only the given key and host-key file, no agent, no config."""
    if host.startswith("-") or not 1 <= port <= 65535:
        raise ValueError("Invalid SSH host or port")
    words = ["ssh", "-F", "/dev/null", "-p", str(port), "-i", str(key)]
    for option in ("BatchMode=yes", "IdentitiesOnly=yes", "StrictHostKeyChecking=yes", f"UserKnownHostsFile={known_hosts}",
                   "GlobalKnownHostsFile=/dev/null", "ConnectTimeout=20", "ServerAliveInterval=15",
                   "ServerAliveCountMax=4", "ControlMaster=no", "ControlPath=none"):
        words += ["-o", option]
    if compress:
        words.append("-C")
    return words + [host]


class Transfer:
    def __init__(self, source_end: Endpoint, dest_end: Endpoint, source: Path, destination: Path, *,
                 chunk_bytes: int = 256 * MIB, connections: int = 8, retries: int = 3, expected_sha256: str | None = None,
                 log=print):
        self.src, self.dst = source_end, dest_end
        self.source, self.destination = source, destination
        self.chunk_bytes, self.connections, self.retries = chunk_bytes, connections, retries
        self.expected = expected_sha256
        self.log = log
        self.cancelled = threading.Event()
        self.live: set[subprocess.Popen] = set()
        self.guard = threading.Lock()

    # -------------------------------------------------------------------------------- processes
    def start(self, endpoint: Endpoint, arguments, **kwargs) -> subprocess.Popen:
        if self.cancelled.is_set():
            raise RuntimeError("Transfer cancelled")
        process = endpoint.popen(arguments, **kwargs)
        with self.guard:
            self.live.add(process)
            if self.cancelled.is_set():
                process.terminate()
        return process

    def cancel(self) -> None:
        self.cancelled.set()
        with self.guard:
            for process in self.live:
                if process.poll() is None:
                    process.terminate()

    def move_chunk(self, manifest: dict, identity: list, index: int) -> dict:
        offset = index * manifest["chunk_size"]
        length = min(manifest["chunk_size"], manifest["size"] - offset)
        started, waited = [], set()
        try:
            reader = self.start(self.src, ["read", self.source, json.dumps(identity), offset, length],
                                stdin=subprocess.DEVNULL, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
            started.append(reader)
            writer = self.start(self.dst, ["write", self.destination, manifest["sha256"], index],
                                stdin=reader.stdout, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
            started.append(writer)
            reader.stdout.close()  # only the writer holds the read end: its failure breaks the reader's pipe
            reader.stdout = None
            out, writer_err = writer.communicate()
            waited.add(writer)
            _, reader_err = reader.communicate()
            waited.add(reader)
            if reader.returncode:
                raise RuntimeError(f"source failed ({reader.returncode}): {reader_err.decode(errors='replace').strip()[-300:]}")
            if writer.returncode:
                raise RuntimeError(f"receiver failed ({writer.returncode}): {writer_err.decode(errors='replace').strip()[-300:]}")
            result = json.loads(out)
            if result["index"] != index or result["sha256"] != manifest["chunk_sha256"][index]:
                raise ValueError("Receiver returned an invalid chunk acknowledgment")
            return result
        finally:
            for process in started:
                if process.poll() is None:
                    process.terminate()
            for process in started:
                if process not in waited:
                    process.communicate()
                with self.guard:
                    self.live.discard(process)

    def move_with_retries(self, manifest, identity, index) -> dict:
        for attempt in range(self.retries):
            try:
                return self.move_chunk(manifest, identity, index)
            except Exception:
                if self.cancelled.is_set() or attempt + 1 == self.retries:
                    raise
                self.cancelled.wait(min(2 ** attempt, 10))
        raise AssertionError

    # ------------------------------------------------------------------------------------- run
    def run(self) -> dict:
        answer = self.src.call(["manifest", self.source, self.chunk_bytes])
        manifest, identity = answer["manifest"], answer["identity"]
        if self.expected is not None and manifest["sha256"] != self.expected:
            raise ValueError("Source SHA256 does not match the expected value")
        self.log(f"Source: {manifest['size']:,} bytes; SHA256 {manifest['sha256']}")
        prepared = self.dst.call(["prepare", self.destination, manifest["sha256"]], json.dumps(manifest).encode())
        if prepared.get("complete"):
            self.log("Destination already exists and its full SHA256 matches.")
            return {"complete": True, "sha256": manifest["sha256"], "sent_chunks": 0, "skipped_chunks": len(manifest["chunk_sha256"])}
        done = set(prepared["completed"])
        pending = [i for i in range(len(manifest["chunk_sha256"])) if i not in done]
        moved, begin = 0, time.monotonic()
        self.log(f"Resuming: {len(done)} verified chunks; {len(pending)} remaining; {self.connections} connections.")
        pool = concurrent.futures.ThreadPoolExecutor(max_workers=self.connections)
        try:
            futures = [pool.submit(self.move_with_retries, manifest, identity, i) for i in pending]
            for future in concurrent.futures.as_completed(futures):
                result = future.result()
                done.add(result["index"])
                moved += result["bytes"]
                rate = moved / max(time.monotonic() - begin, 1e-3) / MIB
                self.log(f"{len(done)}/{len(manifest['chunk_sha256'])} chunks  {rate:.1f} MiB/s")
        except BaseException:
            self.cancel()
            pool.shutdown(wait=True, cancel_futures=True)
            raise
        pool.shutdown(wait=True)
        if self.src.call(["identity", self.source, json.dumps(identity)])["identity"] != identity:
            raise ValueError("Source changed during transfer; refusing final publication")
        final = self.dst.call(["finalize", self.destination, manifest["sha256"]])
        if not final["complete"] or final["sha256"] != manifest["sha256"]:
            raise ValueError("Invalid final verification response")
        self.log(f"Complete: {self.destination}; SHA256 {final['sha256']}")
        return {"complete": True, "sha256": final["sha256"], "sent_chunks": len(pending),
                "skipped_chunks": len(manifest["chunk_sha256"]) - len(pending)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("source", type=agent.confined)
    p.add_argument("destination", type=agent.confined)
    p.add_argument("--host", required=True, help="user@hostname")
    p.add_argument("--port", type=int, default=22)
    p.add_argument("--key", type=agent.confined, required=True)
    p.add_argument("--known-hosts", type=agent.confined, required=True, help="verified host-key file inside the workspace")
    p.add_argument("--connections", type=int, default=8)
    p.add_argument("--chunk-mib", type=int, default=256)
    p.add_argument("--retries", type=int, default=3)
    p.add_argument("--compress", action="store_true")
    p.add_argument("--pull", action="store_true", help="download SOURCE from the host instead of uploading it")
    p.add_argument("--expected-sha256")
    p.add_argument("--manifest-dir", type=agent.confined, default=None)
    a = p.parse_args(argv)
    if min(a.connections, a.chunk_mib, a.retries) < 1:
        p.error("connections, chunk size and retries must be positive")
    if a.expected_sha256 is not None:
        if re.fullmatch(r"[0-9a-fA-F]{64}", a.expected_sha256) is None:
            p.error("--expected-sha256 must contain exactly 64 hexadecimal digits")
        a.expected_sha256 = a.expected_sha256.lower()
    remote = Endpoint(ssh_prefix(a.host, a.port, a.key, a.known_hosts, a.compress))
    local = Endpoint()
    source_end, dest_end = (remote, local) if a.pull else (local, remote)
    transfer = Transfer(source_end, dest_end, a.source, a.destination, chunk_bytes=a.chunk_mib * MIB,
                        connections=a.connections, retries=a.retries, expected_sha256=a.expected_sha256,
                        log=lambda m: print(m, flush=True))
    try:
        result = transfer.run()
    except KeyboardInterrupt:
        print("Interrupted; verified chunks are retained for resume.", file=sys.stderr)
        return 130
    if a.manifest_dir is not None:  # informational record; every run re-hashes its source
        a.manifest_dir.mkdir(parents=True, exist_ok=True)
        name = hashlib.sha256(f"{a.host}:{a.port}:{a.source}:{a.pull}".encode()).hexdigest()[:20] + ".json"
        (a.manifest_dir / name).write_text(json.dumps({"source": str(a.source), **result}, indent=2) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
