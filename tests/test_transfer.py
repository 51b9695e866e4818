"""Artifact transfer without an SSH server: both endpoints are local agent processes, one of them
reached through a shell-string prefix (the quoting path an ssh command takes).  Covers parallel
upload + verified publication, resume with corrupt receipts, never-overwrite, path confinement,
changed-source rejection and failed-chunk retention (reference test_artifact_transfer.py:58-248)."""
import hashlib
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from warpstate_ai_b200.orchestration import transfer as T
from warpstate_ai_b200.orchestration import transfer_agent as A


@pytest.fixture()
def ws(tmp_path, monkeypatch):
    root = (tmp_path / "ws").resolve()
    root.mkdir()
    monkeypatch.setenv("WARPSTATE_WORKSPACE", str(root))
    source = root / "out/model.pt"
    source.parent.mkdir()
    source.write_bytes(os.urandom(5 * 4096 + 123))
    return root, source


def shell_endpoint(root: Path) -> T.Endpoint:
    """Stands in for `ssh host`: a prefix that receives ONE shell string, like a remote shell."""
    return T.Endpoint(prefix=["sh", "-c"], python=sys.executable, env={"WARPSTATE_WORKSPACE": str(root)})


def make(root, source, dest, **kw):
    return T.Transfer(T.Endpoint(), shell_endpoint(root), source, dest, chunk_bytes=4096, connections=3, retries=2,
                      log=lambda m: None, **kw)


def sha(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def test_parallel_upload_publishes_only_after_verification(ws):
    root, source = ws
    dest = root / "in/model.pt"
    result = make(root, source, dest).run()
    assert result["sent_chunks"] == 6 and dest.read_bytes() == source.read_bytes()
    assert not Path(f"{dest}.uploading").exists()
    again = make(root, source, dest).run()  # destination already complete
    assert again["sent_chunks"] == 0 and again["skipped_chunks"] == 6


def test_resume_rehashes_receipts_and_resends_corrupt_chunks(ws):
    root, source = ws
    dest = root / "in/model.pt"
    t = make(root, source, dest)
    answer = t.src.call(["manifest", source, 4096])
    manifest, identity = answer["manifest"], answer["identity"]
    t.dst.call(["prepare", dest, manifest["sha256"]], json.dumps(manifest).encode())
    for index in (0, 1, 2):
        t.move_chunk(manifest, identity, index)
    partial = Path(f"{dest}.uploading")
    with partial.open("r+b") as f:  # damage chunk 1 behind its receipt
        f.seek(4096 + 7)
        f.write(b"\x00\x01\x02")
    result = make(root, source, dest).run()
    assert result["skipped_chunks"] == 2 and result["sent_chunks"] == 4
    assert sha(dest) == manifest["sha256"]


def test_existing_destination_and_foreign_partial_are_protected(ws):
    root, source = ws
    dest = root / "in/model.pt"
    dest.parent.mkdir()
    dest.write_bytes(b"someone else's file")
    with pytest.raises(RuntimeError, match="never overwritten"):
        make(root, source, dest).run()
    assert dest.read_bytes() == b"someone else's file"
    other = root / "in/other.pt"
    Path(f"{other}.uploading").write_bytes(b"x")
    with pytest.raises(RuntimeError, match="sidecars without a manifest"):
        make(root, source, other).run()
    # a partial upload of a different source is not adopted either
    third = root / "in/third.pt"
    make(root, source, third).src.call(["manifest", source, 4096])
    t = make(root, source, third)
    m = t.src.call(["manifest", source, 4096])["manifest"]
    t.dst.call(["prepare", third, m["sha256"]], json.dumps(m).encode())
    source2 = root / "out/model2.pt"
    source2.write_bytes(os.urandom(9000))
    with pytest.raises(RuntimeError, match="another source"):
        make(root, source2, third).run()


def test_paths_outside_the_workspace_and_symlinks_are_rejected(ws, tmp_path):
    root, source = ws
    with pytest.raises(ValueError):
        A.confined(tmp_path / "elsewhere.pt")
    with pytest.raises(ValueError):
        A.confined(root)
    link = root / "link"
    link.symlink_to(root / "out")
    with pytest.raises(ValueError, match="symlink"):
        A.confined(link / "model.pt")
    with pytest.raises(RuntimeError, match="symlink"):
        make(root, link / "model.pt", root / "in/model.pt").run()
    with pytest.raises(RuntimeError, match="is not below"):
        make(root, source, tmp_path / "escape.pt").run()


def test_wrong_expected_hash_and_changed_source_are_rejected(ws):
    root, source = ws
    dest = root / "in/model.pt"
    with pytest.raises(ValueError, match="expected"):
        make(root, source, dest, expected_sha256="0" * 64).run()
    t = make(root, source, dest)
    answer = t.src.call(["manifest", source, 4096])
    manifest, identity = answer["manifest"], answer["identity"]
    t.dst.call(["prepare", dest, manifest["sha256"]], json.dumps(manifest).encode())
    source.write_bytes(source.read_bytes()[:-1] + b"!")  # same size, new content and mtime
    with pytest.raises(RuntimeError, match="source file changed"):
        t.move_chunk(manifest, identity, 0)
    assert not dest.exists()


def test_corrupt_stream_keeps_partial_and_never_publishes(ws):
    root, source = ws
    dest = root / "in/model.pt"
    t = make(root, source, dest)
    manifest = t.src.call(["manifest", source, 4096])["manifest"]
    t.dst.call(["prepare", dest, manifest["sha256"]], json.dumps(manifest).encode())
    # feed the receiver a chunk whose bytes do not match the manifest
    bad = t.dst.popen(["write", dest, manifest["sha256"], 0], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                      stderr=subprocess.PIPE)
    _, err = bad.communicate(b"\x00" * 4096)
    assert bad.returncode != 0 and b"chunk SHA256 mismatch" in err
    with pytest.raises(RuntimeError, match="receipt"):
        t.dst.call(["finalize", dest, manifest["sha256"]])
    assert not dest.exists() and Path(f"{dest}.uploading").exists()
    # a destination that appears before finalize is preserved
    result = make(root, source, root / "in/b.pt")
    m2 = result.src.call(["manifest", source, 4096])
    result.dst.call(["prepare", root / "in/b.pt", manifest["sha256"]], json.dumps(manifest).encode())
    for i in range(6):
        result.move_chunk(m2["manifest"], m2["identity"], i)
    (root / "in/b.pt").write_bytes(b"raced")
    with pytest.raises(RuntimeError, match="never overwritten"):
        result.dst.call(["finalize", root / "in/b.pt", manifest["sha256"]])
    assert (root / "in/b.pt").read_bytes() == b"raced"


def test_pull_direction_and_cli_arguments(ws, monkeypatch):
    root, source = ws
    dest = root / "pulled/model.pt"
    t = T.Transfer(shell_endpoint(root), T.Endpoint(), source, dest, chunk_bytes=4096, connections=2, log=lambda m: None)
    assert t.run()["sent_chunks"] == 6 and sha(dest) == sha(source)
    prefix = T.ssh_prefix("user@box", 2222, root / "key", root / "known")
    assert prefix[0] == "ssh" and "StrictHostKeyChecking=yes" in prefix and prefix[-1] == "user@box"
    with pytest.raises(ValueError):
        T.ssh_prefix("-oProxyCommand=x", 22, root / "key", root / "known")
