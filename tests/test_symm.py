"""Symmetric memory (`parallel/symm.py` over `ops/csrc/symm_alloc.cpp`).

CPU (3 gloo ranks): the descriptor exchange -- every rank's file descriptor reaches every other rank over
abstract Unix sockets, and the one-to-all form delivers rank 0's only -- checked by reading through the
received descriptors.  GPU (2 ranks, needs two devices): a buffer from the package's own allocator is mapped by
both ranks (peer stores land, peer loads see them), the multimem address reduces and broadcasts when the fabric
offers one, the in-kernel all-reduce runs on it, and dropping the buffer releases every mapping.
The file doubles as the worker.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def spawn(mode: str, world: int, tmp_path: Path, env_extra=None, timeout=300):
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    env.update(env_extra or {})
    procs = [subprocess.Popen([sys.executable, __file__, mode, str(rank), str(world), str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outputs.append(out)
    for rank, p in enumerate(procs):
        assert p.returncode == 0, f"rank {rank} failed:\n{outputs[rank][-3000:]}"
    return [json.loads((tmp_path / f"report-{rank}.json").read_text()) for rank in range(world)]


def worker(mode: str, rank: int, world: int, out_dir: Path) -> None:
    import torch.distributed as dist
    from warpstate_ai_b200.parallel import symm
    cuda = mode.startswith("gpu")
    device = torch.device("cuda", rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dist.init_process_group("nccl" if cuda else "gloo", init_method=(out_dir / "rendezvous").as_uri(), rank=rank,
                            world_size=world, **({"device_id": device} if cuda else {}))
    report = {}
    if mode == "cpu_fds":
        mine = out_dir / f"payload-{rank}.txt"
        mine.write_text(f"hello from {rank}")
        fd = os.open(mine, os.O_RDONLY)
        got = symm.exchange_descriptors(fd, rank, world, None)
        report["all_to_all"] = {str(source): os.pread(peer, 64, 0).decode() for source, peer in got.items()}
        for peer in got.values():
            os.close(peer)
        got = symm.exchange_descriptors(fd if rank == 0 else -1, rank, world, None, only_from=0)
        report["from_zero"] = {str(source): os.pread(peer, 64, 0).decode() for source, peer in got.items()}
        for peer in got.values():
            os.close(peer)
        os.close(fd)
    elif mode == "cpu_vote":
        # a local step that fails on ONE rank must end as the same error on EVERY rank (nobody is left in a collective)
        owner = symm._OwnAllocation.__new__(symm._OwnAllocation)
        owner.group, owner.rank, owner.world, owner.handle = None, rank, world, None

        def step():
            if rank == 1:
                raise RuntimeError("cuMemCreate refused (simulated)")

        try:
            owner._together(step, "allocation")
            report["raised"] = None
        except symm.SymmetricAllocationError as error:
            report["raised"] = str(error)
        owner._together(lambda: None, "allocation")      # and a step that works everywhere goes on
        report["went_on"] = True
    elif mode == "gpu_buffer":
        import ctypes
        from warpstate_ai_b200.ops import _ext
        _ext.require()
        assert symm.provider() == "own"
        n = 1 << 20
        buf = symm.allocate(n, torch.float32, device)
        report["peers_distinct"] = len(set(buf.peer_ptrs)) == world and all(buf.peer_ptrs)
        report["multicast"] = bool(buf.multicast_ptr)
        buf.tensor.fill_(float(rank + 1))
        buf.barrier()
        # the peer's mapping in THIS process: read what the peer wrote, then write into it (driver copies: no
        # library kernel is handed a peer address)
        peer = (rank + 1) % world
        scratch = torch.zeros(1, dtype=torch.float32, device=device)
        torch.cuda.synchronize()
        symm.copy_bytes(scratch.data_ptr(), buf.peer_ptrs[peer] + 4 * 123, 4)
        report["peer_read"] = float(scratch[0])
        buf.barrier()
        scratch.fill_(100.0 + rank)
        torch.cuda.synchronize()
        symm.copy_bytes(buf.peer_ptrs[peer] + 4 * 7, scratch.data_ptr(), 4)
        buf.barrier()
        report["peer_wrote_here"] = float(buf.tensor[7])
        # the in-kernel all-reduce on the own allocator (peer loads, and multimem when there is an address)
        flags = symm.allocate(64, torch.int32, device)
        status = torch.zeros(8, dtype=torch.int32, device=device)
        for label, mc in (("p2p", 0), ("nvls", buf.multicast_ptr)):
            if label == "nvls" and not mc:
                report["nvls"] = "unavailable"
                continue
            src = torch.full((n,), float(rank + 1), device=device) + torch.arange(n, device=device) % 7
            buf.tensor.copy_(src)
            want = src.clone()
            dist.all_reduce(want)
            want /= world
            buf.barrier()
            torch.ops.ws_b200.grad_allreduce(buf.peer_ptrs, flags.peer_ptrs, mc, rank, world, 0, n, 0 if label == "p2p" else 1,
                                             1, 1.0 / world, True, 16, None, status, 20.0)
            torch.cuda.synchronize()
            buf.barrier()
            report[label] = float((buf.tensor - want).abs().max())
        report["status"] = int(status[0])
        before = torch.cuda.mem_get_info(device)[0]
        del buf, flags
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        report["freed_bytes"] = torch.cuda.mem_get_info(device)[0] - before
    (out_dir / f"report-{rank}.json").write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


def test_descriptor_exchange_between_three_processes(tmp_path):
    reports = spawn("cpu_fds", 3, tmp_path, env_extra={"CUDA_VISIBLE_DEVICES": ""})
    for rank, report in enumerate(reports):
        others = {str(r): f"hello from {r}" for r in range(3) if r != rank}
        assert report["all_to_all"] == others
        assert report["from_zero"] == ({} if rank == 0 else {"0": "hello from 0"})


def test_a_failure_on_one_rank_is_raised_on_every_rank(tmp_path):
    reports = spawn("cpu_vote", 3, tmp_path, env_extra={"CUDA_VISIBLE_DEVICES": ""})
    for report in reports:
        assert report["raised"] == "symmetric memory (allocation) failed: rank 1: cuMemCreate refused (simulated)"
        assert report["went_on"] is True


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two CUDA devices")
def test_own_allocator_maps_peers_and_serves_the_collectives(tmp_path):
    reports = spawn("gpu_buffer", 2, tmp_path)
    for rank, report in enumerate(reports):
        peer = (rank + 1) % 2
        assert report["peers_distinct"] and report["status"] == 0
        assert report["peer_read"] == float(peer + 1)            # what the peer filled its buffer with
        assert report["peer_wrote_here"] == 100.0 + peer         # the peer's store landed in this rank's memory
        assert report["p2p"] < 1e-6
        assert report["nvls"] == "unavailable" or report["nvls"] < 1e-5
        assert report["freed_bytes"] > 0                          # dropping the buffers returned device memory


if __name__ == "__main__":
    worker(sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), Path(sys.argv[4]))
