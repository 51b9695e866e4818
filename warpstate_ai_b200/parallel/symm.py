"""Symmetric memory: buffers that every rank of a single-node job can address directly.

A `SymmetricBuffer` is a CUDA tensor over memory that all ranks map, the table of peer addresses *as seen
from this process* and, when the NVSwitch fabric offers it, a multimem address whose loads reduce and whose
stores broadcast inside the switch (NVLS).

Two providers:

* ``own`` (default): this package's allocator.  `ops/csrc/symm_alloc.cpp` creates the physical allocation with
  the CUDA virtual-memory API, exports it as a file descriptor, imports and maps the peers' and sets up the
  multicast object; this module moves the descriptors between the processes -- every rank listens on an
  abstract Unix socket whose name is agreed over the process group, and sends its descriptor to every peer with
  ``SCM_RIGHTS`` -- and wraps the local mapping in a tensor.  Nothing but the driver and sockets is involved.
* ``torch``: PyTorch's ``torch.distributed._symmetric_memory`` (a private API), kept as a fallback selected
  with ``WARPSTATE_SYMM=torch``.

Everything that touches the memory afterwards is this package's own kernels (`ops/csrc/comm.cu`,
`gemm2_kernel<GATHER>`): plain loads and stores or ``multimem`` instructions only; no tensor map ever covers a
peer's mapping and no library kernel is given one.

The reference has no counterpart (its collectives are NCCL's, reference run_40b.py:601-603).
"""
from __future__ import annotations

import ctypes
import os
import socket
import uuid
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor          # this rank's buffer
    peer_ptrs: list[int]          # device addresses of every rank's buffer in this process
    multicast_ptr: int            # multimem address or 0
    rank: int
    world: int
    handle: object = None         # provider "torch": its rendezvous handle
    _owner: object = field(default=None, repr=False)   # provider "own": keeps the mappings alive

    def barrier(self) -> None:
        """Every rank has reached this point (host-side for the own provider, device-side for torch's)."""
        if self.handle is not None:
            self.handle.barrier()
        elif self.world > 1:
            torch.cuda.current_stream(self.tensor.device).synchronize()
            dist.barrier(group=self._owner.group)


def nvls_allowed() -> bool:
    """NVLS (multimem) is used unless disabled; failure-handling tests turn it off."""
    return os.environ.get("WARPSTATE_NVLS", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


def provider() -> str:
    return os.environ.get("WARPSTATE_SYMM", "own")


# ----------------------------------------------------------------------------------- own allocator
class _Library:
    """ctypes view of the allocator's C entry points."""

    def __init__(self):
        from ..ops import _ext
        lib = _ext.cdll()
        u64p, intp = ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_int)
        lib.ws_symm_last_error.restype = ctypes.c_char_p
        lib.ws_symm_padded_size.restype = ctypes.c_longlong
        lib.ws_symm_padded_size.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int]
        lib.ws_symm_create.argtypes = [ctypes.c_int, ctypes.c_longlong, u64p, u64p, intp]
        lib.ws_symm_import.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_longlong, u64p, u64p]
        lib.ws_symm_multicast_create.argtypes = [ctypes.c_longlong, ctypes.c_int, u64p, intp]
        lib.ws_symm_multicast_import.argtypes = [ctypes.c_int, u64p]
        lib.ws_symm_multicast_add_device.argtypes = [ctypes.c_ulonglong, ctypes.c_int]
        lib.ws_symm_multicast_bind.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_longlong, ctypes.c_int, u64p]
        lib.ws_symm_multicast_release.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_longlong, ctypes.c_int,
                                                  ctypes.c_int]
        lib.ws_symm_release.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_longlong]
        lib.ws_symm_multicast_supported.argtypes = [ctypes.c_int]
        lib.ws_symm_copy.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_longlong]
        self.lib = lib

    def check(self, code: int, what: str) -> None:
        if code < 0:
            raise RuntimeError(f"symmetric memory: {what}: {self.lib.ws_symm_last_error().decode()} (code {code})")


_library = None


def _lib() -> _Library:
    global _library
    if _library is None:
        _library = _Library()
    return _library


def copy_bytes(dst_ptr: int, src_ptr: int, nbytes: int) -> None:
    """Synchronous copy between mapped device ranges, peers' included, by the driver (no library kernel is handed
    a peer address)."""
    api = _lib()
    api.check(api.lib.ws_symm_copy(dst_ptr, src_ptr, nbytes), "copy")


class _DeviceMemory:
    """`__cuda_array_interface__` over a raw device range, so that torch can view it without owning it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def exchange_descriptors(fd: int, rank: int, world: int, group, only_from: int | None = None) -> dict[int, int]:
    """Every rank's ``fd`` delivered to every other rank (or rank ``only_from``'s to all): ``{source rank: fd}``.

    Rank r listens on an abstract Unix socket (no file system entry) whose name all ranks learn through the
    process group; a sender connects, says who it is and passes the descriptor as ancillary data."""
    name = f"\0warpstate-symm-{os.getpid()}-{uuid.uuid4().hex}"
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(name)
    server.listen(world)
    names = [None] * world
    dist.all_gather_object(names, name, group=group)
    senders = [r for r in range(world) if r != rank] if only_from is None else ([only_from] if rank != only_from else [])
    targets = [r for r in range(world) if r != rank] if only_from in (None, rank) else []
    received: dict[int, int] = {}
    try:
        for target in targets:
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as out:
                out.connect(names[target])
                socket.send_fds(out, [rank.to_bytes(4, "little")], [fd])
        for _ in senders:
            connection, _ = server.accept()
            with connection:
                message, fds, _, _ = socket.recv_fds(connection, 4, 1)
                if len(message) != 4 or len(fds) != 1:
                    raise RuntimeError("symmetric memory: a peer closed the descriptor channel early")
                received[int.from_bytes(message, "little")] = fds[0]
    finally:
        server.close()
    dist.barrier(group=group)      # nobody tears its listener down while a peer still connects
    return received


class SymmetricAllocationError(RuntimeError):
    """Raised on every rank of the group together when the library's own allocator could not build a buffer."""


class _OwnAllocation:
    """The mappings of one symmetric buffer in this process; released when the buffer is dropped."""

    def __init__(self, nbytes: int, device: torch.device, group, want_multicast: bool):
        api = _lib()
        lib = api.lib
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device_index = device.index if device.index is not None else torch.cuda.current_device()
        multicast = bool(want_multicast and self.world > 1 and lib.ws_symm_multicast_supported(self.device_index) == 1)
        # every rank must take the same decision and the same padded size
        votes = [None] * self.world
        dist.all_gather_object(votes, multicast, group=group)
        multicast = all(votes)
        self.handle, self.ptr = None, 0
        self.imports: list[tuple[int, int]] = []
        self.mc, self.mc_ptr, self.mc_bound = 0, 0, False
        self.peer_ptrs = [0] * self.world
        fd = ctypes.c_int(-1)

        def create() -> None:
            self.bytes = int(lib.ws_symm_padded_size(self.device_index, nbytes, self.world, int(multicast)))
            api.check(self.bytes, "sizing the allocation")
            handle, ptr = ctypes.c_ulonglong(), ctypes.c_ulonglong()
            api.check(lib.ws_symm_create(self.device_index, self.bytes, ctypes.byref(handle), ctypes.byref(ptr), ctypes.byref(fd)),
                      "creating the local allocation")
            self.handle, self.ptr = handle.value, ptr.value
            self.peer_ptrs[self.rank] = self.ptr

        self._together(create, "allocation")
        try:
            incoming = exchange_descriptors(fd.value, self.rank, self.world, group)
        finally:
            lib.ws_symm_close_fd(fd.value)

        def map_peers() -> None:
            try:
                for source, peer_fd in sorted(incoming.items()):
                    peer_handle, peer_ptr = ctypes.c_ulonglong(), ctypes.c_ulonglong()
                    api.check(lib.ws_symm_import(self.device_index, peer_fd, self.bytes, ctypes.byref(peer_handle),
                                                 ctypes.byref(peer_ptr)), f"mapping rank {source}'s allocation")
                    self.imports.append((peer_handle.value, peer_ptr.value))
                    self.peer_ptrs[source] = peer_ptr.value
            finally:
                for peer_fd in incoming.values():
                    lib.ws_symm_close_fd(peer_fd)

        self._together(map_peers, "peer mapping")
        if multicast:
            self._join_multicast(api)

    def _together(self, step, what: str) -> None:
        """Run a local step on every rank, then let the ranks tell one another how it went: either all go on, or
        all release what they hold and raise `SymmetricAllocationError` -- no rank is left waiting in a collective
        for a peer that has already given up."""
        problem = None
        try:
            step()
        except Exception as error:     # reported to every rank below, then re-raised as one common error
            problem = f"rank {self.rank}: {error}"
        reports = [None] * self.world
        dist.all_gather_object(reports, problem, group=self.group)
        failed = [r for r in reports if r]
        if failed:
            self.close()
            raise SymmetricAllocationError(f"symmetric memory ({what}) failed: " + "; ".join(failed))

    def _join_multicast(self, api: _Library) -> None:
        """Join the ranks' allocations in one multicast object.  Any rank's failure makes every rank go on without
        a multimem address (peer loads still work)."""
        lib = api.lib
        mc, fd = ctypes.c_ulonglong(), ctypes.c_int(-1)
        created = 0
        if self.rank == 0:
            created = lib.ws_symm_multicast_create(self.bytes, self.world, ctypes.byref(mc), ctypes.byref(fd))
        outcome = [created]
        dist.broadcast_object_list(outcome, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                                   group=self.group)
        if outcome[0] < 0:
            return                      # the fabric refused the object: every rank goes on without multimem
        incoming = exchange_descriptors(fd.value if self.rank == 0 else -1, self.rank, self.world, self.group, only_from=0)

        def agreed(step) -> bool:
            fine = True
            try:
                step()
            except Exception:
                fine = False
            votes = [None] * self.world
            dist.all_gather_object(votes, fine, group=self.group)
            return all(votes)

        def join() -> None:
            if self.rank == 0:
                lib.ws_symm_close_fd(fd.value)
            else:
                try:
                    api.check(lib.ws_symm_multicast_import(incoming[0], ctypes.byref(mc)), "importing the multicast object")
                finally:
                    lib.ws_symm_close_fd(incoming[0])
            self.mc = mc.value
            api.check(lib.ws_symm_multicast_add_device(self.mc, self.device_index), "adding the device to the multicast object")

        def bind() -> None:
            mc_ptr = ctypes.c_ulonglong()
            api.check(lib.ws_symm_multicast_bind(self.mc, self.handle, self.bytes, self.device_index, ctypes.byref(mc_ptr)),
                      "binding to the multicast object")
            self.mc_ptr, self.mc_bound = mc_ptr.value, True

        # all devices are members before anyone binds; every rank is bound before anyone issues a multimem instruction
        if not (agreed(join) and agreed(bind)):
            if self.mc:
                lib.ws_symm_multicast_release(self.mc, self.mc_ptr, self.bytes, self.device_index, int(self.mc_bound))
            self.mc, self.mc_ptr, self.mc_bound = 0, 0, False

    def close(self) -> None:
        if getattr(self, "handle", None) is None:
            return
        lib = _lib().lib
        if self.mc:
            lib.ws_symm_multicast_release(self.mc, self.mc_ptr, self.bytes, self.device_index, int(self.mc_bound))
            self.mc = 0
        for handle, ptr in self.imports:
            lib.ws_symm_release(handle, ptr, self.bytes)
        self.imports = []
        lib.ws_symm_release(self.handle, self.ptr, self.bytes)
        self.handle = None

    def __del__(self):
        try:
            torch.cuda.synchronize(self.device_index)
            self.close()
        except Exception:       # interpreter shutdown: the driver reclaims the mappings with the process
            pass


def _allocate_own(numel: int, dtype: torch.dtype, device: torch.device, group) -> SymmetricBuffer:
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    owner = _OwnAllocation(max(nbytes, 16), device, group, want_multicast=nvls_allowed())
    with torch.cuda.device(device):
        raw = torch.as_tensor(_DeviceMemory(owner.ptr, owner.bytes), device=device)
    tensor = raw[:nbytes].view(dtype)
    tensor._ws_symmetric_owner = owner          # the mapping lives as long as any view of it
    tensor.zero_()
    torch.cuda.current_stream(device).synchronize()
    dist.barrier(group=group)                   # zeroed everywhere before a peer reads or writes
    return SymmetricBuffer(tensor, list(owner.peer_ptrs), owner.mc_ptr if nvls_allowed() else 0, owner.rank, owner.world,
                           None, owner)


# ----------------------------------------------------------------------------------- torch's allocator
def _allocate_torch(numel: int, dtype: torch.dtype, device: torch.device, group) -> SymmetricBuffer:
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", FutureWarning)
        import torch.distributed._symmetric_memory as symm_mem
        name = group.group_name
        enable = getattr(symm_mem, "enable_symm_mem_for_group", None)
        enabled = getattr(symm_mem, "is_symm_mem_enabled_for_group", None)
        if enable is not None and not (enabled is not None and enabled(name)):
            enable(name)
        tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        tensor.zero_()
        handle = symm_mem.rendezvous(tensor, group=name)
    ptrs = [int(p) for p in handle.buffer_ptrs]
    mc = int(getattr(handle, "multicast_ptr", 0) or 0) if nvls_allowed() else 0
    return SymmetricBuffer(tensor, ptrs, mc, handle.rank, handle.world_size, handle)


def allocate(numel: int, dtype: torch.dtype, device: torch.device, group=None) -> SymmetricBuffer:
    """``numel`` elements of ``dtype`` on ``device``, zero-filled, mapped by every rank of ``group`` (collective)."""
    group = group if group is not None else dist.group.WORLD
    if provider() == "torch":
        return _allocate_torch(numel, dtype, device, group)
    try:
        return _allocate_own(numel, dtype, device, group)
    except SymmetricAllocationError as error:
        # raised on every rank together, so every rank takes the other allocator together
        if dist.get_rank(group) == 0:
            print(f"warpstate_ai_b200: {error}; using torch.distributed._symmetric_memory instead", flush=True)
        return _allocate_torch(numel, dtype, device, group)
