"""Symmetric memory: one allocation of the same size on every rank, each rank able to address every peer's copy
over NVLink, plus one multicast (NVLS) mapping of all copies where the fabric offers one. Everything that happens in
the memory afterwards is this library's own kernels.

Two allocation back ends (`B2_SYMM_BACKEND`):
  vmm    this library's own heap (`csrc/runtime/symm_heap.cpp`): cuMemCreate per rank, the allocation exported as a
         file descriptor, sent to the peers over AF_UNIX sockets (SCM_RIGHTS), imported and mapped with cuMemMap; the
         multicast object created by rank 0, shared the same way, bound with cuMulticastBindMem
  torch  `torch.distributed._symmetric_memory` (the same driver calls behind PyTorch's rendezvous)
The default tries `vmm` and falls back to `torch` when the driver refuses a step (all ranks decide together).

On CPU (tests of the host-side protocol) the region is a POSIX shared-memory segment per rank, mapped by all.
"""
from __future__ import annotations

import os
import socket
import uuid

import numpy as np
import torch
import torch.distributed as dist

from .dist import DistInfo


def _align(n: int, a: int = 1024) -> int:
    return (n + a - 1) // a * a


class _DevicePointer:
    """Lets torch wrap a raw device address (a mapping made with cuMemMap) as a tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def _exchange_fds(info: DistInfo, tag: str, my_fd: int | None, senders: list[int]) -> dict[int, int]:
    """Every rank in `senders` gives a duplicate of its descriptor to every other rank over abstract AF_UNIX sockets
    (SCM_RIGHTS); returns {sender rank: received descriptor}. `my_fd` is closed by the caller."""
    group = info.host_group or info.group
    rank, world = info.rank, info.world_size
    expect = [r for r in senders if r != rank]
    name = f"\0b2symm-{tag}-{rank}"
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name)
    srv.listen(world)
    dist.barrier(group=group)          # every listener is up
    if rank in senders:
        for peer in range(world):
            if peer == rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.connect(f"\0b2symm-{tag}-{peer}")
            socket.send_fds(c, [rank.to_bytes(4, "little")], [my_fd])
            c.close()
    got: dict[int, int] = {}
    srv.settimeout(60.0)
    while len(got) < len(expect):
        conn, _ = srv.accept()
        msg, fds, _, _ = socket.recv_fds(conn, 4, 1)
        conn.close()
        got[int.from_bytes(msg, "little")] = fds[0]
    srv.close()
    dist.barrier(group=group)
    return got


def _all_ok(info: DistInfo, ok: bool) -> bool:
    flag = torch.tensor([1 if ok else 0], dtype=torch.int64)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=info.host_group or info.group)
    return bool(flag[0])


class SymmRegion:
    """`nbytes` of zero-initialised symmetric memory. `ptrs[r]` is the address of rank r's copy as seen from
    this process; `local` is a uint8 tensor over this rank's copy. A band of `GUARD_BYTES` of a known pattern
    follows the region in the same allocation: a local or peer write past `nbytes` lands there and
    `check_guard()` counts it."""

    GUARD_BYTES = 4096
    GUARD_PATTERN = 0xA5

    def __init__(self, nbytes: int, info: DistInfo):
        self.info = info
        self.nbytes = _align(nbytes)
        self.mc_ptr = 0
        self._hdl = None
        if info.device.type != "cuda":
            raise RuntimeError("SymmRegion needs CUDA; use CpuSymmRegion for host-side protocol tests")
        if info.world_size == 1:
            self._raw = torch.zeros(self.nbytes + self.GUARD_BYTES, dtype=torch.uint8, device=info.device)
            self._raw[self.nbytes:].fill_(self.GUARD_PATTERN)
            self.local = self._raw[: self.nbytes]
            self.ptrs = [self.local.data_ptr()]
            return
        backend = os.environ.get("B2_SYMM_BACKEND", "auto")
        self.backend = "torch"
        self._seg = None
        if backend in ("auto", "vmm") and self._init_vmm(info):
            self.backend = "vmm"
            return
        if backend == "vmm":
            raise RuntimeError("B2_SYMM_BACKEND=vmm: the VMM symmetric heap could not be set up on this machine")
        import torch.distributed._symmetric_memory as symm_mem

        group = info.group
        self._raw = symm_mem.empty(self.nbytes + self.GUARD_BYTES, dtype=torch.uint8, device=info.device)
        self._hdl = symm_mem.rendezvous(self._raw, group=group.group_name)
        self.local = self._raw[: self.nbytes]
        self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        try:
            self.mc_ptr = int(self._hdl.multicast_ptr or 0)
        except Exception:  # noqa: BLE001
            self.mc_ptr = 0
        self.local.zero_()
        self._raw[self.nbytes:].fill_(self.GUARD_PATTERN)
        torch.cuda.synchronize(info.device)
        dist.barrier(group=group)

    def _init_vmm(self, info: DistInfo) -> bool:
        """Own heap: allocate, exchange descriptors, map peers, bind the multicast object. Every step is agreed on by
        all ranks (a rank that fails makes all fall back together); returns False when the fall-back should be used."""
        from .. import _ext

        C = _ext.require()
        if not hasattr(C, "SymmHeapSegment"):
            return False
        rank, world, dev = info.rank, info.world_size, info.device
        tag = None
        box = [uuid.uuid4().hex[:12] if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=info.host_group or info.group)
        tag = box[0]
        seg = C.SymmHeapSegment()
        total = self.nbytes + self.GUARD_BYTES
        ok = True
        try:
            seg.create(dev.index if dev.index is not None else torch.cuda.current_device(), rank, world, total, True)
        except RuntimeError:
            ok = False
        if not _all_ok(info, ok):
            seg.close()
            return False
        fd = seg.export_fd()
        got = _exchange_fds(info, tag + "a", fd, list(range(world)))
        os.close(fd)
        try:
            for peer, pfd in got.items():
                seg.map_peer(peer, pfd)
        except RuntimeError:
            ok = False
        if not _all_ok(info, ok):
            seg.close()
            return False
        mc_ptr = 0
        if _all_ok(info, bool(seg.multicast_supported())):
            # rank 0 creates the multicast object; a failure at any step only costs the multicast mapping
            mc_ok, mfd = True, None
            if rank == 0:
                try:
                    mfd = seg.mc_create()
                except RuntimeError:
                    mc_ok = False
            if _all_ok(info, mc_ok):
                got = _exchange_fds(info, tag + "m", mfd, [0])
                if rank == 0:
                    os.close(mfd)
                try:
                    if rank != 0:
                        seg.mc_import(got[0])
                    seg.mc_add_device()
                except RuntimeError:
                    mc_ok = False
                if _all_ok(info, mc_ok):        # every device has been added: the allocations can be bound
                    try:
                        seg.mc_bind_and_map()
                    except RuntimeError:
                        mc_ok = False
                    if _all_ok(info, mc_ok):
                        mc_ptr = int(seg.mc_ptr())
        self._seg = seg
        self._raw = torch.as_tensor(_DevicePointer(seg.ptr(rank), total), device=dev)
        self.local = self._raw[: self.nbytes]
        self.ptrs = [int(seg.ptr(r)) for r in range(world)]
        self.mc_ptr = mc_ptr
        self._raw[self.nbytes:].fill_(self.GUARD_PATTERN)     # the allocation itself was cleared when it was created
        torch.cuda.synchronize(dev)
        dist.barrier(group=info.host_group or info.group)
        return True

    def check_guard(self) -> int:
        """Number of bytes of the band after the region that no longer hold the pattern (0 = nothing wrote past the end)."""
        return int((self._raw[self.nbytes:] != self.GUARD_PATTERN).sum().item())

    def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + n].view(dtype).view(*shape)


class CpuSymmRegion:
    """Software model of the symmetric heap for CPU ranks: one shared-memory segment per rank, all mapped by all
    ranks as numpy arrays. Used to test indexing, flag protocols and timeouts without GPUs."""

    def __init__(self, nbytes: int, info: DistInfo, tag: str):
        from multiprocessing import shared_memory

        self.info = info
        self.nbytes = _align(nbytes)
        name = f"b2symm_{tag}_{info.rank}"
        try:
            old = shared_memory.SharedMemory(name=name)
            old.close()
            old.unlink()
        except FileNotFoundError:
            pass
        self._own = shared_memory.SharedMemory(name=name, create=True, size=self.nbytes)
        np.frombuffer(self._own.buf, dtype=np.uint8)[:] = 0
        if info.world_size > 1:
            dist.barrier(group=info.host_group or info.group)
        self._peers = []
        self.bufs = []
        for r in range(info.world_size):
            shm = self._own if r == info.rank else shared_memory.SharedMemory(name=f"b2symm_{tag}_{r}")
            self._peers.append(shm)
            self.bufs.append(np.frombuffer(shm.buf, dtype=np.uint8))
        if info.world_size > 1:
            dist.barrier(group=info.host_group or info.group)

    def array(self, rank: int, offset: int, shape, dtype) -> np.ndarray:
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return self.bufs[rank][offset:offset + n].view(dtype).reshape(shape)

    def close(self) -> None:
        self.bufs = []
        for r, shm in enumerate(self._peers):
            try:
                shm.close()
            except BufferError:
                pass
        try:
            self._own.unlink()
        except FileNotFoundError:
            pass
