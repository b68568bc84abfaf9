"""Symmetric memory: one allocation of the same size on every rank, each rank able to address every peer's copy
over NVLink. Allocation and handle exchange go through `torch.distributed._symmetric_memory` (CUDA VMM handles
exchanged at rendezvous; NVLS multicast mapping when the fabric offers one); everything that happens in the
memory afterwards is this library's own kernels.

On CPU (tests of the host-side protocol) the region is a POSIX shared-memory segment per rank, mapped by all.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from .dist import DistInfo


def _align(n: int, a: int = 1024) -> int:
    return (n + a - 1) // a * a


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
