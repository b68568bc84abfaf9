"""Guard bands around device buffers that kernels index with run-time metadata.

A memory checker cannot be attached to the device code on every machine, so the buffers whose indices come from
block tables, slot mappings and peer offsets (the KV pool, the symmetric-memory regions) can carry a band of a
known byte pattern on each side. A kernel that writes one page, one row or one tile past its buffer lands in a
band instead of in a neighbouring allocation, and `check()` after a step or at the end of a test reports it as
a count of changed bytes instead of as a wrong token much later. The reference relies on `debug_assert` modes
for the same purpose (stdlib/src/builtin/debug_assert.mojo:35-57); this is the analogue for writes that no
assertion saw.

`B2_GUARD=1` makes the models allocate their KV caches through `guarded_zeros`; symmetric regions always carry a
tail band (a few KB). Checking is explicit: `check_all()` raises `GuardError` naming the buffers that were hit.
"""
from __future__ import annotations

import os
import weakref

import torch

GUARD_BYTES = 4096
PATTERN = 0xA5

_registry: list[tuple[str, weakref.ReferenceType]] = []


class GuardError(RuntimeError):
    pass


def enabled() -> bool:
    return os.environ.get("B2_GUARD", "0") not in ("", "0")


class GuardedBuffer:
    """`nbytes` of zeroed payload with `GUARD_BYTES` of pattern before and after it, in one allocation."""

    def __init__(self, nbytes: int, device, name: str = "buffer", guard_bytes: int = GUARD_BYTES):
        self.name = name
        self.guard = int(guard_bytes)
        self.nbytes = (int(nbytes) + 255) // 256 * 256       # keeps the payload and the tail band 256-byte aligned
        self.raw = torch.empty(self.nbytes + 2 * self.guard, dtype=torch.uint8, device=device)
        self.raw[: self.guard].fill_(PATTERN)
        self.raw[self.guard: self.guard + self.nbytes].zero_()
        self.raw[self.guard + self.nbytes:].fill_(PATTERN)
        _registry.append((name, weakref.ref(self)))

    @property
    def payload(self) -> torch.Tensor:
        return self.raw[self.guard: self.guard + self.nbytes]

    def view(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        n *= torch.empty((), dtype=dtype).element_size()
        if n > self.nbytes:
            raise ValueError(f"{self.name}: view of {n} bytes does not fit {self.nbytes}")
        t = self.payload[:n].view(dtype).view(*shape)
        t._b2_guard = self   # keeps the allocation (and its registry entry) alive as long as the view
        return t

    def corrupted(self) -> tuple[int, int]:
        """(changed bytes in the band before the payload, changed bytes in the band after it)."""
        head = int((self.raw[: self.guard] != PATTERN).sum().item())
        tail = int((self.raw[self.guard + self.nbytes:] != PATTERN).sum().item())
        return head, tail

    def check(self) -> None:
        head, tail = self.corrupted()
        if head or tail:
            raise GuardError(f"{self.name}: {head} byte(s) written before the buffer, {tail} after it")


def guarded_zeros(shape, dtype: torch.dtype, device, name: str = "buffer") -> torch.Tensor:
    """A zero tensor of this shape inside its own guarded allocation."""
    n = 1
    for s in shape:
        n *= int(s)
    buf = GuardedBuffer(n * torch.empty((), dtype=dtype).element_size(), device, name)
    return buf.view(shape, dtype)


def zeros(shape, dtype: torch.dtype, device, name: str = "buffer") -> torch.Tensor:
    """`guarded_zeros` when `B2_GUARD` is set, plain `torch.zeros` otherwise."""
    if enabled():
        return guarded_zeros(shape, dtype, device, name)
    return torch.zeros(shape, dtype=dtype, device=device)


def live() -> list[GuardedBuffer]:
    out = []
    for _, ref in list(_registry):
        b = ref()
        if b is not None:
            out.append(b)
    _registry[:] = [(n, r) for n, r in _registry if r() is not None]
    return out


def check_all() -> int:
    """Check every guarded buffer that is still alive; returns how many were checked. Raises `GuardError` listing
    every buffer whose bands changed."""
    bad = []
    bufs = live()
    for b in bufs:
        head, tail = b.corrupted()
        if head or tail:
            bad.append(f"{b.name}: {head} before / {tail} after")
    if bad:
        raise GuardError("guard bands overwritten: " + "; ".join(bad))
    return len(bufs)
