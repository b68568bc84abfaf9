"""Standalone collectives over symmetric memory: the small-message and test counterparts of the collectives that
the fused GEMM / MoE kernels carry inside them. One kernel per call, no NCCL; every wait is bounded and reports
through the device status word (`ops.check_status`).

    coll = SymmCollectives(info, max_bytes=8 << 20)
    y = coll.all_reduce(x)                    # one-shot below 256 KiB, two-shot above, in-switch when `nvls=True`
    s = coll.reduce_scatter(x)                # this rank's 1/tp of the sum
    g = coll.all_gather(x)                    # [tp, *x.shape] view into the receive buffer
    r, counts = coll.all_to_all(blocks, send_counts)
    tok = coll.vocab_argmax(logits_shard)     # greedy sampling over a vocabulary split across ranks

Views returned by all_gather / all_to_all / two-shot all_reduce point into a double-buffered receive area: they
stay valid until the second collective launched after the one that produced them.
"""
from __future__ import annotations

import torch

from .. import _ext, ops
from ..ops import _state
from .dist import DistInfo
from .symm import SymmRegion, _align


class SymmCollectives:
    ONE_SHOT_MAX_BYTES = 256 << 10
    # all-reduce + residual + RMSNorm: above this many bytes per rank the in-switch form (each rank reduces 1 / tp of the
    # rows through the multicast mapping) replaces the one-shot form (each rank reads every peer's whole message)
    NVLS_NORM_MIN_BYTES = 128 << 10

    def __init__(self, info: DistInfo, max_bytes: int = 8 << 20, timeout_s: float = 20.0, nvls: bool = False):
        self.info = info
        self.world_size, self.rank = info.world_size, info.rank
        self.C = _ext.require()
        tp = self.world_size
        lay = self.C.CollLayout()
        off = 0

        def take(n):
            nonlocal off
            o = off
            off = _align(off + n)
            return o

        lay.buf_half_bytes = _align(max_bytes)
        lay.off_buf = take(2 * lay.buf_half_bytes)
        lay.out_half_bytes = _align(max_bytes * tp)
        lay.off_out = take(2 * lay.out_half_bytes)
        lay.off_flags_a = take(64)
        lay.off_flags_b = take(64)
        lay.off_counts = take(64)
        lay.off_done = take(64)
        lay.off_epoch = take(64)
        lay.total_bytes = off
        self.layout = lay
        self.max_bytes = max_bytes
        self.region = SymmRegion(off, info)
        self.peers = self.region.ptrs
        self.mc_ptr = self.region.mc_ptr if nvls else 0
        self.timeout_ns = int(timeout_s * 1e9)
        self.status = _state.get(info.device).status
        self._calls = 0

    def _slot(self) -> int:
        s = self._calls & 1
        self._calls += 1
        return s

    def _stage(self, x: torch.Tensor, slot: int) -> int:
        """Copy x (bf16) into this rank's input half, zero-padded to a multiple of 8 * tp elements."""
        assert x.dtype == torch.bfloat16 and x.is_cuda
        n = x.numel()
        unit = 8 * self.world_size
        n_pad = (n + unit - 1) // unit * unit
        assert n_pad * 2 <= self.max_bytes, "message larger than the collective buffer"
        buf = self.region.view(self.layout.off_buf + slot * self.layout.buf_half_bytes, (n_pad,), torch.bfloat16)
        buf[:n].copy_(x.reshape(-1))
        if n_pad > n:
            buf[n:].zero_()
        return n_pad

    def staging_view(self, shape, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """The input half of the NEXT collective as a tensor of `shape`: a producer (e.g. a GEMM) can write its result
        straight into it and call `all_reduce_staged(shape)` instead of `all_reduce(x)`, saving the staging copy."""
        n = 1
        for d in shape:
            n *= int(d)
        assert n * torch.empty((), dtype=dtype).element_size() <= self.max_bytes, "message larger than the collective buffer"
        slot = self._calls & 1
        return self.region.view(self.layout.off_buf + slot * self.layout.buf_half_bytes, tuple(shape), dtype)

    def all_reduce_staged(self, shape, algo: str = "auto") -> torch.Tensor:
        """All-reduce of what was written into `staging_view(shape)` (bf16; numel a multiple of 8 * world size)."""
        n = 1
        for d in shape:
            n *= int(d)
        assert n % (8 * self.world_size) == 0
        slot = self._slot()
        if algo == "auto":
            algo = "one_shot" if n * 2 <= self.ONE_SHOT_MAX_BYTES else ("nvls" if self.mc_ptr else "two_shot")
        code = {"one_shot": 0, "two_shot": 1, "nvls": 2}[algo]
        out = torch.empty(n, dtype=torch.bfloat16, device=self.info.device) if code == 0 else None
        self.C.coll_all_reduce(self.rank, self.peers, self.layout, self.mc_ptr, out, n, code, slot, self.timeout_ns, self.status)
        ops._count()
        if out is None:
            out = self.region.view(self.layout.off_out + slot * self.layout.out_half_bytes, (n,), torch.bfloat16)
        return out.view(*shape)

    def all_reduce_rmsnorm_staged(self, shape, weight: torch.Tensor, eps: float, residual: torch.Tensor | None, form: str = "auto"):
        """One kernel for all-reduce + residual add + RMSNorm of the [rows, hidden] partials written into
        `staging_view(shape)`: new stream = residual (bf16 [rows, hidden]; None = no residual) + sum; returns
        (rmsnorm(new stream) * weight, new stream). The one-shot form updates `residual` in place and returns it; the
        in-switch form (multicast mapping present, message large enough) leaves `residual` untouched and returns views
        into the symmetric result half. Callers must use the returned stream. `form`: "one_shot", "nvls" or "auto"."""
        rows, hidden = int(shape[0]), int(shape[1])
        slot = self._slot()
        nbytes = rows * hidden * 2
        if form == "auto":
            form = "nvls" if (self.mc_ptr and nbytes >= self.NVLS_NORM_MIN_BYTES and 2 * nbytes <= self.layout.out_half_bytes) else "one_shot"
        if form == "nvls":
            if not self.mc_ptr or 2 * nbytes > self.layout.out_half_bytes:
                raise RuntimeError("in-switch all-reduce + norm needs a multicast mapping and room for two result tensors")
            # in-switch reduction; the normalised rows and the new residual stream land in the symmetric result half of
            # every rank (valid until the second collective after this one; `residual` itself is only read)
            self.C.coll_all_reduce_rmsnorm_nvls(self.rank, self.peers, self.layout, self.mc_ptr, residual, weight, rows, eps, slot,
                                                self.timeout_ns, self.status)
            ops._count()
            base = self.layout.off_out + slot * self.layout.out_half_bytes
            return (self.region.view(base, (rows, hidden), torch.bfloat16), self.region.view(base + nbytes, (rows, hidden), torch.bfloat16))
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=self.info.device)
        self.C.coll_all_reduce_rmsnorm(self.rank, self.peers, self.layout, residual, weight, out, eps, slot, self.timeout_ns, self.status)
        ops._count()
        return out, residual

    def p2p_probe(self, nbytes: int, n_peers: int = 1, senders: int | None = None, pull: bool = False, ctas: int = 148) -> None:
        """One launch of the link probe: every rank in the `senders` bit mask (default: all) moves `nbytes` to (push) or
        from (pull) each of its next `n_peers` ranks with the library's own peer stores / loads. Time it with CUDA events."""
        if self.world_size == 1:
            return
        senders = (1 << self.world_size) - 1 if senders is None else int(senders)
        self.C.coll_p2p_probe(self.rank, self.peers, self.layout, int(nbytes), int(n_peers), senders, bool(pull), int(ctas), self._slot(),
                              self.timeout_ns, self.status)
        ops._count()

    def all_reduce(self, x: torch.Tensor, algo: str = "auto") -> torch.Tensor:
        if self.world_size == 1:
            return x
        slot = self._slot()
        n_pad = self._stage(x, slot)
        if algo == "auto":
            algo = "one_shot" if n_pad * 2 <= self.ONE_SHOT_MAX_BYTES else ("nvls" if self.mc_ptr else "two_shot")
        code = {"one_shot": 0, "two_shot": 1, "nvls": 2}[algo]
        if code == 2 and not self.mc_ptr:
            raise RuntimeError("in-switch all-reduce needs a multicast mapping (construct with nvls=True on an NVLS fabric)")
        out = torch.empty(n_pad, dtype=torch.bfloat16, device=x.device) if code == 0 else None
        self.C.coll_all_reduce(self.rank, self.peers, self.layout, self.mc_ptr, out, n_pad, code, slot, self.timeout_ns, self.status)
        ops._count()
        if out is None:
            out = self.region.view(self.layout.off_out + slot * self.layout.out_half_bytes, (n_pad,), torch.bfloat16)
        return out[: x.numel()].view(x.shape)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """x: [tp * r, ...] on every rank -> sum over ranks of rows [rank * r, (rank + 1) * r)."""
        if self.world_size == 1:
            return x
        assert x.shape[0] % self.world_size == 0 and (x.numel() // self.world_size) % 8 == 0
        slot = self._slot()
        n = self._stage(x, slot)
        out = torch.empty(x.shape[0] // self.world_size, *x.shape[1:], dtype=x.dtype, device=x.device)
        self.C.coll_reduce_scatter(self.rank, self.peers, self.layout, out, n, slot, self.timeout_ns, self.status)
        ops._count()
        return out

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x.unsqueeze(0)
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        assert nbytes % 16 == 0 and nbytes <= self.max_bytes
        slot = self._slot()
        self.C.coll_all_gather(self.rank, self.peers, self.layout, x, slot, self.timeout_ns, self.status)
        ops._count()
        return self.region.view(self.layout.off_out + slot * self.layout.out_half_bytes, (self.world_size, *x.shape), x.dtype)

    def all_to_all(self, blocks: torch.Tensor, send_counts: list[int]):
        """blocks [tp, max_rows, row]: rows [0, send_counts[j]) of block j go to rank j. Returns the receive view
        [tp, max_rows, row] (block s = rows from rank s) and an int32 [tp] device tensor of received row counts."""
        tp = self.world_size
        blocks = blocks.contiguous()
        if tp == 1:
            return blocks, torch.tensor(send_counts, dtype=torch.int32, device=blocks.device)
        assert blocks.shape[0] == tp and (blocks.shape[2] * blocks.element_size()) % 16 == 0
        assert blocks.numel() * blocks.element_size() <= self.layout.out_half_bytes
        slot = self._slot()
        self.C.coll_all_to_all(self.rank, self.peers, self.layout, blocks, [int(c) for c in send_counts], slot, self.timeout_ns, self.status)
        ops._count()
        recv = self.region.view(self.layout.off_out + slot * self.layout.out_half_bytes, tuple(blocks.shape), blocks.dtype)
        counts = self.region.view(self.layout.off_counts + slot * 32, (8,), torch.int32)[:tp]
        return recv, counts

    def vocab_argmax(self, logits: torch.Tensor, vocab_stride: int | None = None) -> torch.Tensor:
        """logits [S, v] bf16: the valid columns of this rank's vocabulary shard (unit inner stride; rank r's column c
        is token r * vocab_stride + c, default stride v) -> int64 [S] global arg-max tokens, identical on all ranks."""
        vocab_stride = vocab_stride or logits.shape[1]
        local = ops.argmax(logits)
        if self.world_size == 1:
            return local
        tokens = torch.empty_like(local)
        slot = self._slot()
        self.C.coll_vocab_argmax(self.rank, self.peers, self.layout, logits, local, tokens, vocab_stride, slot, self.timeout_ns, self.status)
        ops._count()
        return tokens
