"""Tensor-parallel communicators for row-parallel GEMMs and the vocab-parallel LM head.

`NcclTPComm` is the baseline named in the project's performance contract: a separate GEMM kernel followed by
an NCCL collective. `FusedTPComm` (see `fused.py`) replaces each GEMM + collective pair by one kernel that
moves tiles over peer memory while the tensor cores run.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from .dist import DistInfo


class NcclTPComm:
    def __init__(self, info: DistInfo):
        self.info = info
        self.world_size = info.world_size
        self.rank = info.rank
        self.group = info.group

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def linear_all_reduce(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Row-parallel linear: every rank multiplies its K-shard, partial sums are all-reduced."""
        y = ops.linear(x, w)
        self.all_reduce(y)
        if residual is not None:
            y = y + residual
        return y

    def linear_fp8_all_reduce(self, x, w_q: torch.Tensor, w_scale: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Row-parallel block-scaled fp8 linear followed by an all-reduce of the partial sums."""
        y = self.all_reduce(ops.linear_fp8(x, w_q, w_scale))
        if residual is not None:
            y = y + residual
        return y

    def all_gather_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        """[S, V/tp] per rank -> [S, V] on every rank."""
        if self.world_size == 1:
            return logits
        parts = [torch.empty_like(logits) for _ in range(self.world_size)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)
