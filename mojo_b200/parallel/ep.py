"""Expert parallelism for mixture-of-experts layers.

`local_moe` runs all experts on one GPU (grouped tcgen05 GEMM over tokens sorted by expert). `EPComm` spreads the
routed experts over the ranks: tokens are dispatched to the rank that owns each of their top-k experts by a kernel
that writes rows straight into the destination's expert-sorted receive buffer over NVLink, the local experts run as
a grouped GEMM, and a combine kernel sends results back and forms the weighted sum (see csrc/kernels/moe_ep.cu).
"""
from __future__ import annotations

import torch

from .. import _ext, ops
from ..ops import reference


class EPComm:
    """Expert-parallel MoE over `info.world_size` ranks (1 rank: same kernels against the local buffer).

    Experts are stored per rank as w_gu [e_local, 2F, H] (gate/up rows interleaved in blocks of 16, see
    `reference.interleave_gate_up`) and w_down [e_local, H, F]. `moe()` runs router + dispatch, the two grouped GEMMs
    and combine; every rank must call it the same number of times (ranks without tokens pass T = 0)."""

    def __init__(self, info, n_experts: int, hidden: int, ffn: int, top_k: int, max_tokens: int, timeout_s: float = 20.0):
        from .symm import SymmRegion, _align

        self.info = info
        self.world_size, self.rank = info.world_size, info.rank
        self.C = _ext.require()
        assert n_experts % self.world_size == 0
        self.n_experts, self.e_local, self.hidden, self.ffn, self.top_k = n_experts, n_experts // self.world_size, hidden, ffn, top_k
        self.t_cap = max_tokens
        # an expert can receive every token of every rank once
        self.cap = (max_tokens * self.world_size + 255) // 256 * 256
        lay = self.C.EpLayout()
        off = 0

        def take(n):
            nonlocal off
            o = off
            off = _align(off + n)
            return o

        lay.cap, lay.e_local, lay.hidden, lay.top_k, lay.t_cap = self.cap, self.e_local, hidden, top_k, max_tokens
        lay.off_recv_x = take(self.e_local * self.cap * hidden * 2)
        lay.off_recv_meta = take(self.e_local * self.cap * 4)
        lay.off_recv_count = take(2 * self.e_local * 4)
        lay.off_ret_y = take(max_tokens * top_k * hidden * 2)
        lay.off_disp_done = take(64)
        lay.off_comb_done = take(64)
        lay.off_epoch = take(64)
        lay.total_bytes = off
        self.layout = lay
        self.region = SymmRegion(off, info)
        self.peers = self.region.ptrs
        self.timeout_ns = int(timeout_s * 1e9)
        self._calls = 0
        dev = info.device
        self.act = torch.empty(self.e_local * self.cap, ffn, dtype=torch.bfloat16, device=dev)
        self.y_local = torch.empty(self.e_local * self.cap, hidden, dtype=torch.bfloat16, device=dev)
        from ..ops import _state

        self.status = _state.get(dev).status

    def _bn(self, tokens_per_expert: float) -> int:
        for bn in (16, 32, 64, 128):
            if tokens_per_expert <= bn:
                return bn
        return 256

    def moe(self, x: torch.Tensor, router_logits: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor,
            shared: torch.Tensor | None = None, norm_topk: bool = False, route_scale: float = 1.0) -> torch.Tensor:
        """x [T, H] bf16, router_logits [T, E] bf16 -> sum_k w_k * expert_k(x) (+ shared) as bf16 [T, H]."""
        T = x.shape[0]
        lay, C = self.layout, self.C
        slot = self._calls & 1
        self._calls += 1
        weights = torch.empty(T, self.top_k, dtype=torch.float32, device=x.device)
        ids = torch.empty(T, self.top_k, dtype=torch.int32, device=x.device)
        C.ep_dispatch(x, router_logits, weights, ids, self.rank, self.peers, lay, self.top_k, norm_topk, route_scale, slot,
                      self.timeout_ns, self.status)
        recv_x = self.region.view(lay.off_recv_x, (self.e_local * self.cap, self.hidden), torch.bfloat16)
        counts = self.region.view(lay.off_recv_count + slot * self.e_local * 4, (self.e_local,), torch.int32)
        bn = self._bn(T * self.world_size * self.top_k / max(self.n_experts, 1))
        C.moe_grouped_gemm(recv_x, w_gu, counts, self.act, self.cap, True, bn, self.status)
        C.moe_grouped_gemm(self.act, w_down, counts, self.y_local, self.cap, False, bn, self.status)
        out = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=x.device)
        C.ep_combine(self.y_local, weights, shared, out, self.rank, self.peers, lay, self.top_k, slot, self.timeout_ns, self.status)
        ops._count(4)
        self.last_weights, self.last_ids = weights, ids
        return out


def local_moe(x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Single-rank MoE: x [T, H], weights/ids [T, k], w_gu [E, 2F, H] (gate rows, then up rows), w_down [E, H, F]."""
    if not x.is_cuda:
        return reference.moe_forward(x, w_gu, w_down, weights, ids).to(x.dtype)
    # expert loop on the plain GEMM with pre-computed routing (oracle for the fused path; `EPComm.moe` is the product path)
    T, k = ids.shape
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=w_gu.shape[0]).tolist()
    tok = (order // k)
    xs = x[tok]
    out = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device)
    f = w_gu.shape[1] // 2
    o = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        xe = xs[o:o + n].contiguous()
        gu = ops.linear(xe, w_gu[e])
        act = ops.swiglu(gu)
        y = ops.linear(act, w_down[e]).float()
        wsel = weights.reshape(-1)[order[o:o + n]].unsqueeze(1).float()
        out.index_add_(0, tok[o:o + n], y * wsel)
        o += n
    return out.to(x.dtype)


