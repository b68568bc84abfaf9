"""Turns a scheduler batch into device tensors, runs the model and the sampler.

All integer metadata of a step (token ids, positions, KV slots, sequence offsets, block tables, rows to sample,
sampling parameters) is packed into one pinned host buffer and moved with a single host->device copy; the only
device->host traffic is the vector of sampled token ids. Decode-only steps replay a CUDA graph captured per
batch-size bucket, so their ~10 launches per layer cost one `cudaGraphLaunch`.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops


def _align(n: int, a: int = 16) -> int:
    return (n + a - 1) // a * a


class _Staging:
    """Pinned host buffer + same-sized device buffer, carved into typed segments per step."""

    def __init__(self, nbytes: int, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        self.host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.cuda)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(nbytes, dtype=torch.uint8, device=device) if self.cuda else self.host
        self.off = 0
        self.segments = []

    def begin(self):
        self.off = 0
        self.segments = []

    def put(self, arr: np.ndarray, dtype) -> tuple[int, int, torch.dtype, tuple]:
        arr = np.ascontiguousarray(arr, dtype=dtype)
        n = arr.nbytes
        if self.off + n > self.host_np.size:
            raise RuntimeError("staging buffer too small for this batch")
        self.host_np[self.off:self.off + n] = arr.view(np.uint8).reshape(-1)
        seg = (self.off, n, arr.shape)
        self.off = _align(self.off + n)
        return seg

    def flush(self) -> int:
        """Issue the single host->device copy of everything staged; returns bytes copied."""
        if self.cuda and self.off:
            self.dev[:self.off].copy_(self.host[:self.off], non_blocking=True)
        return self.off

    def view(self, seg, dtype: torch.dtype) -> torch.Tensor:
        off, n, shape = seg
        return self.dev[off:off + n].view(dtype).view(*shape)


class ModelRunner:
    def __init__(self, model, kv_caches, cfg):
        self.model = model
        self.kv_caches = kv_caches
        self.cfg = cfg
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        max_blocks = (cfg.max_model_len + cfg.page_size - 1) // cfg.page_size
        nbytes = cfg.max_num_batched_tokens * 24 + cfg.max_num_seqs * (max_blocks * 4 + 64) + (1 << 16)
        self.staging = _Staging(nbytes, self.device)
        self.max_blocks = max_blocks
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.ids_host = torch.empty(cfg.max_num_seqs, dtype=torch.int64, pin_memory=self.cuda)
        self.graphs: dict[int, tuple] = {}
        self.use_graphs = bool(cfg.use_cuda_graphs and self.cuda)
        self.graph_launches = 0
        self.launches_per_graph: dict[int, int] = {}

    # ------------------------------------------------------------------------------------------------
    def execute(self, batch, states, step: int) -> list[int]:
        st = self.staging
        st.begin()
        T, B = int(batch.num_tokens), int(batch.num_seqs)
        seg_tok = st.put(batch.token_ids, np.int64)
        seg_slot = st.put(batch.slots, np.int64)
        seg_pos = st.put(batch.positions, np.int32)
        seg_cu = st.put(batch.cu_q, np.int32)
        seg_ctx = st.put(batch.ctx_lens, np.int32)
        seg_bt = st.put(batch.block_tables, np.int32)
        sample_rows = batch.sample_rows
        S = len(sample_rows)
        seg_rows = st.put(sample_rows.astype(np.int64), np.int64)
        greedy = all(s.params.temperature <= 0.0 for s in states)
        if not greedy:
            seg_temp = st.put(np.array([s.params.temperature for s in states], dtype=np.float32), np.float32)
            seg_topk = st.put(np.array([s.params.top_k for s in states], dtype=np.int32), np.int32)
            seg_topp = st.put(np.array([s.params.top_p for s in states], dtype=np.float32), np.float32)
        self.h2d_bytes = st.flush()

        token_ids = st.view(seg_tok, torch.int64)
        slots = st.view(seg_slot, torch.int64)
        positions = st.view(seg_pos, torch.int32)
        ctx_np = batch.ctx_lens
        meta = ops.AttnMeta(st.view(seg_cu, torch.int32), st.view(seg_ctx, torch.int32), st.view(seg_bt, torch.int32),
                            batch.num_decode, batch.max_q_len, int(ctx_np.max()) if B else 0)
        rows = st.view(seg_rows, torch.int64)
        if S == 0:
            # pure mid-prompt chunks: run the layers for their KV side effect, nothing to sample
            self.model.forward(token_ids, positions, slots, meta, self.kv_caches, rows)
            self.d2h_bytes = 0
            return []
        logits = self.model.forward(token_ids, positions, slots, meta, self.kv_caches, rows)
        if greedy:
            ids = ops.argmax(logits)
        else:
            seed = self.cfg.seed if states[0].params.seed is None else states[0].params.seed
            ids = ops.sample(logits.float() if not self.cuda else logits, st.view(seg_temp, torch.float32),
                             st.view(seg_topk, torch.int32), st.view(seg_topp, torch.float32), seed, step)
        if self.cuda:
            self.ids_host[:S].copy_(ids, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            out = self.ids_host[:S].tolist()
        else:
            out = ids.tolist()
        self.d2h_bytes = S * 8
        return out
