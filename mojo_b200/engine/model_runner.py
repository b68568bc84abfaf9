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
        self.graphs: dict[int, "_DecodeGraph"] = {}
        self.use_graphs = bool(cfg.use_cuda_graphs and self.cuda)
        self.graph_launches = 0          # graph replays
        self.graph_kernel_launches = 0   # kernels executed inside replayed graphs
        self.step_events = None          # optional (start, end) CUDA events recorded around the device work
        self.last_num_tokens = 0
        self.last_logprobs = None        # per sampled row (logprob of the chosen token, [(id, logprob)] top-k) of the last step, on request
        b, self.buckets = 1, []
        while b < cfg.max_num_seqs:
            self.buckets.append(b)
            b = b * 2 if b < 16 else b + max(16, b // 4) // 16 * 16
        self.buckets.append(cfg.max_num_seqs)
        self.graph_pool = None           # memory pool shared by the decode graphs (they never replay concurrently)
        self.failed_buckets: dict[int, str] = {}   # buckets whose capture failed: their steps run eagerly
        # Expert parallelism: every rank must run the same number of MoE layer calls per step, so a decode graph can
        # only be captured when all ranks capture together (at start-up); a bucket that is missing runs eagerly.
        ep = getattr(model, "ep", None)
        self.ep = ep if ep is not None and getattr(ep, "world_size", 1) > 1 else None

    def capture_graphs(self, buckets=None) -> int:
        """Capture the decode graph of every batch-size bucket now, largest first so that the smaller ones reuse its
        memory pool. Without this a bucket is captured the first time a decode-only step needs it, which puts a
        capture (an eager pass plus the captured pass) into some request's inter-token latency. Returns the number
        of graphs captured. Tensor-parallel ranks must all call it (the passes contain collectives)."""
        if not self.use_graphs:
            return 0
        n = 0
        for bb in sorted(set(buckets if buckets is not None else self.buckets), reverse=True):
            if bb not in self.graphs and bb not in self.failed_buckets and self._capture(bb) is not None:
                n += 1
        if self.cuda:
            torch.cuda.synchronize(self.device)
            ops.check_status(self.device)
        return n

    def _capture(self, bb: int):
        """Capture one bucket. A capture that fails (an operation that a capturing stream does not allow) is not fatal:
        the bucket is remembered as failed and its steps run eagerly. The failure is the same on every rank of a
        tensor-parallel group (same shapes, same code), so the ranks keep taking the same path."""
        try:
            g = _DecodeGraph(self, bb)
        except Exception as e:  # noqa: BLE001
            import warnings

            self.failed_buckets[bb] = repr(e)
            if self.cuda:
                torch.cuda.synchronize(self.device)
            warnings.warn(f"mojo_b200: CUDA-graph capture of the {bb}-sequence decode step failed ({e!r}); such steps run eagerly", stacklevel=2)
            return None
        self.graphs[bb] = g
        return g

    def autotune(self, verbose: bool = False) -> dict:
        """Measure the GEMM configurations of this model's weight shapes at the token counts the engine produces
        (decode graph buckets, then multiples of 128 up to the token budget). A second or two, once, before serving."""
        if not self.cuda or not hasattr(self.model, "gemm_shapes"):
            return {}
        counts = ops.autotune.default_token_counts(self.cfg.max_num_batched_tokens, self.buckets)
        report = {}
        for N, K, epi, max_m in self.model.gemm_shapes():
            ms = [m for m in counts if not max_m or m <= max_m]
            report[(N, K, epi)] = ops.autotune.tune(N, K, epi, ms, self.device)
            if verbose:
                for m, (cfg, us, us_auto) in report[(N, K, epi)].items():
                    print(f"[autotune] N={N} K={K} epi={epi} M={m}: {ops.autotune.describe(cfg)} {us:.1f} us (rule: {us_auto:.1f} us)")
        comm = getattr(self.model, "comm", None)
        if comm is not None and hasattr(comm, "tune_all_reduce") and hasattr(self.model, "row_parallel_shapes"):
            # fused GEMM+all-reduce kernel or GEMM -> symmetric all-reduce kernel: whichever is faster per token count
            for N, K in self.model.row_parallel_shapes():
                report[("all_reduce", N, K)] = comm.tune_all_reduce(N, K, [m for m in counts if m >= 8])
        torch.cuda.synchronize(self.device)
        ops.check_status(self.device)
        return report

    # ------------------------------------------------------------------------------------------------
    def execute(self, batch, states, step: int) -> list[int]:
        self.last_num_tokens = int(batch.num_tokens)
        self.last_logprobs = None
        top_lp = max((s.params.logprobs for s in states if s.params.logprobs is not None), default=None)
        if (top_lp is None and self.use_graphs and batch.num_prefill == 0 and batch.num_decode > 0
                and all(s.params.temperature <= 0.0 for s in states)):
            bb = self._bucket(int(batch.num_seqs))
            g = self.graphs.get(bb)
            if g is None and self.ep is None and bb not in self.failed_buckets:
                g = self._capture(bb)          # first use of a bucket that was not captured at start-up
            if g is not None and g.usable():
                return self._execute_decode_graph(batch)
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
        if self.step_events is not None:
            self.step_events[0].record()
        comm = getattr(self.model, "comm", None)
        if comm is not None and hasattr(comm, "begin_graph"):
            # cross-rank barrier kernel: eager steps and graph replays interleave, and each keeps its own count of
            # double-buffer halves; after the barrier no peer is still reading a half this step overwrites
            comm.begin_graph()
        if S == 0:
            # pure mid-prompt chunks: run the layers for their KV side effect, nothing to sample
            self.model.forward(token_ids, positions, slots, meta, self.kv_caches, rows)
            if self.step_events is not None:
                self.step_events[1].record()
            self.d2h_bytes = 0
            return []
        # log-probabilities need the logits themselves: no arg-max inside the forward pass for such a step
        fused_greedy = greedy and top_lp is None and getattr(self.model, "greedy_in_forward", False)
        if fused_greedy:
            ids = self.model.forward(token_ids, positions, slots, meta, self.kv_caches, rows, greedy=True)
        else:
            logits = self.model.forward(token_ids, positions, slots, meta, self.kv_caches, rows)
        if fused_greedy:
            pass
        elif greedy:
            ids = ops.argmax(logits)
        else:
            seed = self.cfg.seed if states[0].params.seed is None else states[0].params.seed
            ids = ops.sample(logits.float() if not self.cuda else logits, st.view(seg_temp, torch.float32),
                             st.view(seg_topk, torch.int32), st.view(seg_topp, torch.float32), seed, step)
        if top_lp is not None:
            # optional diagnostic output, off the measured path: plain tensor ops on the step's logits
            lp = torch.log_softmax(logits.float(), dim=-1)
            chosen = lp.gather(1, ids.view(-1, 1).long()).view(-1).tolist()
            if top_lp > 0:
                tv, ti = lp.topk(min(top_lp, lp.shape[1]), dim=-1)
                tv, ti = tv.tolist(), ti.tolist()
                self.last_logprobs = [(chosen[r], list(zip(ti[r], tv[r]))) for r in range(S)]
            else:
                self.last_logprobs = [(chosen[r], []) for r in range(S)]
        if self.step_events is not None:
            self.step_events[1].record()
        if self.cuda:
            self.ids_host[:S].copy_(ids, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            out = self.ids_host[:S].tolist()
        else:
            out = ids.tolist()
        self.d2h_bytes = S * 8
        return out

    # ------------------------------------------------------------------------------------------------
    # decode-only steps: CUDA graph per batch-size bucket
    # ------------------------------------------------------------------------------------------------
    def _bucket(self, b: int) -> int:
        for x in self.buckets:
            if x >= b:
                return x
        return self.buckets[-1]

    def _execute_decode_graph(self, batch) -> list[int]:
        B = int(batch.num_seqs)
        bb = self._bucket(B)
        g = self.graphs[bb]
        self.h2d_bytes = g.stage(batch, B)
        if self.step_events is not None:
            self.step_events[0].record()
        g.graph.replay()
        if self.step_events is not None:
            self.step_events[1].record()
        self.graph_launches += 1
        self.graph_kernel_launches += g.kernel_launches
        if self.ep is not None:
            self.ep._calls += g.ep_calls     # the replay ran that many MoE layers: keep the buffer-bank parity in step
        self.ids_host[:B].copy_(g.ids[:B], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        self.d2h_bytes = B * 8
        return self.ids_host[:B].tolist()


class _DecodeGraph:
    """Static input buffers + captured forward/argmax for one decode batch-size bucket. Padding rows carry
    slot -1 (no KV write) and context length 0 (attention produces zeros)."""

    def __init__(self, runner: ModelRunner, bb: int):
        self.runner, self.bb = runner, bb
        mb = runner.max_blocks
        dev = runner.device
        # host layout: tok i64[bb] | slot i64[bb] | pos i32[bb] | ctx i32[bb] | bt i32[bb * mb]
        self.o_tok, self.o_slot = 0, 8 * bb
        self.o_pos, self.o_ctx = 16 * bb, 20 * bb
        self.o_bt = _align(24 * bb)
        nbytes = self.o_bt + 4 * bb * mb
        self.host = torch.zeros(nbytes, dtype=torch.uint8, pin_memory=True)
        self.np = self.host.numpy()
        self.dev = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        d = self.dev
        self.tok = d[self.o_tok:self.o_tok + 8 * bb].view(torch.int64)
        self.slot = d[self.o_slot:self.o_slot + 8 * bb].view(torch.int64)
        self.pos = d[self.o_pos:self.o_pos + 4 * bb].view(torch.int32)
        self.ctx = d[self.o_ctx:self.o_ctx + 4 * bb].view(torch.int32)
        self.bt = d[self.o_bt:self.o_bt + 4 * bb * mb].view(torch.int32).view(bb, mb)
        self.cu = torch.arange(bb + 1, dtype=torch.int32, device=dev)
        self.h_tok = self.np[self.o_tok:self.o_tok + 8 * bb].view(np.int64)
        self.h_slot = self.np[self.o_slot:self.o_slot + 8 * bb].view(np.int64)
        self.h_pos = self.np[self.o_pos:self.o_pos + 4 * bb].view(np.int32)
        self.h_ctx = self.np[self.o_ctx:self.o_ctx + 4 * bb].view(np.int32)
        self.h_bt = self.np[self.o_bt:self.o_bt + 4 * bb * mb].view(np.int32).reshape(bb, mb)
        self.h_slot[:] = -1
        self.dev.copy_(self.host)
        self.meta = ops.AttnMeta(self.cu, self.ctx, self.bt, bb, 1, runner.cfg.max_model_len)
        model, caches = runner.model, runner.kv_caches

        comm = getattr(model, "comm", None)
        ep = runner.ep
        calls0 = ep._calls if ep is not None else 0

        def run():
            if comm is not None and hasattr(comm, "begin_graph"):
                comm.begin_graph()
            if getattr(model, "greedy_in_forward", False):
                return model.forward(self.tok, self.pos, self.slot, self.meta, caches, None, greedy=True)
            logits = model.forward(self.tok, self.pos, self.slot, self.meta, caches, None)
            return ops.argmax(logits)

        # one eager pass on a side stream: one-time kernel attribute set-up must not happen under capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            run()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        # the eager pass ran its MoE layers on the device; the captured pass below only records them
        self.ep_calls = (ep._calls - calls0) if ep is not None else 0
        self.ep_parity = (ep._calls & 1) if ep is not None else 0
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=runner.graph_pool):
            self.ids = run()
        if runner.graph_pool is None:
            runner.graph_pool = self.graph.pool()
        self.kernel_launches = ops.launch_count - before
        ops.launch_count = before
        if ep is not None:
            ep._calls -= self.ep_calls

    def usable(self) -> bool:
        """Under expert parallelism the graph holds the receive-buffer bank (call parity) of each MoE layer as it was at
        capture: it may replay only from the same parity, which an even number of MoE layers per step guarantees."""
        ep = self.runner.ep
        return ep is None or (self.ep_calls % 2 == 0 and (ep._calls & 1) == self.ep_parity)

    def stage(self, batch, B: int) -> int:
        bb = self.bb
        self.h_tok[:B] = batch.token_ids
        self.h_slot[:B] = batch.slots
        self.h_pos[:B] = batch.positions
        self.h_ctx[:B] = batch.ctx_lens
        if B < bb:
            self.h_tok[B:] = 0
            self.h_slot[B:] = -1
            self.h_pos[B:] = 0
            self.h_ctx[B:] = 0
        bt = batch.block_tables
        self.h_bt[:B, :bt.shape[1]] = bt
        self.dev.copy_(self.host, non_blocking=True)
        return self.host.numel()
