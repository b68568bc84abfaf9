"""Turns a scheduler batch into device tensors, runs the model and the sampler.

All integer metadata of a step (token ids, positions, KV slots, sequence offsets, block tables, rows to sample,
sampling parameters) is packed into one pinned host buffer and moved with a single host->device copy; the only
device->host traffic is the vector of sampled token ids.

Greedy steps replay CUDA graphs, so the ten-odd launches per layer cost one `cudaGraphLaunch`:
  * decode-only steps: one graph per batch-size bucket (`_DecodeGraph`);
  * steps that also carry prefill chunks, which under continuous batching is nearly every step: one graph per
    (token-count bucket, decode-row bucket, prefill-sequence bucket) (`_MixedGraph`). Tokens are padded to the bucket
    (slot -1: nothing is written for a padding row); the decode-attention launch covers a fixed number of rows and
    reads a context length of 0 for the rows that are not decode sequences; the prefill-attention launch covers a
    fixed number of (sequence, query tile) work items of which the device-side count says how many are real.
Everything else (sampling with temperature, log-probabilities, models without the static attention form) runs the
launch sequence eagerly.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops


def _align(n: int, a: int = 16) -> int:
    return (n + a - 1) // a * a


class _Staging:
    """Pinned host buffers + one device buffer of the same size, carved into typed segments per step.

    The host->device copy of a step is asynchronous, and a step with nothing to sample never waits for the device, so
    the copy of step k may still be queued when step k + 1 is staged: the host side alternates between two pinned
    buffers, and a buffer is refilled only after the copy that last read it has completed (an event recorded right
    behind that copy)."""

    def __init__(self, nbytes: int, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        n_host = 2 if self.cuda else 1
        self.hosts = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.cuda) for _ in range(n_host)]
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.copied = [torch.cuda.Event() if self.cuda else None for _ in range(n_host)]
        self.turn = 0
        self.host, self.host_np = self.hosts[0], self.hosts_np[0]
        self.dev = torch.empty(nbytes, dtype=torch.uint8, device=device) if self.cuda else self.host
        self.off = 0

    def begin(self):
        self.off = 0
        if self.cuda:
            self.turn ^= 1
            self.copied[self.turn].synchronize()    # no-op unless the copy two steps back is still in flight
            self.host, self.host_np = self.hosts[self.turn], self.hosts_np[self.turn]

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
            self.copied[self.turn].record()
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
        # sampled ids come back through two pinned slots, so that a step can be launched before the previous one is read
        self.ids_slots = [torch.empty(cfg.max_num_seqs, dtype=torch.int64, pin_memory=self.cuda) for _ in range(2)]
        self.ids_events = [torch.cuda.Event() if self.cuda else None for _ in range(2)]
        self.ids_turn = 0
        self.steps_launched = 0          # steps handed to the device so far (a pipelined `step()` call may launch none)
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
        self.graph_pool = None           # memory pool shared by all graphs (they never replay concurrently)
        self.failed_buckets: dict = {}   # buckets / mixed-step keys whose capture failed: their steps run eagerly
        # mixed steps (decode rows + prefill chunks) as graphs: token-count buckets are the counts the GEMM tables are
        # measured at; decode rows and prefill sequences come in two sizes each
        self.mixed_graphs: dict[tuple, "_MixedGraph"] = {}
        self.mixed_launches = 0
        self.use_mixed_graphs = bool(self.use_graphs and getattr(cfg, "mixed_step_graphs", True)
                                     and getattr(model, "supports_static_attention", lambda *_: False)(cfg.page_size))
        tb = [t for t in (16, 32, 64, 128, 192, 256) if t < cfg.max_num_batched_tokens]
        t = 384
        while t < cfg.max_num_batched_tokens:
            tb.append(t)
            t += 128
        tb.append(cfg.max_num_batched_tokens)
        self.token_buckets = tb
        self.prefill_seq_buckets = (4, 32)
        self.decode_row_buckets = (min(32, cfg.max_num_seqs), cfg.max_num_seqs)
        # Expert parallelism: every rank must run the same number of MoE layer calls per step, so a decode graph can
        # only be captured when all ranks capture together (at start-up); a bucket that is missing runs eagerly.
        ep = getattr(model, "ep", None)
        self.ep = ep if ep is not None and getattr(ep, "world_size", 1) > 1 else None

    def capture_graphs(self, buckets=None, mixed: bool = False) -> int:
        """Capture the decode graph of every batch-size bucket now, largest first so that the smaller ones reuse its
        memory pool. Without this a bucket is captured the first time a decode-only step needs it, which puts a
        capture (an eager pass plus the captured pass) into some request's inter-token latency. With `mixed` the
        graphs of steps that carry prefill chunks are captured too (every token-count bucket times two decode-row and
        two prefill-sequence sizes). Returns the number of graphs captured. Tensor-parallel ranks must all call it
        (the passes contain collectives)."""
        if not self.use_graphs:
            return 0
        n = 0
        if mixed and self.use_mixed_graphs:
            # the shapes of a loaded server (decode rows at the large bucket); the cold-start shapes are captured at first use
            steady = [k for k in self.mixed_keys() if k[1] == min(self.decode_row_buckets[-1], k[0])]
            for key in sorted(steady, reverse=True):
                if key not in self.mixed_graphs and key not in self.failed_buckets and self._capture_mixed(key) is not None:
                    n += 1
        for bb in sorted(set(buckets if buckets is not None else self.buckets), reverse=True):
            if bb not in self.graphs and bb not in self.failed_buckets and self._capture(bb) is not None:
                n += 1
        if self.cuda:
            torch.cuda.synchronize(self.device)
            ops.check_status(self.device)
        return n

    def mixed_keys(self) -> list[tuple]:
        """Every (token bucket, decode rows, prefill-sequence bucket) a mixed step can map to."""
        keys = set()
        for tb in self.token_buckets:
            for db in (0,) + tuple(self.decode_row_buckets):
                for pb in self.prefill_seq_buckets:
                    keys.add((tb, min(db, tb), min(pb, tb)))
        return sorted(keys)

    def mixed_key(self, T: int, nd: int, P: int):
        """Bucket of a step with T tokens, nd decode sequences and P prefill chunks; None if no graph shape covers it."""
        if P < 1 or P > self.prefill_seq_buckets[-1] or T > self.token_buckets[-1]:
            return None
        tb = next(t for t in self.token_buckets if t >= T)
        pb = min(next(p for p in self.prefill_seq_buckets if p >= P), tb)
        db = 0 if nd == 0 else min(next(d for d in self.decode_row_buckets if d >= nd), tb)
        return (tb, db, pb)

    def _capture_mixed(self, key):
        try:
            g = _MixedGraph(self, *key)
        except Exception as e:  # noqa: BLE001
            import warnings

            self.failed_buckets[key] = repr(e)
            if self.cuda:
                torch.cuda.synchronize(self.device)
            warnings.warn(f"mojo_b200: CUDA-graph capture of the mixed step {key} failed ({e!r}); such steps run eagerly", stacklevel=2)
            return None
        self.mixed_graphs[key] = g
        return g

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
        if comm is not None and hasattr(comm, "tune_all_reduce_norm") and hasattr(self.model, "row_parallel_shapes"):
            # row-parallel linear + all-reduce + residual + norm: one-shot kernel, in-switch kernel, all-reduce kernel + norm,
            # or the fused GEMM+all-reduce kernel + norm: whichever measures fastest per token count
            for N, K in self.model.row_parallel_shapes():
                report[("all_reduce_norm", N, K)] = comm.tune_all_reduce_norm(N, K, [m for m in counts if m >= 8])
        elif comm is not None and hasattr(comm, "tune_all_reduce") and hasattr(self.model, "row_parallel_shapes"):
            for N, K in self.model.row_parallel_shapes():
                report[("all_reduce", N, K)] = comm.tune_all_reduce(N, K, [m for m in counts if m >= 8])
        torch.cuda.synchronize(self.device)
        ops.check_status(self.device)
        return report

    # ------------------------------------------------------------------------------------------------
    def execute(self, batch, states, step: int) -> list[int]:
        """Run one step and return its sampled tokens (launch, then wait for the result)."""
        return self.collect(self.launch(batch, states, step))

    def collect(self, h: "StepHandle") -> list[int]:
        """The sampled token ids of a launched step: waits for its device->host copy."""
        if h.tokens is not None:
            return h.tokens
        if h.S == 0:
            return []
        h.event.synchronize()
        return self.ids_slots[h.slot][:h.S].tolist()

    def _finish_launch(self, ids, S: int) -> "StepHandle":
        """Queue the copy of the sampled ids into a pinned slot (two slots: a step is collected before the launch after
        the next reuses its slot) and return the handle that `collect` waits on."""
        self.d2h_bytes = S * 8
        if not self.cuda:
            return StepHandle(S, ids, tokens=ids.tolist() if S else [])
        if S == 0:
            return StepHandle(0, ids)
        self.ids_turn ^= 1
        slot = self.ids_turn
        self.ids_slots[slot][:S].copy_(ids[:S], non_blocking=True)
        self.ids_events[slot].record()
        return StepHandle(S, ids, slot=slot, event=self.ids_events[slot])

    def _patch_plan(self, batch, prev):
        """Rows of this batch whose input token is still a placeholder (-1): the token the previous step sampled for that
        sequence, not yet read back by the host. Returns (row indices, indices into the previous step's sampled ids)."""
        tok = batch.token_ids
        neg = np.nonzero(tok < 0)[0]
        if neg.size == 0:
            return None
        if prev is None:
            raise RuntimeError("a placeholder token without a step in flight to take it from")
        _, prev_seq_ids = prev
        where = {int(r): j for j, r in enumerate(prev_seq_ids)}
        seq_of_row = np.searchsorted(batch.cu_q, neg, side="right") - 1
        seq_ids = batch.seq_ids
        src = np.fromiter((where[int(seq_ids[i])] for i in seq_of_row), dtype=np.int32, count=neg.size)
        return neg.astype(np.int32), src

    def launch(self, batch, states, step: int, prev=None) -> "StepHandle":
        """Stage and launch one step without waiting for it. `prev` = (handle of the step launched before this one, the
        sequence ids of its sampled rows) when the host has not read that step's tokens yet: decode rows whose input is
        such a token carry -1 in the batch and are filled on the device from the previous step's output."""
        self.last_num_tokens = int(batch.num_tokens)
        self.last_logprobs = None
        self.steps_launched += 1
        plan = self._patch_plan(batch, prev)
        prev_ids = prev[0].ids if (plan is not None) else None
        top_lp = max((s.params.logprobs for s in states if s.params.logprobs is not None), default=None)
        if (top_lp is None and self.use_graphs and batch.num_prefill == 0 and batch.num_decode > 0
                and all(s.params.temperature <= 0.0 for s in states)):
            bb = self._bucket(int(batch.num_seqs))
            g = self.graphs.get(bb)
            if g is None and self.ep is None and bb not in self.failed_buckets:
                g = self._capture(bb)          # first use of a bucket that was not captured at start-up
            if g is not None and g.usable():
                return self._launch_decode_graph(batch, plan, prev_ids)
        if (top_lp is None and self.use_mixed_graphs and batch.num_prefill > 0
                and all(s.params.temperature <= 0.0 for s in states)):
            key = self.mixed_key(int(batch.num_tokens), int(batch.num_decode), int(batch.num_prefill))
            if key is not None:
                g = self.mixed_graphs.get(key)
                if g is None and key not in self.failed_buckets:
                    g = self._capture_mixed(key)      # first use of a shape that was not captured at start-up
                if g is not None:
                    return self._launch_mixed_graph(g, batch, plan, prev_ids)
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
        seg_work, n_items = None, 0
        if self.cuda and batch.num_prefill > 0 and getattr(self.model, "supports_static_attention", lambda *_: False)(self.cfg.page_size):
            # one CTA per (sequence, query tile) of the chunks, longest context first, instead of a padded grid
            work = ops.prefill_work_items(batch.cu_q, batch.ctx_lens, int(batch.num_decode))
            n_items = int(work.shape[0])
            if n_items:
                seg_work = st.put(work, np.int32)
        greedy = all(s.params.temperature <= 0.0 for s in states)
        if not greedy:
            seg_temp = st.put(np.array([s.params.temperature for s in states], dtype=np.float32), np.float32)
            seg_topk = st.put(np.array([s.params.top_k for s in states], dtype=np.int32), np.int32)
            seg_topp = st.put(np.array([s.params.top_p for s in states], dtype=np.float32), np.float32)
        if plan is not None:
            seg_prow, seg_psrc = st.put(plan[0], np.int32), st.put(plan[1], np.int32)
        self.h2d_bytes = st.flush()

        token_ids = st.view(seg_tok, torch.int64)
        if plan is not None:
            self._patch(token_ids, st.view(seg_prow, torch.int32), st.view(seg_psrc, torch.int32), prev_ids, len(plan[0]))
        slots = st.view(seg_slot, torch.int64)
        positions = st.view(seg_pos, torch.int32)
        ctx_np = batch.ctx_lens
        meta = ops.AttnMeta(st.view(seg_cu, torch.int32), st.view(seg_ctx, torch.int32), st.view(seg_bt, torch.int32),
                            batch.num_decode, batch.max_q_len, int(ctx_np.max()) if B else 0,
                            work=st.view(seg_work, torch.int32) if seg_work is not None else None, n_items=n_items)
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
            return self._finish_launch(None, 0)
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
        return self._finish_launch(ids, S)

    def _patch(self, token_ids, rows, src, prev_ids, n: int) -> None:
        if token_ids.is_cuda:
            from .. import _ext

            _ext.require().patch_tokens(token_ids, rows, src, prev_ids, n, ops._state.get(self.device).status)
            ops._count()
        else:
            token_ids[rows[:n].long()] = prev_ids[src[:n].long()].to(token_ids.dtype)

    # ------------------------------------------------------------------------------------------------
    # decode-only steps: CUDA graph per batch-size bucket
    # ------------------------------------------------------------------------------------------------
    def _bucket(self, b: int) -> int:
        for x in self.buckets:
            if x >= b:
                return x
        return self.buckets[-1]

    def _launch_decode_graph(self, batch, plan=None, prev_ids=None) -> "StepHandle":
        B = int(batch.num_seqs)
        bb = self._bucket(B)
        g = self.graphs[bb]
        self.h2d_bytes = g.stage(batch, B, plan)
        if plan is not None:
            self._patch(g.tok, g.fix_rows, g.fix_src, prev_ids, len(plan[0]))
        if self.step_events is not None:
            self.step_events[0].record()
        g.graph.replay()
        if self.step_events is not None:
            self.step_events[1].record()
        self.graph_launches += 1
        self.graph_kernel_launches += g.kernel_launches
        if self.ep is not None:
            self.ep._calls += g.ep_calls     # the replay ran that many MoE layers: keep the buffer-bank parity in step
        return self._finish_launch(g.ids, B)

    def _execute_decode_graph(self, batch) -> list[int]:
        return self.collect(self._launch_decode_graph(batch))

    def _launch_mixed_graph(self, g: "_MixedGraph", batch, plan=None, prev_ids=None) -> "StepHandle":
        S = int(len(batch.sample_rows))
        self.h2d_bytes = g.stage(batch, plan)
        if plan is not None:
            self._patch(g.tok, g.fix_rows, g.fix_src, prev_ids, len(plan[0]))
        if self.step_events is not None:
            self.step_events[0].record()
        g.graph.replay()
        if self.step_events is not None:
            self.step_events[1].record()
        self.graph_launches += 1
        self.mixed_launches += 1
        self.graph_kernel_launches += g.kernel_launches
        return self._finish_launch(g.ids, S)     # S == 0: mid-prompt chunks only, nothing to read back


class StepHandle:
    """A launched step: `ids` is the device tensor of its sampled token ids (first `S` entries), of which a copy is on
    its way into pinned slot `slot` (`event` marks its arrival); `tokens` holds them already when nothing was queued."""

    __slots__ = ("S", "ids", "slot", "event", "tokens")

    def __init__(self, S, ids, slot=0, event=None, tokens=None):
        self.S, self.ids, self.slot, self.event, self.tokens = S, ids, slot, event, tokens


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
        self.o_fix = _align(self.o_bt + 4 * bb * mb)      # rows / sources of tokens still on the device (pipelined stepping)
        nbytes = self.o_fix + 8 * bb
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
        self.fix_rows = d[self.o_fix:self.o_fix + 4 * bb].view(torch.int32)
        self.fix_src = d[self.o_fix + 4 * bb:self.o_fix + 8 * bb].view(torch.int32)
        self.h_fix = self.np[self.o_fix:self.o_fix + 8 * bb].view(np.int32)
        self.copied = torch.cuda.Event()
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

    def stage(self, batch, B: int, plan=None) -> int:
        bb = self.bb
        self.copied.synchronize()       # the previous copy out of this block has been consumed
        if plan is not None:
            n = len(plan[0])
            self.h_fix[:n] = plan[0]
            self.h_fix[bb:bb + n] = plan[1]
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
        self.copied.record()
        return self.host.numel()


class _MixedGraph:
    """Static buffers + captured forward/argmax for steps with `tb` tokens (padded), up to `db` decode rows and up to
    `pb` prefill chunks. One pinned block is filled on the host and moved with one copy; the graph reads everything
    that varies (ids, positions, slots, context lengths, block tables, work items and their count, rows to sample)
    from the device copy of that block."""

    def __init__(self, runner: ModelRunner, tb: int, db: int, pb: int):
        self.runner, self.tb, self.db, self.pb = runner, tb, db, pb
        mb, dev = runner.max_blocks, runner.device
        self.max_items = tb // 128 + pb
        self.sb = max(1, min(db + pb, tb))          # rows that can be sampled in one step
        lay, off = {}, 0

        def seg(name, nbytes):
            nonlocal off
            lay[name] = (off, nbytes)
            off = _align(off + nbytes)

        seg("tok", 8 * tb); seg("slot", 8 * tb); seg("pos", 4 * tb)
        seg("d_ctx", 4 * max(db, 1)); seg("d_bt", 4 * max(db, 1) * mb)
        seg("p_cu", 4 * (pb + 1)); seg("p_ctx", 4 * pb); seg("p_bt", 4 * pb * mb)
        seg("work", 8 * self.max_items); seg("n_work", 4); seg("rows", 8 * self.sb)
        seg("fix_rows", 4 * self.sb); seg("fix_src", 4 * self.sb)   # tokens still on the device (pipelined stepping)
        self.nbytes = off
        self.host = torch.zeros(off, dtype=torch.uint8, pin_memory=True)
        self.dev = torch.zeros(off, dtype=torch.uint8, device=dev)
        self.copied = torch.cuda.Event()
        hn = self.host.numpy()

        def hv(name, dtype, shape=None):
            o, n = lay[name]
            a = hn[o:o + n].view(dtype)
            return a.reshape(shape) if shape is not None else a

        def dv(name, dtype, shape=None):
            o, n = lay[name]
            t = self.dev[o:o + n].view(dtype)
            return t.view(*shape) if shape is not None else t

        self.h = {"tok": hv("tok", np.int64), "slot": hv("slot", np.int64), "pos": hv("pos", np.int32),
                  "d_ctx": hv("d_ctx", np.int32), "d_bt": hv("d_bt", np.int32, (max(db, 1), mb)),
                  "p_cu": hv("p_cu", np.int32), "p_ctx": hv("p_ctx", np.int32), "p_bt": hv("p_bt", np.int32, (pb, mb)),
                  "work": hv("work", np.int32, (self.max_items, 2)), "n_work": hv("n_work", np.int32), "rows": hv("rows", np.int64),
                  "fix_rows": hv("fix_rows", np.int32), "fix_src": hv("fix_src", np.int32)}
        self.h["slot"][:] = -1
        self.dev.copy_(self.host)
        self.tok, self.slot, self.pos = dv("tok", torch.int64), dv("slot", torch.int64), dv("pos", torch.int32)
        self.rows = dv("rows", torch.int64)
        self.fix_rows, self.fix_src = dv("fix_rows", torch.int32), dv("fix_src", torch.int32)
        n_kv = runner.kv_caches[0][0].shape[1]
        static = ops.StaticAttn(db, dv("d_ctx", torch.int32), dv("d_bt", torch.int32, (max(db, 1), mb)),
                                ops._decode_splits(db, n_kv, runner.cfg.max_model_len) if db else 1,
                                dv("p_cu", torch.int32), dv("p_ctx", torch.int32), dv("p_bt", torch.int32, (pb, mb)),
                                dv("work", torch.int32, (self.max_items, 2)), dv("n_work", torch.int32), self.max_items, tb)
        self.meta = ops.AttnMeta(None, None, None, 0, tb, runner.cfg.max_model_len, static=static)
        model, caches = runner.model, runner.kv_caches
        comm = getattr(model, "comm", None)

        def run():
            if comm is not None and hasattr(comm, "begin_graph"):
                comm.begin_graph()
            if getattr(model, "greedy_in_forward", False):
                return model.forward(self.tok, self.pos, self.slot, self.meta, caches, self.rows, greedy=True)
            return ops.argmax(model.forward(self.tok, self.pos, self.slot, self.meta, caches, self.rows))

        # one eager pass on a side stream (one-time kernel attribute set-up must not happen under capture); the block
        # is all padding at this point: slots -1, no decode context, no work items, so the pass touches no KV page
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            run()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=runner.graph_pool):
            self.ids = run()
        if runner.graph_pool is None:
            runner.graph_pool = self.graph.pool()
        self.kernel_launches = ops.launch_count - before
        ops.launch_count = before

    def stage(self, batch, plan=None) -> int:
        """Fill the pinned block from the scheduler's batch and start its copy. Returns the bytes copied."""
        self.copied.synchronize()       # the previous copy out of this block has been consumed
        h = self.h
        if plan is not None:
            n = len(plan[0])
            if n > self.sb:
                raise RuntimeError(f"mixed-step graph {self.tb, self.db, self.pb}: {n} device-side tokens exceed {self.sb}")
            h["fix_rows"][:n] = plan[0]
            h["fix_src"][:n] = plan[1]
        T, B, nd = int(batch.num_tokens), int(batch.num_seqs), int(batch.num_decode)
        P = B - nd
        h["tok"][:T] = batch.token_ids
        h["tok"][T:] = 0
        h["slot"][:T] = batch.slots
        h["slot"][T:] = -1
        h["pos"][:T] = batch.positions
        h["pos"][T:] = 0
        ctx, cu, bt = batch.ctx_lens, batch.cu_q, batch.block_tables
        w = bt.shape[1]
        if self.db:
            h["d_ctx"][:nd] = ctx[:nd]
            h["d_ctx"][nd:] = 0
            h["d_bt"][:nd, :w] = bt[:nd]
        h["p_cu"][:P + 1] = cu[nd:]
        h["p_cu"][P + 1:] = cu[-1]
        h["p_ctx"][:P] = ctx[nd:]
        h["p_ctx"][P:] = 0
        h["p_bt"][:P, :w] = bt[nd:]
        work = ops.prefill_work_items(cu, ctx, nd)
        n = work.shape[0]
        if n > self.max_items:
            raise RuntimeError(f"mixed-step graph {self.tb, self.db, self.pb}: {n} attention work items exceed {self.max_items}")
        h["work"][:n] = work
        h["n_work"][0] = n
        rows = batch.sample_rows
        S = len(rows)
        if S > self.sb:
            raise RuntimeError(f"mixed-step graph {self.tb, self.db, self.pb}: {S} rows to sample exceed {self.sb}")
        h["rows"][:S] = rows
        h["rows"][S:] = 0
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        return self.nbytes
