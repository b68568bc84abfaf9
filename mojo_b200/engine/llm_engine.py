"""The serving engine: request queue -> continuous-batching scheduler (C++) -> model runner -> sampler.

`LLMEngine.step()` is one iteration of the hot loop: the scheduler packs decode tokens and prefill chunks under
a token budget and hands back flat metadata; the runner stages it in pinned memory, copies it to the device in
one transfer, runs the model and the sampler, and reads the sampled ids back. Works on CPU (fp32 reference
ops, the numerics oracle) and on CUDA (sm_100a kernels) with the same code.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import _ext, ops
from ..models import build_model
from ..models.config import ModelConfig
from ..utils import trace


@dataclass
class SamplingParams:
    temperature: float = 0.0          # 0 = greedy
    top_k: int = 0                    # 0 = off
    top_p: float = 1.0                # 1 = off
    max_tokens: int = 16
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    seed: int | None = None
    logprobs: int | None = None       # None: off; k >= 0: log-probability of each sampled token plus the k most likely ones

    def __post_init__(self):
        # one place for every entry point (Python API, server, CLI): a value the sampling kernel would misread is refused here
        if not (0.0 <= float(self.temperature) <= 100.0):      # also false for NaN
            raise ValueError("temperature must be between 0 and 100")
        if not (0.0 < float(self.top_p) <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if int(self.top_k) < 0:
            raise ValueError("top_k must be 0 (off) or positive")
        if int(self.max_tokens) < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.logprobs is not None and not (0 <= int(self.logprobs) <= 20):
            raise ValueError("logprobs must be between 0 and 20")


@dataclass
class EngineConfig:
    model: ModelConfig = None
    device: str = "cpu"
    dtype: torch.dtype = torch.float32
    page_size: int = 16
    num_pages: int | None = None          # None: size from free device memory
    gpu_memory_utilization: float = 0.9
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096
    enable_prefix_cache: bool = False
    enable_chunked_prefill: bool = True
    eos_token_id: int | None = None
    seed: int = 0
    use_cuda_graphs: bool = True
    capture_graphs_at_start: bool = True  # capture every decode bucket before serving instead of at first use
    mixed_step_graphs: bool = True        # steps that carry prefill chunks replay CUDA graphs too (captured at first use of a shape)
    capture_mixed_graphs_at_start: bool = False   # capture every mixed-step shape before serving (a few seconds for an 8B model)
    tp_size: int = 1
    ep_size: int = 1
    lockstep: bool = False                # data-parallel attention + expert parallelism: a rank without work still joins every MoE layer
    autotune: bool = False                # measure GEMM configurations for this model's shapes at start-up
    # Pipelined stepping: step k + 1 is scheduled, staged and launched while the device still runs step k, so the host's
    # per-step work (scheduler, staging, output bookkeeping) is hidden behind the device. `step()` then returns the
    # outputs of the step launched one call earlier. Off in lock-step (expert-parallel) engines.
    async_scheduling: bool = False


@dataclass
class RequestState:
    request_id: int
    prompt_len: int
    params: SamplingParams
    arrival: float
    output_ids: list = field(default_factory=list)
    token_times: list = field(default_factory=list)
    first_token_time: float | None = None
    finished: bool = False
    finish_reason: str | None = None
    logprobs: list = field(default_factory=list)   # per generated token: (logprob, [(token id, logprob), ...]) when requested


@dataclass
class RequestOutput:
    request_id: int
    new_token_ids: list
    output_ids: list
    finished: bool
    finish_reason: str | None
    logprobs: list | None = None      # for the new tokens, when the request asked for them


class LLMEngine:
    def __init__(self, cfg: EngineConfig, model=None, comm=None):
        self.cfg = cfg
        self.C = _ext.require()
        self.device = torch.device(cfg.device)
        self.model = model if model is not None else build_model(cfg.model, self.device, cfg.dtype, comm=comm).init_random(cfg.seed)
        self.comm = comm
        # positions beyond the model's rotary table do not exist: the context limit cannot exceed it
        max_pos = int(getattr(self.model.cfg, "max_position_embeddings", 0) or 0)
        if max_pos and cfg.max_model_len > max_pos:
            cfg.max_model_len = max_pos
        num_pages = cfg.num_pages or self._auto_num_pages()
        self.kv_caches = self.model.allocate_kv_cache(num_pages, cfg.page_size)
        self.kv = self.C.KVCacheManager(num_pages, cfg.page_size, cfg.enable_prefix_cache)
        sc = self.C.SchedulerConfig()
        sc.max_num_seqs = cfg.max_num_seqs
        sc.max_num_batched_tokens = cfg.max_num_batched_tokens
        sc.max_model_len = cfg.max_model_len
        sc.enable_chunked_prefill = cfg.enable_chunked_prefill
        self.scheduler = self.C.Scheduler(sc, self.kv)
        self.requests: dict[int, RequestState] = {}
        self._prompts: dict[int, np.ndarray] = {}
        # running latency histograms (Prometheus-style cumulative buckets are derived on read); they survive `forget`
        self.ttft_bounds_ms = np.array([10, 25, 50, 100, 250, 500, 1000, 2500, 5000, 10000, 30000], dtype=np.float64)
        self.itl_bounds_ms = np.array([1, 2, 5, 10, 20, 50, 100, 250, 1000], dtype=np.float64)
        self._ttft_hist = np.zeros(len(self.ttft_bounds_ms) + 1, dtype=np.int64)
        self._itl_hist = np.zeros(len(self.itl_bounds_ms) + 1, dtype=np.int64)
        self._ttft_sum_ms = self._itl_sum_ms = 0.0
        self.finished_requests = 0
        self.generated_tokens = 0
        self._next_id = 0
        self.step_count = 0
        # failure detection (all optional, all on the host): see engine/watchdog.py and utils/fault.py
        from ..utils import fault as _fault

        rank = getattr(comm, "rank", 0) if comm is not None else 0
        self.fault = _fault.FaultInjector(_fault.from_env(), rank)
        self.watchdog = None
        self.heartbeat = None
        self.skipped_launches = 0
        from .model_runner import ModelRunner

        self.runner = ModelRunner(self.model, self.kv_caches, cfg)
        self._inflight = None     # pipelined stepping: the launched step whose tokens the host has not read yet
        if cfg.async_scheduling and not cfg.lockstep:
            self.scheduler.set_auto_commit(False)   # a batch is confirmed when its tokens have been read, not when the next is scheduled
        self.tune_report = self.runner.autotune() if cfg.autotune else {}
        if cfg.use_cuda_graphs and cfg.capture_graphs_at_start:
            # after tuning: the captured launches carry the tuned configurations
            self.runner.capture_graphs(mixed=cfg.capture_mixed_graphs_at_start)

    def _auto_num_pages(self) -> int:
        cfg = self.cfg
        per_page = self.model.kv_bytes_per_page(cfg.page_size)
        if self.device.type != "cuda":
            return max(64, (cfg.max_num_seqs * cfg.max_model_len) // cfg.page_size // 8)
        free, total = torch.cuda.mem_get_info(self.device)
        budget = int(total * cfg.gpu_memory_utilization) - (total - free)
        # activations of one full token budget + logits, with slack
        budget -= 8 << 30
        need_max = (cfg.max_num_seqs * cfg.max_model_len + cfg.page_size - 1) // cfg.page_size
        return int(max(16, min(budget // per_page, need_max)))

    # ------------------------------------------------------------------------------------------------
    def add_request(self, prompt_ids, params: SamplingParams | None = None, arrival: float | None = None,
                    request_id: int | None = None) -> int:
        params = params or SamplingParams()
        rid = self._next_id if request_id is None else request_id
        self._next_id = max(self._next_id, rid) + 1
        prompt = np.asarray(prompt_ids, dtype=np.int32)
        self.check_prompt_len(len(prompt))
        max_new = max(1, min(params.max_tokens, self.cfg.max_model_len - len(prompt)))
        now = time.perf_counter() if arrival is None else arrival
        self.scheduler.add_request(rid, prompt, max_new, now)
        self.requests[rid] = RequestState(rid, len(prompt), params, now)
        self._prompts[rid] = prompt
        return rid

    def check_prompt_len(self, n: int) -> None:
        """A request needs at least one prompt token and room for at least one generated token."""
        if n < 1:
            raise ValueError("empty prompt")
        if n >= self.cfg.max_model_len:
            raise ValueError(f"prompt of {n} tokens does not fit the context limit of {self.cfg.max_model_len} tokens")
        if not self.cfg.enable_chunked_prefill and n > self.cfg.max_num_batched_tokens:
            raise ValueError(f"prompt of {n} tokens exceeds the per-step token budget of {self.cfg.max_num_batched_tokens} and chunked prefill is off")

    def prompt_of(self, rid: int) -> np.ndarray:
        return self._prompts[rid]

    def readmit(self, rid: int, prompt_ids, max_new: int, state: RequestState) -> None:
        """Put an aborted request back in the queue under its old id (recovery: recompute from the prompt plus
        the tokens already produced). The request's state object, and with it its output so far, is kept."""
        prompt = np.asarray(prompt_ids, dtype=np.int32)
        max_new = max(1, min(max_new, self.cfg.max_model_len - len(prompt)))
        self.scheduler.add_request(rid, prompt, max_new, state.arrival)
        self.requests[rid] = state

    def attach_watchdog(self, limit_s: float = 60.0, on_stall=None):
        from .watchdog import Watchdog

        self.watchdog = Watchdog(limit_s, on_stall).start()
        return self.watchdog

    def attach_heartbeat(self, store, rank: int, world_size: int, limit_s: float = 30.0):
        from .watchdog import Heartbeat

        self.heartbeat = Heartbeat(store, rank, world_size, limit_s)
        return self.heartbeat

    def abort_request(self, rid: int) -> None:
        if rid in self.requests:
            self.scheduler.abort(rid)
            self.requests[rid].finished = True
            self.requests[rid].finish_reason = "abort"

    def abort_all(self) -> list[int]:
        """Abort every request that has not finished (after a failed step the batch's state is unknown: the KV written
        by the step may be partial). Returns their ids."""
        self.discard_inflight()
        rids = [rid for rid, st in self.requests.items() if not st.finished]
        for rid in rids:
            self.abort_request(rid)
        return rids

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    # ------------------------------------------------------------------------------------------------
    def step(self) -> list[RequestOutput]:
        """One engine iteration. Returns outputs for every sequence that produced a token.

        Before anything is launched the host-side failure hooks run: an injected fault may raise, sleep or skip the
        launch, and the heartbeat check raises `WorkerLost` when a peer rank has left or gone silent."""
        if self.cfg.async_scheduling and not self.cfg.lockstep:
            return self._step_pipelined()
        skip = self.fault.before_step(self.step_count)
        if self.heartbeat is not None:
            self.heartbeat.check()
        if skip:
            self.skipped_launches += 1
            self.step_count += 1
            return []
        with trace.span("engine.schedule"):
            batch = self.scheduler.step()
        if batch.num_seqs == 0:
            if self.cfg.lockstep and hasattr(self.model, "forward_idle"):
                self.model.forward_idle()
                self.step_count += 1
            return []
        sample_ids = batch.sample_seq_ids
        states = [self.requests[int(r)] for r in sample_ids]
        if self.watchdog is not None:
            self.watchdog.begin_step()
        with trace.span("engine.execute"):
            tokens = self.runner.execute(batch, states, self.step_count)
        self.fault.after_execute(self.step_count)
        # the step ran: its full pages may enter the prefix cache (a step that raised never gets here, and the abort
        # that follows it drops the pages it may have half written)
        self.scheduler.commit_step()
        if self.watchdog is not None:
            self.watchdog.end_step(self.step_count)
        if self.heartbeat is not None:
            self.heartbeat.beat(self.step_count)
        self.step_count += 1
        return self._deliver(sample_ids, tokens, states, self.runner.last_logprobs, None)

    def _deliver(self, sample_ids, tokens, states, step_lp, pending) -> list[RequestOutput]:
        """Book the sampled tokens of one step: append them to their sequences, time them, decide who has finished.
        `pending` is None for a step that was waited for; for a pipelined step it holds, per sampled row, the position
        the placeholder took in the sequence and whether the sequence reached its length limit at launch."""
        now = time.perf_counter()
        outs = []
        ttfts, itls = [], []
        for row, (rid, tok, st) in enumerate(zip(sample_ids, tokens, states)):
            rid, tok = int(rid), int(tok)
            if pending is None:
                hit_max = self.scheduler.append_token(rid, tok)
            else:
                if st.finished:
                    continue      # stopped (EOS, stop token, abort) after this step had been launched: its token is dropped
                pos, hit_max = pending[row]
                self.scheduler.set_token(rid, pos, tok)
            st.output_ids.append(tok)
            new_lp = None
            if step_lp is not None and st.params.logprobs is not None:
                lp, top = step_lp[row]
                new_lp = [(lp, top[: st.params.logprobs])]
                st.logprobs.extend(new_lp)
            if st.first_token_time is None:
                st.first_token_time = now
                ttfts.append(now - st.arrival)
            else:
                itls.append(now - st.token_times[-1])
            st.token_times.append(now)
            reason = None
            eos = self.cfg.eos_token_id
            if not st.params.ignore_eos and eos is not None and tok == eos:
                reason = "stop"
            elif tok in st.params.stop_token_ids:
                reason = "stop"
            elif hit_max:
                reason = "length"
            if reason is not None:
                st.finished, st.finish_reason = True, reason
                self.scheduler.finish(rid)      # (a pipelined step that ran into its length limit was finished at launch: no-op)
                self.finished_requests += 1
            outs.append(RequestOutput(rid, [tok], st.output_ids, st.finished, reason, new_lp))
        self.generated_tokens += len(outs)
        if ttfts:
            v = np.asarray(ttfts) * 1e3
            np.add.at(self._ttft_hist, np.searchsorted(self.ttft_bounds_ms, v, side="left"), 1)
            self._ttft_sum_ms += float(v.sum())
        if itls:
            v = np.asarray(itls) * 1e3
            np.add.at(self._itl_hist, np.searchsorted(self.itl_bounds_ms, v, side="left"), 1)
            self._itl_sum_ms += float(v.sum())
        return outs

    def _step_pipelined(self) -> list[RequestOutput]:
        """One iteration with the host one step ahead of the device: schedule and launch the next step, then read and
        book the tokens of the step launched by the previous call (which the device has been running meanwhile).

        A sequence sampled by the step in flight gets a placeholder token at once, so the scheduler can plan its next
        decode row; the row's input is filled on the device from the in-flight step's output. Whether a sequence reaches
        its length limit is known at launch, so it leaves the batch without delay; a stop token shows only when the
        tokens are read, one step later, and the token the sequence produced in between is dropped."""
        skip = self.fault.before_step(self.step_count)
        if self.heartbeat is not None:
            self.heartbeat.check()
        if skip:
            self.skipped_launches += 1
            self.step_count += 1
            return self.flush()
        prev = self._inflight
        with trace.span("engine.schedule"):
            batch = self.scheduler.step()
        launched = None
        if batch.num_seqs > 0:
            sample_ids = batch.sample_seq_ids
            states = [self.requests[int(r)] for r in sample_ids]
            if self.watchdog is not None:
                self.watchdog.begin_step()
            with trace.span("engine.execute"):
                handle = self.runner.launch(batch, states, self.step_count, prev=(prev[0], prev[1]) if prev is not None else None)
            self.fault.after_execute(self.step_count)
            pending = []
            for rid in sample_ids:
                rid = int(rid)
                hit_max = self.scheduler.append_token(rid, -1)
                pending.append((self.scheduler.num_tokens(rid) - 1, hit_max))
                if hit_max:
                    self.scheduler.finish(rid)      # leaves the batch now; its last token is booked when it is read
            launched = (handle, sample_ids, states, self.runner.last_logprobs, pending)
            self.step_count += 1
        outs = self._collect(prev)
        self._inflight = launched
        if launched is not None and self.runner.last_logprobs is not None:
            # a step that computed log-probabilities waited for the device anyway: deliver it in the same call
            outs += self.flush()
        return outs

    def _collect(self, inflight) -> list[RequestOutput]:
        if inflight is None:
            return []
        handle, sample_ids, states, step_lp, pending = inflight
        tokens = self.runner.collect(handle)
        self.scheduler.commit_step()      # that step has completed: its full pages may enter the prefix cache
        if self.watchdog is not None:
            self.watchdog.end_step(self.step_count)
        if self.heartbeat is not None:
            self.heartbeat.beat(self.step_count)
        return self._deliver(sample_ids, tokens, states, step_lp, pending)

    def discard_inflight(self) -> None:
        """Pipelined stepping: wait for the step in flight and drop its tokens unbooked (before aborting or re-queueing
        requests: their sequences still hold that step's placeholders)."""
        inflight, self._inflight = self._inflight, None
        if inflight is not None:
            try:
                self.runner.collect(inflight[0])
            except Exception:  # noqa: BLE001 - the step is being thrown away
                pass

    def flush(self) -> list[RequestOutput]:
        """Pipelined stepping: wait for the step in flight and return its outputs (no-op otherwise)."""
        inflight, self._inflight = self._inflight, None
        return self._collect(inflight)

    def forget(self, rid: int) -> None:
        """Drop the bookkeeping of a finished (or aborted) request. A long-running server calls this when a stream
        ends; the latency histograms and counters keep what they recorded."""
        st = self.requests.get(rid)
        if st is not None and st.finished:
            del self.requests[rid]
            self._prompts.pop(rid, None)

    def histograms(self) -> dict:
        """{"ttft_ms" | "itl_ms": {"bounds": [...], "counts": per-bucket counts (last = above the top bound), "sum": ms}}"""
        return {"ttft_ms": {"bounds": self.ttft_bounds_ms.tolist(), "counts": self._ttft_hist.tolist(), "sum": self._ttft_sum_ms},
                "itl_ms": {"bounds": self.itl_bounds_ms.tolist(), "counts": self._itl_hist.tolist(), "sum": self._itl_sum_ms}}

    def generate(self, prompts, params: SamplingParams | list | None = None) -> list[list[int]]:
        """Blocking convenience: run a list of token-id prompts to completion, return generated ids in order."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        self.run_until_done()
        if self.device.type == "cuda":
            ops.check_status(self.device)
        return [list(self.requests[r].output_ids) for r in rids]

    def run_until_done(self) -> None:
        """Step until every admitted request has finished. In lock-step mode (data-parallel attention with
        expert-parallel MoE) ranks serve different requests but must take the same number of steps: go on, with idle
        steps that only join the MoE layers, until no rank has work left."""
        if self.cfg.lockstep and self._lockstep_group() is not None:
            while self._any_rank_busy():
                self.step()
        else:
            while self.has_unfinished():
                self.step()

    def _lockstep_group(self):
        ep = getattr(self.model, "ep", None)
        info = getattr(ep, "info", None)
        if info is None or info.world_size == 1:
            return None
        return getattr(info, "host_group", None)

    def _any_rank_busy(self) -> bool:
        import torch.distributed as dist

        flag = torch.tensor([1 if self.has_unfinished() else 0], dtype=torch.int64)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self._lockstep_group())
        return bool(flag[0])

    # ------------------------------------------------------------------------------------------------
    def metrics(self) -> dict:
        """TTFT / ITL percentiles and throughput over finished requests."""
        ttft, itl, n_out = [], [], 0
        t0, t1 = float("inf"), 0.0
        for st in self.requests.values():
            if not st.token_times:
                continue
            ttft.append(st.first_token_time - st.arrival)
            tt = st.token_times
            itl.extend(b - a for a, b in zip(tt[:-1], tt[1:]))
            n_out += len(tt)
            t0, t1 = min(t0, st.arrival), max(t1, tt[-1])
        stats = self.kv.stats()
        return {
            "requests": len(ttft), "output_tokens": n_out,
            "ttft_p50_ms": 1e3 * float(np.median(ttft)) if ttft else None,
            "ttft_p99_ms": 1e3 * float(np.percentile(ttft, 99)) if ttft else None,
            "itl_p50_ms": 1e3 * float(np.median(itl)) if itl else None,
            "itl_p99_ms": 1e3 * float(np.percentile(itl, 99)) if itl else None,
            "output_tok_per_s": n_out / (t1 - t0) if t1 > t0 else None,
            "steps": self.step_count, "preemptions": self.scheduler.total_preemptions(),
            "kv_pages": stats.num_pages, "kv_free_pages": stats.free_pages, "prefix_hits": stats.prefix_hits,
        }
