"""Headline benchmark: output tokens/s of the serving engine on Llama-3.1-8B (bf16, random-init weights,
synthetic prompts) under continuous batching with a paged KV cache of page size 128.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A "step" is one engine iteration (one scheduler decision + one model forward over the decode tokens and prefill
chunks it packed + sampling). The request stream is the 512-request Poisson trace (prompt U[128, 2048], output
U[64, 512], greedy); when it runs dry it continues with fresh requests from the same distribution, so any K
measures the same regime. Before the W warm-up steps the engine is ramped until the first request completes, so
the timed region sees the steady mix of decode tokens and prefill chunks, not the cold start.

The K-step window is timed `--repeats` times back to back (default 5); `value` is the median window and `spread`
holds the fastest and slowest one. Two numbers come out of the same steps:
  value      output tokens / device time: CUDA events around each step's device work (model + sampler), summed,
             max over ranks
  e2e.value  output tokens / wall time of `LLMEngine.step()`: scheduler, pinned staging, the host->device copy
             of the step's metadata, the model, the sampler and the device->host read of the sampled ids. The engine
             steps pipelined (the host schedules step k + 1 while the device runs step k), so most of the host's
             share is hidden; `--no-async` gives the step-by-step figure.
With all eight GPUs the same process then measures the two other named serving configurations, each as one window
that runs its whole fixed batch from the first prefill chunk to the last token (prefill inside the timed region):
Llama-3.3-70B fp8 block-scaled at TP = 8 and DeepSeek-V2-Lite with data-parallel attention + expert-parallel MoE.
They ride in the same JSON line under `secondary`. Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


METRIC_NAMES = {"llama-3.1-8b": "Llama-3.1-8B bf16", "llama-3.3-70b-fp8": "Llama-3.3-70B fp8 block-scaled",
                "deepseek-v2-lite": "DeepSeek-V2-Lite bf16 (MLA + MoE)"}
# configurations that are one fixed batch present at t = 0: (requests, prompt tokens, output tokens)
FIXED = {"llama-3.3-70b-fp8": (256, 1024, 256), "deepseek-v2-lite": (512, 512, 256), "tiny-deepseek": (64, 64, 16)}
SECONDARY_DEADLINE_S = 420.0     # the two extra configurations together; past it the headline line goes out without them
SECONDARY_GRACE_S = 90.0         # after the deadline the runs stop between steps; only if that does not happen either, every rank leaves
ABANDON = threading.Event()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5, help="how many times the K-step window is timed (median reported)")
    ap.add_argument("--impl", default="mojo_b200", choices=["mojo_b200", "reference", "torch-baseline", "vllm-yardstick"])
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--rate", type=float, default=1000.0,
                    help="Poisson arrival rate, requests/s; the default keeps the queue non-empty at every GPU count, so the number is capacity, not offered load")
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-batched-tokens", type=int, default=4096)
    ap.add_argument("--page-size", type=int, default=128)
    ap.add_argument("--max-ramp-steps", type=int, default=400)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-mixed-graphs", action="store_true", help="CUDA graphs for decode-only steps only; steps with prefill chunks launch eagerly")
    ap.add_argument("--no-autotune", action="store_true", help="skip the start-up measurement of GEMM configurations")
    ap.add_argument("--no-async", action="store_true", help="step by step: the host waits for every step's tokens before it schedules the next")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--ar-mode", default="auto", choices=["auto", "fused", "split"],
                    help="row-parallel linear + all-reduce: the single fused kernel, GEMM -> symmetric-memory all-reduce kernel, "
                         "or whichever was measured faster per token count at start-up (no NCCL in any of them)")
    ap.add_argument("--sp", action="store_true", help="sequence-parallel dataflow: all-gather -> GEMM and GEMM -> reduce-scatter kernels")
    ap.add_argument("--secondary", default="auto", choices=["auto", "on", "off"],
                    help="also measure the 70B fp8 and DeepSeek configurations (auto: when the headline model runs on 8 GPUs)")
    ap.add_argument("--whole-batch", action="store_true", help="time one window that runs the whole request set to completion (the mode of the fixed-batch configurations)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: marks the result invalid")
    ap.add_argument("--profile", default=None, help="debug only: write a per-kernel table of a few steps to this file")
    ap.add_argument("--tune-report", default=None, help="debug only: append the start-up tuning tables (GEMM configurations, all-reduce forms) to this file")
    return ap.parse_args()


def reference_arm(args) -> None:
    # The reference tree is the Mojo standard library, docs and examples: it has no setup.py / pyproject.toml,
    # no engine, no model code and no prebuilt payload, so there is nothing to install or run.
    print(json.dumps({
        "impl": "reference",
        "unavailable": "pip install of the reference fails: directory is not installable (neither setup.py nor "
                       "pyproject.toml); the tree holds only the Mojo stdlib/docs/examples, no MAX engine or LLM code",
    }))


class Run:
    """One model + engine + request stream on the current process group."""

    def __init__(self, args, model_name: str, info):
        import torch

        from mojo_b200.engine import EngineConfig, LLMEngine
        from mojo_b200.models import build_model, get_config
        from mojo_b200.utils.workload import fixed_batch, poisson_trace

        self.args, self.info, self.model_name = args, info, model_name
        rank, world, device = info.rank, info.world_size, info.device
        mcfg = get_config(model_name)
        self.debug_invalid = False
        if args.layers is not None:
            mcfg.num_layers = args.layers
            self.debug_invalid = True
        # Named configurations: the Llama models are tensor-parallel over all GPUs; the DeepSeek MoE model runs
        # data-parallel attention (every rank serves its own requests from its own KV cache) with the routed experts
        # spread over all GPUs (expert parallelism) and every rank in lock-step through the MoE layers.
        self.ep_mode = ep_mode = mcfg.architecture == "deepseek_v2"
        comm = ep = None
        self.comm_name = "none"
        if ep_mode:
            from mojo_b200.parallel.ep import EPComm

            ep = EPComm(info, mcfg.n_routed_experts, mcfg.hidden_size, mcfg.moe_intermediate_size, mcfg.num_experts_per_tok,
                        max_tokens=args.max_batched_tokens, timeout_s=30.0)
        elif world > 1:
            if args.comm == "fused" and args.impl == "mojo_b200":
                from mojo_b200.parallel.fused import FusedTPComm

                comm = FusedTPComm(info, max_tokens=args.max_batched_tokens, hidden=mcfg.hidden_size, max_k=mcfg.hidden_size)
                comm.ar_mode = args.ar_mode
                self.comm_name = "fused"
            else:
                from mojo_b200.parallel.tp import NcclTPComm

                comm = NcclTPComm(info)
                self.comm_name = "nccl"
        graphs = not args.no_graphs
        if args.impl == "torch-baseline":
            from mojo_b200.ops import torch_baseline

            torch_baseline.enable()
            graphs = False
        self.fixed = fixed = FIXED.get(model_name)
        max_model_len = 2048 + 512 + 128 if fixed is None else fixed[1] + fixed[2] + 128
        self.max_num_seqs = args.max_num_seqs if fixed is None else max(1, fixed[0] // (world if ep_mode else 1))
        self.n_requests = args.requests if fixed is None else fixed[0]
        self.ecfg = EngineConfig(model=mcfg, device=str(device), dtype=torch.bfloat16, page_size=args.page_size,
                                 max_num_seqs=self.max_num_seqs, max_num_batched_tokens=args.max_batched_tokens,
                                 max_model_len=max_model_len, seed=0, use_cuda_graphs=graphs, tp_size=1 if ep_mode else world,
                                 ep_size=world if ep_mode else 1, lockstep=ep_mode and world > 1,
                                 mixed_step_graphs=not args.no_mixed_graphs, capture_mixed_graphs_at_start=True,
                                 async_scheduling=(args.impl == "mojo_b200" and not args.no_async and not ep_mode),
                                 autotune=(args.impl == "mojo_b200" and not args.no_autotune and device.type == "cuda"))
        self.model = build_model(mcfg, device, torch.bfloat16, comm=comm, ep=ep).init_random(0)
        if args.sp and world > 1 and self.comm_name == "fused":
            self.model.sequence_parallel = True
        self.engine = LLMEngine(self.ecfg, model=self.model, comm=comm)
        self.mcfg, self.comm, self.ep = mcfg, comm, ep
        if fixed is None:
            self.trace = poisson_trace(self.n_requests, args.rate, (128, 2048), (64, 512), mcfg.vocab_size, seed=1)
        else:
            self.trace = fixed_batch(fixed[0], fixed[1], fixed[2], mcfg.vocab_size, seed=1)   # one batch, all present at t = 0
        if ep_mode and world > 1:
            self.trace = self.trace[rank::world]      # data-parallel attention: every rank serves its own share of the requests
        self.state = {"next": 0, "t0": None}
        self.finite = fixed is not None     # whole-batch runs of the Poisson trace also end with its last request
        self.ev_pairs: list = []
        report = getattr(self.engine, "tune_report", None)
        if args.tune_report and rank == 0 and report:
            with open(args.tune_report, "a") as f:
                for key, table in report.items():
                    f.write(json.dumps({"model": model_name, "key": [str(k) for k in key], "table": {str(m): v for m, v in table.items()}}, default=str) + "\n")

    # ---- request stream ----
    def feed(self) -> None:
        """Admit every request whose arrival time has passed (rank 0's clock decides for all ranks)."""
        from mojo_b200.engine import SamplingParams
        from mojo_b200.parallel import host_broadcast_object

        args, trace, state, world = self.args, self.trace, self.state, self.info.world_size
        now = time.perf_counter() - state["t0"]
        n = 0
        while True:
            i = state["next"] + n
            if self.finite and i >= len(trace):
                break           # fixed-batch configurations are one batch, present at t = 0: nothing arrives later
            req = trace[i % len(trace)]
            arrival = req.arrival + (i // len(trace)) * (trace[-1].arrival + 1.0 / max(args.rate, 1e-9))
            if arrival > now:
                break
            n += 1
            if n > 4096:
                break
        n = host_broadcast_object(n, self.info) if world > 1 else n
        for _ in range(n):
            i = state["next"]
            req = trace[i % len(trace)]
            self.engine.add_request(req.prompt, SamplingParams(max_tokens=req.max_tokens, ignore_eos=True), arrival=time.perf_counter())
            state["next"] += 1

    def one_step(self, timed: bool):
        import torch

        engine = self.engine
        self.feed()
        lock = self.ep_mode and self.info.world_size > 1
        if not engine.has_unfinished() and not lock:
            # idle gap in the arrival process: wait for the next arrival without burning a step
            # (expert-parallel ranks never skip: a rank without work still joins every MoE layer of the step)
            time.sleep(0.0005)
            return None
        if timed and self.ep_mode:
            # a rank may have an idle step (it only serves peers' tokens in the MoE layers): bracket the whole step
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            engine.runner.step_events = None
            s.record()
            outs = engine.step()
            e.record()
            self.ev_pairs.append((s, e))
            return outs
        if timed:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            engine.runner.step_events = (s, e)
        else:
            engine.runner.step_events = None
        before = engine.runner.steps_launched
        outs = engine.step()
        if timed and engine.runner.steps_launched > before:      # a pipelined call that only collected launched nothing
            self.ev_pairs.append(engine.runner.step_events)
        return outs

    def ramp_and_warm(self) -> int:
        """Steady-state runs: step until the first request has completed, then the W warm-up steps. Returns the ramp length."""
        import torch

        from mojo_b200 import ops

        args, info = self.args, self.info
        lock = self.ep_mode and info.world_size > 1
        ramp = finished = 0
        while ramp < args.max_ramp_steps and finished == 0:
            outs = self.one_step(False)
            if outs is None:
                continue
            ramp += 1
            finished += sum(o.finished for o in outs)
            if ramp % 8 == 1:
                ops.check_status(info.device)   # a kernel that gave up (bounded wait) ends the run here instead of after every step
            if lock:
                # ranks serve different requests: agree on when the ramp ends so that all take the same number of steps
                flag = torch.tensor([finished], dtype=torch.int64)
                torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX, group=info.host_group)
                finished = int(flag[0])
        w = 0
        while w < args.warmup:
            if self.one_step(False) is not None:
                w += 1
        self.sync()
        ops.check_status(info.device)
        return ramp

    def abandoned(self) -> bool:
        """True on every rank once rank 0's deadline for the secondary configurations has passed (rank 0 decides, the
        others hear it over the host group, so that all ranks stop after the same step)."""
        import torch

        if self.info.world_size == 1:
            return ABANDON.is_set()
        flag = torch.tensor([1 if ABANDON.is_set() else 0], dtype=torch.int64)
        torch.distributed.broadcast(flag, src=0, group=self.info.host_group)
        return bool(flag[0])

    def sync(self) -> None:
        import torch

        torch.cuda.synchronize()
        if self.info.world_size > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize()

    def window(self, steps: int | None) -> dict:
        """Time `steps` engine steps (None: until every request of the fixed batch has finished, on every rank)."""
        import torch

        from mojo_b200 import ops

        engine, info, world = self.engine, self.info, self.info.world_size
        lock = self.ep_mode and world > 1
        ops.reset_launch_count()
        engine.runner.graph_launches = 0
        engine.runner.graph_kernel_launches = 0
        self.ev_pairs = []
        tokens = h2d = d2h = prefill_tokens = k = 0
        t_begin = time.perf_counter()
        if steps is None:
            self.feed()      # the whole batch is present at t = 0
        while True:
            if steps is not None and k >= steps:
                break
            if steps is None and not (engine._any_rank_busy() if lock else (engine.has_unfinished() or self.state["next"] < len(self.trace))):
                break
            outs = self.one_step(True)
            if outs is None:
                continue
            k += 1
            if steps is None and k % 32 == 0 and self.abandoned():
                # every rank leaves at the same step, with nothing of the next one launched
                engine.discard_inflight()
                self.sync()
                raise TimeoutError(f"abandoned after {k} steps: the time allowed for the secondary configurations ran out")
            tokens += len(outs)
            h2d += engine.runner.h2d_bytes
            d2h += engine.runner.d2h_bytes
            prefill_tokens += engine.runner.last_num_tokens - len(outs)
        self.sync()
        t_wall = time.perf_counter() - t_begin
        launches = ops.reset_launch_count() + engine.runner.graph_kernel_launches
        replays = engine.runner.graph_launches
        ops.check_status(info.device)
        dev_ms = sum(s.elapsed_time(e) for s, e in self.ev_pairs if s is not None)
        times = torch.tensor([dev_ms, t_wall * 1e3, float(k)], dtype=torch.float64, device=info.device)
        if world > 1:
            torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
        dev_ms, wall_ms, k = float(times[0]), float(times[1]), int(times[2])
        if lock:
            # data-parallel ranks produce different tokens: the job's output is their sum
            counts = torch.tensor([tokens, prefill_tokens, h2d, d2h, launches], dtype=torch.float64, device=info.device)
            torch.distributed.all_reduce(counts)
            tokens, prefill_tokens, h2d, d2h, launches = (int(c) for c in counts.tolist())
        return {"tokens": tokens, "prefill_tokens": prefill_tokens, "dev_ms": dev_ms, "wall_ms": wall_ms, "steps": k, "h2d": h2d, "d2h": d2h,
                "launches": launches, "graph_replays": replays, "t_begin": t_begin, "t_end": t_begin + t_wall}

    def latencies(self, t_begin: float, t_end: float) -> dict:
        """p50 time-to-first-token of the requests whose first token was produced inside [t_begin, t_end] (from their
        arrival, which under a saturating arrival rate lies before the window: the figure is mostly queueing), and p50
        inter-token latency of the token pairs produced there (host clock)."""
        import numpy as np

        ttft, itl = [], []
        for st in self.engine.requests.values():
            tt = st.token_times
            if not tt:
                continue
            if st.first_token_time is not None and t_begin <= st.first_token_time <= t_end:
                ttft.append(st.first_token_time - st.arrival)
            itl.extend(b - a for a, b in zip(tt[:-1], tt[1:]) if a >= t_begin and b <= t_end)
        return {"ttft_p50_ms": round(1e3 * float(np.median(ttft)), 3) if ttft else None, "ttft_requests": len(ttft),
                "itl_p50_ms": round(1e3 * float(np.median(itl)), 3) if itl else None, "itl_samples": len(itl)}

    def config(self, ramp, mode: str) -> dict:
        args, world, fixed = self.args, self.info.world_size, self.fixed
        coll = getattr(self.comm, "_coll", None)
        return {
            "model": self.model_name, "global_batch": self.max_num_seqs * (world if self.ep_mode else 1),
            "seq_len": "prompt U[128,2048] + output U[64,512]" if fixed is None else f"prompt {fixed[1]} + output {fixed[2]}",
            "parallelism": (f"dp{world}-attention + ep{world}-experts" if self.ep_mode else f"tp{world}"), "requests": self.n_requests,
            "poisson_rate_per_s": args.rate if fixed is None else None, "max_num_batched_tokens": args.max_batched_tokens, "page_size": args.page_size,
            "ramp_steps": ramp, "timed_region": mode,
            "l2": "inputs larger than L2: every step streams this rank's full weight set (GBs) through the 126 MB L2",
            "pipelined_stepping": bool(self.ecfg.async_scheduling and not self.ecfg.lockstep),
            "cuda_graphs": bool(self.ecfg.use_cuda_graphs), "mixed_step_graphs": bool(self.engine.runner.use_mixed_graphs),
            "gemm_autotune": bool(self.ecfg.autotune), "comm": self.comm_name if world > 1 else "none",
            "all_reduce_form": (args.ar_mode if world > 1 and self.comm_name == "fused" and not self.ep_mode else None),
            "in_switch_reduction": bool(getattr(self.comm, "nvls", False) and getattr(coll, "mc_ptr", 0)),
            "sequence_parallel": bool(getattr(self.model, "sequence_parallel", False)),
        }

    def close(self) -> None:
        """Drop the engine, the model and its symmetric regions so that the next configuration has the memory."""
        import torch

        self.sync()
        if self.engine is not None:
            self.engine.runner.graphs.clear()
            self.engine.runner.mixed_graphs.clear()
        self.engine = self.model = self.comm = self.ep = None
        gc.collect()
        torch.cuda.empty_cache()
        self.sync()


def line_from(run: Run, args, windows: list, clocks: dict, ramp, mode: str) -> dict:
    """The JSON record of one configuration: the median window is `value`; min / max go to `spread`."""
    world, mcfg = run.info.world_size, run.mcfg
    rates = [w["tokens"] / (w["dev_ms"] / 1e3) for w in windows]
    order = sorted(range(len(windows)), key=lambda i: rates[i])
    mid = windows[order[len(order) // 2]]
    value = mid["tokens"] / (mid["dev_ms"] / 1e3)
    e2e_rates = [w["tokens"] / (w["wall_ms"] / 1e3) for w in windows]
    lat = run.latencies(windows[0]["t_begin"], windows[-1]["t_end"])
    cfg = run.config(ramp, mode)
    cfg.update({"prefill_tokens_in_timed_region": mid["prefill_tokens"], "output_tokens_in_timed_region": mid["tokens"], "graph_replays": mid["graph_replays"]})
    line = {
        "metric": f"output tok/s/box, {METRIC_NAMES.get(run.model_name, run.model_name)}, continuous batching (paged KV, page {args.page_size})",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": mid["steps"], "warmup": args.warmup,
        "ms_per_step": round(mid["dev_ms"] / max(mid["steps"], 1), 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8 block-scaled weights and GEMMs, bf16 activations" if mcfg.quantization == "fp8_block" else "bf16",
        "data": "synthetic: uniform-random token ids, random-init N(0,0.02) weights of the named architecture",
        "impl": args.impl, "config": cfg,
        "spread": {"repeats": len(windows), "min": round(min(rates), 2), "max": round(max(rates), 2), "values": [round(r, 2) for r in rates]},
        "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons", "power_w_max")},
        "e2e": {"value": round(statistics.median(e2e_rates), 2), "unit": "tok/s", "h2d_bytes_per_step": mid["h2d"] // max(mid["steps"], 1),
                "d2h_bytes_per_step": mid["d2h"] // max(mid["steps"], 1), "ms_per_step": round(mid["wall_ms"] / max(mid["steps"], 1), 4),
                "min": round(min(e2e_rates), 2), "max": round(max(e2e_rates), 2)},
        "gpu_launches": mid["launches"],
        "ttft_p50_ms": lat["ttft_p50_ms"], "itl_p50_ms": lat["itl_p50_ms"], "latency_samples": {"ttft_requests": lat["ttft_requests"], "itl": lat["itl_samples"]},
    }
    if run.debug_invalid:
        line["invalid"] = "--layers override: not the named model"
    return line


def measure(args, model_name: str, info, whole_batch: bool) -> dict:
    """Build the configuration, run it, return its record (rank 0's is printed)."""
    from mojo_b200.utils.clocks import ClockSampler

    run = Run(args, model_name, info)
    try:
        run.state["t0"] = time.perf_counter()
        if whole_batch:
            # graphs and GEMM tables exist from engine start; the window starts with the first prefill chunk
            run.finite = True
            run.sync()
            with ClockSampler(info.local_rank) as clocks:
                windows = [run.window(None)]
            return line_from(run, args, windows, clocks.summary(), None, "whole batch: first prefill chunk to last token")
        ramp = run.ramp_and_warm()
        if args.profile:
            # diagnostic only (numbers taken under a profiler are never reported as results)
            import torch
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                n = 0
                while n < 6:
                    if run.one_step(False) is not None:
                        n += 1
                torch.cuda.synchronize()
            if info.rank == 0:
                with open(args.profile, "w") as f:
                    f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=90))
        repeats = max(1, args.repeats)
        with ClockSampler(info.local_rank) as clocks:
            windows = [run.window(args.steps) for _ in range(repeats)]
        return line_from(run, args, windows, clocks.summary(), ramp, f"steady state: {repeats} windows of {args.steps} steps after ramp and warm-up")
    finally:
        run.close()


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.impl == "vllm-yardstick":
        from mojo_b200.utils import yardstick

        yardstick.main(args)
        return

    import torch

    from mojo_b200.parallel import init_distributed

    info = init_distributed("cuda")
    if info.world_size != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={info.world_size}; launch with torch.distributed.run")
    if args.impl == "torch-baseline":
        args.comm = "nccl"
    world = info.world_size
    line = measure(args, args.model, info, whole_batch=args.whole_batch or args.model in FIXED)
    want_secondary = args.secondary == "on" or (args.secondary == "auto" and world == 8 and args.model == "llama-3.1-8b"
                                                and args.impl == "mojo_b200" and args.layers is None and not args.profile)
    if want_secondary:
        line["secondary"] = {}

        def give_up():
            # a secondary configuration that hangs must not cost the headline: every rank leaves, rank 0 prints what it has
            if info.rank == 0:
                line["secondary"].setdefault("error", f"not finished within {SECONDARY_DEADLINE_S + SECONDARY_GRACE_S:.0f} s")
                print(json.dumps(line), flush=True)
            os._exit(0)

        soft = threading.Timer(SECONDARY_DEADLINE_S, ABANDON.set)       # stop between steps, on all ranks together
        timer = threading.Timer(SECONDARY_DEADLINE_S + SECONDARY_GRACE_S, give_up)
        for t in (soft, timer):
            t.daemon = True
            t.start()
        for name in ("llama-3.3-70b-fp8", "deepseek-v2-lite"):
            t0 = time.perf_counter()
            try:
                rec = measure(args, name, info, whole_batch=True)
                rec["wall_s_including_setup"] = round(time.perf_counter() - t0, 1)
            except Exception as e:  # noqa: BLE001 - a secondary configuration must not take the headline down with it
                rec = {"error": repr(e)[:400]}
            line["secondary"][name] = rec
            # every rank agrees on whether to go on (after a failure on any rank the process group may be out of step)
            ok = torch.tensor([0 if "error" in rec else 1], dtype=torch.int64)
            if world > 1:
                torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN, group=info.host_group)
            if int(ok[0]) == 0:
                break
        soft.cancel()
        timer.cancel()
    if info.rank == 0:
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    if world > 1:
        # NCCL collectives captured in CUDA graphs make process-group teardown unreliable; leave together instead
        torch.distributed.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
