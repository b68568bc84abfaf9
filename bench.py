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

Two numbers come out of the same K steps:
  value      output tokens / device time: CUDA events around each step's device work (model + sampler), summed,
             max over ranks
  e2e.value  output tokens / wall time of `LLMEngine.step()`: scheduler, pinned staging, the host->device copy
             of the step's metadata, the model, the sampler and the device->host read of the sampled ids
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


METRIC_NAMES = {"llama-3.1-8b": "Llama-3.1-8B bf16", "llama-3.3-70b-fp8": "Llama-3.3-70B fp8 block-scaled",
                "deepseek-v2-lite": "DeepSeek-V2-Lite bf16 (MLA + MoE)"}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=192)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="mojo_b200", choices=["mojo_b200", "reference", "torch-baseline"])
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
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--ar-mode", default="auto", choices=["auto", "fused", "split"],
                    help="row-parallel linear + all-reduce: the single fused kernel, GEMM -> symmetric-memory all-reduce kernel, "
                         "or whichever was measured faster per token count at start-up (no NCCL in any of them)")
    ap.add_argument("--sp", action="store_true", help="sequence-parallel dataflow: all-gather -> GEMM and GEMM -> reduce-scatter kernels")
    ap.add_argument("--layers", type=int, default=None, help="debug only: marks the result invalid")
    ap.add_argument("--profile", default=None, help="debug only: write a per-kernel table of a few steps to this file")
    return ap.parse_args()


def reference_arm(args) -> None:
    # The reference tree is the Mojo standard library, docs and examples: it has no setup.py / pyproject.toml,
    # no engine, no model code and no prebuilt payload, so there is nothing to install or run.
    print(json.dumps({
        "impl": "reference",
        "unavailable": "pip install of the reference fails: directory is not installable (neither setup.py nor "
                       "pyproject.toml); the tree holds only the Mojo stdlib/docs/examples, no MAX engine or LLM code",
    }))


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch

    from mojo_b200 import ops
    from mojo_b200.engine import EngineConfig, LLMEngine, SamplingParams
    from mojo_b200.models import build_model, get_config
    from mojo_b200.parallel import init_distributed, host_broadcast_object
    from mojo_b200.utils.clocks import ClockSampler
    from mojo_b200.utils.workload import poisson_trace

    info = init_distributed("cuda")
    if info.world_size != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={info.world_size}; launch with torch.distributed.run")
    rank, world, device = info.rank, info.world_size, info.device

    mcfg = get_config(args.model)
    debug_invalid = False
    if args.layers is not None:
        mcfg.num_layers = args.layers
        debug_invalid = True
    if args.impl == "torch-baseline":
        args.comm = "nccl"
    # Named configurations: the Llama models are tensor-parallel over all GPUs; the DeepSeek MoE model runs
    # data-parallel attention (every rank serves its own requests from its own KV cache) with the routed experts
    # spread over all GPUs (expert parallelism) and every rank in lock-step through the MoE layers.
    ep_mode = mcfg.architecture == "deepseek_v2"
    comm = None
    ep = None
    if ep_mode:
        from mojo_b200.parallel.ep import EPComm

        ep = EPComm(info, mcfg.n_routed_experts, mcfg.hidden_size, mcfg.moe_intermediate_size, mcfg.num_experts_per_tok,
                    max_tokens=args.max_batched_tokens, timeout_s=30.0)
    elif world > 1:
        if args.comm == "fused" and args.impl == "mojo_b200":
            from mojo_b200.parallel.fused import FusedTPComm

            comm = FusedTPComm(info, max_tokens=args.max_batched_tokens, hidden=mcfg.hidden_size, max_k=mcfg.hidden_size)
            comm.ar_mode = args.ar_mode
        else:
            from mojo_b200.parallel.tp import NcclTPComm

            comm = NcclTPComm(info)
    if args.impl == "torch-baseline":
        from mojo_b200.ops import torch_baseline

        torch_baseline.enable()
        args.no_graphs = True
        args.comm = "nccl"

    fixed = {"llama-3.3-70b-fp8": (256, 1024, 256), "deepseek-v2-lite": (512, 512, 256), "tiny-deepseek": (64, 64, 16)}.get(args.model)
    max_model_len = 2048 + 512 + 128 if fixed is None else fixed[1] + fixed[2] + 128
    if fixed is not None:
        args.max_num_seqs = max(1, fixed[0] // (world if ep_mode else 1))
        args.requests = fixed[0]
    ecfg = EngineConfig(model=mcfg, device=str(device), dtype=torch.bfloat16, page_size=args.page_size,
                        max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_batched_tokens,
                        max_model_len=max_model_len, seed=0, use_cuda_graphs=not args.no_graphs, tp_size=1 if ep_mode else world,
                        ep_size=world if ep_mode else 1, lockstep=ep_mode and world > 1,
                        mixed_step_graphs=not args.no_mixed_graphs, capture_mixed_graphs_at_start=True,
                        autotune=(args.impl == "mojo_b200" and not args.no_autotune and device.type == "cuda"))
    model = build_model(mcfg, device, torch.bfloat16, comm=comm, ep=ep).init_random(0)
    if args.sp and world > 1 and args.comm == "fused":
        model.sequence_parallel = True
    engine = LLMEngine(ecfg, model=model, comm=comm)

    if fixed is None:
        trace = poisson_trace(args.requests, args.rate, (128, 2048), (64, 512), mcfg.vocab_size, seed=1)
    else:
        from mojo_b200.utils.workload import fixed_batch

        trace = fixed_batch(fixed[0], fixed[1], fixed[2], mcfg.vocab_size, seed=1)   # one batch, all present at t = 0
    if ep_mode and world > 1:
        trace = trace[rank::world]      # data-parallel attention: every rank serves its own share of the requests
    state = {"next": 0, "epoch": 0, "t0": None, "offset": 0.0}

    def feed() -> None:
        """Admit every request whose arrival time has passed (rank 0's clock decides for all ranks)."""
        now = time.perf_counter() - state["t0"]
        n = 0
        while True:
            i = state["next"] + n
            if fixed is not None and i >= len(trace):
                break           # fixed-batch configurations are one batch, present at t = 0: nothing arrives later
            req = trace[i % len(trace)]
            arrival = req.arrival + (i // len(trace)) * (trace[-1].arrival + 1.0 / max(args.rate, 1e-9))
            if arrival > now:
                break
            n += 1
            if n > 4096:
                break
        n = host_broadcast_object(n, info) if world > 1 else n
        for _ in range(n):
            i = state["next"]
            req = trace[i % len(trace)]
            engine.add_request(req.prompt, SamplingParams(max_tokens=req.max_tokens, ignore_eos=True),
                               arrival=time.perf_counter())
            state["next"] += 1

    ev_pairs = []

    def one_step(timed: bool):
        feed()
        if not engine.has_unfinished() and not (ep_mode and world > 1):
            # idle gap in the arrival process: wait for the next arrival without burning a step
            # (expert-parallel ranks never skip: a rank without work still joins every MoE layer of the step)
            time.sleep(0.0005)
            return None
        if timed and ep_mode:
            # a rank may have an idle step (it only serves peers' tokens in the MoE layers): bracket the whole step
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            engine.runner.step_events = None
            s.record()
            outs = engine.step()
            e.record()
            ev_pairs.append((s, e))
            return outs
        if timed:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            engine.runner.step_events = (s, e)
        else:
            engine.runner.step_events = None
        outs = engine.step()
        if timed:
            ev_pairs.append(engine.runner.step_events)
        return outs

    state["t0"] = time.perf_counter()
    # ---- ramp: until the first request has completed (steady mix of decode + prefill) ----
    ramp = 0
    finished = 0
    while ramp < args.max_ramp_steps and finished == 0:
        outs = one_step(False)
        if outs is None:
            continue
        ramp += 1
        finished += sum(o.finished for o in outs)
        if ramp % 8 == 1:
            ops.check_status(device)   # a kernel that gave up (bounded wait) ends the run here instead of after every step
        if ep_mode and world > 1:
            # ranks serve different requests: agree on when the ramp ends so that all take the same number of steps
            flag = torch.tensor([finished], dtype=torch.int64)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX, group=info.host_group)
            finished = int(flag[0])
    # ---- warm-up ----
    w = 0
    while w < args.warmup:
        if one_step(False) is not None:
            w += 1
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
        torch.cuda.synchronize()
    ops.check_status(device)

    if args.profile:
        # diagnostic only (numbers taken under a profiler are never reported as results)
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            n = 0
            while n < 6:
                if one_step(False) is not None:
                    n += 1
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.profile, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=90))

    # ---- timed region: exactly K engine steps ----
    ops.reset_launch_count()
    engine.runner.graph_launches = 0
    engine.runner.graph_kernel_launches = 0
    tokens = 0
    h2d = d2h = 0
    prefill_tokens = 0
    with ClockSampler(info.local_rank) as clocks:
        t_start = time.perf_counter()
        k = 0
        while k < args.steps:
            outs = one_step(True)
            if outs is None:
                continue
            k += 1
            tokens += len(outs)
            h2d += engine.runner.h2d_bytes
            d2h += engine.runner.d2h_bytes
            prefill_tokens += engine.runner.last_num_tokens - len(outs)
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize()
        t_wall = time.perf_counter() - t_start
    launches = ops.reset_launch_count() + engine.runner.graph_kernel_launches
    ops.check_status(device)
    dev_ms = sum(s.elapsed_time(e) for s, e in ev_pairs if s is not None)
    times = torch.tensor([dev_ms, t_wall * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    dev_ms, wall_ms = float(times[0]), float(times[1])
    if ep_mode and world > 1:
        # data-parallel ranks produce different tokens: the job's output is their sum
        counts = torch.tensor([tokens, prefill_tokens, h2d, d2h, launches], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(counts)
        tokens, prefill_tokens, h2d, d2h, launches = (int(c) for c in counts.tolist())

    if rank == 0:
        m = engine.metrics()
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (wall_ms / 1e3)
        line = {
            "metric": f"output tok/s/box, {METRIC_NAMES.get(args.model, args.model)}, continuous batching (paged KV, page {args.page_size})",
            "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8 block-scaled weights and GEMMs, bf16 activations" if mcfg.quantization == "fp8_block" else "bf16",
            "data": "synthetic: uniform-random token ids, random-init N(0,0.02) weights of the named architecture",
            "impl": args.impl,
            "config": {
                "model": args.model, "global_batch": args.max_num_seqs * (world if ep_mode else 1),
                "seq_len": "prompt U[128,2048] + output U[64,512]" if fixed is None else f"prompt {fixed[1]} + output {fixed[2]}",
                "parallelism": (f"dp{world}-attention + ep{world}-experts" if ep_mode else f"tp{world}"), "requests": args.requests, "poisson_rate_per_s": args.rate,
                "max_num_batched_tokens": args.max_batched_tokens, "page_size": args.page_size, "ramp_steps": ramp,
                "l2": "inputs larger than L2: every step streams this rank's full weight set (GBs) through the 126 MB L2",
                "cuda_graphs": not args.no_graphs, "mixed_step_graphs": bool(engine.runner.use_mixed_graphs), "graph_replays": engine.runner.graph_launches, "gemm_autotune": bool(ecfg.autotune), "comm": args.comm if world > 1 else "none", "all_reduce_form": (args.ar_mode if world > 1 and args.comm == "fused" and not ep_mode else None), "sequence_parallel": bool(getattr(model, "sequence_parallel", False)),
                "prefill_tokens_in_timed_region": prefill_tokens, "output_tokens_in_timed_region": tokens,
            },
            "clocks": {k: clocks.summary().get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons", "power_w_max")},
            "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d // max(args.steps, 1),
                    "d2h_bytes_per_step": d2h // max(args.steps, 1), "ms_per_step": round(wall_ms / args.steps, 4)},
            "gpu_launches": launches,
            "ttft_p50_ms": m["ttft_p50_ms"], "itl_p50_ms": m["itl_p50_ms"],
        }
        if debug_invalid:
            line["invalid"] = "--layers override: not the named model"
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    if world > 1:
        # NCCL collectives captured in CUDA graphs make process-group teardown unreliable; leave together instead
        torch.distributed.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
