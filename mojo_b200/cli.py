"""Command line: `python -m mojo_b200.cli {serve,generate,bench,bench-ops,deviceinfo}`.

  serve       OpenAI-compatible HTTP server
  generate    run prompts (token ids, or text with --tokenizer) to completion and print the outputs
  bench       synthetic serving benchmark (Poisson or fixed-batch trace) with TTFT / ITL / tok/s; JSON (+CSV) out
  bench-ops   fused tensor-parallel op sweep (run under torch.distributed.run)
  deviceinfo  capability probe of the visible GPUs
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _cmd_serve(a) -> None:
    import uvicorn

    from .pipelines import LLM, PipelineConfig
    from .serve import build_app

    llm = LLM(PipelineConfig.from_args(a))
    comm, ep = getattr(llm, "comm", None), getattr(llm, "ep", None)
    info = None
    if comm is not None and getattr(comm, "world_size", 1) > 1:
        info, data_parallel = comm.info, False      # tensor parallelism: every rank admits every request
    elif ep is not None and getattr(ep, "world_size", 1) > 1:
        info, data_parallel = ep.info, True         # data-parallel attention + expert parallelism: requests are routed to an owner rank
    elif getattr(llm, "dist_info", None) is not None and llm.dist_info.world_size > 1:
        info, data_parallel = llm.dist_info, True   # whole-model replicas behind one endpoint
    if info is not None:
        # rank 0 serves HTTP and broadcasts its commands once per engine iteration, the other ranks follow
        from .serve.api_server import RankSync, follower_loop

        sync = RankSync(info, data_parallel=data_parallel)
        if not sync.leader:
            follower_loop(llm, sync)
            return
        app = build_app(llm, model_name=a.model, sync=sync)
        try:
            uvicorn.run(app, host=a.host, port=a.port, log_level="info")
        finally:
            app.state.engine.shutdown()
        return
    uvicorn.run(build_app(llm, model_name=a.model), host=a.host, port=a.port, log_level="info")


def _cmd_generate(a) -> None:
    from .pipelines import LLM, PipelineConfig, SamplingParams

    llm = LLM(PipelineConfig.from_args(a))
    prompts = []
    for p in a.prompt:
        prompts.append([int(t) for t in p.split(",")] if a.token_ids else p)
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, max_tokens=a.max_tokens)
    for o in llm.generate(prompts, sp):
        print(json.dumps({"request_id": o.request_id, "token_ids": o.token_ids, "text": o.text, "finish_reason": o.finish_reason}))


def _cmd_bench(a) -> None:
    import numpy as np
    import torch

    from .pipelines import LLM, PipelineConfig, SamplingParams
    from .utils.workload import fixed_batch, poisson_trace

    cfg = PipelineConfig.from_args(a)
    cfg.random_init = True
    llm = LLM(cfg)
    eng = llm.engine
    vocab = llm.model_config.vocab_size
    # keep prompt + output inside the engine's context limit (it is capped by the model's position range)
    room = eng.cfg.max_model_len - 1
    a.output_max = max(1, min(a.output_max, room // 2))
    a.output_min = min(a.output_min, a.output_max)
    a.prompt_max = max(1, min(a.prompt_max, room - a.output_max))
    a.prompt_min = min(a.prompt_min, a.prompt_max)
    if a.trace == "poisson":
        trace = poisson_trace(a.requests, a.rate, (a.prompt_min, a.prompt_max), (a.output_min, a.output_max), vocab, seed=a.seed)
    else:
        trace = fixed_batch(a.requests, a.prompt_max, a.output_max, vocab, seed=a.seed)
    t0 = time.perf_counter()
    nxt = 0
    while nxt < len(trace) or eng.has_unfinished():
        now = time.perf_counter() - t0
        while nxt < len(trace) and trace[nxt].arrival <= now:
            eng.add_request(trace[nxt].prompt, SamplingParams(max_tokens=trace[nxt].max_tokens, ignore_eos=True),
                            arrival=t0 + trace[nxt].arrival)
            nxt += 1
        if eng.has_unfinished():
            eng.step()
        else:
            time.sleep(0.0005)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    m = eng.metrics()
    m["wall_s"] = time.perf_counter() - t0
    m["config"] = json.loads(cfg.to_json())
    m["trace"] = {"kind": a.trace, "requests": a.requests, "rate": a.rate, "prompt": [a.prompt_min, a.prompt_max],
                  "output": [a.output_min, a.output_max]}
    print(json.dumps(m))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(m, f, indent=1)
    if a.csv:
        with open(a.csv, "w") as f:
            f.write("request,prompt_len,output_len,ttft_ms,mean_itl_ms\n")
            for st in eng.requests.values():
                if st.token_times:
                    itl = np.diff(st.token_times).mean() * 1e3 if len(st.token_times) > 1 else 0.0
                    f.write(f"{st.request_id},{st.prompt_len},{len(st.output_ids)},{(st.first_token_time - st.arrival) * 1e3:.3f},{itl:.3f}\n")


def _cmd_deviceinfo(a) -> None:
    from .examples.deviceinfo import main as info_main

    info_main()


def main(argv=None) -> None:
    from .pipelines import PipelineConfig

    ap = argparse.ArgumentParser(prog="mojo_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    PipelineConfig.add_cli_args(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.set_defaults(fn=_cmd_serve)
    g = sub.add_parser("generate")
    PipelineConfig.add_cli_args(g)
    g.add_argument("--prompt", action="append", required=True)
    g.add_argument("--token-ids", action="store_true", help="prompts are comma-separated token ids")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.set_defaults(fn=_cmd_generate)
    b = sub.add_parser("bench")
    PipelineConfig.add_cli_args(b)
    b.add_argument("--trace", choices=["poisson", "fixed"], default="poisson")
    b.add_argument("--requests", type=int, default=512)
    b.add_argument("--rate", type=float, default=64.0)
    b.add_argument("--prompt-min", type=int, default=128)
    b.add_argument("--prompt-max", type=int, default=2048)
    b.add_argument("--output-min", type=int, default=64)
    b.add_argument("--output-max", type=int, default=512)
    b.add_argument("--out", default=None)
    b.add_argument("--csv", default=None)
    b.set_defaults(fn=_cmd_bench)
    o = sub.add_parser("bench-ops", help="run as: python -m torch.distributed.run ... -m mojo_b200.bench_ops")
    o.set_defaults(fn=lambda a: print("launch with: python -m torch.distributed.run --nproc-per-node N -m mojo_b200.bench_ops"))
    sub.add_parser("bench-kernels", help="micro-benchmarks of kernels and host runtime; options as in python -m mojo_b200.bench_kernels --help")
    d = sub.add_parser("deviceinfo")
    d.set_defaults(fn=_cmd_deviceinfo)
    import sys

    args = list(sys.argv[1:] if argv is None else argv)
    if args and args[0] == "bench-kernels":      # its own option parser takes the rest of the line
        from . import bench_kernels

        bench_kernels.main(args[1:])
        return
    a = ap.parse_args(args)
    a.fn(a)


if __name__ == "__main__":
    main()
