"""Tracing helpers, all off unless asked for.

`B2_NVTX=1`   NVTX ranges around each engine step and its phases (schedule / stage / forward / sample / readback), so
              a timeline tool shows them against the kernels.
`B2_TRACE=1`  per-phase host wall-clock accumulators (`summary()`), cheap enough to leave on during a bench.
`timeline()`  per-request records (arrival, first token, every token time) for TTFT / ITL analysis.
"""
from __future__ import annotations

import json
import os
import time
from collections import defaultdict
from contextlib import contextmanager

NVTX = os.environ.get("B2_NVTX", "0") == "1"
TRACE = os.environ.get("B2_TRACE", "0") == "1"
_acc: dict[str, list] = defaultdict(lambda: [0, 0.0])


@contextmanager
def span(name: str):
    """A named phase: NVTX range and/or wall-clock accumulation, nothing when both switches are off."""
    if not (NVTX or TRACE):
        yield
        return
    if NVTX:
        import torch

        torch.cuda.nvtx.range_push(name)
    t0 = time.perf_counter()
    try:
        yield
    finally:
        if TRACE:
            a = _acc[name]
            a[0] += 1
            a[1] += time.perf_counter() - t0
        if NVTX:
            import torch

            torch.cuda.nvtx.range_pop()


def summary() -> dict:
    """{phase: {"calls": n, "total_ms": t, "mean_us": m}} since the last `reset()`."""
    return {k: {"calls": n, "total_ms": round(t * 1e3, 3), "mean_us": round(t / n * 1e6, 2) if n else 0.0} for k, (n, t) in _acc.items()}


def reset() -> None:
    _acc.clear()


def timeline(engine) -> list[dict]:
    """One record per request of `engine`: arrival, first-token and token times relative to the first arrival."""
    reqs = list(engine.requests.values())
    if not reqs:
        return []
    t0 = min(r.arrival for r in reqs)
    out = []
    for r in reqs:
        out.append({
            "request_id": r.request_id, "prompt_len": r.prompt_len, "output_len": len(r.output_ids),
            "arrival_s": round(r.arrival - t0, 6),
            "ttft_s": None if r.first_token_time is None else round(r.first_token_time - r.arrival, 6),
            "token_times_s": [round(t - t0, 6) for t in r.token_times],
            "finish_reason": r.finish_reason,
        })
    return out


def dump_timeline(engine, path: str) -> None:
    with open(path, "w") as f:
        json.dump(timeline(engine), f)
