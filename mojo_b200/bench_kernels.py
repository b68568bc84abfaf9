"""Micro-benchmarks of the library's building blocks: `python -m mojo_b200.bench_kernels [--suite host|gpu|all]`.

The counterpart of the reference's `stdlib/benchmarks/` tree (e.g. stdlib/benchmarks/math/bench_math.mojo:113-131,
collections/bench_dict.mojo, hashlib/bench_hash.mojo: one function per primitive, run serially by
stdlib/scripts/run-benchmarks.sh:17-35), on the harness of `mojo_b200.utils.bench`:

* suite `host`: the C++ runtime pieces every serving step goes through (page hash, KV manager allocate / free /
  prefix lookup, one scheduler iteration with 256 running sequences, the CPU-rank collective simulator). Runs anywhere.
* suite `gpu`: every single-kernel case of `mojo_b200.utils.kernel_driver` (GEMMs, attention, MLA, RMSNorm, sampling)
  with CUDA-event timing; inputs are larger than L2 or rotate through copies that are.

`--test` runs every benchmark once (a smoke test of the suite); `--out file.json|file.csv` also writes the report.
"""
from __future__ import annotations

import argparse

import numpy as np

from . import _ext
from .utils.bench import Bench, BenchConfig, BenchId, Mode


def host_suite(b: Bench) -> None:
    C = _ext.require()
    rng = np.random.default_rng(0)
    page = rng.integers(0, 128256, size=128, dtype=np.int32)
    b.bench_function(BenchId("hash_page", "128 tokens"), lambda: C.hash_page(0x9E3779B97F4A7C15, page), throughput_elems=128)

    prompt = rng.integers(0, 128256, size=2048, dtype=np.int32)

    def kv_cycle():
        kv = kv_cycle.kv
        for i in range(64):
            kv.add_sequence(i, prompt)
            kv.reserve(i, 2048)
        for i in range(64):
            kv.free_sequence(i)

    kv_cycle.kv = C.KVCacheManager(4096, 128, False)
    b.bench_function(BenchId("kv_manager", "64 x (add + reserve 16 pages + free)"), kv_cycle, throughput_elems=64)

    def kv_prefix():
        kv = kv_prefix.kv
        for i in range(1, 33):
            kv.add_sequence(i, prompt)       # 16 full pages found in the prefix cache
            kv.free_sequence(i)

    kv_prefix.kv = C.KVCacheManager(4096, 128, True)
    kv_prefix.kv.add_sequence(0, prompt)
    kv_prefix.kv.reserve(0, 2048)
    kv_prefix.kv.commit(0, prompt, 2048)
    b.bench_function(BenchId("kv_manager", "32 x prefix lookup of 16 pages"), kv_prefix, throughput_elems=32)

    def make_sched():
        kv = C.KVCacheManager(8192, 128, False)
        sc = C.SchedulerConfig()
        sc.max_num_seqs, sc.max_num_batched_tokens, sc.max_model_len = 256, 4096, 4096
        s = C.Scheduler(sc, kv)
        for i in range(256):
            s.add_request(i, prompt[:256], 1 << 20, 0.0)
        # prefill everything, so that the timed iterations are steady-state decode steps of 256 sequences
        while True:
            batch = s.step()
            for rid in batch.sample_seq_ids:
                s.append_token(int(rid), 1)
            if batch.num_prefill == 0:
                break
        return kv, s

    state = {}

    def sched_step():
        if "s" not in state or state["n"] > 1500:
            state["kv"], state["s"] = make_sched()
            state["n"] = 0
        batch = state["s"].step()
        for rid in batch.sample_seq_ids:
            state["s"].append_token(int(rid), 1)
        state["n"] += 1

    b.bench_function(BenchId("scheduler", "decode step, 256 sequences"), sched_step, throughput_elems=256)
    b.bench_function(BenchId("symm_sim", "one-shot all-reduce, 4 ranks x 4096 floats x 8 steps"),
                     lambda: C.symm_sim_run(4, 4096, 8, "one_shot", "", 2000), throughput_elems=8)


def gpu_suite(b: Bench, cases=None) -> None:
    from .utils import kernel_driver

    for name in cases or kernel_driver.CASES:
        fn, flops, nbytes = kernel_driver._case(name)
        b.bench_function(BenchId(name), fn, bytes_per_iter=nbytes or None, flops_per_iter=flops or None)


def main(argv=None) -> Bench:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--suite", choices=["host", "gpu", "all"], default="all")
    ap.add_argument("--cases", default=None, help="comma-separated kernel_driver cases for the gpu suite")
    ap.add_argument("--test", action="store_true", help="run every benchmark once")
    ap.add_argument("--min-runtime", type=float, default=0.3)
    ap.add_argument("--max-runtime", type=float, default=1.5)
    ap.add_argument("--repetitions", type=int, default=1)
    ap.add_argument("--json", action="store_true", help="one JSON object per line instead of the CSV table")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    import torch

    have_gpu = torch.cuda.is_available()
    cfg = BenchConfig(out_file=a.out, min_runtime_secs=a.min_runtime, max_runtime_secs=a.max_runtime, num_repetitions=a.repetitions,
                      tabular_view=not a.json)
    mode = Mode.Test if a.test else Mode.Benchmark
    if a.suite in ("host", "all"):
        hb = Bench(BenchConfig(**{**cfg.__dict__, "device": "cpu", "out_file": None}), mode)
        host_suite(hb)
    else:
        hb = None
    gb = None
    if a.suite in ("gpu", "all") and (have_gpu or a.suite == "gpu"):
        if not have_gpu:
            raise SystemExit("the gpu suite needs a CUDA device")
        gb = Bench(BenchConfig(**{**cfg.__dict__, "device": "cuda", "out_file": None}), mode)
        gpu_suite(gb, a.cases.split(",") if a.cases else None)
    out = Bench(cfg, mode)
    for part in (hb, gb):
        if part is not None:
            out.info_vec.extend(part.info_vec)
    out.dump_report()
    return out


if __name__ == "__main__":
    main()
