"""Benchmark harness: run a function until a time budget is met, report per-iteration time and throughput.

The shape follows the reference's `benchmark` package as far as its public description goes
(stdlib/docs/bencher/BenchConfig.md:16-33: `out_file`, `min_runtime_secs`, `max_runtime_secs`, `min_warmuptime_secs`,
`max_batch_size`, `max_iters`, `num_repetitions`, `tabular_view`; Bench.md: `bench_function`, `bench_with_input`,
`dump_report`; Mode.md: benchmark mode and a test mode that runs everything once), re-thought for a GPU:

* device work is timed with CUDA events on the launching stream, one event pair around a batch of launches, never by
  wall clock; host-only functions (the scheduler, the KV manager) fall back to `time.perf_counter_ns`;
* `flush_l2=True` writes a buffer larger than the 126 MB L2 before every timed launch and then times launches one by
  one, so that every launch sees cold caches (the reference's `flush_denormals` has no meaning here and is absent);
* throughput is reported in elements, bytes and floating-point operations per second when the caller states them.

Typical use:

    b = Bench(BenchConfig(min_runtime_secs=0.2, max_runtime_secs=1.0))
    b.bench_function(BenchId("rmsnorm", "65536x4096"), lambda: ops.rms_norm(x, w, 1e-5), bytes_per_iter=x.numel() * 4)
    b.dump_report()
"""
from __future__ import annotations

import csv
import enum
import io
import json
import math
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

try:  # the harness itself runs without torch (host-only benchmarks)
    import torch
except Exception:  # noqa: BLE001
    torch = None

L2_FLUSH_BYTES = 256 << 20


class Mode(enum.Enum):
    Benchmark = 0
    Test = 1          # run every benchmark exactly once: a smoke test of the benchmark suite itself


@dataclass
class BenchConfig:
    out_file: str | Path | None = None      # write the report here as well (.json -> JSON, anything else -> CSV)
    min_runtime_secs: float = 0.5           # keep measuring until this much time has been measured ...
    max_runtime_secs: float = 2.0           # ... but never beyond this
    min_warmuptime_secs: float = 0.1        # untimed warm-up before the first measurement (at least 3 calls)
    max_batch_size: int = 0                 # launches per time measurement (0: sized so that a batch takes about 2 ms)
    max_iters: int = 1_000_000
    num_repetitions: int = 1                # independent repetitions; the report keeps all and summarises
    flush_l2: bool = False
    show_progress: bool = False
    tabular_view: bool = True               # CSV table on stdout (False: one JSON object per line)
    device: str | None = None               # "cuda", "cpu" or None (CUDA when available)


@dataclass(frozen=True)
class BenchId:
    func_name: str
    input_id: str | None = None

    def __str__(self) -> str:
        return self.func_name if self.input_id is None else f"{self.func_name}/{self.input_id}"


@dataclass
class BenchmarkInfo:
    name: str
    iters: int
    mean_us: float
    min_us: float
    max_us: float
    stdev_us: float
    repetitions: int
    elems_per_s: float | None = None
    gbytes_per_s: float | None = None
    tflops: float | None = None
    samples_us: list = field(default_factory=list, repr=False)


class Bencher:
    """Handed to a benchmark body that wants to control what is timed: `iter(fn)` times calls of `fn`,
    `iter_custom(fn)` lets `fn(n)` run n iterations itself and return the elapsed nanoseconds."""

    def __init__(self, bench: "Bench"):
        self._bench = bench
        self.samples_us: list[float] = []
        self.iters = 0

    def iter(self, fn) -> None:
        self.samples_us, self.iters = self._bench._measure(fn)

    def iter_custom(self, fn) -> None:
        cfg, mode = self._bench.config, self._bench.mode
        if mode is Mode.Test:
            self.samples_us, self.iters = [fn(1) / 1e3], 1
            return
        fn(3)
        n, total_ns, samples, iters = 1, 0.0, [], 0
        while total_ns < cfg.min_runtime_secs * 1e9 and total_ns < cfg.max_runtime_secs * 1e9 and iters < cfg.max_iters:
            ns = float(fn(n))
            samples.append(ns / 1e3 / n)
            total_ns += ns
            iters += n
            if ns < 2e6 and (cfg.max_batch_size == 0 or n < cfg.max_batch_size):
                n *= 2
        self.samples_us, self.iters = samples, iters


class Bench:
    def __init__(self, config: BenchConfig | None = None, mode: Mode = Mode.Benchmark):
        self.config = config or BenchConfig()
        self.mode = mode
        self.info_vec: list[BenchmarkInfo] = []
        dev = self.config.device
        if dev is None:
            dev = "cuda" if (torch is not None and torch.cuda.is_available()) else "cpu"
        self.cuda = dev.startswith("cuda")
        self._flush_buf = None

    # ---- timing primitives -------------------------------------------------------------------------------------
    def _sync(self) -> None:
        if self.cuda:
            torch.cuda.synchronize()

    def _time_batch_us(self, fn, n: int) -> float:
        """Elapsed microseconds of n back-to-back calls (device time on CUDA)."""
        if self.cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(n):
                fn()
            e.record()
            e.synchronize()
            return s.elapsed_time(e) * 1e3
        t0 = time.perf_counter_ns()
        for _ in range(n):
            fn()
        return (time.perf_counter_ns() - t0) / 1e3

    def _flush(self) -> None:
        if not self.cuda:
            return
        if self._flush_buf is None:
            self._flush_buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
        self._flush_buf.zero_()

    def _measure(self, fn) -> tuple[list[float], int]:
        cfg = self.config
        if self.mode is Mode.Test:
            us = self._time_batch_us(fn, 1)
            self._sync()
            return [us], 1
        # warm-up: at least three calls, at least min_warmuptime_secs
        t0 = time.perf_counter()
        calls = 0
        while calls < 3 or time.perf_counter() - t0 < cfg.min_warmuptime_secs:
            fn()
            calls += 1
            if calls % 8 == 0:
                self._sync()
        self._sync()
        per_call_us = max(self._time_batch_us(fn, 3) / 3, 1e-3)
        if cfg.flush_l2:
            batch = 1
        elif cfg.max_batch_size > 0:
            batch = cfg.max_batch_size
        else:
            batch = max(1, min(1024, int(2000.0 / per_call_us)))
        samples, iters, measured_us = [], 0, 0.0
        wall0 = time.perf_counter()
        while True:
            if cfg.flush_l2:
                self._flush()
            us = self._time_batch_us(fn, batch)
            samples.append(us / batch)
            iters += batch
            measured_us += us
            if measured_us >= cfg.min_runtime_secs * 1e6 or iters >= cfg.max_iters:
                break
            if time.perf_counter() - wall0 >= cfg.max_runtime_secs:
                break
        return samples, iters

    # ---- public API --------------------------------------------------------------------------------------------
    def bench_function(self, bench_id: BenchId | str, fn, throughput_elems: int | None = None, bytes_per_iter: float | None = None,
                       flops_per_iter: float | None = None) -> BenchmarkInfo:
        """Benchmark `fn()` (no arguments). With `fn` taking a `Bencher`, the body decides what is timed."""
        name = str(bench_id)
        takes_bencher = getattr(fn, "__code__", None) is not None and fn.__code__.co_argcount == 1
        all_samples: list[float] = []
        iters = 0
        reps = 1 if self.mode is Mode.Test else max(1, self.config.num_repetitions)
        for r in range(reps):
            if self.config.show_progress:
                print(f"[bench] {name} repetition {r + 1}/{reps}", file=sys.stderr, flush=True)
            if takes_bencher:
                b = Bencher(self)
                fn(b)
                s, n = b.samples_us, b.iters
            else:
                s, n = self._measure(fn)
            all_samples.extend(s)
            iters += n
        mean = sum(all_samples) / len(all_samples)
        var = sum((x - mean) ** 2 for x in all_samples) / len(all_samples)
        info = BenchmarkInfo(name=name, iters=iters, mean_us=mean, min_us=min(all_samples), max_us=max(all_samples), stdev_us=math.sqrt(var),
                             repetitions=reps, samples_us=all_samples)
        if throughput_elems:
            info.elems_per_s = throughput_elems / (mean * 1e-6)
        if bytes_per_iter:
            info.gbytes_per_s = bytes_per_iter / (mean * 1e-6) / 1e9
        if flops_per_iter:
            info.tflops = flops_per_iter / (mean * 1e-6) / 1e12
        self.info_vec.append(info)
        return info

    def bench_with_input(self, bench_id: BenchId | str, input, fn, **throughput) -> BenchmarkInfo:  # noqa: A002
        """Benchmark `fn(input)`; `fn(bencher, input)` when it wants the `Bencher`."""
        if getattr(fn, "__code__", None) is not None and fn.__code__.co_argcount == 2:
            return self.bench_function(bench_id, lambda b: fn(b, input), **throughput)
        return self.bench_function(bench_id, lambda: fn(input), **throughput)

    # ---- reporting ---------------------------------------------------------------------------------------------
    COLUMNS = ("name", "iters", "mean_us", "min_us", "max_us", "stdev_us", "repetitions", "elems_per_s", "gbytes_per_s", "tflops")

    def _rows(self) -> list[dict]:
        rows = []
        for i in self.info_vec:
            d = asdict(i)
            d.pop("samples_us")
            rows.append({k: (round(v, 4) if isinstance(v, float) else v) for k, v in d.items()})
        return rows

    def to_csv(self) -> str:
        buf = io.StringIO()
        w = csv.DictWriter(buf, fieldnames=self.COLUMNS)
        w.writeheader()
        for r in self._rows():
            w.writerow({k: ("" if r[k] is None else r[k]) for k in self.COLUMNS})
        return buf.getvalue()

    def to_json(self) -> str:
        return json.dumps({"mode": self.mode.name, "config": {k: (str(v) if isinstance(v, Path) else v) for k, v in asdict(self.config).items()},
                           "results": self._rows()})

    def dump_report(self, file=None) -> None:
        out = file or sys.stdout
        if self.config.tabular_view:
            out.write(self.to_csv())
        else:
            for r in self._rows():
                out.write(json.dumps(r) + "\n")
        if self.config.out_file is not None:
            p = Path(self.config.out_file)
            p.write_text(self.to_json() if p.suffix == ".json" else self.to_csv())
