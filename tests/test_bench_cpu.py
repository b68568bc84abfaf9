"""The benchmark harness (`mojo_b200.utils.bench`) and the micro-benchmark suite: test mode runs everything once,
benchmark mode honours its time budget and repetition count, reports come out as CSV and JSON."""
import csv
import io
import json
import time

import pytest

from mojo_b200.utils.bench import Bench, BenchConfig, Bencher, BenchId, Mode


def _work():
    s = 0
    for i in range(2000):
        s += i * i
    return s


def test_test_mode_runs_each_benchmark_once():
    calls = []
    b = Bench(BenchConfig(device="cpu"), Mode.Test)
    b.bench_function(BenchId("f", "a"), lambda: calls.append(1))
    b.bench_with_input(BenchId("g"), 7, lambda x: calls.append(x))
    assert calls == [1, 7]
    assert [i.name for i in b.info_vec] == ["f/a", "g"] and all(i.iters == 1 for i in b.info_vec)


def test_benchmark_mode_respects_budget_repetitions_and_reports_throughput(tmp_path):
    out = tmp_path / "r.json"
    cfg = BenchConfig(out_file=out, min_runtime_secs=0.05, max_runtime_secs=0.5, min_warmuptime_secs=0.01, num_repetitions=2,
                      device="cpu", tabular_view=True)
    b = Bench(cfg)
    t0 = time.perf_counter()
    info = b.bench_function("work", _work, throughput_elems=2000, bytes_per_iter=16000, flops_per_iter=4000)
    assert time.perf_counter() - t0 < 3.0
    assert info.repetitions == 2 and info.iters >= 6
    assert info.min_us <= info.mean_us <= info.max_us and info.mean_us > 0
    assert info.elems_per_s == pytest.approx(2000 / (info.mean_us * 1e-6))
    assert info.gbytes_per_s == pytest.approx(16000 / (info.mean_us * 1e-6) / 1e9)
    assert info.tflops == pytest.approx(4000 / (info.mean_us * 1e-6) / 1e12)
    buf = io.StringIO()
    b.dump_report(buf)
    rows = list(csv.DictReader(io.StringIO(buf.getvalue())))
    assert rows[0]["name"] == "work" and float(rows[0]["mean_us"]) > 0 and rows[0]["tflops"] != ""
    rep = json.loads(out.read_text())
    assert rep["mode"] == "Benchmark" and rep["results"][0]["name"] == "work" and rep["config"]["num_repetitions"] == 2


def test_bencher_bodies_control_what_is_timed():
    b = Bench(BenchConfig(min_runtime_secs=0.02, max_runtime_secs=0.2, min_warmuptime_secs=0.0, device="cpu", tabular_view=False))
    seen = []

    def body(bench: Bencher):
        data = list(range(1000))           # set-up outside the timed region
        bench.iter(lambda: sum(data))

    def custom(bench: Bencher):
        def run(n):
            seen.append(n)
            t0 = time.perf_counter_ns()
            for _ in range(n):
                _work()
            return time.perf_counter_ns() - t0
        bench.iter_custom(run)

    a = b.bench_function("iter", body)
    c = b.bench_with_input(BenchId("custom", "x"), None, lambda bench, _inp: custom(bench))
    assert a.iters > 0 and c.iters == sum(seen) - 3          # the first custom call of 3 iterations is warm-up
    buf = io.StringIO()
    b.dump_report(buf)
    lines = [json.loads(l) for l in buf.getvalue().splitlines()]
    assert [l["name"] for l in lines] == ["iter", "custom/x"]


def test_host_micro_benchmark_suite_in_test_mode(capsys):
    from mojo_b200 import bench_kernels

    out = bench_kernels.main(["--suite", "host", "--test"])
    names = [i.name for i in out.info_vec]
    assert any(n.startswith("scheduler/") for n in names) and any(n.startswith("kv_manager/") for n in names) and len(names) >= 5
    assert capsys.readouterr().out.startswith("name,iters,mean_us")


@pytest.mark.gpu
def test_gpu_micro_benchmark_suite_in_test_mode():
    from mojo_b200 import bench_kernels, ops

    out = bench_kernels.main(["--suite", "gpu", "--test", "--cases", "rmsnorm,sampling,gemm_decode,mla_prefill"])
    assert [i.name for i in out.info_vec] == ["rmsnorm", "sampling", "gemm_decode", "mla_prefill"]
    assert all(i.mean_us > 0 for i in out.info_vec)
    ops.check_status()
