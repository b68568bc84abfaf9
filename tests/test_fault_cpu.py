"""Failure detection and fault injection, all on the host: the CPU-rank simulator of the symmetric-memory protocol,
the engine's fault hooks, the watchdog, the cross-rank heartbeat (gloo-free: a FileStore shared by child processes)
and recovery by re-queueing. No GPU is involved, let alone faulted."""
import os
import subprocess
import sys
import time

import pytest
import torch

from mojo_b200 import _ext
from mojo_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
from mojo_b200.engine.watchdog import Heartbeat, Watchdog, WorkerLost, recover
from mojo_b200.models.config import tiny_llama
from mojo_b200.utils import fault

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("algo", ["one_shot", "two_shot", "all_to_all"])
@pytest.mark.parametrize("world", [2, 5, 8])
def test_simulated_ranks_run_the_flag_protocol_clean(algo, world):
    r = _ext.require().symm_sim_run(world, 97, 40, algo, "", 5000)
    assert all(x["code"] == 0 and x["wrong_steps"] == 0 and x["timeouts"] == 0 for x in r["ranks"]), r


@pytest.mark.parametrize("algo", ["one_shot", "two_shot"])
def test_dropped_signal_times_out_cleanly_within_the_limit(algo):
    C = _ext.require()
    steps, bad = 12, 2
    t0 = time.perf_counter()
    r = C.symm_sim_run(4, 64, steps, algo, f"drop_signal:rank={bad}:step={steps - 1}", 150)
    assert time.perf_counter() - t0 < 5.0
    for x in r["ranks"]:
        # every rank (the faulty one waits for its own slot too) reports TIMEOUT on flag A of the faulty rank at that step
        assert x["code"] == 1 and x["step"] == steps - 1 and x["peer"] == bad and x["which"] == 0, r
        assert x["wrong_steps"] == 0


def test_skipped_launch_is_seen_by_the_peers_only():
    r = _ext.require().symm_sim_run(4, 64, 10, "one_shot", "skip_launch:rank=1:step=9", 150)
    codes = [x["code"] for x in r["ranks"]]
    assert codes == [1, 0, 1, 1], r
    assert all(x["peer"] == 1 for i, x in enumerate(r["ranks"]) if i != 1)


def test_short_delay_is_absorbed_and_a_mid_run_drop_heals():
    C = _ext.require()
    r = C.symm_sim_run(4, 64, 10, "two_shot", "delay:rank=0:step=3:ms=60", 3000)
    assert all(x["code"] == 0 and x["wrong_steps"] == 0 for x in r["ranks"]), r
    # flags only grow: the signal of the next step releases whoever still waits for the dropped one
    r = C.symm_sim_run(4, 64, 10, "one_shot", "drop_signal:rank=2:step=4", 100)
    assert all(x["wrong_steps"] == 0 for x in r["ranks"]), r
    assert all(x["step"] in (-1, 4) for x in r["ranks"]), r


def test_fault_spec_parsing():
    f = fault.parse("delay:rank=3:step=17:ms=250")
    assert (f.kind, f.rank, f.step, f.ms) == ("delay", 3, 17, 250) and str(f) == "delay:rank=3:step=17:ms=250"
    assert fault.parse("") is None and fault.parse("none") is None
    with pytest.raises(ValueError):
        fault.parse("explode:rank=1")
    with pytest.raises(ValueError):
        fault.parse("raise:rank=x")
    with pytest.raises(ValueError):
        _ext.require().symm_sim_run(2, 8, 2, "one_shot", "explode:rank=1", 100)


def _engine():
    cfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=8,
                       max_num_batched_tokens=64, max_model_len=256)
    return LLMEngine(cfg)


def test_engine_fault_hooks_raise_skip_and_recover_to_the_same_tokens():
    prompts = [[1, 2, 3, 4, 5], list(range(10, 40)), [7] * 12]
    sp = SamplingParams(max_tokens=10)
    want = _engine().generate(prompts, sp)

    # a rank that raises mid-run: the caller recovers by re-queueing; greedy outputs are unchanged
    eng = _engine()
    eng.fault = fault.FaultInjector("raise:rank=0:step=4", 0)
    rids = [eng.add_request(p, sp) for p in prompts]
    raised = 0
    while eng.has_unfinished():
        try:
            eng.step()
        except fault.InjectedFault:
            raised += 1
            redo = recover(eng)
            assert set(redo) <= set(rids) and redo
    assert raised == 1
    assert [eng.requests[r].output_ids for r in rids] == want

    # a skipped launch produces no tokens for that step and nothing else changes
    eng = _engine()
    eng.fault = fault.FaultInjector("skip_launch:rank=0:step=2", 0)
    assert eng.generate(prompts, sp) == want and eng.skipped_launches == 1

    # a fault addressed to another rank does nothing here
    eng = _engine()
    eng.fault = fault.FaultInjector("raise:rank=1:step=0", 0)
    assert eng.generate(prompts, sp) == want


def test_watchdog_reports_a_stalled_step_and_recovers():
    seen = []
    wd = Watchdog(limit_s=0.15, on_stall=lambda w: seen.append(w.last_step), poll_s=0.02, dump_stacks=False).start()
    try:
        wd.begin_step()
        wd.end_step(0)
        time.sleep(0.3)           # idle between steps is not a stall
        assert wd.healthy and not seen
        wd.begin_step()
        time.sleep(0.4)           # a step that does not finish
        assert not wd.healthy and seen == [0] and wd.stalls == 1
        wd.end_step(1)
        assert wd.healthy
    finally:
        wd.stop()


_WORKER = r"""
import sys, time
import torch.distributed as dist
sys.path.insert(0, {root!r})
from mojo_b200.engine.watchdog import Heartbeat, WorkerLost
rank, world, path, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
store = dist.FileStore(path, world)
hb = Heartbeat(store, rank, world, limit_s=2.0)
# processes start seconds apart on a busy machine: meet, beat afresh, meet again, so that no first check sees a
# heartbeat that is stale only because its owner was still importing
for gate in ("ready", "go"):
    store.add(gate, 1)
    while int(store.add(gate, 0)) < world:
        time.sleep(0.01)
    hb.beat(-1)
for step in range(200):
    try:
        hb.check()
    except WorkerLost as e:
        print("LOST", rank, step, e.ranks, e.reason.split()[0], flush=True)
        sys.exit(0)
    if rank == 1 and step == 5:
        if mode == "leave":
            hb.leave()            # between steps, nothing in flight
        sys.exit(0)               # mode "die": no word, the heartbeat just stops
    time.sleep(0.02)              # the step
    hb.beat(step)
print("DONE", rank, flush=True)
"""


@pytest.mark.parametrize("mode", ["leave", "die"])
def test_ranks_learn_on_the_host_that_a_peer_is_gone(tmp_path, mode):
    world = 3
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT))
    store = str(tmp_path / "store")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), store, mode], stdout=subprocess.PIPE, text=True)
             for r in range(world)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs)
    for r in (0, 2):
        assert outs[r].startswith("LOST"), outs
        _, rank, step, lost, why = outs[r].split(maxsplit=4)
        assert "1" in lost and (why.startswith("left") if mode == "leave" else why.startswith("sent"))
        assert int(step) >= 5
    assert outs[1] == ""


def test_a_failed_step_leaves_no_prefix_cache_entry_and_recovery_matches_the_clean_run():
    """With the prefix cache on, a step that fails before its KV is written must not leave its pages shareable:
    recovery re-queues the same prompts, and a cache hit on a half-written page would feed garbage to attention."""
    def engine():
        cfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=8,
                           max_num_batched_tokens=64, max_model_len=256, enable_prefix_cache=True)
        return LLMEngine(cfg)

    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (50, 37, 20)]
    sp = SamplingParams(max_tokens=6)
    want = engine().generate(prompts, sp)

    eng = engine()
    real = eng.runner.execute
    calls = {"n": 0}

    def failing_execute(batch, states, step):
        calls["n"] += 1
        if calls["n"] == 1:
            raise fault.InjectedFault("the launch failed: nothing was written")   # scheduled, never computed
        return real(batch, states, step)

    eng.runner.execute = failing_execute
    rids = [eng.add_request(p, sp) for p in prompts]
    with pytest.raises(fault.InjectedFault):
        eng.step()
    assert recover(eng)
    assert eng.kv.stats().cached_pages == 0        # the failed step's full pages did not enter the cache
    eng.run_until_done()
    assert [eng.requests[r].output_ids for r in rids] == want
    assert eng.kv.check_invariants() == ""
    # pages of completed steps are shared as before: the same prompts again hit the cache
    hits0 = eng.kv.stats().prefix_hits
    assert eng.generate(prompts, sp) == want and eng.kv.stats().prefix_hits > hits0


def test_prompts_beyond_the_token_budget_are_refused_when_chunked_prefill_is_off():
    cfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=4,
                       max_num_batched_tokens=32, max_model_len=256, enable_chunked_prefill=False)
    eng = LLMEngine(cfg)
    with pytest.raises(ValueError):
        eng.add_request(list(range(40)), SamplingParams(max_tokens=4))
    # a prompt that fits runs, and nothing is left waiting behind a request that can never be scheduled
    assert len(eng.generate([list(range(30))], SamplingParams(max_tokens=4))[0]) == 4
    assert not eng.has_unfinished()
