"""Config 1: tiny Llama in fp32 on CPU through the real engine (paged KV, page 16, continuous batching).
Greedy tokens must equal a straightforward dense forward pass that knows nothing about pages or chunks."""
import numpy as np
import pytest
import torch

from mojo_b200.engine import EngineConfig, LLMEngine, SamplingParams
from mojo_b200.models import build_model
from mojo_b200.models.config import tiny_llama
from mojo_b200.ops import reference as ref


def dense_forward(model, ids):
    """Whole-sequence forward with plain tensor ops: returns logits for the last position."""
    cfg = model.cfg
    T, d = len(ids), cfg.head_dim
    h = model.embed[torch.tensor(ids)].float()
    pos = torch.arange(T)
    for lw in model.layers:
        x, _ = ref.rms_norm(h, lw.attn_norm, cfg.rms_norm_eps)
        qkv = x @ lw.wqkv.float().t()
        nq, nkv = cfg.num_heads, cfg.num_kv_heads
        q = ref.apply_rope(qkv[:, :nq * d].reshape(T, nq, d), pos, model.cos_sin)
        k = ref.apply_rope(qkv[:, nq * d:(nq + nkv) * d].reshape(T, nkv, d), pos, model.cos_sin)
        v = qkv[:, (nq + nkv) * d:].reshape(T, nkv, d)
        k = k.repeat_interleave(nq // nkv, dim=1)
        v = v.repeat_interleave(nq // nkv, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) / d ** 0.5
        s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, -1)
        h = h + a @ lw.wo.float().t()
        x, _ = ref.rms_norm(h, lw.mlp_norm, cfg.rms_norm_eps)
        h = h + ref.linear_swiglu_interleaved(x, lw.w_gu) @ lw.w_down.float().t()
    x, _ = ref.rms_norm(h, model.final_norm, cfg.rms_norm_eps)
    return x[-1] @ model.lm_head.float().t()


def make_engine(**kw):
    cfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64,
                       max_num_seqs=8, max_num_batched_tokens=kw.pop("budget", 256), max_model_len=512, seed=0, **kw)
    return LLMEngine(cfg)


def test_config1_greedy_matches_dense_reference():
    eng = make_engine()
    prompt = torch.randint(0, 32000, (64,), generator=torch.Generator().manual_seed(1)).tolist()
    out = eng.generate([prompt], SamplingParams(max_tokens=32))[0]
    assert len(out) == 32
    ids = list(prompt)
    for t in range(32):
        nxt = int(torch.argmax(dense_forward(eng.model, ids)))
        assert nxt == out[t], f"token {t}: engine {out[t]} vs dense {nxt}"
        ids.append(nxt)
    # 64 + 31 cached positions -> ceil(95 / 16) = 6 pages were in use; all returned after finish
    assert eng.kv.stats().free_pages == 64
    assert eng.kv.check_invariants() == ""


def test_chunked_prefill_and_batching_do_not_change_tokens():
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (5, 70, 33, 16, 100)]
    base = make_engine(budget=512).generate(prompts, SamplingParams(max_tokens=12))
    chunked = make_engine(budget=24).generate(prompts, SamplingParams(max_tokens=12))   # prompts split in chunks
    assert base == chunked
    one_by_one = [make_engine().generate([p], SamplingParams(max_tokens=12))[0] for p in prompts[:2]]
    assert one_by_one == base[:2]


def test_prefix_cache_reuses_pages_and_keeps_tokens():
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, 32000, (48,), generator=g).tolist()
    p1, p2 = shared + [11, 12, 13], shared + [21, 22]
    ref_out = make_engine().generate([p1, p2], SamplingParams(max_tokens=8))
    eng = make_engine(enable_prefix_cache=True)
    o1 = eng.generate([p1], SamplingParams(max_tokens=8))
    o2 = eng.generate([p2], SamplingParams(max_tokens=8))
    assert [o1[0], o2[0]] == ref_out
    assert eng.kv.stats().prefix_hits == 3  # three full pages of the shared 48 tokens
    assert eng.kv.check_invariants() == ""


def test_preemption_recomputes_and_matches():
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 32000, (40,), generator=g).tolist() for _ in range(4)]
    want = make_engine().generate(prompts, SamplingParams(max_tokens=40))
    cfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=12,
                       max_num_seqs=8, max_num_batched_tokens=256, max_model_len=512, seed=0)
    eng = LLMEngine(cfg)   # 12 pages cannot hold 4 x 80 tokens: someone gets preempted and recomputed
    got = eng.generate(prompts, SamplingParams(max_tokens=40))
    assert got == want
    assert eng.scheduler.total_preemptions() > 0
    assert eng.kv.check_invariants() == ""


def test_sampling_params_and_metrics():
    eng = make_engine()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 32000, (20,), generator=g).tolist() for _ in range(3)]
    sp = [SamplingParams(max_tokens=6), SamplingParams(temperature=0.8, top_k=50, max_tokens=6),
          SamplingParams(temperature=1.0, top_p=0.9, max_tokens=6)]
    a = eng.generate(prompts, sp)
    b = make_engine().generate(prompts, sp)
    assert a == b, "sampling must be reproducible for a fixed seed"
    m = eng.metrics()
    assert m["requests"] == 3 and m["output_tokens"] == 18 and m["ttft_p50_ms"] > 0


def test_fp8_block_quantised_llama_runs_and_tracks_the_bf16_model():
    """fp8 (128x128 block-scaled) weights through the same engine: on CPU the linears dequantise to fp32, so the
    logits must stay close to the unquantised model's and generation must be deterministic."""
    import copy

    from mojo_b200.models import build_model
    from mojo_b200 import ops

    cfg = tiny_llama()
    cfg.hidden_size, cfg.intermediate_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = 256, 768, 4, 2, 64
    qcfg = copy.deepcopy(cfg)
    qcfg.quantization = "fp8_block"
    full = build_model(cfg, "cpu", torch.float32).init_random(0, std=0.05)
    quant = build_model(qcfg, "cpu", torch.float32).init_random(0, std=0.05)
    T = 40
    ids = torch.randint(0, 32000, (T,), generator=torch.Generator().manual_seed(1))
    pos, slots = torch.arange(T, dtype=torch.int32), torch.arange(T, dtype=torch.int64)
    meta = ops.AttnMeta(torch.tensor([0, T], dtype=torch.int32), torch.tensor([T], dtype=torch.int32),
                        torch.arange(3, dtype=torch.int32).unsqueeze(0), 0, T, T)
    a = full.forward(ids, pos, slots, meta, full.allocate_kv_cache(4, 16), None).float()
    b = quant.forward(ids, pos, slots, meta, quant.allocate_kv_cache(4, 16), None).float()
    assert quant.layers[0].wqkv.dtype == torch.float8_e4m3fn and quant.layers[0].s_qkv.shape == (4, 2)
    rel = (a - b).norm() / a.norm()
    assert rel < 0.2, rel       # e4m3 keeps 3 mantissa bits on both operands; K = 256 averages little


def test_trace_spans_and_request_timeline(monkeypatch):
    from mojo_b200.utils import trace

    monkeypatch.setattr(trace, "TRACE", True)
    trace.reset()
    eng = _engine() if "_engine" in globals() else None
    if eng is None:
        from mojo_b200.engine.llm_engine import EngineConfig, LLMEngine
        from mojo_b200.models.config import tiny_llama

        eng = LLMEngine(EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=8,
                                     max_num_batched_tokens=64, max_model_len=256))
    from mojo_b200.engine.llm_engine import SamplingParams

    eng.generate([[1, 2, 3], list(range(5, 30))], SamplingParams(max_tokens=5))
    s = trace.summary()
    assert s["engine.schedule"]["calls"] >= 5 and s["engine.execute"]["calls"] >= 5 and s["engine.execute"]["total_ms"] > 0
    tl = trace.timeline(eng)
    assert len(tl) == 2 and all(len(r["token_times_s"]) == 5 and r["ttft_s"] is not None and r["ttft_s"] >= 0 for r in tl)
    trace.reset()


def test_guard_bands_report_writes_outside_the_buffer():
    from mojo_b200.utils import guard

    t = guard.guarded_zeros((3, 5), torch.float32, "cpu", "scratch")
    assert t.shape == (3, 5) and t.abs().sum() == 0
    t.fill_(1.0)
    n = guard.check_all()
    assert n >= 1
    buf = t._b2_guard
    assert buf.corrupted() == (0, 0)
    buf.raw[buf.guard - 1] = 0            # one byte before the payload
    buf.raw[buf.guard + buf.nbytes + 7] = 1
    assert buf.corrupted() == (1, 1)
    with pytest.raises(guard.GuardError, match="scratch: 1 before / 1 after"):
        guard.check_all()
    with pytest.raises(guard.GuardError):
        buf.check()
    buf.raw[buf.guard - 1] = guard.PATTERN
    buf.raw[buf.guard + buf.nbytes + 7] = guard.PATTERN
    guard.check_all()
    del t, buf
    import gc

    gc.collect()
    assert all(b.name != "scratch" for b in guard.live())


def test_kv_caches_are_guarded_when_the_switch_is_set(monkeypatch):
    from mojo_b200.utils import guard

    monkeypatch.setenv("B2_GUARD", "1")
    model = build_model(tiny_llama(), "cpu", torch.float32).init_random(0)
    caches = model.allocate_kv_cache(4, 16)
    assert all(hasattr(k, "_b2_guard") and hasattr(v, "_b2_guard") for k, v in caches)
    assert guard.check_all() >= 2 * len(caches)
    monkeypatch.setenv("B2_GUARD", "0")
    plain = model.allocate_kv_cache(4, 16)
    assert not hasattr(plain[0][0], "_b2_guard")


def test_context_limit_is_capped_by_the_position_table_and_enforced_at_admission():
    cfg = tiny_llama()
    ecfg = EngineConfig(model=cfg, device="cpu", dtype=torch.float32, page_size=16, num_pages=32, max_num_seqs=2,
                        max_num_batched_tokens=64, max_model_len=1 << 20)
    eng = LLMEngine(ecfg)
    assert eng.cfg.max_model_len == cfg.max_position_embeddings
    with pytest.raises(ValueError, match="context limit"):
        eng.add_request(list(range(cfg.max_position_embeddings)))
    with pytest.raises(ValueError, match="empty prompt"):
        eng.add_request([])


def test_logprobs_match_the_models_own_distribution():
    """SamplingParams.logprobs: the log-probability of each generated token and the k most likely alternatives, equal
    to log_softmax of the logits the model produces for the same prefix; requests without the option are unaffected."""
    from mojo_b200 import ops

    cfg = tiny_llama()
    ecfg = EngineConfig(model=cfg, device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=4,
                        max_num_batched_tokens=64, max_model_len=256)
    eng = LLMEngine(ecfg)
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(9)).tolist()
    plain = eng.generate([prompt], SamplingParams(max_tokens=5))[0]
    r_lp = eng.add_request(prompt, SamplingParams(max_tokens=5, logprobs=3))
    r_no = eng.add_request(prompt[:7], SamplingParams(max_tokens=5))
    eng.run_until_done()
    st = eng.requests[r_lp]
    assert st.output_ids == plain and len(st.logprobs) == 5
    assert eng.requests[r_no].logprobs == []
    ids = list(prompt)
    for tok, (lp, top) in zip(st.output_ids, st.logprobs):
        T = len(ids)
        caches = eng.model.allocate_kv_cache((T + 15) // 16 + 1, 16)
        bt = torch.arange((T + 15) // 16, dtype=torch.int32).unsqueeze(0)
        meta = ops.AttnMeta(torch.tensor([0, T], dtype=torch.int32), torch.tensor([T], dtype=torch.int32), bt, 0, T, T)
        logits = eng.model.forward(torch.tensor(ids), torch.arange(T, dtype=torch.int32), torch.arange(T, dtype=torch.int64), meta, caches,
                                   torch.tensor([T - 1]))[0].float()
        want = torch.log_softmax(logits, -1)
        assert abs(lp - want[tok].item()) < 1e-4
        assert len(top) == 3 and top[0][0] == tok                       # greedy: the chosen token is the most likely one
        assert [t for t, _ in top] == want.topk(3).indices.tolist()
        assert all(abs(v - want[t].item()) < 1e-4 for t, v in top)
        ids.append(tok)


def test_decode_graph_dispatch_and_fallback_when_a_capture_fails(monkeypatch):
    """The runner's choice between graph replay and eager execution, exercised on CPU with stand-ins for the graph
    objects: a bucket is captured at first use, a capture that raises is remembered and its steps run eagerly (with
    the same tokens), and other buckets keep replaying."""
    import warnings

    from mojo_b200.engine import model_runner as mr

    ecfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=4,
                        max_num_batched_tokens=64, max_model_len=128)
    eng = LLMEngine(ecfg)
    runner = eng.runner
    prompts = [[3, 4, 5, 6], [9, 8, 7]]
    want = LLMEngine(ecfg).generate(prompts, SamplingParams(max_tokens=6))
    captured, replayed = [], []

    class FakeGraph:
        def __init__(self, r, bb):
            if bb == 2:
                raise RuntimeError("operation not permitted when stream is capturing")
            captured.append(bb)
            self.ep_calls = 0

        def usable(self):
            return True

    def fake_replay(batch, plan=None, prev_ids=None):
        replayed.append(int(batch.num_seqs))
        runner.use_graphs = False                      # compute the step's tokens through the eager path
        try:
            toks = runner.execute(batch, [eng.requests[int(r)] for r in batch.sample_seq_ids], 0)
        finally:
            runner.use_graphs = True
        return mr.StepHandle(len(toks), None, tokens=toks)

    monkeypatch.setattr(mr, "_DecodeGraph", FakeGraph)
    monkeypatch.setattr(runner, "_launch_decode_graph", fake_replay)
    runner.use_graphs = True
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        got = eng.generate(prompts, SamplingParams(max_tokens=6))          # two sequences decode together: bucket 2 fails
        one = eng.generate([prompts[0]], SamplingParams(max_tokens=6))     # one sequence: bucket 1 captures and replays
    assert got == want and one == [want[0]]
    assert list(runner.failed_buckets) == [2] and captured == [1] and replayed and set(replayed) == {1}
    assert sum("capture" in str(x.message) for x in w) == 1                # warned once, not once per step
    assert runner.capture_graphs() == 1 and sorted(captured) == [1, 4]     # the remaining bucket; the failed one is not retried


def test_prefill_work_items_cover_every_query_tile_once_longest_first():
    import numpy as np

    from mojo_b200 import ops

    rng = np.random.default_rng(0)
    for _ in range(20):
        nd, P = int(rng.integers(0, 5)), int(rng.integers(1, 6))
        q = np.concatenate([np.ones(nd, dtype=np.int64), rng.integers(1, 700, P)])
        ctx = q + np.concatenate([rng.integers(0, 900, nd), rng.integers(0, 3, P) * 128])   # chunks start at page boundaries or 0
        cu = np.concatenate([[0], np.cumsum(q)])
        w = ops.prefill_work_items(cu, ctx, nd)
        want = {(s, t) for s in range(P) for t in range((q[nd + s] + 127) // 128)}
        assert len(w) == len(want) and {(int(a), int(b)) for a, b in w} == want
        cost = [min((ctx[nd + s] - q[nd + s] + t * 128 + min(128, q[nd + s] - t * 128) + 127) // 128, (ctx[nd + s] + 127) // 128) for s, t in w]
        assert cost == sorted(cost, reverse=True)
        assert len(w) <= cu[-1] // 128 + P     # the bound the captured launch's grid is sized with


def test_mixed_step_buckets_cover_every_schedulable_batch():
    ecfg = EngineConfig(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=48,
                        max_num_batched_tokens=1000, max_model_len=128)
    r = LLMEngine(ecfg).runner
    assert r.token_buckets[-1] == 1000 and r.token_buckets == sorted(set(r.token_buckets))
    keys = set(r.mixed_keys())
    for T, nd, P in [(1000, 48, 1), (17, 16, 1), (5, 0, 1), (300, 33, 4), (300, 2, 30), (129, 0, 32), (16, 3, 13)]:
        k = r.mixed_key(T, nd, P)
        tb, db, pb = k
        assert k in keys and tb >= T and db >= nd and pb >= P and db <= tb and pb <= tb
    assert r.mixed_key(300, 2, 33) is None and r.mixed_key(300, 300, 0) is None     # too many chunks / no chunk: not a mixed step


def test_torch_baseline_attention_matches_the_oracle():
    """The comparison arm's attention (two padded scaled_dot_product_attention calls) against the fp32 oracle on a batch
    of decode rows and prefill chunks with cached prefixes."""
    from mojo_b200 import ops
    from mojo_b200.ops import reference, torch_baseline

    g = torch.Generator().manual_seed(5)
    n_q, n_kv, D, page = 4, 2, 32, 16
    q_lens, ctx = [1, 1, 7, 20, 3], [9, 33, 7, 36, 19]          # two decode rows; chunks with 0, 16 and 16 cached tokens
    T, B = sum(q_lens), len(q_lens)
    pages_per = [(c + page - 1) // page for c in ctx]
    num_pages = sum(pages_per) + 1
    kc, vc = torch.randn(num_pages, n_kv, page, D, generator=g), torch.randn(num_pages, n_kv, page, D, generator=g)
    bt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(pages_per):
        bt[b, :n] = torch.arange(nxt, nxt + n)
        nxt += n
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    q = torch.randn(T, n_q * D, generator=g)
    meta = ops.AttnMeta(cu, torch.tensor(ctx, dtype=torch.int32), bt, 2, max(q_lens), max(ctx))
    want = reference.paged_attention(q.reshape(T, n_q, D), kc, vc, cu, meta.ctx_lens, bt, 0.2).reshape(T, -1)
    got = torch_baseline._paged_attention(q, kc, vc, meta, 0.2, D)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)


def _pipelined_engine(**kw):
    base = dict(model=tiny_llama(), device="cpu", dtype=torch.float32, page_size=16, num_pages=64, max_num_seqs=8,
                max_num_batched_tokens=64, max_model_len=256, seed=0, async_scheduling=True)
    base.update(kw)
    return LLMEngine(EngineConfig(**base))


def test_pipelined_stepping_gives_the_same_tokens_one_call_later():
    """The host schedules one step ahead: placeholders stand in for tokens not read yet, decode rows take their input
    from the in-flight step's output, length limits take effect at launch. Same tokens as the step-by-step engine."""
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (5, 70, 33, 16, 100, 3)]
    params = [SamplingParams(max_tokens=m) for m in (12, 1, 7, 30, 2, 9)]
    want = make_engine(budget=64).generate(prompts, params)
    eng = _pipelined_engine()
    got = eng.generate(prompts, params)
    assert got == want
    assert eng._inflight is None and not eng.has_unfinished() and eng.kv.check_invariants() == ""
    assert eng.kv.stats().free_pages == eng.kv.stats().num_pages          # every page came back
    # outputs trail the launches by one call
    eng = _pipelined_engine()
    eng.add_request(prompts[0], SamplingParams(max_tokens=3))
    assert eng.step() == []                                # prefill launched, nothing read yet
    first = eng.step()
    assert len(first) == 1 and len(first[0].output_ids) == 1


def test_pipelined_stepping_drops_the_token_after_a_stop_token_and_recovers_from_preemption():
    g = torch.Generator().manual_seed(32)
    prompts = [torch.randint(0, 32000, (40,), generator=g).tolist() for _ in range(4)]
    ref = make_engine().generate(prompts, SamplingParams(max_tokens=40))
    # a stop token that appears in the reference output ends that request there, also when the next step was already in flight
    stop = ref[1][5]
    params = SamplingParams(max_tokens=40, stop_token_ids=(stop,))
    want = make_engine().generate(prompts, params)
    assert any(len(w) < 40 for w in want)
    got = _pipelined_engine(max_num_batched_tokens=256, max_model_len=512).generate(prompts, params)
    assert got == want
    # twelve pages cannot hold four sequences of 80 tokens: someone is preempted with a placeholder pending
    eng = _pipelined_engine(num_pages=12, max_num_batched_tokens=256, max_model_len=512)
    assert eng.generate(prompts, SamplingParams(max_tokens=40)) == ref
    assert eng.scheduler.total_preemptions() > 0 and eng.kv.check_invariants() == ""


def test_pipelined_stepping_with_prefix_cache_and_recovery():
    from mojo_b200.engine.watchdog import recover
    from mojo_b200.utils import fault

    g = torch.Generator().manual_seed(33)
    shared = torch.randint(0, 32000, (48,), generator=g).tolist()
    prompts = [shared + [11, 12, 13], shared + [21, 22], shared[:20]]
    sp = SamplingParams(max_tokens=8)
    want = make_engine().generate(prompts, sp)
    eng = _pipelined_engine(enable_prefix_cache=True)
    assert eng.generate(prompts[:1], sp) == want[:1]
    assert eng.generate(prompts[1:], sp) == want[1:]
    assert eng.kv.stats().prefix_hits >= 3 and eng.kv.check_invariants() == ""
    # a fault after a launch: the step in flight is discarded, the requests are re-queued, the tokens are unchanged
    eng = _pipelined_engine()
    eng.fault = fault.FaultInjector("raise_after:rank=0:step=3", 0)
    rids = [eng.add_request(p, sp) for p in prompts]
    raised = 0
    while eng.has_unfinished():
        try:
            eng.step()
        except fault.InjectedFault:
            raised += 1
            assert recover(eng)
    assert raised == 1 and [eng.requests[r].output_ids for r in rids] == want


@pytest.mark.parametrize("bad", [dict(temperature=-1.0), dict(temperature=float("nan")), dict(top_p=0.0), dict(top_p=1.01), dict(top_k=-2),
                                 dict(max_tokens=0), dict(logprobs=21)])
def test_sampling_params_refuse_values_the_kernels_would_misread(bad):
    with pytest.raises(ValueError):
        SamplingParams(**bad)
    SamplingParams(temperature=0.0, top_p=1.0, top_k=0, max_tokens=1, logprobs=0)      # the edges themselves are fine
