"""Host runtime unit tests: paged KV manager (alloc/free/prefix cache/fork/eviction), scheduler (token budget,
chunked prefill, preemption), hashing and the bit-exact dtype helpers. No GPU."""
import numpy as np
import pytest
import torch

from mojo_b200 import _ext

C = _ext.require()


def toks(*v):
    return np.array(v, dtype=np.int32)


def test_kv_pages_are_ceil_len_over_page():
    kv = C.KVCacheManager(32, 16, False)
    kv.add_sequence(1, np.arange(40, dtype=np.int32))
    assert kv.reserve(1, 40)
    assert len(kv.block_table(1)) == 3            # ceil(40 / 16)
    assert kv.reserve(1, 48) and len(kv.block_table(1)) == 3
    assert kv.reserve(1, 49) and len(kv.block_table(1)) == 4
    assert kv.slot(1, 17) == kv.block_table(1)[1] * 16 + 1
    with pytest.raises(IndexError):
        kv.slot(1, 64)
    assert kv.available_pages() == 28
    kv.free_sequence(1)
    assert kv.available_pages() == 32 and kv.check_invariants() == ""


def test_kv_reserve_fails_without_side_effects():
    kv = C.KVCacheManager(4, 16, False)
    kv.add_sequence(1, np.zeros(1, dtype=np.int32))
    kv.add_sequence(2, np.zeros(1, dtype=np.int32))
    assert kv.reserve(1, 48)
    assert not kv.reserve(2, 33)                  # needs 3, only 1 left
    assert len(kv.block_table(2)) == 0 and kv.available_pages() == 1
    assert kv.check_invariants() == ""


def test_prefix_cache_hit_eviction_and_never_whole_prompt():
    kv = C.KVCacheManager(8, 4, True)
    a = np.arange(12, dtype=np.int32)
    assert kv.add_sequence(1, a) == 0
    kv.reserve(1, 12)
    kv.commit(1, a, 12)
    kv.free_sequence(1)                           # three cached, evictable pages
    assert kv.stats().cached_pages == 3 and kv.available_pages() == 8
    # same prompt again: only 2 of the 3 pages may be reused (one token must be computed)
    assert kv.add_sequence(2, a) == 8
    b = np.concatenate([a[:8], toks(99, 98, 97, 96, 95)])
    assert kv.add_sequence(3, b) == 8             # shares the first two pages with seq 2
    t2, t3 = kv.block_table(2), kv.block_table(3)
    assert list(t2[:2]) == list(t3[:2])
    assert kv.check_invariants() == ""
    kv.free_sequence(2)
    kv.free_sequence(3)
    # fill the cache with something else: cached pages get evicted oldest-first, leaves before roots
    kv.add_sequence(4, np.full(32, 7, dtype=np.int32))
    assert kv.reserve(4, 32)
    assert kv.stats().evictions == 3 and kv.stats().cached_pages == 0
    assert kv.check_invariants() == ""


def test_fork_shares_full_pages_and_copies_the_tail():
    kv = C.KVCacheManager(8, 4, False)
    kv.add_sequence(1, np.zeros(1, dtype=np.int32))
    kv.reserve(1, 10)                             # 2 full pages + partial third
    ok, copies = kv.fork(1, 2)
    assert ok and len(copies) == 1
    t1, t2 = kv.block_table(1), kv.block_table(2)
    assert list(t1[:2]) == list(t2[:2]) and t1[2] != t2[2] and copies[0] == (int(t1[2]), int(t2[2]))
    kv.free_sequence(1)
    assert kv.available_pages() == 8 - 3          # shared pages still referenced by seq 2
    kv.free_sequence(2)
    assert kv.available_pages() == 8 and kv.check_invariants() == ""


def test_hash_page_chains_and_is_never_zero():
    a = C.hash_page(0, toks(1, 2, 3, 4))
    assert a != 0 and a == C.hash_page(0, toks(1, 2, 3, 4))
    assert a != C.hash_page(0, toks(1, 2, 4, 3)) and a != C.hash_page(1, toks(1, 2, 3, 4))
    assert len({C.hash_page(0, toks(i, i + 1, i + 2)) for i in range(2000)}) == 2000


def make_sched(pages=64, page=16, budget=64, seqs=8, chunked=True, max_len=512):
    kv = C.KVCacheManager(pages, page, False)
    sc = C.SchedulerConfig()
    sc.max_num_seqs, sc.max_num_batched_tokens, sc.max_model_len, sc.enable_chunked_prefill = seqs, budget, max_len, chunked
    return C.Scheduler(sc, kv), kv


def test_scheduler_budget_chunking_and_decode_first():
    s, kv = make_sched(budget=64)
    s.add_request(1, np.arange(100, dtype=np.int32), 4)
    s.add_request(2, np.arange(10, dtype=np.int32), 4)
    b = s.step()
    assert list(b.seq_ids) == [1] and list(b.q_lens) == [64] and len(b.sample_rows) == 0   # first chunk, nothing to sample
    b = s.step()
    assert list(b.seq_ids) == [1, 2] and list(b.q_lens) == [36, 10]
    assert list(b.sample_seq_ids) == [1, 2] and list(b.sample_rows) == [35, 45]
    assert list(b.positions[:3]) == [64, 65, 66] and list(b.cu_q) == [0, 36, 46]
    s.append_token(1, 7)
    s.append_token(2, 8)
    b = s.step()
    assert b.num_decode == 2 and b.num_prefill == 0 and list(b.ctx_lens) == [101, 11] and list(b.token_ids) == [7, 8]
    assert b.block_tables.shape == (2, 7)
    s.add_request(3, np.arange(5, dtype=np.int32), 2)
    s.append_token(1, 1)
    s.append_token(2, 1)
    b = s.step()                                   # decode sequences are emitted before the new prefill
    assert list(b.seq_ids) == [1, 2, 3] and b.num_decode == 2 and b.num_prefill == 1
    assert kv.check_invariants() == ""


def test_scheduler_without_chunking_waits_for_budget():
    s, _ = make_sched(budget=32, chunked=False)
    s.add_request(1, np.arange(20, dtype=np.int32), 2)
    s.add_request(2, np.arange(20, dtype=np.int32), 2)
    b = s.step()
    assert list(b.seq_ids) == [1]                 # the second prompt does not fit whole
    s.append_token(1, 0)
    b = s.step()
    assert list(b.seq_ids) == [1, 2] and list(b.q_lens) == [1, 20]


def test_scheduler_preempts_latest_and_requeues_front():
    s, kv = make_sched(pages=4, page=16, budget=256)
    for i in (1, 2):
        s.add_request(i, np.arange(30, dtype=np.int32), 30)
    b = s.step()
    assert list(b.seq_ids) == [1, 2] and kv.available_pages() == 0
    for _ in range(3):
        s.append_token(1, 5)
        s.append_token(2, 5)
        b = s.step()
    # sequence 1 needs a third page at position 32: the newer sequence 2 is preempted
    assert list(b.preempted) == [2] and list(b.seq_ids) == [1]
    assert s.num_waiting() == 1 and s.request_info(2)["computed"] == 0 and s.total_preemptions() == 1
    s.finish(1)
    b = s.step()
    assert list(b.seq_ids) == [2] and b.q_lens[0] == 33      # recompute prompt + the three generated tokens
    assert kv.check_invariants() == ""


def test_scheduler_rejects_impossible_requests():
    s, _ = make_sched(pages=2, page=16, max_len=64)
    with pytest.raises(ValueError):
        s.add_request(1, np.arange(80, dtype=np.int32), 4)       # longer than max_model_len
    with pytest.raises(ValueError):
        s.add_request(2, np.arange(40, dtype=np.int32), 4)       # can never fit in 2 pages
    with pytest.raises(ValueError):
        s.add_request(3, np.zeros(0, dtype=np.int32), 4)


def test_dtype_helpers_match_torch_bit_for_bit():
    g = torch.Generator().manual_seed(0)
    vals = torch.cat([torch.randn(2000, generator=g) * 10, torch.tensor([0.0, -0.0, 448.0, 500.0, -1e9, 2 ** -9, 2 ** -10, 3e-4, 1.0625, 0.0166])])
    for v in vals.tolist():
        assert C.f32_to_bf16_bits(v) == (torch.tensor(v).bfloat16().view(torch.int16).item() & 0xFFFF)
        want = torch.tensor(v).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).item()
        assert C.f32_to_e4m3_bits(v) == want, v
    for b in range(256):
        t = torch.tensor([b], dtype=torch.uint8)
        a, w = C.e4m3_bits_to_f32(b), t.view(torch.float8_e4m3fn).float().item()
        assert (a != a and w != w) or a == w
        a, w = C.e5m2_bits_to_f32(b), t.view(torch.float8_e5m2).float().item()
        assert (a != a and w != w) or a == w
    assert C.bf16_bits_to_f32(0x3F80) == 1.0


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_host_runtime_selftest_under_sanitizer(sanitizer, tmp_path):
    """The KV manager, the scheduler and the threaded collective simulator, driven by random traffic in a plain
    executable built with AddressSanitizer+UBSan and with ThreadSanitizer: any report makes the run exit non-zero."""
    import subprocess

    from mojo_b200 import build

    exe = build.build_selftest(sanitizer, out_dir=tmp_path)
    env = {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "halt_on_error=1", "TSAN_OPTIONS": "halt_on_error=1",
           "PATH": "/usr/bin:/bin"}
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    assert "runtime self-test: ok" in p.stdout


def test_safetensors_reader_matches_the_reference_writer(tmp_path):
    """Files written by the `safetensors` package read back bit for bit through the C++ reader: every dtype the
    loaders use, zero-copy views, whole-tensor reads through the worker pool, metadata, and clean errors."""
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(0)
    tensors = {
        "a.bf16": torch.randn(33, 64, generator=g).bfloat16(), "b.f32": torch.randn(7, generator=g), "c.f16": torch.randn(3, 5, 2, generator=g).half(),
        "d.i64": torch.arange(10), "e.u8": torch.randint(0, 255, (9 << 20,), generator=g, dtype=torch.uint8),
        "f.e4m3": torch.randn(128, 256, generator=g).to(torch.float8_e4m3fn), "g.scalar": torch.tensor(3.5), "h.empty": torch.zeros(0, 4),
    }
    path = tmp_path / "t.safetensors"
    save_file(tensors, str(path), metadata={"format": "pt", "who": "test \"quoted\""})
    f = C.SafetensorsFile(str(path))
    assert sorted(f.keys()) == sorted(tensors) and f.has("a.bf16") and not f.has("zzz")
    assert f.metadata()["who"] == 'test "quoted"'
    for name, want in tensors.items():
        dtype, shape, nbytes = f.info(name)
        assert list(shape) == list(want.shape) and nbytes == want.numel() * want.element_size()
        got = f.get(name)
        assert got.dtype == want.dtype and got.shape == want.shape
        def raw(t):      # compare bit patterns (fp8 has no equality kernel on CPU)
            return t.reshape(-1).view(torch.uint8) if t.numel() else t

        assert torch.equal(raw(got), raw(want))
        dst = torch.empty_like(want)
        f.read_into(name, dst)
        assert torch.equal(raw(dst), raw(want))
    view = f.get("a.bf16")
    del f
    import gc

    gc.collect()
    assert torch.equal(view, tensors["a.bf16"])          # the view keeps the mapping alive
    with pytest.raises(KeyError):
        C.SafetensorsFile(str(path)).get("zzz")
    with pytest.raises(ValueError):
        C.SafetensorsFile(str(path)).read_into("b.f32", torch.empty(8))
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(RuntimeError, match="header length"):
        C.SafetensorsFile(str(bad))
    with pytest.raises(RuntimeError, match="cannot open"):
        C.SafetensorsFile(str(tmp_path / "missing.safetensors"))


def test_worker_pool_and_context():
    info = C.context_info()
    assert info["pool_threads"] >= 1 and info["hardware_threads"] >= 1
    src = torch.randint(0, 255, (40 << 20,), dtype=torch.uint8)
    dst = torch.zeros_like(src)
    C.parallel_copy(dst, src)
    assert torch.equal(dst, src)
    dst.zero_()
    C.parallel_copy(dst, src, 2)
    assert torch.equal(dst, src)
    with pytest.raises(ValueError):
        C.parallel_copy(torch.zeros(3), src)


@pytest.mark.parametrize("mode,ran_cheap,cheap,ran_costly,costly", [(0, 1, "TIMEOUT", 1, "OK"), (1, 1, "ASSERT", 1, "OK"), (2, 0, "ASSERT", 1, "OK"),
                                                                 (3, 0, "ASSERT", 0, "ASSERT")])
def test_assertion_modes_config_matrix(mode, ran_cheap, cheap, ran_costly, costly, tmp_path):
    """The same source under the four assertion modes (none / warn / safe / all): what gets recorded and whether the
    guarded access still runs. In mode none the failed check leaves the word empty, so the program's later explicit
    TIMEOUT record is the first one and is what shows."""
    import subprocess
    from pathlib import Path

    import mojo_b200

    csrc = Path(mojo_b200.__file__).parent / "csrc"
    exe = tmp_path / f"assert_modes_{mode}"
    subprocess.run(["g++", "-std=c++17", f"-DB2_ASSERT_MODE={mode}", f"-I{csrc / 'include'}", str(csrc / "tests" / "assert_modes.cpp"), "-o", str(exe)],
                   check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    got = dict(kv.split("=") for kv in out)
    assert got["mode"] == str(mode)
    assert (int(got["ran_cheap"]), got["cheap"], int(got["ran_costly"]), got["costly"]) == (ran_cheap, cheap, ran_costly, costly)
    assert got["ran_passing"] == "1" and got["passing"] == "OK"
    if cheap == "ASSERT":      # the first record is kept: site kSiteTest with the offending index and its limit
        assert (got["site"], got["a"], got["b"]) == ("15", "41", "8")


def test_symmetric_heap_rendezvous_passes_descriptors_between_ranks():
    """The side channel of the VMM symmetric heap (descriptors over AF_UNIX sockets with SCM_RIGHTS, all ranks agreeing on
    every step) with three CPU ranks and ordinary files standing in for the device allocations."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29655", os.path.join(root, "tests", "mp_fd_exchange_cpu.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=180, cwd=root)
    assert "FD_EXCHANGE_OK 3" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
