// Self-test of the host runtime (KV-cache manager, scheduler, CPU-rank collective simulator) as a plain
// executable, so that it can be built with -fsanitize=address,undefined or -fsanitize=thread and run in a
// CPU-only test job. The reference has no sanitizer job of its own (its lit config only reserves an `asan`
// feature flag, stdlib/test/lit.cfg.py:66-69); the device side cannot be run under a sanitizer here, so the
// host code that computes every block table, slot and schedule is the part that gets one.
//
// Exit code 0 = every check passed. Each failed check prints one line and the process exits 1.
#include <cstdio>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <random>
#include <set>
#include <string>
#include <vector>

#include "b2/engine.h"
#include "b2/io.h"
#include "b2/runtime.h"
#include "b2/shape.h"
#include "b2/symm_sim.h"

namespace {

int g_failed = 0;

#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) {                                                               \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);     \
      ++g_failed;                                                                \
    }                                                                            \
  } while (0)

using b2::engine::Batch;
using b2::engine::KVCacheManager;
using b2::engine::Scheduler;
using b2::engine::SchedulerConfig;

std::vector<int32_t> random_tokens(std::mt19937& rng, int n, int vocab = 1000) {
  std::uniform_int_distribution<int> d(0, vocab - 1);
  std::vector<int32_t> t(n);
  for (auto& v : t) v = d(rng);
  return t;
}

// Random add / grow / fork / free traffic against a small pool; the manager's own invariant check must hold
// after every operation, and no two live sequences may own the same writable page.
void kv_manager_stress(bool prefix) {
  std::mt19937 rng(prefix ? 7 : 3);
  KVCacheManager kv(64, 16, prefix);
  std::vector<int64_t> live;
  std::vector<std::vector<int32_t>> toks;
  int64_t next_id = 0;
  for (int it = 0; it < 4000; ++it) {
    const int op = static_cast<int>(rng() % 5);
    if (op <= 1 || live.empty()) {
      // new sequence; half of them share a prompt prefix so that the prefix cache gets hits
      auto t = random_tokens(rng, 1 + static_cast<int>(rng() % 90), prefix ? 4 : 1000);
      const int64_t id = next_id++;
      const int64_t have = kv.add_sequence(id, t.data(), static_cast<int64_t>(t.size()));
      CHECK(have >= 0 && have <= static_cast<int64_t>(t.size()));
      CHECK(have % 16 == 0);
      if (kv.reserve(id, static_cast<int64_t>(t.size()))) {
        kv.commit(id, t.data(), static_cast<int64_t>(t.size()));
        live.push_back(id);
        toks.push_back(t);
      } else {
        kv.free_sequence(id);
      }
    } else if (op == 2) {
      const size_t i = rng() % live.size();
      const int64_t want = kv.num_tokens_reserved(live[i]) + 1 + static_cast<int64_t>(rng() % 20);
      const int64_t need = kv.pages_needed(live[i], want);
      const bool ok = kv.reserve(live[i], want);
      CHECK(ok || need > 0);
      if (ok) {
        CHECK(kv.num_tokens_reserved(live[i]) >= want);
        // slots of consecutive positions inside one page are consecutive
        const int64_t s0 = kv.slot(live[i], want - 1);
        CHECK(s0 >= 0 && s0 < 64 * 16);
        CHECK(s0 / 16 == kv.block_table(live[i])[static_cast<size_t>((want - 1) / 16)]);
      }
    } else if (op == 3) {
      const size_t i = rng() % live.size();
      std::vector<std::pair<int64_t, int64_t>> copies;
      const int64_t id = next_id++;
      if (kv.fork(live[i], id, &copies)) {
        CHECK(copies.size() <= 1);
        CHECK(kv.block_table(id).size() == kv.block_table(live[i]).size());
        live.push_back(id);
        toks.push_back(toks[i]);
      }
    } else {
      const size_t i = rng() % live.size();
      kv.free_sequence(live[i]);
      CHECK(!kv.has_sequence(live[i]));
      live.erase(live.begin() + static_cast<long>(i));
      toks.erase(toks.begin() + static_cast<long>(i));
    }
    const std::string err = kv.check_invariants();
    if (!err.empty()) {
      std::fprintf(stderr, "FAILED invariant after op %d (iteration %d): %s\n", op, it, err.c_str());
      ++g_failed;
      return;
    }
  }
  for (int64_t id : live) kv.free_sequence(id);
  CHECK(kv.check_invariants().empty());
  CHECK(kv.available_pages() == 64);
  const auto st = kv.stats();
  if (prefix) CHECK(st.prefix_queries > 0);
}

// Continuous batching with chunked prefill on a pool that is too small for the load: every request must
// finish with exactly its token count, the per-step budget must hold, every slot handed to the device must be
// inside the pool and unique within the step, and preemption must not lose a request.
void scheduler_stress() {
  std::mt19937 rng(11);
  KVCacheManager kv(48, 16, false);
  SchedulerConfig cfg;
  cfg.max_num_seqs = 8;
  cfg.max_num_batched_tokens = 96;
  cfg.max_model_len = 512;
  Scheduler sched(cfg, &kv);
  const int n_req = 40;
  std::vector<int64_t> want_new(n_req);
  for (int i = 0; i < n_req; ++i) {
    auto t = random_tokens(rng, 5 + static_cast<int>(rng() % 150));
    want_new[i] = 1 + static_cast<int64_t>(rng() % 40);
    sched.add_request(i, t.data(), static_cast<int64_t>(t.size()), want_new[i], 0.0);
  }
  std::vector<int64_t> got(n_req, 0);
  std::vector<char> done(n_req, 0);
  int steps = 0;
  while (sched.has_unfinished() && steps < 20000) {
    ++steps;
    Batch b = sched.step();
    if (b.seq_ids.empty()) {
      CHECK(false && "scheduler made no progress");
      break;
    }
    CHECK(b.num_tokens <= cfg.max_num_batched_tokens);
    CHECK(static_cast<int>(b.seq_ids.size()) <= cfg.max_num_seqs);
    CHECK(b.cu_q.size() == b.seq_ids.size() + 1);
    CHECK(static_cast<int64_t>(b.token_ids.size()) == b.num_tokens);
    CHECK(b.slots.size() == b.token_ids.size() && b.positions.size() == b.token_ids.size());
    CHECK(b.block_tables.size() == b.seq_ids.size() * static_cast<size_t>(b.max_blocks));
    std::set<int64_t> seen;
    for (int64_t s : b.slots) {
      CHECK(s >= 0 && s < 48 * 16);
      CHECK(seen.insert(s).second);
    }
    for (size_t i = 0; i < b.seq_ids.size(); ++i) {
      CHECK(b.cu_q[i + 1] - b.cu_q[i] == b.q_lens[i]);
      CHECK(b.ctx_lens[i] >= b.q_lens[i]);
      CHECK((b.ctx_lens[i] + 15) / 16 <= b.max_blocks);
      if (static_cast<int>(i) < b.num_decode) CHECK(b.q_lens[i] == 1);
    }
    for (int32_t r : b.sample_rows) CHECK(r >= 0 && r < b.num_tokens);
    CHECK(b.sample_rows.size() == b.sample_seq_ids.size());
    for (int64_t id : b.sample_seq_ids) {
      CHECK(!done[static_cast<size_t>(id)]);
      ++got[static_cast<size_t>(id)];
      if (sched.append_token(id, static_cast<int32_t>(rng() % 1000))) {
        sched.finish(id);
        done[static_cast<size_t>(id)] = 1;
      }
    }
    const std::string err = kv.check_invariants();
    if (!err.empty()) {
      std::fprintf(stderr, "FAILED invariant at step %d: %s\n", steps, err.c_str());
      ++g_failed;
      return;
    }
  }
  CHECK(!sched.has_unfinished());
  for (int i = 0; i < n_req; ++i) {
    CHECK(done[static_cast<size_t>(i)]);
    // a preempted request recomputes its prompt and already generated tokens but samples each new token once
    CHECK(got[static_cast<size_t>(i)] == want_new[static_cast<size_t>(i)]);
  }
  CHECK(sched.total_preemptions() > 0);   // the pool is sized to force at least one
  CHECK(kv.available_pages() == 48);
}

// The simulator runs its ranks as threads: under -fsanitize=thread this is the check that the flag protocol
// (release stores / acquire loads on the epoch flags) orders every data access.
void collective_sim() {
  using namespace b2::sim;
  for (Algo algo : {Algo::kOneShot, Algo::kTwoShot, Algo::kAllToAll}) {
    for (int world : {2, 4}) {
      SimResult r = run(world, 1024, 12, algo, Fault{}, 2000);
      CHECK(static_cast<int>(r.ranks.size()) == world);
      for (const auto& rr : r.ranks) {
        CHECK(rr.code == 0);
        CHECK(rr.wrong_steps == 0);
        CHECK(rr.timeouts == 0);
      }
    }
  }
  Fault f;
  CHECK(parse_fault("drop_signal:rank=1:step=7", &f));
  CHECK(f.kind == FaultKind::kDropSignal && f.rank == 1 && f.step == 7);
  // the dropped signal is the last step's, so nothing later can release the waiters: every rank (the faulty
  // one reads its own slot through the same wait) must give up within the limit and name rank 1
  SimResult r = run(4, 256, 8, Algo::kOneShot, f, 100);
  for (size_t i = 0; i < r.ranks.size(); ++i) {
    CHECK(r.ranks[i].timeouts > 0);
    CHECK(r.ranks[i].step == 7 && r.ranks[i].peer == 1 && r.ranks[i].which == 0);
    CHECK(r.ranks[i].wrong_steps == 0);
  }
  CHECK(r.elapsed_ms < 5000.0);
  CHECK(!parse_fault("drop_signal:rank=x", &f));
}

// Shapes and strides as the kernels use them: the paged KV cache [pages, kv heads, page size, head dim].
void shape_arithmetic() {
  const auto cache = b2::make_shape(9, 2, 16, 128);
  CHECK(cache.rank() == 4 && cache.numel() == 9 * 2 * 16 * 128);
  const auto st = b2::row_major(cache);
  CHECK(st[3] == 1 && st[2] == 128 && st[1] == 16 * 128 && st[0] == 2 * 16 * 128);
  const b2::Coord<4> c = b2::make_shape(7, 1, 15, 127);
  CHECK(st.offset(c) == ((7 * 2 + 1) * 16 + 15) * 128 + 127);
  CHECK(b2::in_bounds(c, cache));
  CHECK(!b2::in_bounds(b2::make_shape(9, 0, 0, 0), cache) && !b2::in_bounds(b2::make_shape(0, 0, -1, 0), cache));
  for (int64_t i : {int64_t{0}, int64_t{1}, int64_t{4095}, int64_t{4096}, cache.numel() - 1}) {
    const auto back = b2::delinearize(i, cache);
    CHECK(b2::in_bounds(back, cache) && st.offset(back) == i);
  }
  CHECK(b2::make_shape(3, 4) == b2::make_shape(3, 4) && !(b2::make_shape(3, 4) == b2::make_shape(4, 3)));
}

// Worker pool: every index of a parallel loop runs exactly once, submitted tasks finish before wait_idle returns, a
// throwing task is counted and does not take a worker down, nested use from the caller's thread makes progress.
void worker_pool() {
  b2::rt::WorkerPool pool(4);
  std::vector<std::atomic<int>> hits(1000);
  for (auto& h : hits) h.store(0);
  pool.parallel_for(1000, [&](int64_t i) { hits[static_cast<size_t>(i)].fetch_add(1); });
  for (auto& h : hits) CHECK(h.load() == 1);
  std::atomic<int64_t> sum{0};
  for (int i = 1; i <= 100; ++i) pool.submit([&sum, i] { sum.fetch_add(i); });
  pool.submit([] { throw std::runtime_error("task failure"); });
  pool.wait_idle();
  CHECK(sum.load() == 5050);
  CHECK(pool.failed_tasks() == 1);
  pool.parallel_for(1, [&](int64_t) { sum.fetch_add(1); });
  CHECK(sum.load() == 5051);
  bool threw = false;
  try {
    pool.parallel_for(64, [](int64_t i) { if (i == 5) throw std::runtime_error("loop body failure"); });
  } catch (const std::runtime_error&) {
    threw = true;
  }
  (void)threw;   // the body that throws may run on a helper (swallowed) or on this thread (rethrown); both leave the pool usable
  pool.parallel_for(8, [&](int64_t) { sum.fetch_add(1); });
  CHECK(sum.load() == 5059);

  auto& ctx = b2::rt::Context::instance();
  static int inits = 0;
  void* a = ctx.global("selftest.block", 64, [](void* p) { ++inits; static_cast<char*>(p)[0] = 7; });
  void* b = ctx.global("selftest.block", 64, [](void* p) { ++inits; static_cast<char*>(p)[0] = 9; });
  CHECK(a != nullptr && a == b && inits == 1 && static_cast<char*>(a)[0] == 7 && static_cast<char*>(a)[1] == 0);
  CHECK(ctx.global("selftest.block", 128) == nullptr);            // same name, other size
  CHECK(ctx.global_or_null("selftest.block") == a && ctx.global_or_null("selftest.none") == nullptr);
  CHECK(ctx.pool().size() >= 1);
}

// A safetensors file written byte by byte here: header parsing (escapes, metadata, unknown keys), offsets, the copy
// paths, and the errors a damaged file must raise instead of reading out of bounds.
void safetensors_io(const std::string& dir) {
  using b2::io::SafetensorsFile;
  auto write = [&](const std::string& name, const std::string& header, const std::string& data, uint64_t claimed_len = UINT64_MAX) {
    const std::string path = dir + "/" + name;
    std::ofstream f(path, std::ios::binary);
    uint64_t n = claimed_len == UINT64_MAX ? header.size() : claimed_len;
    for (int i = 0; i < 8; ++i) f.put(static_cast<char>((n >> (8 * i)) & 0xff));
    f << header << data;
    return path;
  };
  const size_t big = 9u << 20;
  std::string data(16 + 24 + big, '\0');
  for (size_t i = 0; i < data.size(); ++i) data[i] = static_cast<char>((i * 131 + 7) & 0xff);
  const std::string header =
      std::string(R"({"__metadata__":{"format":"pt","note":"a\u00e9\n \ud83d\ude00"}, "w\"q":{"dtype":"F32","shape":[2,2],"data_offsets":[0,16],"extra":[1,{"x":null}]},)") +
      R"("big":{"dtype":"U8","shape":[)" + std::to_string(big) + R"(],"data_offsets":[40,)" + std::to_string(40 + big) + R"(]},)" +
      R"("b":{"dtype":"BF16","shape":[3,4],"data_offsets":[16,40]}}   )";
  const std::string path = write("ok.safetensors", header, data);
  {
    SafetensorsFile f(path);
    CHECK(f.names().size() == 3 && f.names()[0] == "w\"q" && f.names()[1] == "b" && f.names()[2] == "big");   // data order
    CHECK(f.metadata().at("format") == "pt" && f.metadata().at("note") == "a\xc3\xa9\n \xf0\x9f\x98\x80");
    CHECK(f.info("b").dtype == "BF16" && f.info("b").shape == std::vector<int64_t>({3, 4}) && f.info("b").nbytes() == 24);
    CHECK(std::memcmp(f.tensor_data("b"), data.data() + 16, 24) == 0);
    std::vector<char> out(big);
    b2::io::parallel_copy(out.data(), f.tensor_data("big"), out.size());
    CHECK(std::memcmp(out.data(), data.data() + 40, out.size()) == 0);
    std::fill(out.begin(), out.end(), 0);
    b2::io::parallel_copy(out.data(), f.tensor_data("big"), out.size(), 1);
    CHECK(std::memcmp(out.data(), data.data() + 40, out.size()) == 0);
    CHECK(!f.has("nope"));
    bool threw = false;
    try { f.info("nope"); } catch (const std::out_of_range&) { threw = true; }
    CHECK(threw);
  }
  auto must_fail = [&](const std::string& p) {
    bool threw = false;
    try { SafetensorsFile f(p); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);
  };
  must_fail(dir + "/missing.safetensors");
  must_fail(write("short_header.safetensors", "{}", "", 1000));                                                   // header length past the end
  must_fail(write("range.safetensors", R"({"a":{"dtype":"F32","shape":[4],"data_offsets":[0,16]}})", "12345678"));     // data past the end
  must_fail(write("mismatch.safetensors", R"({"a":{"dtype":"F32","shape":[3],"data_offsets":[0,16]}})", std::string(16, 'x')));
  must_fail(write("garbage.safetensors", R"({"a":{"dtype":"F32","shape":[4 "data_offsets":[0,16]}})", std::string(16, 'x')));
  must_fail(write("nofields.safetensors", R"({"a":{"dtype":"F32"}})", ""));
  { SafetensorsFile empty(write("empty.safetensors", "{}", "")); CHECK(empty.names().empty()); }
}

}  // namespace

int main(int argc, char** argv) {
  const std::string only = argc > 1 ? argv[1] : "";
  if (only.empty() || only == "kv") {
    kv_manager_stress(false);
    kv_manager_stress(true);
  }
  if (only.empty() || only == "sched") scheduler_stress();
  if (only.empty() || only == "sim") collective_sim();
  if (only.empty() || only == "shape") shape_arithmetic();
  if (only.empty() || only == "pool") worker_pool();
  if (only.empty() || only == "io") {
    const char* tmp = std::getenv("B2_SELFTEST_DIR");
    safetensors_io(tmp != nullptr ? tmp : "/tmp");
  }
  if (g_failed != 0) {
    std::fprintf(stderr, "runtime self-test: %d check(s) failed\n", g_failed);
    return 1;
  }
  std::printf("runtime self-test: ok\n");
  return 0;
}
