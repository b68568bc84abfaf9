// Self-test of the host runtime (KV-cache manager, scheduler, CPU-rank collective simulator) as a plain
// executable, so that it can be built with -fsanitize=address,undefined or -fsanitize=thread and run in a
// CPU-only test job. The reference has no sanitizer job of its own (its lit config only reserves an `asan`
// feature flag, stdlib/test/lit.cfg.py:66-69); the device side cannot be run under a sanitizer here, so the
// host code that computes every block table, slot and schedule is the part that gets one.
//
// Exit code 0 = every check passed. Each failed check prints one line and the process exits 1.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <set>
#include <string>
#include <vector>

#include "b2/engine.h"
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
  if (g_failed != 0) {
    std::fprintf(stderr, "runtime self-test: %d check(s) failed\n", g_failed);
    return 1;
  }
  std::printf("runtime self-test: ok\n");
  return 0;
}
