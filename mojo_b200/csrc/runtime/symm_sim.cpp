// CPU-rank simulator of the symmetric-memory collectives: see b2/symm_sim.h.
#include "b2/symm_sim.h"

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <memory>
#include <sstream>
#include <thread>

#include "b2/status.h"

namespace b2 {
namespace sim {
namespace {

constexpr int kMaxWorld = 8;
using Clock = std::chrono::steady_clock;

// One rank's "symmetric region": everything peers may touch.
struct Region {
  std::vector<float> buf[2];            // input halves (peers read)
  std::vector<float> out[2];            // result / receive halves (peers write)
  std::atomic<uint32_t> flag_a[kMaxWorld];
  std::atomic<uint32_t> flag_b[kMaxWorld];
  std::atomic<uint32_t> counts[2][kMaxWorld];
  Region() {
    for (int i = 0; i < kMaxWorld; ++i) {
      flag_a[i].store(0);
      flag_b[i].store(0);
      counts[0][i].store(0);
      counts[1][i].store(0);
    }
  }
};

// Deterministic input of (rank, step, element): small integers, so float sums are exact in any order.
inline float input_value(int rank, int step, int i) { return static_cast<float>(((rank + 1) * 7 + step * 3 + i) % 17 - 8); }

bool wait_ge(const std::atomic<uint32_t>& f, uint32_t want, int timeout_ms) {
  if (f.load(std::memory_order_acquire) >= want) return true;
  const auto t0 = Clock::now();
  int spins = 0;
  while (f.load(std::memory_order_acquire) < want) {
    if (++spins > 64) {
      std::this_thread::sleep_for(std::chrono::microseconds(50));
      if (Clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) return f.load(std::memory_order_acquire) >= want;
    }
  }
  return true;
}

struct World {
  int world, n, steps, timeout_ms;
  Algo algo;
  Fault fault;
  std::vector<std::unique_ptr<Region>> regions;
};

void note_timeout(RankReport& rep, int step, int peer, int which) {
  ++rep.timeouts;
  if (rep.code == 0) {
    rep.code = kTimeout;
    rep.step = step;
    rep.peer = peer;
    rep.which = which;
  }
}

void rank_main(World& w, int rank, RankReport& rep) {
  Region& self = *w.regions[rank];
  const int tp = w.world;
  for (int step = 0; step < w.steps; ++step) {
    const uint32_t epoch = static_cast<uint32_t>(step) + 1u;
    const int half = step & 1;
    const bool mine = w.fault.kind != FaultKind::kNone && w.fault.rank == rank && w.fault.step == step;
    if (mine && w.fault.kind == FaultKind::kSkipLaunch) continue;
    if (mine && w.fault.kind == FaultKind::kDelay) std::this_thread::sleep_for(std::chrono::milliseconds(w.fault.delay_ms));
    // stage the input (the copy that precedes the kernel on the stream)
    if (w.algo != Algo::kAllToAll)
      for (int i = 0; i < w.n; ++i) self.buf[half][i] = input_value(rank, step, i);
    // flag A on every peer
    if (!(mine && w.fault.kind == FaultKind::kDropSignal))
      for (int r = 0; r < tp; ++r) w.regions[r]->flag_a[rank].store(epoch, std::memory_order_release);
    bool ok = true;
    for (int r = 0; r < tp; ++r)
      if (!wait_ge(self.flag_a[r], epoch, w.timeout_ms)) {
        note_timeout(rep, step, r, 0);
        ok = false;
      }
    bool step_failed = !ok;
    std::vector<float> result;
    if (w.algo == Algo::kOneShot) {
      if (ok) {
        result.assign(w.n, 0.0f);
        for (int r = 0; r < tp; ++r)
          for (int i = 0; i < w.n; ++i) result[i] += w.regions[r]->buf[half][i];
      }
    } else {
      if (ok) {
        if (w.algo == Algo::kTwoShot) {
          const int per = (w.n + tp - 1) / tp;
          const int lo = per * rank, hi = std::min(w.n, lo + per);
          for (int i = lo; i < hi; ++i) {
            float s = 0.0f;
            for (int r = 0; r < tp; ++r) s += w.regions[r]->buf[half][i];
            for (int r = 0; r < tp; ++r) w.regions[r]->out[half][i] = s;
          }
        } else {
          // all-to-all: block j of my data goes to rank j, count = (rank + j + step) % (n + 1) elements
          for (int j = 0; j < tp; ++j) {
            const int cnt = (rank + j + step) % (w.n + 1);
            float* dst = w.regions[j]->out[half].data() + static_cast<size_t>(rank) * w.n;
            for (int i = 0; i < cnt; ++i) dst[i] = input_value(rank, step, j * w.n + i);
            w.regions[j]->counts[half][rank].store(static_cast<uint32_t>(cnt), std::memory_order_relaxed);
          }
        }
      }
      // flag B is owed even after a failed wait, so that peers do not wait for this rank in turn
      for (int r = 0; r < tp; ++r) w.regions[r]->flag_b[rank].store(epoch, std::memory_order_release);
      for (int r = 0; r < tp; ++r)
        if (!wait_ge(self.flag_b[r], epoch, w.timeout_ms)) {
          note_timeout(rep, step, r, 1);
          step_failed = true;
        }
      if (!step_failed && w.algo == Algo::kTwoShot) result.assign(self.out[half].begin(), self.out[half].begin() + w.n);
    }
    if (step_failed) continue;
    // verify
    bool good = true;
    if (w.algo == Algo::kAllToAll) {
      for (int s = 0; s < tp && good; ++s) {
        const int cnt = (s + rank + step) % (w.n + 1);
        if (static_cast<int>(self.counts[half][s].load(std::memory_order_relaxed)) != cnt) good = false;
        const float* src = self.out[half].data() + static_cast<size_t>(s) * w.n;
        for (int i = 0; i < cnt && good; ++i)
          if (src[i] != input_value(s, step, rank * w.n + i)) good = false;
      }
    } else {
      for (int i = 0; i < w.n && good; ++i) {
        float want = 0.0f;
        for (int r = 0; r < tp; ++r) want += input_value(r, step, i);
        if (result[i] != want) good = false;
      }
    }
    if (!good) ++rep.wrong_steps;
  }
}

}  // namespace

bool parse_fault(const std::string& spec, Fault* out) {
  Fault f;
  if (spec.empty() || spec == "none") {
    *out = f;
    return true;
  }
  std::stringstream ss(spec);
  std::string tok;
  bool first = true;
  while (std::getline(ss, tok, ':')) {
    if (first) {
      first = false;
      if (tok == "drop_signal") f.kind = FaultKind::kDropSignal;
      else if (tok == "delay") f.kind = FaultKind::kDelay;
      else if (tok == "skip_launch") f.kind = FaultKind::kSkipLaunch;
      else return false;
      continue;
    }
    const size_t eq = tok.find('=');
    if (eq == std::string::npos) return false;
    const std::string key = tok.substr(0, eq), val = tok.substr(eq + 1);
    char* end = nullptr;
    const long v = std::strtol(val.c_str(), &end, 10);
    if (end == val.c_str() || *end != '\0' || v < 0) return false;
    if (key == "rank") f.rank = static_cast<int>(v);
    else if (key == "step") f.step = static_cast<int>(v);
    else if (key == "ms") f.delay_ms = static_cast<int>(v);
    else return false;
  }
  *out = f;
  return true;
}

SimResult run(int world, int n, int steps, Algo algo, const Fault& fault, int timeout_ms) {
  SimResult res;
  if (world < 1 || world > kMaxWorld || n < 1 || steps < 0 || timeout_ms < 1) return res;
  World w{world, n, steps, timeout_ms, algo, fault, {}};
  for (int r = 0; r < world; ++r) {
    auto reg = std::make_unique<Region>();
    for (int h = 0; h < 2; ++h) {
      reg->buf[h].assign(n, 0.0f);
      reg->out[h].assign(static_cast<size_t>(n) * world, 0.0f);
    }
    w.regions.push_back(std::move(reg));
  }
  res.ranks.resize(world);
  const auto t0 = Clock::now();
  std::vector<std::thread> threads;
  for (int r = 0; r < world; ++r) threads.emplace_back(rank_main, std::ref(w), r, std::ref(res.ranks[r]));
  for (auto& t : threads) t.join();
  res.elapsed_ms = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
  return res;
}

}  // namespace sim
}  // namespace b2
