// CPU-rank simulator of the symmetric-memory collective protocol (csrc/runtime/symm_sim.cpp).
//
// N host threads play N ranks over plain host memory, running the same steps as the device kernels in
// csrc/kernels/symm_coll.cu: epoch-valued flags A ("my input is in place") and B ("my writes into your memory
// are complete"), inputs double-buffered by launch parity, bounded waits that record a TIMEOUT status and
// return. Faults are injected here, on the host, never on a GPU: a rank that drops one signal, starts a
// step late, or skips a launch altogether. No counterpart in the reference, which has no multi-device code.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace b2 {
namespace sim {

enum class Algo : int { kOneShot = 0, kTwoShot = 1, kAllToAll = 2 };

enum class FaultKind : int {
  kNone = 0,
  kDropSignal = 1,   // `rank` does not raise flag A at `step` (peers time out; the next step heals, flags only grow)
  kDelay = 2,        // `rank` starts `step` `delay_ms` late (peers wait; no error if the limit is longer)
  kSkipLaunch = 3,   // `rank` does not run `step` at all: no signals, no data
};

struct Fault {
  FaultKind kind = FaultKind::kNone;
  int rank = 0;
  int step = 0;
  int delay_ms = 0;
};

// "drop_signal:rank=3:step=17", "delay:rank=1:step=2:ms=50", "skip_launch:rank=0:step=4", "" or "none".
// Returns false on a malformed spec.
bool parse_fault(const std::string& spec, Fault* out);

struct RankReport {
  int code = 0;        // b2::StatusCode of the first failed wait (0 = OK)
  int step = -1;       // step at which it happened
  int peer = -1;       // peer whose flag did not arrive
  int which = 0;       // 0 = flag A, 1 = flag B
  int wrong_steps = 0; // steps whose result differed from the expected sum (excluding steps that reported a timeout)
  int timeouts = 0;    // number of waits that ran out
};

struct SimResult {
  std::vector<RankReport> ranks;
  double elapsed_ms = 0.0;
};

// Runs `steps` collectives of `n` floats on `world` ranks (2..8). Every wait gives up after `timeout_ms`.
SimResult run(int world, int n, int steps, Algo algo, const Fault& fault, int timeout_ms);

}  // namespace sim
}  // namespace b2
