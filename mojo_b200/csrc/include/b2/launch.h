// Launch-side helpers shared by every kernel file: return codes that keep the CUDA error they came from, and
// one-time kernel attribute set-up that is remembered per device.
//
// A launcher returns 0, a negative b2::StatusCode for a request it refuses before launching (kBadArgument,
// kTooLarge), or -(kCudaErrorBase + cudaError_t) when the CUDA runtime refused something: a launch under a stream
// capture that does not allow it, an attribute the device does not support, a sticky error left by earlier work.
// Folding all of these into kBadArgument would hide which one it was.
#pragma once
#include <atomic>
#include <cuda_runtime.h>
#include "b2/status.h"

namespace b2 {

constexpr int kCudaErrorBase = 1000;

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? 0 : -(kCudaErrorBase + static_cast<int>(e)); }
// After a `<<<>>>` launch: 0, or the code of the error the launch left behind (which this call also clears).
inline int last_launch_rc() { return cuda_rc(cudaGetLastError()); }
// True when `rc` carries a cudaError_t; `cuda_error_of(rc)` recovers it.
inline bool is_cuda_rc(int rc) { return rc <= -kCudaErrorBase; }
inline cudaError_t cuda_error_of(int rc) { return static_cast<cudaError_t>(-rc - kCudaErrorBase); }

// Attributes set with cudaFuncSetAttribute belong to the (kernel, device) pair, so "done once" has to be kept per
// device: a process that drives two GPUs must set the attribute on each. `run(f)` calls f() (returning a
// cudaError_t) unless it already succeeded with the current device current; safe to call from several host threads
// (the worst case is that two of them both set the attribute).
class DeviceOnce {
 public:
  template <class F>
  int run(F&& f) {
    int dev = -1;
    const bool known = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices;
    if (known && done_[dev].load(std::memory_order_acquire)) return 0;
    const cudaError_t e = f();
    if (e != cudaSuccess) {
      cudaGetLastError();
      return cuda_rc(e);
    }
    if (known) done_[dev].store(1, std::memory_order_release);
    return 0;
  }
  // The usual case: opt one kernel into `bytes` of dynamic shared memory.
  template <class Kernel>
  int max_smem(Kernel kernel, int bytes) {
    return run([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); });
  }

 private:
  static constexpr int kMaxDevices = 64;
  std::atomic<unsigned char> done_[kMaxDevices] = {};
};

}  // namespace b2
