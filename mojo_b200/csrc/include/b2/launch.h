// Launch-side helpers shared by every kernel file: return codes that keep the CUDA error they came from, and
// one-time kernel attribute set-up that is remembered per device.
//
// A launcher returns 0, a negative b2::StatusCode for a request it refuses before launching (kBadArgument,
// kTooLarge), or -(kCudaErrorBase + cudaError_t) when the CUDA runtime refused something: a launch under a stream
// capture that does not allow it, an attribute the device does not support, a sticky error left by earlier work.
// Folding all of these into kBadArgument would hide which one it was.
#pragma once
#include <atomic>
#include <cstdlib>
#include <utility>
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

// Programmatic dependent launch. A kernel launched through `launch_pdl` may be scheduled while the kernel before it in
// the stream is still running: its CTAs start, run whatever precedes their `ptx::grid_dep_wait()` (barrier and TMEM
// set-up in the GEMMs, nothing in the small kernels) and block there until the earlier kernel has completed and its
// writes are visible. That takes the launch latency, and for the tensor-core kernels the prologue, off the critical
// path of a step made of hundreds of short dependent kernels; stream capture records the same edges in a CUDA graph.
// Rules every kernel launched this way follows: (1) every thread executes grid_dep_wait() before its first global
// memory access and before any return; (2) `ptx::grid_dep_launch()` right after it lets the next kernel be scheduled.
// A kernel that never calls them behaves exactly as under an ordinary launch. The attribute is off unless B2_PDL=1:
// measured on the 8B serving step at one and two GPUs it changed nothing (10.75 / 10.88 ms per step with it, 10.85 /
// 10.83 ms without), so ordinary stream order stays the default and the switch stays for shapes where it may pay.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("B2_PDL");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace b2
