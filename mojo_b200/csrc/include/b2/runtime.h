// Process-wide host runtime: a small worker pool, lazily created named singletons and cached device capabilities.
//
// The reference leans on a closed task runtime for the same three jobs: a thread pool behind `parallelize`
// (KGEN_CompilerRT_AsyncRT_CreateRuntime, stdlib/src/builtin/_startup.mojo:23-36), a registry of named globals
// created on first use and destroyed at exit (`_Global` / `_get_global_or_null`, stdlib/src/sys/ffi.mojo:412-462)
// and core-count queries (stdlib/src/sys/info.mojo:788-818). On this target the GPU work is ordered by CUDA
// streams, so the pool only serves host chores that are worth spreading over cores: faulting in and copying
// memory-mapped checkpoint tensors, and whatever the bindings hand it. Plain C++17, no CUDA dependency.
#pragma once
#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace b2 {
namespace rt {

class WorkerPool {
 public:
  explicit WorkerPool(int threads);
  ~WorkerPool();
  WorkerPool(const WorkerPool&) = delete;
  WorkerPool& operator=(const WorkerPool&) = delete;

  int size() const { return static_cast<int>(workers_.size()); }
  void submit(std::function<void()> task);
  // Blocks until every task submitted so far has finished. Exceptions thrown by tasks are swallowed by the pool and
  // counted: `failed_tasks()` tells how many.
  void wait_idle();
  int64_t failed_tasks() const;
  // fn(i) for i in [0, n), spread over the pool (the caller's thread takes part); returns when all are done.
  void parallel_for(int64_t n, const std::function<void(int64_t)>& fn);

 private:
  void worker_loop();

  std::vector<std::thread> workers_;
  std::deque<std::function<void()>> queue_;
  mutable std::mutex mu_;
  std::condition_variable cv_task_, cv_idle_;
  int64_t in_flight_ = 0, failed_ = 0;
  bool stop_ = false;
};

// One per process. Everything is created on first use and torn down in reverse order of creation at exit.
class Context {
 public:
  static Context& instance();

  // Pool sized min(8, hardware threads), or B2_HOST_THREADS when that is set.
  WorkerPool& pool();
  int hardware_threads() const;

  // Named singleton of `bytes` zero-initialised bytes, created by the first caller (`init`, if given, runs once on
  // the fresh block; `fini` runs at teardown). Later callers get the same block; a size mismatch returns nullptr.
  void* global(const std::string& name, size_t bytes, void (*init)(void*) = nullptr, void (*fini)(void*) = nullptr);
  void* global_or_null(const std::string& name) const;
  size_t num_globals() const;

  ~Context();

 private:
  Context() = default;
  struct Global {
    std::unique_ptr<uint8_t[]> mem;
    size_t bytes;
    void (*fini)(void*);
  };
  mutable std::mutex mu_;
  std::unique_ptr<WorkerPool> pool_;
  std::unordered_map<std::string, Global> globals_;
  std::vector<std::string> order_;
};

}  // namespace rt
}  // namespace b2
