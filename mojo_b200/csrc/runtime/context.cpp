// Worker pool and process-wide context (see b2/runtime.h).
#include "b2/runtime.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <exception>

namespace b2 {
namespace rt {

WorkerPool::WorkerPool(int threads) {
  threads = std::max(1, threads);
  workers_.reserve(static_cast<size_t>(threads));
  for (int i = 0; i < threads; ++i) workers_.emplace_back([this] { worker_loop(); });
}

WorkerPool::~WorkerPool() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_task_.notify_all();
  for (auto& t : workers_) t.join();
}

void WorkerPool::worker_loop() {
  for (;;) {
    std::function<void()> task;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_task_.wait(lk, [this] { return stop_ || !queue_.empty(); });
      if (queue_.empty()) return;  // stop_ and nothing left to run
      task = std::move(queue_.front());
      queue_.pop_front();
    }
    bool failed = false;
    try {
      task();
    } catch (...) {
      failed = true;
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (failed) ++failed_;
      if (--in_flight_ == 0) cv_idle_.notify_all();
    }
  }
}

void WorkerPool::submit(std::function<void()> task) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    queue_.push_back(std::move(task));
    ++in_flight_;
  }
  cv_task_.notify_one();
}

void WorkerPool::wait_idle() {
  std::unique_lock<std::mutex> lk(mu_);
  cv_idle_.wait(lk, [this] { return in_flight_ == 0; });
}

int64_t WorkerPool::failed_tasks() const {
  std::lock_guard<std::mutex> lk(mu_);
  return failed_;
}

void WorkerPool::parallel_for(int64_t n, const std::function<void(int64_t)>& fn) {
  if (n <= 0) return;
  // Work is claimed index by index from a shared counter, so uneven items balance themselves. The state lives on
  // this frame: the call returns only after every helper has finished with it.
  struct Shared {
    std::atomic<int64_t> next{0};
    std::atomic<int> helpers_left{0};
    std::mutex mu;
    std::condition_variable cv;
  } sh;
  const int helpers = static_cast<int>(std::min<int64_t>(size(), n - 1));
  sh.helpers_left.store(helpers);
  auto drain = [&sh, &fn, n] {
    for (;;) {
      const int64_t i = sh.next.fetch_add(1);
      if (i >= n) break;
      fn(i);
    }
  };
  for (int h = 0; h < helpers; ++h) {
    submit([&sh, drain] {
      try {
        drain();
      } catch (...) {
      }
      std::lock_guard<std::mutex> lk(sh.mu);
      if (sh.helpers_left.fetch_sub(1) == 1) sh.cv.notify_all();
    });
  }
  std::exception_ptr err;
  try {
    drain();
  } catch (...) {
    err = std::current_exception();
    sh.next.store(n);  // nothing more is handed out; helpers finish the item they hold
  }
  {
    std::unique_lock<std::mutex> lk(sh.mu);
    sh.cv.wait(lk, [&sh] { return sh.helpers_left.load() == 0; });
  }
  if (err) std::rethrow_exception(err);
}

Context& Context::instance() {
  static Context ctx;
  return ctx;
}

int Context::hardware_threads() const {
  const unsigned n = std::thread::hardware_concurrency();
  return n == 0 ? 1 : static_cast<int>(n);
}

WorkerPool& Context::pool() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!pool_) {
    int n = std::min(8, hardware_threads());
    if (const char* e = std::getenv("B2_HOST_THREADS")) {
      const int v = std::atoi(e);
      if (v >= 1 && v <= 256) n = v;
    }
    pool_ = std::make_unique<WorkerPool>(n);
  }
  return *pool_;
}

void* Context::global(const std::string& name, size_t bytes, void (*init)(void*), void (*fini)(void*)) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = globals_.find(name);
  if (it != globals_.end()) return it->second.bytes == bytes ? it->second.mem.get() : nullptr;
  Global g{std::unique_ptr<uint8_t[]>(new uint8_t[bytes == 0 ? 1 : bytes]), bytes, fini};
  std::memset(g.mem.get(), 0, bytes);
  if (init != nullptr) init(g.mem.get());
  void* p = g.mem.get();
  globals_.emplace(name, std::move(g));
  order_.push_back(name);
  return p;
}

void* Context::global_or_null(const std::string& name) const {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = globals_.find(name);
  return it == globals_.end() ? nullptr : it->second.mem.get();
}

size_t Context::num_globals() const {
  std::lock_guard<std::mutex> lk(mu_);
  return globals_.size();
}

Context::~Context() {
  pool_.reset();  // joins the workers before anything they might touch goes away
  for (auto it = order_.rbegin(); it != order_.rend(); ++it) {
    auto g = globals_.find(*it);
    if (g != globals_.end() && g->second.fini != nullptr) g->second.fini(g->second.mem.get());
  }
}

}  // namespace rt
}  // namespace b2
