// Priority thread pool of the CPU tier.
//
// Same contract as the reference's pool (backend/src/engine/threadpool.h:18-99): jobs carry an integer
// priority, the smallest runs first (older iteration, then earlier layer), ties run in submission
// order, every worker has a stable id for per-worker resources.  Added here: parallel_for for the SIMD
// kernels, and a bounded shutdown that drops queued jobs instead of blocking on them.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <future>
#include <mutex>
#include <queue>
#include <string>
#include <thread>
#include <vector>

namespace stc {

class ThreadPool {
 public:
  explicit ThreadPool(size_t workers, const std::string& name_prefix = "Worker");
  ~ThreadPool();
  ThreadPool(const ThreadPool&) = delete;
  ThreadPool& operator=(const ThreadPool&) = delete;

  std::future<void> enqueue(int64_t priority, std::function<void()> fn);
  // Splits [0, n) into ranges of at least `grain` and runs fn(begin, end) on the workers and on the
  // calling thread; returns when every range is done.  Safe to call from a worker.
  void parallel_for(size_t n, size_t grain, const std::function<void(size_t, size_t)>& fn);

  size_t size() const { return threads_.size(); }
  size_t pending() const;
  static int worker_id();   // -1 outside a worker

 private:
  struct Job {
    int64_t priority;
    uint64_t seq;
    std::function<void()> fn;
    std::shared_ptr<std::promise<void>> done;
  };
  struct Later {
    bool operator()(const Job& a, const Job& b) const {
      return a.priority != b.priority ? a.priority > b.priority : a.seq > b.seq;
    }
  };
  void worker_main(int id, const std::string& name);
  bool run_one();

  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::priority_queue<Job, std::vector<Job>, Later> queue_;
  std::vector<std::thread> threads_;
  uint64_t seq_ = 0;
  bool stop_ = false;
};

}  // namespace stc
