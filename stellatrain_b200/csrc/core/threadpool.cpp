#include "threadpool.h"

#include <pthread.h>
#include <signal.h>

#include <algorithm>

namespace stc {

static thread_local int tl_worker_id = -1;

int ThreadPool::worker_id() { return tl_worker_id; }

ThreadPool::ThreadPool(size_t workers, const std::string& name_prefix) {
  workers = std::max<size_t>(1, workers);
  threads_.reserve(workers);
  for (size_t i = 0; i < workers; ++i)
    threads_.emplace_back([this, i, name_prefix] { worker_main(static_cast<int>(i), name_prefix + "-" + std::to_string(i)); });
}

ThreadPool::~ThreadPool() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
    while (!queue_.empty()) {   // dropped jobs report broken_promise to whoever waits on them
      queue_.pop();
    }
  }
  cv_.notify_all();
  for (auto& t : threads_) t.join();
}

size_t ThreadPool::pending() const {
  std::lock_guard<std::mutex> lk(mu_);
  return queue_.size();
}

std::future<void> ThreadPool::enqueue(int64_t priority, std::function<void()> fn) {
  auto done = std::make_shared<std::promise<void>>();
  std::future<void> fut = done->get_future();
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (stop_) throw std::runtime_error("enqueue on a stopped ThreadPool");
    queue_.push(Job{priority, seq_++, std::move(fn), std::move(done)});
  }
  cv_.notify_one();
  return fut;
}

bool ThreadPool::run_one() {
  Job job;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (queue_.empty()) return false;
    job = queue_.top();
    queue_.pop();
  }
  try {
    job.fn();
    job.done->set_value();
  } catch (...) {
    job.done->set_exception(std::current_exception());
  }
  return true;
}

void ThreadPool::worker_main(int id, const std::string& name) {
  tl_worker_id = id;
  pthread_setname_np(pthread_self(), name.substr(0, 15).c_str());
  // termination signals are the main thread's business (cf. reference threadpool.cpp:16-20)
  sigset_t set;
  sigemptyset(&set);
  sigaddset(&set, SIGTERM);
  sigaddset(&set, SIGHUP);
  pthread_sigmask(SIG_BLOCK, &set, nullptr);
  for (;;) {
    Job job;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [this] { return stop_ || !queue_.empty(); });
      if (stop_ && queue_.empty()) return;
      job = queue_.top();
      queue_.pop();
    }
    try {
      job.fn();
      job.done->set_value();
    } catch (...) {
      job.done->set_exception(std::current_exception());
    }
  }
}

void ThreadPool::parallel_for(size_t n, size_t grain, const std::function<void(size_t, size_t)>& fn) {
  if (n == 0) return;
  grain = std::max<size_t>(1, grain);
  const size_t max_parts = threads_.size() + 1;
  size_t parts = std::min(max_parts, (n + grain - 1) / grain);
  if (parts <= 1) {
    fn(0, n);
    return;
  }
  const size_t step = (n + parts - 1) / parts;
  struct Shared {
    std::mutex mu;
    std::condition_variable cv;
    size_t left;
    std::exception_ptr err;
  };
  auto sh = std::make_shared<Shared>();
  sh->left = parts - 1;
  for (size_t p = 1; p < parts; ++p) {
    const size_t b = p * step, e = std::min(n, b + step);
    enqueue(INT64_MIN, [sh, b, e, &fn] {   // helpers of a running job go first
      try {
        if (b < e) fn(b, e);
      } catch (...) {
        std::lock_guard<std::mutex> lk(sh->mu);
        sh->err = std::current_exception();
      }
      std::lock_guard<std::mutex> lk(sh->mu);
      if (--sh->left == 0) sh->cv.notify_all();
    });
  }
  fn(0, std::min(n, step));
  // a worker that waits here helps to drain the queue, so nested use cannot deadlock the pool
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(sh->mu);
      if (sh->left == 0) break;
      if (tl_worker_id < 0) {
        sh->cv.wait(lk, [&] { return sh->left == 0; });
        break;
      }
    }
    if (!run_one()) std::this_thread::yield();
  }
  if (sh->err) std::rethrow_exception(sh->err);
}

}  // namespace stc
