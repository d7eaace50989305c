// A stand-in for the CUDA runtime calls of cuda_api.h on machines without a GPU.
//
// Every stream is a worker thread that runs its queue in order; the null stream runs work at once on the caller;
// events carry a generation counter; "device memory" is host memory.  An optional delay per copy makes the streams
// fall behind the host the way a busy GPU does, which is the situation the slot and ordering rules of the engine
// exist for.  Used by the tests of the engine's own device copies; never installed unless a test asks for it.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <future>
#include <mutex>
#include <thread>

#include "cuda_api.h"

namespace stc {

namespace {

std::atomic<int> copy_delay_ms{0};
std::atomic<long> copies_d2h{0}, copies_h2d{0}, host_funcs{0};

struct FakeStream {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::function<void()>> q;
  bool stop = false;
  std::thread th;
  FakeStream() : th([this] { run(); }) {}
  ~FakeStream() {
    {
      std::lock_guard<std::mutex> lk(mu);
      stop = true;
    }
    cv.notify_all();
    th.join();
  }
  void run() {
    for (;;) {
      std::function<void()> fn;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [this] { return stop || !q.empty(); });
        if (q.empty()) return;
        fn = std::move(q.front());
        q.pop_front();
      }
      fn();
    }
  }
  void push(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> lk(mu);
      q.push_back(std::move(fn));
    }
    cv.notify_one();
  }
};

struct FakeEvent {
  std::mutex mu;
  std::condition_variable cv;
  uint64_t recorded = 0, done = 0;
};

void on_stream(void* stream, std::function<void()> fn) {
  if (stream) static_cast<FakeStream*>(stream)->push(std::move(fn));
  else fn();
}

int f_stream_create(void** s) { *s = new FakeStream(); return 0; }
int f_stream_destroy(void* s) { delete static_cast<FakeStream*>(s); return 0; }
int f_stream_sync(void* s) {
  if (!s) return 0;
  auto done = std::make_shared<std::promise<void>>();
  auto fut = done->get_future();
  on_stream(s, [done] { done->set_value(); });
  return fut.wait_for(std::chrono::seconds(30)) == std::future_status::ready ? 0 : 1;
}
int f_event_create(void** e) { *e = new FakeEvent(); return 0; }
int f_event_destroy(void* e) { delete static_cast<FakeEvent*>(e); return 0; }
int f_event_record(void* e, void* s) {
  auto* ev = static_cast<FakeEvent*>(e);
  uint64_t gen;
  {
    std::lock_guard<std::mutex> lk(ev->mu);
    gen = ++ev->recorded;
  }
  on_stream(s, [ev, gen] {
    {
      std::lock_guard<std::mutex> lk(ev->mu);
      if (ev->done < gen) ev->done = gen;
    }
    ev->cv.notify_all();
  });
  return 0;
}
int f_stream_wait(void* s, void* e) {
  auto* ev = static_cast<FakeEvent*>(e);
  uint64_t gen;
  {
    std::lock_guard<std::mutex> lk(ev->mu);
    gen = ev->recorded;
  }
  on_stream(s, [ev, gen] {
    std::unique_lock<std::mutex> lk(ev->mu);
    ev->cv.wait_for(lk, std::chrono::seconds(30), [ev, gen] { return ev->done >= gen; });
  });
  return 0;
}
int f_copy(void* dst, const void* src, size_t n, void* s, std::atomic<long>* counter) {
  on_stream(s, [dst, src, n, counter] {
    if (const int ms = copy_delay_ms.load()) std::this_thread::sleep_for(std::chrono::milliseconds(ms));
    std::memcpy(dst, src, n);
    counter->fetch_add(1);
  });
  return 0;
}
int f_d2h(void* dst, const void* src, size_t n, void* s) { return f_copy(dst, src, n, s, &copies_d2h); }
int f_h2d(void* dst, const void* src, size_t n, void* s) { return f_copy(dst, src, n, s, &copies_h2d); }
int f_host_func(void* s, void (*fn)(void*), void* user) {
  on_stream(s, [fn, user] {
    host_funcs.fetch_add(1);   // before the call: what the callback starts may finish before it returns
    fn(user);
  });
  return 0;
}

std::atomic<int> fake_device{0};
int f_get_device(int* d) { *d = fake_device.load(); return 0; }
int f_set_device(int d) { fake_device = d; return 0; }

const CudaApi kFakeTable = {f_stream_create, f_stream_destroy, f_stream_sync, f_event_create, f_event_destroy,
                            f_event_record,  f_stream_wait,    f_d2h,         f_h2d,          f_host_func,
                            f_get_device,    f_set_device};

}  // namespace

void install_fake_cuda(int delay_ms) {
  copy_delay_ms = delay_ms;
  copies_d2h = copies_h2d = host_funcs = 0;
  set_cuda_api(&kFakeTable);
}
void remove_fake_cuda() { set_cuda_api(nullptr); }
void fake_cuda_counters(long* d2h, long* h2d, long* funcs) {
  *d2h = copies_d2h.load();
  *h2d = copies_h2d.load();
  *funcs = host_funcs.load();
}

}  // namespace stc
