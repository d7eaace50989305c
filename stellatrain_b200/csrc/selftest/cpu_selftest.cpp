// Stand-alone exerciser of the CPU tier for the sanitizers (no Python, no CUDA).
//
// Built by stellatrain_b200/_build.py::build_selftest with -fsanitize=thread or -fsanitize=address and run
// by tests/test_sanitizers.py.  The reference has no sanitizer target (its CMake build knows only
// -march=broadwell, backend/CMakeLists.txt:28-29) and its barrier code loses wake-ups; here the thread
// pool, the task pipeline with both staleness settings, gradient accumulation and a two-node ring over
// loopback TCP (two engines on two threads of this process) all run under the race detector.
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../core/cuda_api.h"
#include "../core/engine.h"
#include "../core/threadpool.h"
#include "../cpu/compressors.h"
#include "../cpu/optimizers.h"
#include "../telemetry/telemetry.h"
#include "../comm/net_util.h"

using namespace stc;

namespace {

#define CHECK(cond)                                                                          \
  do {                                                                                       \
    if (!(cond)) throw std::runtime_error(std::string("check failed: ") + #cond + " at line " + std::to_string(__LINE__)); \
  } while (0)

void test_pool() {
  ThreadPool pool(4);
  std::atomic<int> sum{0};
  std::vector<std::future<void>> futs;
  for (int i = 0; i < 200; ++i) futs.push_back(pool.enqueue(i % 7, [&sum, i] { sum += i; }));
  for (auto& f : futs) f.get();
  CHECK(sum == 199 * 200 / 2);
  // nested parallel_for from inside a worker must not deadlock
  std::vector<int> hits(1 << 16, 0);
  auto outer = pool.enqueue(0, [&] {
    pool.parallel_for(hits.size(), 1024, [&](size_t b, size_t e) {
      for (size_t i = b; i < e; ++i) hits[i] += 1;
    });
  });
  outer.get();
  for (int h : hits) CHECK(h == 1);
}

void test_kernels() {
  ThreadPool pool(3);
  const size_t n = 100000;
  std::vector<float> a(n);
  uint32_t s = 12345;
  for (auto& x : a) { s = s * 1664525u + 1013904223u; x = (static_cast<float>(s >> 8) / 8388608.0f - 1.0f) * 1e-2f; }
  for (const char* method : {"topk", "thresholdv", "thresholdv16", "randomk"}) {
    auto c = make_compressor(method, &pool);
    const uint32_t k = 1000;
    std::vector<uint32_t> idx(k);
    std::vector<float> val(k);
    for (int rep = 0; rep < 3; ++rep) {
      const size_t got = c->compress("t", a.data(), n, k, idx.data(), val.data(), 0);
      // threshold-v may under-fill, down to nothing, while its threshold adapts (as the reference's does)
      if (!(got <= k && (got > 0 || std::string(method) == "thresholdv")))
        throw std::runtime_error(std::string(method) + " returned " + std::to_string(got) + " pairs for k = " + std::to_string(k));
      for (size_t j = 0; j < got; ++j) CHECK(idx[j] < n && val[j] == a[idx[j]]);
    }
  }
  for (const char* kind : {"sgd", "adam"}) {
    auto o = make_optimizer(kind);
    o->configure("lr", 0.1f);
    std::vector<float> p(1000, 1.0f), g(10, 0.5f);
    std::vector<uint32_t> idx = {1, 5, 9, 100, 200, 300, 400, 500, 600, 999};
    o->optimize_raw(p.data(), 1000, "w", g.data(), idx.data(), 10);
    CHECK(p[1] < 1.0f && p[2] == 1.0f);
  }
}

struct Node {
  CpuEngine engine;
  std::vector<std::vector<float>> params;
  std::vector<int> index;
};

void run_node(Node& node, EngineOptions opt, int iters, std::string* error) {
  try {
    node.engine.configure(opt);
    node.engine.set_optimizer("adam");
    node.engine.sparse_optimizer()->configure("lr", 1e-2f);
    const std::vector<uint32_t> sizes = {4096, 17, 70000, 300, 1};
    node.params.resize(sizes.size());
    for (size_t i = 0; i < sizes.size(); ++i) {
      node.params[i].assign(sizes[i], 0.5f);
      node.index.push_back(node.engine.pre_train_init(static_cast<int>(i), "p" + std::to_string(i), sizes[i], node.params[i].data()));
    }
    std::vector<float> grad;
    for (int it = 0; it < iters; ++it) {
      for (size_t i = 0; i < sizes.size(); ++i) node.engine.pre_forward_process(node.index[i]);        // forward
      for (int micro = 0; micro < opt.grad_accumulation; ++micro)
        for (size_t r = sizes.size(); r-- > 0;) {                                                      // backward
          grad.assign(sizes[r], 0.f);
          for (uint32_t j = 0; j < sizes[r]; ++j)
            grad[j] = 1e-3f * static_cast<float>(((j * 2654435761u) >> 20) % 97 + 1) * (opt.rank + 1);
          node.engine.post_backward_process(node.index[r], grad.data());
        }
    }
    node.engine.synchronize();
    for (size_t i = 0; i < sizes.size(); ++i) {
      CHECK(node.engine.model_version(node.index[i]) == iters);
      bool moved = false;
      for (float x : node.params[i]) { CHECK(std::isfinite(x)); moved |= x != 0.5f; }
      CHECK(moved);
    }
  } catch (const std::exception& e) {
    *error = e.what();
  }
}

void test_single_node(int staleness, int accumulation, const char* method) {
  Node node;
  EngineOptions o;
  o.session = static_cast<int64_t>(getpid()) * 100 + staleness * 10 + accumulation;
  o.staleness = staleness;
  o.grad_accumulation = accumulation;
  o.method = method;
  o.ratio = 0.9;
  o.workers = 4;
  o.data_bytes = 16u << 20;
  o.timeout_ms = 20000;
  std::string err;
  run_node(node, o, 12, &err);
  if (!err.empty()) throw std::runtime_error(std::string("single node (") + method + "): " + err);
}

// The engine's own device copies against the stand-in runtime (streams are threads, device memory is host memory):
// gradient copies with host callbacks that start the tasks, parameter copies behind CopyOut, copy streams that lag.
void test_device_copies(int staleness) {
  install_fake_cuda(1);
  std::string err;
  {
    CpuEngine engine;
    EngineOptions o;
    o.session = static_cast<int64_t>(getpid()) * 100 + 70 + staleness;
    o.staleness = staleness;
    o.method = "thresholdv16";
    o.ratio = 0.9;
    o.workers = 4;
    o.data_bytes = 16u << 20;
    o.timeout_ms = 20000;
    try {
      engine.configure(o);
      engine.set_optimizer("adam");
      engine.sparse_optimizer()->configure("lr", 1e-2f);
      const std::vector<uint32_t> sizes = {4096, 17, 70000};
      std::vector<std::vector<float>> device(sizes.size());
      std::vector<std::vector<std::vector<float>>> grads(sizes.size());
      const int iters = 8;
      for (size_t i = 0; i < sizes.size(); ++i) {
        device[i].assign(sizes[i], 0.5f);
        const int idx = engine.pre_train_init(static_cast<int>(i), "d" + std::to_string(i), sizes[i], nullptr, device[i].data());
        CHECK(idx == static_cast<int>(i));
        engine.attach_device_param(idx, device[i].data());
        grads[i].assign(iters, std::vector<float>(sizes[i]));
      }
      for (int it = 0; it < iters; ++it) {
        for (size_t i = 0; i < sizes.size(); ++i) engine.pre_forward_process(static_cast<int>(i));
        for (size_t r = sizes.size(); r-- > 0;) {
          std::vector<float>& g = grads[r][it];                  // stays alive until the copy stream has read it
          for (uint32_t j = 0; j < sizes[r]; ++j) g[j] = 1e-3f * static_cast<float>(((j * 2654435761u) >> 20) % 97 + 1 + it);
          engine.post_backward_device(static_cast<int>(r), g.data(), nullptr, nullptr);
        }
      }
      engine.synchronize();
      for (size_t i = 0; i < sizes.size(); ++i) {
        CHECK(engine.model_version(static_cast<int>(i)) == iters);
        bool moved = false;
        for (float x : device[i]) { CHECK(std::isfinite(x)); moved |= x != 0.5f; }
        CHECK(moved);
      }
      long d2h, h2d, funcs;
      fake_cuda_counters(&d2h, &h2d, &funcs);
      CHECK(d2h == 3 * iters && h2d == 3 * iters);
    } catch (const std::exception& e) {
      err = e.what();
    }
  }   // the engine (and its copy streams) goes away before the stand-in runtime is removed
  remove_fake_cuda();
  if (!err.empty()) throw std::runtime_error("device copies, staleness " + std::to_string(staleness) + ": " + err);
}

// Several tensors as one bundle (one task per iteration, per-member selection): host gradients handed in member by
// member, and the engine's own copies of all members behind one callback.
void test_bundle(bool device_copies) {
  if (device_copies) install_fake_cuda(1);
  std::string err;
  {
    CpuEngine engine;
    EngineOptions o;
    o.session = static_cast<int64_t>(getpid()) * 100 + 80 + (device_copies ? 1 : 0);
    o.staleness = 1;
    o.method = "thresholdv16";
    o.ratio = 0.9;
    o.workers = 4;
    o.data_bytes = 16u << 20;
    o.timeout_ms = 20000;
    try {
      engine.configure(o);
      engine.set_optimizer("adam");
      engine.sparse_optimizer()->configure("lr", 1e-2f);
      const std::vector<uint32_t> sizes = {4096, 17, 70000, 300};
      std::vector<uint32_t> offsets;
      uint32_t total = 0;
      for (uint32_t n : sizes) { offsets.push_back(total); total += (n + 15u) / 16u * 16u; }
      std::vector<float> init(total, 0.f);
      std::vector<std::vector<float>> member(sizes.size());
      std::vector<std::string> keys;
      std::vector<float*> host_ptrs;
      std::vector<void*> dev_ptrs;
      for (size_t m = 0; m < sizes.size(); ++m) {
        member[m].assign(sizes[m], 0.5f);
        std::fill(init.begin() + offsets[m], init.begin() + offsets[m] + sizes[m], 0.5f);
        keys.push_back(std::to_string(m) + "@m" + std::to_string(m));
        host_ptrs.push_back(member[m].data());
        dev_ptrs.push_back(member[m].data());
      }
      const int b = engine.pre_train_init(0, "bundle", total, nullptr, init.data());
      engine.set_param_members(b, keys, offsets, sizes, device_copies ? std::vector<float*>{} : host_ptrs);
      if (device_copies) engine.attach_device_members(b, dev_ptrs);
      const int iters = 8;
      std::vector<std::vector<std::vector<float>>> grads(iters, std::vector<std::vector<float>>(sizes.size()));
      for (int it = 0; it < iters; ++it) {
        engine.pre_forward_process(b);
        std::vector<const void*> ptrs;
        for (size_t m = 0; m < sizes.size(); ++m) {
          std::vector<float>& g = grads[it][m];                  // alive until the copy stream has read it
          g.resize(sizes[m]);
          for (uint32_t j = 0; j < sizes[m]; ++j) g[j] = 1e-3f * static_cast<float>(((j * 2654435761u) >> 20) % 97 + 1 + it + m);
          ptrs.push_back(g.data());
        }
        if (device_copies) {
          engine.post_backward_device_members(b, ptrs, nullptr, nullptr);
        } else {
          for (size_t m = sizes.size(); m-- > 0;) engine.post_backward_member(b, static_cast<int>(m), grads[it][m].data());
        }
      }
      engine.synchronize();
      CHECK(engine.model_version(b) == iters && engine.num_params() == 1);
      for (size_t m = 0; m < sizes.size(); ++m) {
        bool moved = false;
        for (float x : member[m]) { CHECK(std::isfinite(x)); moved |= x != 0.5f; }
        CHECK(moved);
      }
    } catch (const std::exception& e) {
      err = e.what();
    }
  }
  if (device_copies) remove_fake_cuda();
  if (!err.empty()) throw std::runtime_error(std::string("bundle, ") + (device_copies ? "device" : "host") + " copies: " + err);
}

// Telemetry client against a stand-in controller (a thread that acknowledges every frame and answers every fifth
// report with an instruction): ordinary shutdown with reports still queued, and a client whose last owner is a
// callback queued in its own thread, so that it is destroyed on that thread.
void test_telemetry(uint16_t port) {
  uint16_t bound = 0;
  int lfd = tcp_listen(port, &bound, true);
  CHECK(lfd >= 0);
  std::atomic<bool> stop{false};
  std::atomic<int> reports{0};
  std::thread server([&] {
    std::vector<std::thread> conns;
    while (!stop) {
      const int fd = tcp_accept(lfd, 100);
      if (fd < 0) continue;
      conns.emplace_back([fd, &stop, &reports] {
        int cfd = fd;
        while (!stop) {
          if (!wait_readable(cfd, 100)) continue;
          TelemetryFrame f;
          if (!recv_all(cfd, &f, sizeof(f), 1000) || f.magic != kTelemetryMagic) break;
          std::vector<unsigned char> payload(f.payload_len);
          if (f.payload_len && !recv_all(cfd, payload.data(), f.payload_len, 1000)) break;
          if (f.type == kTelLocal && ++reports % 5 == 0) {
            Instruction ins{};
            ins.iter_effective_since = 42;
            ins.config = TrainConfig{8, 1, 0.95};
            TelemetryFrame r{kTelemetryMagic, kTelInstruction, sizeof(ins)};
            if (!send_all(cfd, &r, sizeof(r), 1000) || !send_all(cfd, &ins, sizeof(ins), 1000)) break;
          } else {
            TelemetryFrame r{kTelemetryMagic, kTelOk, 0};
            if (!send_all(cfd, &r, sizeof(r), 1000)) break;
          }
        }
        close_fd(cfd);
      });
    }
    for (auto& c : conns) c.join();
  });
  const std::string uri = "127.0.0.1:" + std::to_string(bound);
  std::atomic<int> instructions{0};
  {
    TelemetryClient client(uri, 0, "cpu", 0, 0, 2000);
    for (int i = 0; i < 50; ++i)
      client.report(i, TrainConfig{4, 1, 0.9}, TrainMeasurement{1, 1, 1, 1, 0, 0},
                    [&instructions](uint64_t since, const TrainConfig& c) { if (since == 42 && c.ubatch_size == 8) ++instructions; });
    const auto t0 = std::chrono::steady_clock::now();
    while (client.sent() < 50 && std::chrono::steady_clock::now() - t0 < std::chrono::seconds(10))
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    CHECK(client.sent() == 50 && instructions == 10);
    for (int i = 0; i < 200; ++i) client.report(100 + i, TrainConfig{4, 1, 0.9}, TrainMeasurement{}, nullptr);
  }   // destroyed with reports still queued: joins its thread
  const uint64_t before = TelemetryClient::destroyed_on_own_thread();
  for (int round = 0; round < 3; ++round) {
    auto owner = std::make_shared<std::unique_ptr<TelemetryClient>>(std::make_unique<TelemetryClient>(uri, 1, "cpu", 0, 1, 2000));
    for (int i = 0; i < 100; ++i)
      (*owner)->report(i, TrainConfig{4, 1, 0.9}, TrainMeasurement{}, [owner](uint64_t, const TrainConfig&) {});
    owner.reset();   // the queued callbacks are now the only owners
  }
  const auto t1 = std::chrono::steady_clock::now();
  while (TelemetryClient::destroyed_on_own_thread() < before + 3 && std::chrono::steady_clock::now() - t1 < std::chrono::seconds(20))
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
  CHECK(TelemetryClient::destroyed_on_own_thread() == before + 3);
  std::this_thread::sleep_for(std::chrono::milliseconds(200));   // the released threads finish on their shared blocks
  stop = true;
  server.join();
  close_fd(lfd);
}

void test_two_nodes(uint16_t port) {
  Node nodes[2];
  std::string errs[2];
  std::thread th[2];
  for (int r = 0; r < 2; ++r) {
    EngineOptions o;
    o.master_port = port;
    o.world = 2;
    o.rank = r;
    o.session = static_cast<int64_t>(getpid()) * 100 + 50 + r;
    o.staleness = 1;
    o.method = "thresholdv16";
    o.ratio = 0.9;
    o.workers = 4;
    o.data_bytes = 16u << 20;
    o.timeout_ms = 20000;
    th[r] = std::thread([&nodes, &errs, o, r] { run_node(nodes[r], o, 10, &errs[r]); });
  }
  for (auto& t : th) t.join();
  for (int r = 0; r < 2; ++r)
    if (!errs[r].empty()) throw std::runtime_error("two nodes, rank " + std::to_string(r) + ": " + errs[r]);
  // both nodes applied the same merged updates to the same start values
  for (size_t i = 0; i < nodes[0].params.size(); ++i)
    for (size_t j = 0; j < nodes[0].params[i].size(); ++j) CHECK(nodes[0].params[i][j] == nodes[1].params[i][j]);
}

}  // namespace

int main(int argc, char** argv) {
  const uint16_t port = argc > 1 ? static_cast<uint16_t>(std::atoi(argv[1])) : 45123;
  try {
    test_pool();
    test_kernels();
    test_single_node(0, 1, "topk");
    test_single_node(1, 1, "thresholdv16");
    test_single_node(1, 2, "thresholdv");
    test_device_copies(0);
    test_device_copies(1);
    test_bundle(false);
    test_bundle(true);
    test_two_nodes(port);
    test_telemetry(static_cast<uint16_t>(port + 7));
  } catch (const std::exception& e) {
    std::fprintf(stderr, "selftest FAILED: %s\n", e.what());
    return 1;
  }
  std::printf("selftest ok\n");
  return 0;
}
