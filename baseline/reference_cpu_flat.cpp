// Times the reference's own CPU kernels on the flat-gradient workload of stellatrain_b200/bench_cpu_flat.py.
//
// Links against the unmodified reference built by baseline/build_reference.sh (libfasterdp_core.so) and calls its
// classes through its own headers: add_arrays (backend/src/misc/array_util.h:12), ThresholdvCompressor16 /
// ThresholdvCompressor / TopkCompressor ::compress (backend/src/compress/*.h) and Adam::optimize_raw
// (backend/src/optim/adam.h).  One step is what the reference's gather, compress and optimise stages do for one tensor
// on one node (backend/src/engine/modules/cpu_gather.cpp:63-82, compress.cpp:44-55 and 172-188, cpu_optimize.cpp:103-108):
//
//     a = g + r;  (idx, val) = compress(a, k);  a[idx] = 0;  r = a;  adam(param, idx, val)
//
// Workload: 11,689,512 fp32 elements ~ N(0, 1e-2), k = 1 %, Adam lr 1e-3, 20 steps, one tensor, world size 1; the
// reference's thread pool has 32 workers as on its node master (backend/src/engine/config.h:7).
// Prints one JSON line per compressor with the median milliseconds per step.
//
// With a third argument (a directory) it also writes the input of the first step (input.f32) and what each compressor
// selected from it (<method>.idx.u32, <method>.val.f32), so that another implementation can be compared on the same data.
#include <algorithm>
#include <chrono>
#include <fstream>
#include <cstdio>
#include <cstring>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "compress/thresholdv.h"
#include "compress/thresholdv16.h"
#include "compress/topk.h"
#include "engine/threadpool.h"
#include "misc/array_util.h"
#include "optim/adam.h"
#include "optim/sgd.h"

int main(int argc, char** argv) {
  const size_t n = argc > 1 ? std::stoull(argv[1]) : 11689512ull;
  const int steps = argc > 2 ? std::atoi(argv[2]) : 20;
  const uint32_t k = static_cast<uint32_t>(std::max<size_t>(1, n / 100));
  const std::string dump = argc > 3 ? argv[3] : "";
  auto write = [&dump](const std::string& name, const void* data, size_t bytes) {
    std::ofstream f(dump + "/" + name, std::ios::binary);
    f.write(static_cast<const char*>(data), static_cast<std::streamsize>(bytes));
  };
  std::unique_ptr<ThreadPool> pool = std::make_unique<ThreadPool>(32);

  for (const std::string method : {"thresholdv16", "thresholdv", "topk"}) {
    std::unique_ptr<Compressor> comp;
    if (method == "thresholdv16") comp = std::make_unique<ThresholdvCompressor16>(pool);
    else if (method == "thresholdv") comp = std::make_unique<ThresholdvCompressor>(pool);
    else comp = std::make_unique<TopkCompressor>(pool);
    Adam adam;
    std::string lr = "lr";
    adam.configure(lr, 1e-3f);

    std::vector<float> grad(n), acc(n), resid(n, 0.f), param(n, 0.f), val(k);
    std::vector<uint32_t> idx(k);
    std::mt19937 rng(0);
    std::normal_distribution<float> dist(0.f, 1e-2f);
    std::vector<double> ms;
    size_t sent = 0;
    for (int s = 0; s < steps; ++s) {
      for (auto& g : grad) g = dist(rng);
      if (!dump.empty() && method == "thresholdv16") {
        std::ofstream f(dump + "/grads.f32", s == 0 ? std::ios::binary : std::ios::binary | std::ios::app);
        f.write(reinterpret_cast<const char*>(grad.data()), static_cast<std::streamsize>(n * sizeof(float)));
      }
      std::memcpy(acc.data(), grad.data(), n * sizeof(float));      // the gradient as it lands in the shared slot (not timed)
      const auto t0 = std::chrono::steady_clock::now();
      add_arrays(acc.data(), resid.data(), n);
      const size_t cnt = comp->compress("flat", {acc.data(), n}, k, {idx.data(), k}, {val.data(), k}, 0);
      if (s == 0 && !dump.empty()) {
        write("input.f32", grad.data(), n * sizeof(float));
        write(method + ".idx.u32", idx.data(), cnt * sizeof(uint32_t));
        write(method + ".val.f32", val.data(), cnt * sizeof(float));
        if (method == "thresholdv") {
          // the reference's optimisers on this selection, two calls each from zero parameters (the second call
          // exercises Adam's step counter and SGD's momentum buffer): parameter values at the selected indices
          std::string opt_lr = "lr", opt_mom = "momentum";
          Adam a2;
          a2.configure(opt_lr, 1e-3f);
          SGD s2;
          s2.configure(opt_lr, 0.1f);
          s2.configure(opt_mom, 0.9f);
          std::vector<float> pa(n, 0.f), ps(n, 0.f), out(cnt);
          for (int rep = 0; rep < 2; ++rep) {
            a2.optimize_raw(pa.data(), static_cast<uint32_t>(n), "parity", val.data(), idx.data(), static_cast<uint32_t>(cnt));
            s2.optimize_raw(ps.data(), static_cast<uint32_t>(n), "parity", val.data(), idx.data(), static_cast<uint32_t>(cnt));
          }
          for (size_t j = 0; j < cnt; ++j) out[j] = pa[idx[j]];
          write("adam.param.f32", out.data(), cnt * sizeof(float));
          for (size_t j = 0; j < cnt; ++j) out[j] = ps[idx[j]];
          write("sgd.param.f32", out.data(), cnt * sizeof(float));
        }
      }
      for (size_t j = 0; j < cnt; ++j) acc[idx[j]] = 0.f;
      std::memcpy(resid.data(), acc.data(), n * sizeof(float));
      adam.optimize_raw(param.data(), static_cast<uint32_t>(n), "flat", val.data(), idx.data(), static_cast<uint32_t>(cnt));
      ms.push_back(std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
      sent += cnt;
    }
    if (!dump.empty()) {
      write(method + ".final_param.f32", param.data(), n * sizeof(float));
      write(method + ".final_resid.f32", resid.data(), n * sizeof(float));
    }
    std::sort(ms.begin(), ms.end());
    std::printf("{\"impl\": \"reference\", \"method\": \"%s\", \"numel\": %zu, \"steps\": %d, \"k\": %u, "
                "\"ms_per_step_median\": %.3f, \"sent_fraction\": %.5f}\n",
                method.c_str(), n, steps, k, ms[ms.size() / 2], static_cast<double>(sent) / (static_cast<double>(steps) * n));
    std::fflush(stdout);
  }
  std::_Exit(0);   // the reference's thread pool has no orderly shutdown in this use
}
