// pybind11 surface of the CPU-offload tier (module `_Ccpu`).  Arrays cross the boundary as raw host
// addresses (integers) owned by Python (torch / numpy), as in the GPU module.  Names follow the
// reference's binding where one exists (backend/src/python/pybind.cpp:18-103): classes SGD and Adam
// with `optimize`, engine functions configure / pre_train_init / pre_forward_process /
// post_backward_process / synchronize / barrier / compress / set_optimizer / configure_optimizer /
// configure_compression(_ratio) / force_model_sync / gradient_accumulation.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <memory>
#include <mutex>

#include "comm/comm_manager.h"
#include "comm/net_util.h"
#include "core/config.h"
#include "core/cuda_api.h"
#include "core/engine.h"
#include "core/logger.h"
#include "core/shm_manager.h"
#include "core/task.h"
#include "core/threadpool.h"
#include "cpu/array_util.h"
#include "cpu/compressors.h"
#include "cpu/optimizers.h"
#include "cpu/xorshift.h"
#include "telemetry/telemetry.h"

namespace py = pybind11;
using namespace stc;

namespace {

template <typename T>
T* P(uint64_t v) { return reinterpret_cast<T*>(static_cast<uintptr_t>(v)); }

ThreadPool& shared_pool() {
  static ThreadPool pool(static_cast<size_t>(std::max(1l, cfg::env_long("STELLATRAIN_CPU_THREADS", 16) - 1)));
  return pool;
}

struct CompressorBox {
  std::unique_ptr<Compressor> c;
  explicit CompressorBox(const std::string& method) : c(make_compressor(method, &shared_pool())) {}
  size_t compress(const std::string& tensor, uint64_t src, size_t n, uint32_t k, uint64_t idx, uint64_t val) {
    py::gil_scoped_release rel;
    return c->compress(tensor, P<const float>(src), n, k, P<uint32_t>(idx), P<float>(val), 0);
  }
  size_t compress_ef(const std::string& tensor, uint64_t grad, uint64_t resid, size_t n, uint32_t k, uint64_t idx, uint64_t val) {
    py::gil_scoped_release rel;
    return compress_with_feedback(*c, tensor, P<const float>(grad), P<float>(resid), n, k, P<uint32_t>(idx), P<float>(val),
                                  &shared_pool());
  }
  py::dict state() {
    py::dict d;
    for (auto& kv : c->export_state()) d[py::str(kv.first)] = py::make_tuple(kv.second.tau, kv.second.tau_inc, kv.second.inited);
    return d;
  }
  void set_state(const std::map<std::string, std::tuple<float, float, bool>>& st) {
    std::map<std::string, ThresholdState> m;
    for (auto& kv : st) m[kv.first] = ThresholdState{std::get<0>(kv.second), std::get<1>(kv.second), std::get<2>(kv.second)};
    c->import_state(m);
  }
};

template <typename Opt>
void bind_optimizer(py::module_& m, const char* name) {
  py::class_<Opt>(m, name)
      .def(py::init([] {
        auto o = std::make_unique<Opt>();
        o->set_pool(&shared_pool());
        return o;
      }))
      .def("optimize", [](Opt& o, uint64_t param, uint32_t n, const std::string& tname, uint64_t grad, uint64_t idx, uint32_t cnt) {
        py::gil_scoped_release rel;
        o.optimize_raw(P<float>(param), n, tname, P<const float>(grad), P<const uint32_t>(idx), cnt);
      })
      .def("configure", [](Opt& o, const std::string& k, py::object v) {
        if (py::isinstance<py::bool_>(v)) o.configure(k, v.cast<bool>());
        else o.configure(k, v.cast<float>());
      })
      .def_property_readonly("lr", &Opt::lr);
}

// Runs jobs that append their tag to a list; used to observe the pool's ordering rule.
std::vector<int> pool_order_probe(const std::vector<int64_t>& priorities) {
  ThreadPool pool(1);
  std::vector<int> order;
  std::mutex mu, gate;
  gate.lock();
  auto blocker = pool.enqueue(INT64_MIN, [&] { std::lock_guard<std::mutex> g(gate); });   // holds the only worker
  std::vector<std::future<void>> futs;
  for (size_t i = 0; i < priorities.size(); ++i)
    futs.push_back(pool.enqueue(priorities[i], [&, i] { std::lock_guard<std::mutex> lk(mu); order.push_back(static_cast<int>(i)); }));
  gate.unlock();
  blocker.get();
  for (auto& f : futs) f.get();
  return order;
}

struct CommBox {
  std::unique_ptr<CommManager> c;
  std::mutex mu;
  std::vector<std::tuple<std::string, int, std::vector<uint32_t>, std::vector<float>>> inbox;
  CommBox(const std::string& addr, uint16_t port, int timeout_ms) : c(new CommManager(addr, port, timeout_ms)) {}
  void post(const std::string& key) {
    c->post_recv(key, [this](SparseMessage&& m) {
      std::lock_guard<std::mutex> lk(mu);
      inbox.emplace_back(m.key, m.flags, std::move(m.idx), std::move(m.val));
    });
  }
  py::list drain() {
    std::lock_guard<std::mutex> lk(mu);
    py::list out;
    for (auto& t : inbox) out.append(py::make_tuple(std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t)));
    inbox.clear();
    return out;
  }
};

}  // namespace

PYBIND11_MODULE(_Ccpu, m) {
  m.doc() = "CPU-offload tier: SIMD compressors and optimisers, thread pool, shm pool, TCP comm manager, telemetry";
  m.attr("__version__") = "1.0.0";
  m.def("best_isa", [] { return std::string(isa_name(best_isa())); });
  m.def("add_arrays", [](uint64_t dst, uint64_t src, size_t n) { add_arrays(P<float>(dst), P<const float>(src), n); });
  m.def("block_l1_norms", [](uint64_t x, size_t n, uint64_t out) { block_l1_norms(P<const float>(x), n, P<float>(out)); });
  m.def("encode_sparse", [](const std::vector<uint32_t>& idx, const std::vector<float>& val, uint32_t numel, bool allow_u16,
                            int value_format, bool allow_blocks) {
    if (idx.size() != val.size()) throw std::invalid_argument("idx and val differ in length");
    EncodedSparse e = encode_sparse(idx.data(), val.data(), idx.size(), numel, allow_u16, value_format, allow_blocks);
    return py::make_tuple(static_cast<int>(e.flags), py::bytes(reinterpret_cast<const char*>(e.payload.data()), e.payload.size()));
  }, py::arg("idx"), py::arg("val"), py::arg("tensor_numel"), py::arg("allow_u16") = true, py::arg("value_format") = 0,
        py::arg("allow_blocks") = true,
        "Payload of one gradient message: (flags, bytes).  Whole aligned runs of 16 indices become block ids.");
  m.def("decode_sparse", [](int flags, const std::string& payload, uint32_t numel) {
    std::vector<uint32_t> idx;
    std::vector<float> val;
    if (!decode_sparse(static_cast<uint8_t>(flags), reinterpret_cast<const unsigned char*>(payload.data()), payload.size(),
                       numel, &idx, &val))
      throw std::invalid_argument("malformed sparse payload");
    return py::make_tuple(idx, val);
  }, py::arg("flags"), py::arg("payload"), py::arg("tensor_numel") = 0);
  m.def("install_fake_cuda", &install_fake_cuda, py::arg("delay_ms") = 0,
        "Replace the CUDA runtime calls of the engine's device copies by worker threads over host memory (tests).");
  m.def("remove_fake_cuda", &remove_fake_cuda);
  m.def("fake_cuda_counters", [] {
    long a, b, c;
    fake_cuda_counters(&a, &b, &c);
    return py::make_tuple(a, b, c);
  });
  m.def("narrow_u32_to_u16", [](uint64_t s, uint64_t d, size_t n) { narrow_u32_to_u16(P<const uint32_t>(s), P<uint16_t>(d), n); });
  m.def("widen_u16_to_u32", [](uint64_t s, uint64_t d, size_t n) { widen_u16_to_u32(P<const uint16_t>(s), P<uint32_t>(d), n); });
  m.def("f32_to_f16", [](uint64_t s, uint64_t d, size_t n) { f32_to_f16(P<const float>(s), P<uint16_t>(d), n); });
  m.def("f16_to_f32", [](uint64_t s, uint64_t d, size_t n) { f16_to_f32(P<const uint16_t>(s), P<float>(d), n); });
  m.def("f32_to_bf16", [](uint64_t s, uint64_t d, size_t n) { f32_to_bf16(P<const float>(s), P<uint16_t>(d), n); });
  m.def("bf16_to_f32", [](uint64_t s, uint64_t d, size_t n) { bf16_to_f32(P<const uint16_t>(s), P<float>(d), n); });
  m.def("sample_without_replacement", [](uint32_t n, uint32_t k, uint64_t seed) {
    std::vector<uint32_t> out(k);
    sample_without_replacement(n, k, seed, out.data());
    return out;
  });
  m.def("xorshift_stream", [](uint64_t seed, int count) {
    XorShift128Plus g(seed);
    std::vector<uint64_t> out(count);
    for (auto& v : out) v = g.next();
    return out;
  });
  m.def("xorshift_lanes8", [](uint64_t seed, int rounds) {
    XorShift128PlusLanes<8> g(seed);
    std::vector<uint64_t> out(static_cast<size_t>(rounds) * 8);
    for (int r = 0; r < rounds; ++r) g.next(out.data() + r * 8);
    return out;
  });
  m.def("merge_streams", [](const std::vector<uint64_t>& idx, const std::vector<uint64_t>& val, const std::vector<size_t>& counts,
                            const std::vector<float>& weights, size_t n) {
    std::vector<const uint32_t*> ip;
    std::vector<const float*> vp;
    size_t total = 0;
    for (size_t s = 0; s < idx.size(); ++s) { ip.push_back(P<const uint32_t>(idx[s])); vp.push_back(P<const float>(val[s])); total += counts[s]; }
    std::vector<float> scratch(n, 0.f);
    std::vector<uint8_t> touched(n, 0);
    std::vector<uint32_t> oi(total);
    std::vector<float> ov(total);
    const size_t cnt = merge_streams(ip.data(), vp.data(), counts.data(), weights.data(), static_cast<int>(idx.size()),
                                     scratch.data(), touched.data(), n, oi.data(), ov.data());
    oi.resize(cnt);
    ov.resize(cnt);
    return py::make_tuple(oi, ov);
  });
  m.def("pool_order_probe", &pool_order_probe);
  m.def("parallel_sum_probe", [](size_t n, size_t workers) {
    ThreadPool pool(workers);
    std::vector<uint64_t> part(n, 0);
    pool.parallel_for(n, 1, [&](size_t b, size_t e) { for (size_t i = b; i < e; ++i) part[i] = i; });
    uint64_t s = 0;
    for (auto v : part) s += v;
    return s;
  });
  m.def("task_transition_allowed", [](int a, int b) { return task_transition_allowed(static_cast<TaskState>(a), static_cast<TaskState>(b)); });
  m.def("task_keys", [](int64_t iter, int layer, const std::string& name) {
    TrainTask t(iter, layer, name);
    return py::make_tuple(t.key, t.persistent_key, t.priority());
  });
  m.def("list_interfaces", [] {
    py::list out;
    for (auto& a : list_interfaces()) out.append(py::make_tuple(a.ifname, a.ip, a.loopback, a.is_private));
    return out;
  });
  m.def("pick_local_ip", &pick_local_ip);
  m.def("set_log_level", [](int l) { Logger::get().set_level(static_cast<LogLevel>(l)); });

  py::class_<CompressorBox>(m, "Compressor")
      .def(py::init<const std::string&>())
      .def("compress", &CompressorBox::compress)
      .def("compress_with_feedback", &CompressorBox::compress_ef)
      .def("state", &CompressorBox::state)
      .def("set_state", &CompressorBox::set_state);

  bind_optimizer<SGD>(m, "SGD");
  bind_optimizer<Adam>(m, "Adam");
  bind_optimizer<SGDNaive>(m, "SGDNaive");

  py::class_<BandwidthMonitor>(m, "BandwidthMonitor")
      .def(py::init<>())
      .def("add", &BandwidthMonitor::add)
      .def("peak_bytes_per_s", &BandwidthMonitor::peak_bytes_per_s)
      .def("mean_bytes_per_s", &BandwidthMonitor::mean_bytes_per_s)
      .def("total_bytes", &BandwidthMonitor::total_bytes);

  py::class_<ShmManager>(m, "ShmManager")
      .def(py::init<bool, int64_t, int, int, size_t, size_t, int>(), py::arg("master"), py::arg("session"), py::arg("local_rank"),
           py::arg("local_world"), py::arg("data_bytes"), py::arg("meta_bytes") = cfg::kShmMetaBytes, py::arg("attach_timeout_ms") = 10000)
      .def("alloc", [](ShmManager& s, size_t bytes) { return reinterpret_cast<uint64_t>(s.alloc(bytes)); })
      .def("offset_of", [](ShmManager& s, uint64_t p) { return s.offset_of(P<void>(p)); })
      .def("from_offset", [](ShmManager& s, uint64_t off) { return reinterpret_cast<uint64_t>(s.from_offset(off)); })
      .def("data_used", &ShmManager::data_used)
      .def("barrier", &ShmManager::barrier, py::call_guard<py::gil_scoped_release>())
      .def("arrive", &ShmManager::arrive)
      .def("complete", &ShmManager::complete)
      .def("depart", &ShmManager::depart)
      .def("pin_for_cuda", &ShmManager::pin_for_cuda)
      .def_static("unlink_session", &ShmManager::unlink_session);

  py::class_<CommBox>(m, "CommManager")
      .def(py::init<const std::string&, uint16_t, int>())
      .def("start_server", [](CommBox& b, int world) { b.c->start_server(world); })
      .def("set_data_transport", [](CommBox& b, const std::string& name, const std::string& libzmq) {
        return b.c->set_data_transport(name, libzmq);
      }, py::arg("name"), py::arg("libzmq") = "")
      .def("data_transport", [](CommBox& b) { return std::string(b.c->data_transport()); })
      .def("start_client", [](CommBox& b, int rank, int world, int gpus) { return b.c->start_client(rank, world, gpus); },
           py::call_guard<py::gil_scoped_release>())
      .def("queue_tx", [](CommBox& b, int64_t prio, const std::string& key, const std::vector<uint32_t>& idx,
                          const std::vector<float>& val, uint32_t numel, bool allow_u16, int value_format,
                          bool allow_blocks) {
        b.c->queue_tx(prio, key, idx.data(), val.data(), idx.size(), numel, allow_u16, value_format, allow_blocks);
      }, py::arg("priority"), py::arg("key"), py::arg("idx"), py::arg("val"), py::arg("tensor_numel"),
           py::arg("allow_u16") = true, py::arg("value_format") = 0, py::arg("allow_blocks") = true)
      .def("post_recv", &CommBox::post)
      .def("drain", &CommBox::drain)
      .def("stashed", [](CommBox& b) { return b.c->stashed(); })
      .def("send_init_model", [](CommBox& b, const std::string& key, const std::vector<float>& v) { return b.c->send_init_model(key, v.data(), v.size()); },
           py::call_guard<py::gil_scoped_release>())
      .def("recv_init_model", [](CommBox& b, const std::string& key, size_t n) {
        std::vector<float> v(n);
        bool ok;
        {
          py::gil_scoped_release rel;
          ok = b.c->recv_init_model(key, v.data(), n);
        }
        return py::make_tuple(ok, v);
      })
      .def("global_barrier", [](CommBox& b) { return b.c->global_barrier(); }, py::call_guard<py::gil_scoped_release>())
      .def("sync_time", [](CommBox& b, int pings) { return b.c->sync_time(pings); }, py::call_guard<py::gil_scoped_release>())
      .def("report_stat", [](CommBox& b, double s, double r) { return b.c->report_stat(s, r); })
      .def("broker_stats", [](CommBox& b) {
        py::list out;
        for (auto& s : b.c->broker_stats()) out.append(py::make_tuple(s.rank, s.send_mbps, s.recv_mbps));
        return out;
      })
      .def("set_tx_rate_limit", [](CommBox& b, double bytes_per_s, size_t burst) { b.c->set_tx_rate_limit(bytes_per_s, burst); },
           py::arg("bytes_per_s"), py::arg("burst_bytes") = 64 << 10)
      .def("drop_keys_containing", [](CommBox& b, const std::string& needle, int delay_ms) {
        b.c->set_tx_fault_hook([needle, delay_ms](const std::string& key, int* delay) {
          if (key.find(needle) == std::string::npos) return false;
          if (delay_ms > 0) { *delay = delay_ms; return false; }
          return true;
        });
      }, py::arg("needle"), py::arg("delay_ms") = 0)
      .def("bytes_sent", [](CommBox& b) { return b.c->bytes_sent(); })
      .def("bytes_received", [](CommBox& b) { return b.c->bytes_received(); })
      .def("rx_peak_bytes_per_s", [](CommBox& b) { return b.c->rx_monitor().peak_bytes_per_s(); })
      .def("failed", [](CommBox& b) { return b.c->failed(); })
      .def("failure", [](CommBox& b) { return b.c->failure(); })
      .def("close", [](CommBox& b) { py::gil_scoped_release rel; b.c.reset(); });

  py::class_<CpuEngine>(m, "CpuEngine")
      .def(py::init<>())
      .def("configure", [](CpuEngine& e, const std::string& addr, uint16_t port, int world, int rank, int64_t session,
                           int local_world, int local_rank, const std::string& method, int grad_acc, int staleness,
                           double ratio, size_t data_bytes, int timeout_ms, int workers, bool pin_cuda, bool debug_accuracy,
                           bool debug_barrier) {
        EngineOptions o;
        o.master_addr = addr; o.master_port = port; o.world = world; o.rank = rank; o.session = session;
        o.local_world = local_world; o.local_rank = local_rank; o.method = method; o.grad_accumulation = grad_acc;
        o.staleness = staleness; o.ratio = ratio; o.data_bytes = data_bytes; o.timeout_ms = timeout_ms; o.workers = workers;
        o.pin_cuda = pin_cuda; o.debug_accuracy = debug_accuracy; o.debug_barrier = debug_barrier;
        py::gil_scoped_release rel;
        e.configure(o);
      }, py::arg("master_addr"), py::arg("master_port"), py::arg("world_size"), py::arg("rank"), py::arg("local_session_id"),
           py::arg("local_world_size") = 1, py::arg("local_rank") = 0, py::arg("method") = "thresholdv16",
           py::arg("gradient_accumulation") = 1, py::arg("staleness") = 1, py::arg("ratio") = 0.99,
           py::arg("data_bytes") = 0, py::arg("timeout_ms") = 30000, py::arg("workers") = 0, py::arg("pin_cuda") = false,
           py::arg("debug_accuracy") = false, py::arg("debug_barrier") = false)
      .def("set_optimizer", &CpuEngine::set_optimizer)
      .def("configure_optimizer", [](CpuEngine& e, const std::string& k, py::object v) {
        if (py::isinstance<py::bool_>(v)) e.sparse_optimizer()->configure(k, v.cast<bool>());
        else e.sparse_optimizer()->configure(k, v.cast<float>());
      })
      .def("configure_compression", &CpuEngine::configure_compression)
      .def("configure_compression_ratio", &CpuEngine::configure_compression_ratio)
      .def("configure_compression_ratio_from", &CpuEngine::configure_compression_ratio_from, py::arg("iteration"), py::arg("ratio"))
      .def("compression_ratio_at", &CpuEngine::compression_ratio_at)
      .def("set_node_weights", &CpuEngine::set_node_weights, py::arg("weights"), py::arg("from_iteration") = 0)
      .def("node_weights_at", &CpuEngine::node_weights_at)
      .def("configure_wire", &CpuEngine::configure_wire, py::arg("blocks") = true, py::arg("value_format") = 0)
      .def("gradient_accumulation", &CpuEngine::gradient_accumulation)
      .def("is_debug_accuracy_mode", [](CpuEngine& e) { return e.options().debug_accuracy; })
      .def("skips_critical_paths", [](CpuEngine& e) { return e.options().skip_critical_paths; })
      .def("barrier", &CpuEngine::barrier, py::call_guard<py::gil_scoped_release>())
      .def("synchronize", &CpuEngine::synchronize, py::call_guard<py::gil_scoped_release>())
      .def("pre_train_init", [](CpuEngine& e, int layer, const std::string& name, uint32_t numel, uint64_t user_param,
                                uint64_t init_values) {
        py::gil_scoped_release rel;
        return e.pre_train_init(layer, name, numel, P<float>(user_param), P<const float>(init_values));
      }, py::arg("layer"), py::arg("name"), py::arg("numel"), py::arg("user_param"), py::arg("init_values") = 0)
      .def("pre_forward_process", &CpuEngine::pre_forward_process, py::call_guard<py::gil_scoped_release>())
      .def("post_backward_process", [](CpuEngine& e, int index, uint64_t grad) {
        py::gil_scoped_release rel;
        e.post_backward_process(index, P<const float>(grad));
      })
      .def("grad_slot", [](CpuEngine& e, int index) { return reinterpret_cast<uint64_t>(e.grad_slot(index)); })
      .def("post_backward_in_slot", &CpuEngine::post_backward_in_slot, py::call_guard<py::gil_scoped_release>())
      .def("master_param", [](CpuEngine& e, int index) { return reinterpret_cast<uint64_t>(e.master_param(index)); })
      .def("pop_ready_updates", &CpuEngine::pop_ready_updates, py::call_guard<py::gil_scoped_release>())
      .def("copy_out_done", &CpuEngine::copy_out_done, py::call_guard<py::gil_scoped_release>())
      .def("force_model_sync", &CpuEngine::force_model_sync, py::call_guard<py::gil_scoped_release>())
      .def("model_version", &CpuEngine::model_version)
      .def("num_params", &CpuEngine::num_params)
      .def("stats_json", &CpuEngine::stats_json)
      .def("comm_bytes", [](CpuEngine& e) {
        const uint64_t tx = e.comm() ? e.comm()->bytes_sent() : 0, rx = e.comm() ? e.comm()->bytes_received() : 0;
        return py::make_tuple(tx, rx);
      })
      .def("claim_grad_slot", [](CpuEngine& e, int i) { return reinterpret_cast<uint64_t>(e.claim_grad_slot(i)); })
      .def("device_copies_available", &CpuEngine::device_copies_available)
      .def("attach_device_param", [](CpuEngine& e, int i, uint64_t dev) { e.attach_device_param(i, P<void>(dev)); })
      .def("post_backward_device", [](CpuEngine& e, int i, uint64_t grad, uint64_t producer_stream, uint64_t copy_stream) {
        e.post_backward_device(i, P<const void>(grad), P<void>(producer_stream), P<void>(copy_stream));
      }, py::arg("param_index"), py::arg("device_grad"), py::arg("producer_stream"), py::arg("copy_stream") = 0)
      .def("set_param_members", [](CpuEngine& e, int i, const std::vector<std::string>& keys, const std::vector<uint32_t>& offsets,
                                   const std::vector<uint32_t>& numels, const std::vector<uint64_t>& user_params) {
        std::vector<float*> up;
        for (uint64_t u : user_params) up.push_back(P<float>(u));
        e.set_param_members(i, keys, offsets, numels, up);
      }, py::arg("param_index"), py::arg("keys"), py::arg("offsets"), py::arg("numels"), py::arg("user_params") = std::vector<uint64_t>{},
           "Declares a registered parameter to be a bundle of tensors laid end to end (offsets in steps of 16).")
      .def("post_backward_member", [](CpuEngine& e, int i, int member, uint64_t grad) {
        py::gil_scoped_release rel;
        e.post_backward_member(i, member, P<const float>(grad));
      })
      .def("attach_device_members", [](CpuEngine& e, int i, const std::vector<uint64_t>& dev) {
        std::vector<void*> v;
        for (uint64_t d : dev) v.push_back(P<void>(d));
        e.attach_device_members(i, v);
      })
      .def("post_backward_device_members", [](CpuEngine& e, int i, const std::vector<uint64_t>& grads, uint64_t producer_stream,
                                              uint64_t copy_stream) {
        std::vector<const void*> v;
        for (uint64_t g : grads) v.push_back(P<const void>(g));
        e.post_backward_device_members(i, v, P<void>(producer_stream), P<void>(copy_stream));
      }, py::arg("param_index"), py::arg("device_grads"), py::arg("producer_stream"), py::arg("copy_stream") = 0)
      .def("set_tx_rate_limit", [](CpuEngine& e, double bytes_per_s, size_t burst) {
        if (e.comm()) e.comm()->set_tx_rate_limit(bytes_per_s, burst);
      }, py::arg("bytes_per_s"), py::arg("burst_bytes") = 64 << 10,
           "Pace this node's gradient sends (a software stand-in for a slow link between nodes); 0 lifts the limit.")
      .def("drop_tx_containing", [](CpuEngine& e, const std::string& needle) {
        if (!e.comm()) return;
        e.comm()->set_tx_fault_hook([needle](const std::string& key, int*) { return key.find(needle) != std::string::npos; });
      })
      .def("grad_residual", [](CpuEngine& e, int i) { return reinterpret_cast<uint64_t>(e.grad_residual(i)); })
      .def("optimizer_kind", [](CpuEngine& e) { return std::string(e.sparse_optimizer()->kind()); })
      .def("optimizer_state", [](CpuEngine& e) {
        // {tensor: ({array name: [float]}, {counter name: int})}
        py::dict out;
        for (auto& kv : e.sparse_optimizer()->export_state()) {
          py::dict arrays, counters;
          for (auto& a : kv.second.arrays)
            arrays[py::str(a.first)] = py::bytes(reinterpret_cast<const char*>(a.second.data()), a.second.size() * sizeof(float));
          for (auto& c : kv.second.counters) counters[py::str(c.first)] = c.second;
          out[py::str(kv.first)] = py::make_tuple(arrays, counters);
        }
        return out;
      }, "Per-tensor optimiser state: {tensor: ({array: bytes of float32}, {counter: int})}")
      .def("set_optimizer_state", [](CpuEngine& e, const std::map<std::string, std::pair<std::map<std::string, std::string>,
                                                                                         std::map<std::string, int64_t>>>& st) {
        std::map<std::string, SparseOptimizer::TensorState> m;
        for (auto& kv : st) {
          SparseOptimizer::TensorState ts;
          for (auto& a : kv.second.first) {
            if (a.second.size() % sizeof(float)) throw std::invalid_argument("array " + a.first + " is not a whole number of floats");
            std::vector<float> v(a.second.size() / sizeof(float));
            std::memcpy(v.data(), a.second.data(), a.second.size());
            ts.arrays[a.first] = std::move(v);
          }
          ts.counters = kv.second.second;
          m[kv.first] = std::move(ts);
        }
        e.sparse_optimizer()->import_state(m);
      })
      .def("set_compressor_state", [](CpuEngine& e, const std::map<std::string, std::tuple<float, float, bool>>& st) {
        std::map<std::string, ThresholdState> m;
        for (auto& kv : st) m[kv.first] = ThresholdState{std::get<0>(kv.second), std::get<1>(kv.second), std::get<2>(kv.second)};
        e.compressor().import_state(m);
      })
      .def("compressor_state", [](CpuEngine& e) {
        py::dict d;
        for (auto& kv : e.compressor().export_state()) d[py::str(kv.first)] = py::make_tuple(kv.second.tau, kv.second.tau_inc, kv.second.inited);
        return d;
      });

  py::class_<TrainConfig>(m, "TrainConfig")
      .def(py::init([](uint32_t ub, uint32_t ga, double cr) { return TrainConfig{ub, ga, cr}; }))
      .def_readwrite("ubatch_size", &TrainConfig::ubatch_size)
      .def_readwrite("gradient_accumulation", &TrainConfig::gradient_accumulation)
      .def_readwrite("compression_rate", &TrainConfig::compression_rate);
  m.def("telemetry_clients_destroyed_on_own_thread", &TelemetryClient::destroyed_on_own_thread);
  // The destructor joins the client's thread, and that thread takes the interpreter lock whenever it calls or releases a
  // Python callback: destroying the client with the lock held would wait for a thread that waits for the lock.
  struct DeleteWithoutGil {
    void operator()(TelemetryClient* c) const {
      py::gil_scoped_release rel;
      delete c;
    }
  };
  py::class_<TelemetryClient, std::unique_ptr<TelemetryClient, DeleteWithoutGil>>(m, "TelemetryClient")
      .def(py::init<const std::string&, uint32_t, const std::string&, uint32_t, uint32_t, int>(), py::arg("uri"), py::arg("gpu_id"),
           py::arg("gpu_name"), py::arg("rank"), py::arg("local_rank"), py::arg("timeout_ms") = 5000,
           py::call_guard<py::gil_scoped_release>())
      .def("report", [](TelemetryClient& c, uint64_t uiter, const TrainConfig& cfg, const std::vector<double>& meas, py::object cb) {
        if (meas.size() != 6) throw std::invalid_argument("six measurements expected");
        TrainMeasurement tm{meas[0], meas[1], meas[2], meas[3], meas[4], meas[5]};
        InstructionCallback fn;
        if (!cb.is_none()) {
          // the callable is released on the client's thread: take the GIL for that too
          std::shared_ptr<py::object> holder(new py::object(cb), [](py::object* p) {
            py::gil_scoped_acquire acq;
            delete p;
          });
          fn = [holder](uint64_t since, const TrainConfig& tc) {
            py::gil_scoped_acquire acq;
            (*holder)(since, tc.ubatch_size, tc.gradient_accumulation, tc.compression_rate);
          };
        }
        c.report(uiter, cfg, tm, fn);
      }, py::arg("uiter"), py::arg("config"), py::arg("measurements"), py::arg("callback") = py::none())
      .def("queued", &TelemetryClient::queued)
      .def("sent", &TelemetryClient::sent)
      .def("alive", &TelemetryClient::alive)
      .def("close", [](TelemetryClient&) {});
  py::class_<TelemetryServer>(m, "TelemetryServer")
      .def(py::init<const std::string&, bool, int>(), py::arg("uri"), py::arg("launch_controller") = false, py::arg("timeout_ms") = 10000,
           py::call_guard<py::gil_scoped_release>())
      .def("send_global_telemetry", &TelemetryServer::send_global_telemetry, py::call_guard<py::gil_scoped_release>())
      .def("terminate", &TelemetryServer::terminate, py::call_guard<py::gil_scoped_release>());
}
