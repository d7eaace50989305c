// pybind11 surface of the GPU-resident tier.  Tensors stay owned by Python (torch); this module
// only sees raw device addresses as integers, so it needs neither torch headers nor torch's ABI.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "bucket_handle.h"
#include "native_engine.h"

namespace py = pybind11;
using st::ApplyArgs;
using st::SelectArgs;

namespace {

template <typename T>
T* as_ptr(uint64_t v) { return reinterpret_cast<T*>(static_cast<uintptr_t>(v)); }

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// One bucket's pre-filled kernel arguments.  Filled once at set-up; `select` and `apply` are then
// a handful of kernel launches without any per-call marshalling.
struct BucketHandle : public st::BucketHandle {
  BucketHandle() {
    std::memset(&sel, 0, sizeof(sel));
    std::memset(&app, 0, sizeof(app));
    std::memset(&grp, 0, sizeof(grp));
    sel.timeout_ns = app.timeout_ns = 2000000000ull;
  }

  // rec: one float4 {accumulator, stamp, m, v} per element of this rank's state range
  void set_data(uint64_t grad, uint64_t grad_tab, uint64_t resid, uint64_t param, uint64_t rec, uint64_t vmax,
                uint64_t last, uint32_t n_total) {
    sel.grad = as_ptr<float>(grad);
    sel.grad_tab = as_ptr<float*>(grad_tab);
    sel.resid = as_ptr<float>(resid);
    sel.n_total = n_total;
    app.param = as_ptr<float>(param);
    app.rec = as_ptr<float4>(rec);
    app.vmax = as_ptr<float>(vmax);
    app.last = as_ptr<uint32_t>(last);
    app.n_total = n_total;
  }

  void set_tables(uint64_t segs, uint64_t state, uint64_t work, uint64_t chunks, uint64_t chunk_cnt,
                  uint64_t chunk_pos, uint64_t hist, uint32_t n_segs, uint32_t n_chunks, uint32_t cap,
                  uint64_t chunk_state, uint32_t max_chunk) {
    sel.chunk_state = as_ptr<uint64_t>(chunk_state);
    max_chunk_len = max_chunk;
    sel.segs = as_ptr<const st::SegDesc>(segs);
    sel.state = as_ptr<st::SegState>(state);
    sel.work = as_ptr<st::SegWork>(work);
    sel.chunks = as_ptr<const st::Chunk>(chunks);
    sel.chunk_cnt = as_ptr<uint32_t>(chunk_cnt);
    sel.chunk_pos = as_ptr<uint32_t>(chunk_pos);
    sel.hist = as_ptr<uint32_t>(hist);
    sel.n_segs = n_segs;
    sel.n_chunks = n_chunks;
    app.cap = cap;
    app.segs = sel.segs;
    app.n_segs = n_segs;
  }

  void set_scratch(uint64_t cand, uint64_t cand_cursor, uint32_t cand_cap) {
    sel.cand = as_ptr<uint2>(cand);
    sel.cand_cursor = as_ptr<uint32_t>(cand_cursor);
    sel.cand_cap = cand_cap;
  }

  // counters: [sel_epoch, app_epoch, sel_done, app_done, 4 spare] as eight u32 words; status: one u32 word
  void set_control(uint64_t counters, uint64_t status, uint64_t opt, uint64_t weight, uint64_t timeout_ns, uint64_t stamps) {
    uint32_t* c = as_ptr<uint32_t>(counters);
    sel.epoch = c + 0;
    app.epoch = c + 1;
    app.sel_epoch = c + 0;
    sel.done_ctr = c + 2;
    app.done_ctr = c + 3;
    sel.status = app.status = as_ptr<uint32_t>(status);
    app.opt = as_ptr<st::OptState>(opt);
    app.weight = as_ptr<const float>(weight);
    sel.timeout_ns = app.timeout_ns = timeout_ns;
    sel.stamps = app.stamps = as_ptr<uint64_t>(stamps);   // 8 u64 words or null
  }

  // Exchange wiring.  recv_local: this rank's receive area [2][world][cap] of (idx,val) pairs.
  // peer_recv[p]: address of peer p's receive area (p == rank: recv_local).  flags/acks likewise:
  // flag areas are [2][world] u64 indexed [slot][source]; ack areas are [2][world] u64 indexed
  // [slot][consumer].
  void set_comm(int world, int rank, uint64_t recv_local, const std::vector<uint64_t>& peer_recv,
                uint64_t recv_mc, uint64_t flag_local, const std::vector<uint64_t>& peer_flag,
                uint64_t ack_local, const std::vector<uint64_t>& peer_ack, bool use_flags, bool use_acks) {
    if (world < 1 || world > st::kMaxWorld) throw std::runtime_error("world size out of range");
    if ((int)peer_recv.size() != world || (int)peer_flag.size() != world || (int)peer_ack.size() != world)
      throw std::runtime_error("peer pointer lists must have one entry per rank");
    const uint64_t cap = app.cap;
    sel.world = app.world = world;
    sel.rank = app.rank = rank;
    sel.slot_stride = app.slot_stride = (uint64_t)world * cap;
    sel.flag_slot_stride = world;
    app.ack_slot_stride = world;
    for (int p = 0; p < world; ++p) {
      sel.out[p] = as_ptr<uint2>(peer_recv[p]) + (uint64_t)rank * cap;
      sel.flag[p] = as_ptr<uint64_t>(peer_flag[p]) + rank;
      app.ack[p] = as_ptr<uint64_t>(peer_ack[p]) + rank;
    }
    sel.out_mc = recv_mc ? as_ptr<uint2>(recv_mc) + (uint64_t)rank * cap : nullptr;
    app.recv = as_ptr<uint2>(recv_local);
    // debug checks are off unless set_debug follows
    sel.cksum_acc = nullptr;
    app.cksum_local = nullptr;
    app.rsum = nullptr;
    app.poison = 0u;
    app.flag_local = as_ptr<const uint64_t>(flag_local);
    sel.ack_local = as_ptr<const uint64_t>(ack_local);
    sel.use_acks = app.use_acks = use_acks ? 1u : 0u;
    sel.publish = app.use_flags = use_flags ? 1u : 0u;
    // replicated optimiser state unless set_owner follows
    sel.owner_mode = app.owner_mode = 0u;
    app.ent_lo = 0u;
    app.ent_hi = (uint32_t)cap;
    app.state_base = 0u;
    app.state_len = app.n_total;
  }

  // Partitioned optimiser state.  bounds: world + 1 stream positions, owner o consumes [bounds[o], bounds[o+1]).
  // state_base/state_len: element range covered by acc, stamp and the optimiser state of this rank.
  // Write-back areas have the shape of the receive areas; pflag areas are [2][world] u64 indexed [slot][owner].
  void set_owner(const std::vector<uint32_t>& bounds, uint32_t state_base, uint32_t state_len, uint64_t wb_local,
                 const std::vector<uint64_t>& peer_wb, uint64_t wb_mc, uint64_t pflag_local,
                 const std::vector<uint64_t>& peer_pflag) {
    const int world = app.world;
    if (world < 1) throw std::runtime_error("set_comm must come first");
    if ((int)bounds.size() != world + 1 || (int)peer_wb.size() != world || (int)peer_pflag.size() != world)
      throw std::runtime_error("set_owner: lists must match the world size");
    for (int o = 0; o <= world; ++o) {
      if (bounds[o] > app.cap || (o > 0 && bounds[o] < bounds[o - 1])) throw std::runtime_error("set_owner: bad bounds");
      app.own_lo[o] = bounds[o];
    }
    if ((uint64_t)state_base + state_len > app.n_total) throw std::runtime_error("set_owner: bad state range");
    sel.owner_mode = app.owner_mode = 1u;
    app.ent_lo = bounds[app.rank];
    app.ent_hi = bounds[app.rank + 1];
    app.state_base = state_base;
    app.state_len = state_len;
    app.wb_local = as_ptr<const uint2>(wb_local);
    app.wb_mc = wb_mc ? as_ptr<uint2>(wb_mc) : nullptr;
    app.pflag_local = as_ptr<const uint64_t>(pflag_local);
    app.pflag_slot_stride = world;
    for (int p = 0; p < world; ++p) {
      app.wb[p] = as_ptr<uint2>(peer_wb[p]);
      app.pflag[p] = as_ptr<uint64_t>(peer_pflag[p]) + app.rank;
    }
  }

  // narrow: some tensors of the bucket carry the narrow-wire flag in their descriptor
  void set_options(uint32_t compressor, bool zero_grad, bool skip_ef, bool narrow, bool deterministic) {
    sel.compressor = compressor;
    sel.zero_grad = zero_grad ? 1u : 0u;
    sel.skip_ef = skip_ef ? 1u : 0u;
    app.narrow = narrow ? 1u : 0u;
    app.deterministic = deterministic ? 1u : 0u;   // one scatter launch per source, in rank order
    app.src_first = 0u;
  }

  // grouped mode -------------------------------------------------------------------------------
  // mates: addresses of the group-mates' flat gradient buffers; flag areas are [group size] u64 words
  // indexed by the local rank of the writer.
  void set_group(uint64_t grad_local, const std::vector<uint64_t>& mate_grad, const std::vector<int>& mate_local,
                 int my_local, uint64_t ready_local, const std::vector<uint64_t>& mate_ready, uint64_t done_local,
                 const std::vector<uint64_t>& mate_done, uint64_t group_done_ctr) {
    if (mate_grad.size() > (size_t)st::kMaxWorld || mate_grad.size() != mate_local.size() ||
        mate_grad.size() != mate_ready.size() || mate_grad.size() != mate_done.size())
      throw std::runtime_error("inconsistent group description");
    std::memset(&grp, 0, sizeof(grp));
    grp.grad_local = as_ptr<float>(grad_local);
    grp.n_mates = (int)mate_grad.size();
    for (int m = 0; m < grp.n_mates; ++m) {
      grp.grad_peer[m] = as_ptr<const float>(mate_grad[m]);
      grp.mate_slot[m] = mate_local[m];
      grp.ready_peer[m] = as_ptr<uint64_t>(mate_ready[m]) + my_local;
      grp.done_peer[m] = as_ptr<uint64_t>(mate_done[m]) + my_local;
    }
    grp.ready_local = as_ptr<const uint64_t>(ready_local);
    grp.done_local = as_ptr<const uint64_t>(done_local);
    grp.done_ctr = as_ptr<uint32_t>(group_done_ctr);
    has_group = grp.n_mates > 0;
  }
  void py_group_reduce(uint64_t stream) {
    check(st::BucketHandle::group_reduce(as_ptr<CUstream_st>(stream)), "launch_group_reduce");
  }

  // The one-pass chain of the threshold compressors runs when it is enabled, possible for this bucket and every
  // tensor has its threshold; otherwise the four-kernel chain.
  void py_select(uint64_t stream) {
    check(st::BucketHandle::select(as_ptr<CUstream_st>(stream)), "launch_select");
  }
  // Debug checks.  cksum areas are [2][world] u32 indexed [slot][source]; cksum_acc has MAX_WORLD words, rsum `world`.
  void set_debug(uint64_t cksum_acc, uint64_t rsum, uint64_t cksum_local, const std::vector<uint64_t>& peer_cksum, bool poison) {
    const int world = app.world;
    if (world < 1) throw std::runtime_error("set_comm must come first");
    if ((int)peer_cksum.size() != world) throw std::runtime_error("set_debug: one checksum area per rank");
    sel.cksum_acc = as_ptr<uint32_t>(cksum_acc);
    sel.cksum_slot_stride = world;
    for (int p = 0; p < world; ++p) sel.cksum[p] = peer_cksum[p] ? as_ptr<uint32_t>(peer_cksum[p]) + app.rank : nullptr;
    app.cksum_local = as_ptr<const uint32_t>(cksum_local);
    app.rsum = as_ptr<uint32_t>(rsum);
    app.poison = poison ? 1u : 0u;
  }

  void py_apply(uint64_t stream, int phase) {
    check(st::BucketHandle::apply(as_ptr<CUstream_st>(stream), phase), "launch_apply");
  }
};

py::bytes ipc_get_handle(uint64_t ptr) {
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, as_ptr<void>(ptr)), "cudaIpcGetMemHandle");
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}

uint64_t ipc_open_handle(const std::string& raw) {
  if (raw.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, raw.data(), sizeof(h));
  void* p = nullptr;
  check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return (uint64_t)(uintptr_t)p;
}

void ipc_close_handle(uint64_t ptr) { check(cudaIpcCloseMemHandle(as_ptr<void>(ptr)), "cudaIpcCloseMemHandle"); }

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "sm_100a kernels of the GPU-resident sparse data-parallel tier";
  m.attr("MAX_WORLD") = st::kMaxWorld;
  m.attr("HIST_BINS") = st::kHistBins;
  m.attr("SENTINEL_IDX") = st::kSentinelIdx;
  m.attr("SIZEOF_SEG_DESC") = sizeof(st::SegDesc);
  m.attr("SIZEOF_SEG_STATE") = sizeof(st::SegState);
  m.attr("SIZEOF_SEG_WORK") = sizeof(st::SegWork);
  m.attr("SIZEOF_CHUNK") = sizeof(st::Chunk);
  m.attr("SIZEOF_OPT_STATE") = sizeof(st::OptState);

  py::class_<BucketHandle>(m, "BucketHandle")
      .def(py::init<>())
      .def("set_data", &BucketHandle::set_data, py::arg("grad"), py::arg("grad_tab"), py::arg("resid"),
           py::arg("param"), py::arg("rec"), py::arg("vmax"), py::arg("last"), py::arg("n_total"))
      .def("set_tables", &BucketHandle::set_tables, py::arg("segs"), py::arg("state"), py::arg("work"),
           py::arg("chunks"), py::arg("chunk_cnt"), py::arg("chunk_pos"), py::arg("hist"), py::arg("n_segs"),
           py::arg("n_chunks"), py::arg("cap"), py::arg("chunk_state") = 0, py::arg("max_chunk") = 0)
      .def("set_scratch", &BucketHandle::set_scratch, py::arg("cand"), py::arg("cand_cursor"), py::arg("cand_cap"))
      .def("set_control", &BucketHandle::set_control, py::arg("counters"), py::arg("status"), py::arg("opt"),
           py::arg("weight"), py::arg("timeout_ns"), py::arg("stamps") = 0)
      .def("set_comm", &BucketHandle::set_comm, py::arg("world"), py::arg("rank"), py::arg("recv_local"),
           py::arg("peer_recv"), py::arg("recv_mc"), py::arg("flag_local"), py::arg("peer_flag"),
           py::arg("ack_local"), py::arg("peer_ack"), py::arg("use_flags"), py::arg("use_acks"))
      .def("set_options", &BucketHandle::set_options, py::arg("compressor"), py::arg("zero_grad"),
           py::arg("skip_ef") = false, py::arg("narrow") = false, py::arg("deterministic") = false)
      .def_readwrite("randomk_seed", &BucketHandle::randomk_seed)
      .def_readwrite("max_ctas_per_source", &BucketHandle::max_ctas_per_source)
      .def("set_group", &BucketHandle::set_group, py::arg("grad_local"), py::arg("mate_grad"), py::arg("mate_local"),
           py::arg("my_local"), py::arg("ready_local"), py::arg("mate_ready"), py::arg("done_local"), py::arg("mate_done"),
           py::arg("group_done_ctr"))
      .def("group_reduce", &BucketHandle::py_group_reduce, py::arg("stream"))
      .def("select", &BucketHandle::py_select, py::arg("stream"))
      .def("can_fuse", [](const BucketHandle& h) { return h.can_fuse(); })
      .def_readwrite("fused_enabled", &BucketHandle::fused_enabled)
      .def_readwrite("thresholds_ready", &BucketHandle::thresholds_ready)
      .def_readonly("last_select_fused", &BucketHandle::last_select_fused)
      .def_property_readonly("select_kernels", [](const BucketHandle& h) { return h.select_kernels(); })
      .def_property_readonly("apply_kernels", [](const BucketHandle& h) { return h.apply_kernels(); })
      .def("set_owner", &BucketHandle::set_owner, py::arg("bounds"), py::arg("state_base"), py::arg("state_len"),
           py::arg("wb_local"), py::arg("peer_wb"), py::arg("wb_mc"), py::arg("pflag_local"), py::arg("peer_pflag"))
      .def("set_debug", &BucketHandle::set_debug, py::arg("cksum_acc"), py::arg("rsum"), py::arg("cksum_local"),
           py::arg("peer_cksum"), py::arg("poison"))
      .def("apply", &BucketHandle::py_apply, py::arg("stream"), py::arg("phase") = 0);

  // Native step engine: C++ hooks on the parameters, bucket bookkeeping, stream and event choreography.
  py::class_<st::NativeEngine>(m, "NativeEngine")
      .def(py::init<int, uint64_t, int, int>(), py::arg("device"), py::arg("sparse_stream"), py::arg("staleness"),
           py::arg("grad_accumulation"))
      .def("add_bucket",
           [](st::NativeEngine& e, BucketHandle& h, py::object select_handle, int n_params, bool steal, uint64_t table_host,
              int table_ring, uint64_t table_dev, py::object flat_grad, const std::vector<uint32_t>& seg_off,
              const std::vector<uint32_t>& seg_numel, uint64_t shaped_bytes) {
             st::NativeBucketSpec spec;
             spec.handle = &h;
             spec.select_handle = select_handle.is_none() ? nullptr : static_cast<st::BucketHandle*>(&select_handle.cast<BucketHandle&>());
             spec.n_params = n_params;
             spec.steal = steal;
             spec.table_host = as_ptr<uint64_t>(table_host);
             spec.table_ring = table_ring;
             spec.table_dev = as_ptr<uint64_t>(table_dev);
             spec.flat_grad = flat_grad.is_none() ? nullptr : flat_grad.ptr();
             spec.seg_off = seg_off;
             spec.seg_numel = seg_numel;
             spec.shaped_bytes = shaped_bytes;
             return e.add_bucket(spec);
           },
           py::arg("handle"), py::arg("select_handle"), py::arg("n_params"), py::arg("steal"), py::arg("table_host"),
           py::arg("table_ring"), py::arg("table_dev"), py::arg("flat_grad"), py::arg("seg_off"), py::arg("seg_numel"),
           py::arg("shaped_bytes") = 0, py::keep_alive<1, 2>())
      .def("add_param", [](st::NativeEngine& e, int bucket, int seg, py::handle p) { e.add_param(bucket, seg, p.ptr()); })
      .def("remove_hooks", &st::NativeEngine::remove_hooks)
      .def("set_shaper", [](st::NativeEngine& e, uint64_t state, uint64_t cap_ns) { e.set_shaper(as_ptr<void>(state), cap_ns); })
      .def("set_shaped_bytes", &st::NativeEngine::set_shaped_bytes)
      .def("wait_applies", &st::NativeEngine::wait_applies, py::arg("stream"), py::arg("bucket") = -1)
      .def("flush", &st::NativeEngine::flush, py::arg("stream"))
      .def("begin_capture", &st::NativeEngine::begin_capture)
      .def("end_capture", [](st::NativeEngine& e) { return py::reinterpret_steal<py::object>(e.end_capture()); })
      .def("select_count", &st::NativeEngine::select_count)
      .def("apply_count", &st::NativeEngine::apply_count)
      .def("pending_apply", &st::NativeEngine::pending_apply)
      .def("pending_hooks", &st::NativeEngine::pending_hooks)
      .def("set_counts", &st::NativeEngine::set_counts)
      .def("kernels_launched", &st::NativeEngine::kernels_launched)
      .def("shaped_bytes", &st::NativeEngine::shaped_bytes)
      .def("last_error", &st::NativeEngine::last_error);

  m.def("max_abs_diff", [](uint64_t a, uint64_t b, uint64_t n, uint64_t out_bits, uint64_t stream) {
    check(st::launch_max_abs_diff(as_ptr<const float>(a), as_ptr<const float>(b), n, as_ptr<uint32_t>(out_bits),
                                  as_ptr<CUstream_st>(stream)), "max_abs_diff");
  });
  m.def("peer_copy", [](uint64_t dst, uint64_t src, uint64_t n, uint64_t stream) {
    check(st::launch_peer_copy(as_ptr<float>(dst), as_ptr<const float>(src), n, as_ptr<CUstream_st>(stream)),
          "peer_copy");
  });
  m.def("delay", [](uint64_t ns_ptr, uint64_t cap_ns, uint64_t stream) {
    check(st::launch_delay(as_ptr<const uint64_t>(ns_ptr), cap_ns, as_ptr<CUstream_st>(stream)), "delay");
  });
  m.attr("SIZEOF_SHAPER_STATE") = sizeof(st::ShaperState);
  m.attr("SHAPER_LEVELS") = st::kShaperLevels;
  m.def("shape", [](uint64_t state, uint64_t nbytes, uint64_t cap_ns, uint64_t stream) {
    check(st::launch_shape(as_ptr<st::ShaperState>(state), nbytes, cap_ns, as_ptr<CUstream_st>(stream)), "shape");
  });
  m.def("stamp", [](uint64_t slot, uint64_t stream) {
    check(st::launch_stamp(as_ptr<uint64_t>(slot), as_ptr<CUstream_st>(stream)), "stamp");
  });
  m.def("link_probe", [](uint64_t dst, uint64_t src, uint64_t n, uint64_t out3, uint64_t ctr, uint64_t stream) {
    check(st::launch_link_probe(as_ptr<float>(dst), as_ptr<const float>(src), n, as_ptr<uint64_t>(out3), as_ptr<uint32_t>(ctr),
                                as_ptr<CUstream_st>(stream)), "link_probe");
  });
  m.def("ipc_get_handle", &ipc_get_handle);
  m.def("ipc_open_handle", &ipc_open_handle);
  m.def("ipc_close_handle", &ipc_close_handle);
}
