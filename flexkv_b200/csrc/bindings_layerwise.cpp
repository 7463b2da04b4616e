// Bindings of the layerwise restore group and the layer stub kernels.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "bindings_common.h"
#include "kernels/layer_sync.h"
#include "layerwise_group.h"
#include "peer_copier.h"
#include "gds_engine.h"

namespace py = pybind11;
using namespace fkv;

void init_layerwise_bindings(py::module_& m) {
  py::class_<LayerwiseResult>(m, "LayerwiseResult")
      .def_readonly("status", &LayerwiseResult::status)
      .def_readonly("epoch", &LayerwiseResult::epoch)
      .def_readonly("total_ms", &LayerwiseResult::total_ms)
      .def_readonly("disk_ms", &LayerwiseResult::disk_ms)
      .def_readonly("layer_done_ms", &LayerwiseResult::layer_done_ms);

  auto parse_options = [](py::dict o) {
    LayerwiseOptions lo;
    lo.group = parse_group_options(o);
    if (o.contains("notify_mode")) lo.notify = parse_notify_mode(o["notify_mode"].cast<std::string>());
    if (o.contains("num_counters")) lo.num_counters = o["num_counters"].cast<int>();
    if (o.contains("layers_per_batch")) lo.layers_per_batch = o["layers_per_batch"].cast<int>();
    if (o.contains("fused_max_bytes")) lo.fused_max_bytes = o["fused_max_bytes"].cast<int64_t>();
    if (o.contains("create_eventfds")) lo.create_eventfds = o["create_eventfds"].cast<bool>();
    if (o.contains("size_table_ptr")) {
      lo.size_table = (uint32_t*)(uintptr_t)o["size_table_ptr"].cast<uint64_t>();
      lo.size_table_layers = o["size_table_layers"].cast<int>();
      lo.size_table_rank_entries = o.contains("size_table_rank_entries") ? o["size_table_rank_entries"].cast<int64_t>() : 0;
      if (o.contains("codec_pipelines")) lo.codec_pipelines = o["codec_pipelines"].cast<int>();
    }
    return lo;
  };

  py::class_<LayerwiseGroup>(m, "LayerwiseGroup")
      .def(py::init([parse_options](py::list gpus, py::dict host, py::dict o) {
             LayerwiseOptions lo = parse_options(o);
             std::vector<GpuSide> gs = parse_gpu_sides(gpus);
             HostSide h = parse_host_side(host);
             py::gil_scoped_release rel;
             return new LayerwiseGroup(std::move(gs), h, lo);
           }))
      // multi-group form: groups = [{"gpus": [...], "host": {...}, "options": {num_layers, kv_dim, chunk_bytes,
      // cpu_tp_stride, shared_kv}}], members[l] = [(group, local_layer), ...], host = the whole block pool
      .def_static("multi_group", [parse_options](py::list groups, py::list members, py::dict host, py::dict o) {
             LayerwiseOptions lo = parse_options(o);
             std::vector<LayerwiseMemberGroup> gs;
             for (py::handle gh : groups) {
               py::dict g = gh.cast<py::dict>();
               LayerwiseMemberGroup mg;
               mg.gpus = parse_gpu_sides(g["gpus"].cast<py::list>());
               mg.host = parse_host_side(g["host"].cast<py::dict>());
               mg.group = parse_group_options(g["options"].cast<py::dict>());
               gs.push_back(std::move(mg));
             }
             std::vector<std::vector<LayerMember>> ms;
             for (py::handle lh : members) {
               std::vector<LayerMember> layer;
               for (py::handle mh : lh.cast<py::list>()) {
                 py::tuple t = mh.cast<py::tuple>();
                 layer.push_back(LayerMember{t[0].cast<int>(), t[1].cast<int>()});
               }
               ms.push_back(std::move(layer));
             }
             HostSide h = parse_host_side(host);
             py::gil_scoped_release rel;
             return new LayerwiseGroup(std::move(gs), std::move(ms), h, lo);
           }, py::arg("groups"), py::arg("members"), py::arg("host"), py::arg("options"))
      .def("update_gpu_ptrs", &LayerwiseGroup::update_gpu_ptrs)
      .def("update_group_gpu_ptrs", &LayerwiseGroup::update_group_gpu_ptrs)
      .def_property_readonly("is_multi_group", &LayerwiseGroup::multi_group)
      .def("restore", [](LayerwiseGroup& g, I64Array gpu_blocks, I64Array cpu_blocks, int counter_id, py::object ssd,
                         py::object ssd_layout, py::object ssd_src, py::object cpu_dst) {
             if (gpu_blocks.size() != cpu_blocks.size()) throw std::invalid_argument("block id arrays differ in size");
             SsdIoEngine* eng = nullptr;
             SsdLayout lay;
             I64Array s, c;
             int64_t nd = 0;
             if (!ssd.is_none() && !ssd_src.is_none()) {
               eng = ssd.cast<SsdIoEngine*>();
               lay = parse_ssd_layout(ssd_layout.cast<py::dict>());
               s = ssd_src.cast<I64Array>();
               c = cpu_dst.cast<I64Array>();
               if (s.size() != c.size()) throw std::invalid_argument("disk id arrays differ in size");
               nd = (int64_t)s.size();
             }
             const int64_t* gp = gpu_blocks.data();
             const int64_t* cp = cpu_blocks.data();
             const int64_t n = (int64_t)gpu_blocks.size();
             const int64_t* sp = nd ? s.data() : nullptr;
             const int64_t* dp = nd ? c.data() : nullptr;
             py::gil_scoped_release rel;
             return g.restore(gp, cp, n, counter_id, eng, nd ? &lay : nullptr, sp, dp, nd);
           }, py::arg("gpu_blocks"), py::arg("cpu_blocks"), py::arg("counter_id") = 0, py::arg("ssd") = py::none(),
           py::arg("ssd_layout") = py::none(), py::arg("ssd_src") = py::none(), py::arg("cpu_dst") = py::none())
      .def("eventfd_of", &LayerwiseGroup::eventfd_of)
      .def("eventfds_flat", &LayerwiseGroup::eventfds_flat)
      .def("set_eventfd", &LayerwiseGroup::set_eventfd)
      .def("device_flags_ptr", &LayerwiseGroup::device_flags_ptr)
      .def("host_flags_ptr", &LayerwiseGroup::host_flags_ptr)
      .def("epoch_of", &LayerwiseGroup::epoch_of)
      .def("begin_restore", &LayerwiseGroup::begin_restore, py::arg("counter"),
           "Reserves and returns the epoch the next restore() on this counter publishes.")
      .def("counter_status", &LayerwiseGroup::counter_status, py::arg("counter"))
      .def("wait_launched", [](LayerwiseGroup& g, int counter, uint32_t epoch, int timeout_ms) {
             py::gil_scoped_release rel;
             return g.wait_launched(counter, epoch, timeout_ms);
           }, py::arg("counter"), py::arg("epoch"), py::arg("timeout_ms") = 10000,
           "Blocks until every rank has queued the launches of the restore publishing `epoch` (or it failed).")
      .def("stream_wait_layer", [](LayerwiseGroup& g, int rank, int counter, int layer, uint64_t stream,
                                   uint32_t epoch) {
             cudaError_t e = g.stream_wait_layer(rank, counter, layer, (cudaStream_t)(uintptr_t)stream, epoch);
             if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(e));
           }, py::arg("rank"), py::arg("counter"), py::arg("layer"), py::arg("stream"), py::arg("epoch") = 0u)
      .def_property_readonly("num_ranks", &LayerwiseGroup::num_ranks)
      .def_property_readonly("num_layers", &LayerwiseGroup::num_layers)
      .def_property_readonly("num_counters", &LayerwiseGroup::num_counters);

  py::class_<PeerCopier>(m, "PeerCopier")
      .def(py::init([](py::list ranks, int num_layers, int kv_dim, int64_t chunk_bytes, int ctas, int tile, int engine,
                       int64_t max_blocks) {
             return new PeerCopier(parse_gpu_sides(ranks), num_layers, kv_dim, chunk_bytes,
                                   KvCopyLaunch{ctas, tile, engine}, max_blocks);
           }), py::arg("ranks"), py::arg("num_layers"), py::arg("kv_dim"), py::arg("chunk_bytes"),
           py::arg("num_ctas") = 64, py::arg("tile_bytes") = 16384, py::arg("engine") = 0,
           py::arg("max_blocks_per_op") = (int64_t)65536)
      .def("pull", [](PeerCopier& c, int dst_rank, int src_rank, I64Array dst_blocks, I64Array src_blocks,
                      int layer_start, int num_layers) {
             if (dst_blocks.size() != src_blocks.size()) throw std::invalid_argument("block id arrays differ in size");
             const int64_t* d = dst_blocks.data();
             const int64_t* s = src_blocks.data();
             const int64_t n = (int64_t)dst_blocks.size();
             py::gil_scoped_release rel;
             return c.pull(dst_rank, src_rank, d, s, n, layer_start, num_layers);
           })
      .def("update_gpu_ptrs", &PeerCopier::update_gpu_ptrs)
      .def("can_access", &PeerCopier::can_access)
      .def_property_readonly("num_ranks", &PeerCopier::num_ranks);

  py::class_<GdsEngine>(m, "GdsEngine")
      .def(py::init<const std::vector<std::vector<std::string>>&, int64_t, int64_t, int>(), py::arg("files"),
           py::arg("block_bytes"), py::arg("blocks_per_file"), py::arg("num_threads") = 8)
      .def_property_readonly("available", &GdsEngine::available)
      .def_property_readonly("why_unavailable", &GdsEngine::why_unavailable)
      .def("register_buffer", &GdsEngine::register_buffer)
      .def("deregister_buffer", &GdsEngine::deregister_buffer)
      .def("transfer", [](GdsEngine& e, uint64_t dev_base, I64Array dev_offsets, I64Array ssd_blocks, bool is_read,
                          int64_t slice_off, int64_t slice_bytes) {
             if (dev_offsets.size() != ssd_blocks.size()) throw std::invalid_argument("arrays differ in size");
             const int64_t n = (int64_t)ssd_blocks.size();
             py::array_t<uint8_t> ok((py::ssize_t)n);
             const int64_t* dp = dev_offsets.data();
             const int64_t* sp = ssd_blocks.data();
             uint8_t* okp = ok.mutable_data();
             int64_t nfail;
             {
               py::gil_scoped_release rel;
               nfail = e.transfer(dev_base, dp, sp, n, is_read, slice_off, slice_bytes, okp);
             }
             return py::make_tuple(nfail, ok);
           });

  m.def("layer_stub", [](uint64_t flag_ptr, uint32_t epoch, uint64_t busy_ns, uint64_t budget_ns, uint64_t status_ptr,
                         uint64_t t_start_ptr, int num_ctas, uint64_t stream) {
    cudaError_t e = launch_layer_stub((const uint32_t*)(uintptr_t)flag_ptr, epoch, busy_ns, budget_ns,
                                      (int32_t*)(uintptr_t)status_ptr, (uint64_t*)(uintptr_t)t_start_ptr, num_ctas,
                                      (cudaStream_t)(uintptr_t)stream);
    if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(e));
  }, py::arg("flag_ptr"), py::arg("epoch"), py::arg("busy_ns"), py::arg("budget_ns") = (uint64_t)1000000000ull,
     py::arg("status_ptr") = (uint64_t)0, py::arg("t_start_ptr") = (uint64_t)0, py::arg("num_ctas") = 1,
     py::arg("stream") = (uint64_t)0);

  m.def("layer_probe", [](uint64_t flag_ptr, uint32_t epoch, uint64_t data_ptr, int64_t num_bytes, uint64_t budget_ns,
                          uint64_t status_ptr, uint64_t out_sum_ptr, int num_ctas, uint64_t stream) {
    cudaError_t e = launch_layer_probe((const uint32_t*)(uintptr_t)flag_ptr, epoch, (const void*)(uintptr_t)data_ptr,
                                       num_bytes, budget_ns, (int32_t*)(uintptr_t)status_ptr,
                                       (uint64_t*)(uintptr_t)out_sum_ptr, num_ctas, (cudaStream_t)(uintptr_t)stream);
    if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(e));
  }, py::arg("flag_ptr"), py::arg("epoch"), py::arg("data_ptr"), py::arg("num_bytes"),
     py::arg("budget_ns") = (uint64_t)2000000000ull, py::arg("status_ptr") = (uint64_t)0, py::arg("out_sum_ptr") = (uint64_t)0,
     py::arg("num_ctas") = 4, py::arg("stream") = (uint64_t)0);

  m.def("set_flags", [](uint64_t flags_ptr, int n, uint32_t value, uint64_t stream) {
    cudaError_t e = launch_set_flags((uint32_t*)(uintptr_t)flags_ptr, n, value, (cudaStream_t)(uintptr_t)stream);
    if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(e));
  });
}
