// dict -> native struct helpers shared by the binding translation units
#pragma once
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "ssd_io.h"
#include "transfer_group.h"

#include "radix_index.h"

namespace fkv {
namespace py = pybind11;

using I64Array = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;
using U64Array = py::array_t<uint64_t, py::array::c_style | py::array::forcecast>;

template <typename T>
inline py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a((py::ssize_t)v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

inline py::object handle_to_py(NodeHandle h) {
  if (h == kNullHandle) return py::none();
  return py::int_(h);
}
inline NodeHandle handle_from_py(const py::object& o) {
  if (o.is_none()) return kNullHandle;
  return o.cast<uint64_t>();
}

// MatchResult as Python sees it (shared by the plain and the lease-aware index bindings)
struct PyMatch {
  MatchResult r;
};

inline std::vector<GpuSide> parse_gpu_sides(const py::list& gpus) {
  std::vector<GpuSide> gs;
  for (auto item : gpus) {
    py::dict d = item.cast<py::dict>();
    GpuSide g;
    g.device = d["device"].cast<int>();
    g.ptrs = d["ptrs"].cast<std::vector<uint64_t>>();
    g.idx_layer_mul = d["idx_layer_mul"].cast<int>();
    g.idx_kv_mul = d["idx_kv_mul"].cast<int>();
    g.layer_stride = d["layer_stride"].cast<int64_t>();
    g.kv_stride = d["kv_stride"].cast<int64_t>();
    g.block_stride = d["block_stride"].cast<int64_t>();
    g.num_blocks = d["num_blocks"].cast<int64_t>();
    gs.push_back(std::move(g));
  }
  return gs;
}

inline HostSide parse_host_side(const py::dict& host) {
  HostSide h;
  h.base = host["base"].cast<uint64_t>();
  h.layer_stride = host["layer_stride"].cast<int64_t>();
  h.kv_stride = host["kv_stride"].cast<int64_t>();
  h.block_stride = host["block_stride"].cast<int64_t>();
  h.num_blocks = host["num_blocks"].cast<int64_t>();
  return h;
}

inline GroupOptions parse_group_options(const py::dict& o) {
  GroupOptions g;
  g.num_layers = o["num_layers"].cast<int>();
  g.kv_dim = o["kv_dim"].cast<int>();
  g.chunk_bytes = o["chunk_bytes"].cast<int64_t>();
  g.cpu_tp_stride = o.contains("cpu_tp_stride") ? o["cpu_tp_stride"].cast<int64_t>() : 0;
  g.shared_kv = o.contains("shared_kv") && o["shared_kv"].cast<bool>();
  if (o.contains("shared_mode")) g.shared_mode = parse_shared_kv_mode(o["shared_mode"].cast<std::string>());
  auto launch = [&](const char* k, KvCopyLaunch& l) {
    if (!o.contains(k)) return;
    py::dict d = o[k].cast<py::dict>();
    if (d.contains("num_ctas")) l.num_ctas = d["num_ctas"].cast<int>();
    if (d.contains("tile_bytes")) l.tile_bytes = d["tile_bytes"].cast<int>();
    if (d.contains("engine")) l.engine = d["engine"].cast<int>();
  };
  launch("h2d", g.h2d);
  launch("d2h", g.d2h);
  if (o.contains("ring_slots")) g.ring_slots = o["ring_slots"].cast<int>();
  if (o.contains("max_blocks_per_op")) g.max_blocks_per_op = o["max_blocks_per_op"].cast<int64_t>();
  if (o.contains("high_priority_stream")) g.high_priority_stream = o["high_priority_stream"].cast<bool>();
  if (o.contains("ce_staging_blocks")) g.ce_staging_blocks = o["ce_staging_blocks"].cast<int64_t>();
  if (o.contains("ce_max_copies")) g.ce_policy.max_copies = o["ce_max_copies"].cast<int64_t>();
  if (o.contains("ce_min_bytes_per_copy")) g.ce_policy.min_bytes_per_copy = o["ce_min_bytes_per_copy"].cast<int64_t>();
  return g;
}

inline SsdLayout parse_ssd_layout(const py::dict& lay) {
  SsdLayout L;
  L.cpu_layer_stride = lay["cpu_layer_stride"].cast<int64_t>();
  L.cpu_kv_stride = lay["cpu_kv_stride"].cast<int64_t>();
  L.cpu_block_stride = lay["cpu_block_stride"].cast<int64_t>();
  L.ssd_layer_stride = lay["ssd_layer_stride"].cast<int64_t>();
  L.ssd_kv_stride = lay["ssd_kv_stride"].cast<int64_t>();
  L.ssd_block_stride = lay["ssd_block_stride"].cast<int64_t>();
  L.chunk_bytes = lay["chunk_bytes"].cast<int64_t>();
  L.num_layers_total = lay["num_layers"].cast<int>();
  L.kv_dim = lay["kv_dim"].cast<int>();
  L.block_first = lay["block_first"].cast<bool>();
  return L;
}

}  // namespace fkv
