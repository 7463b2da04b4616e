// pybind11 surface of flexkv_b200._C. Tensors cross as raw addresses
// (tensor.data_ptr()) and numpy arrays; no torch headers are involved.
// Functional counterpart of the reference's c_ext module (csrc/bindings.cpp:428-1365).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include "hasher.h"
#include "graph_scheduler.h"
#include "native_log.h"
#include "metrics_exposer.h"
#include "host_mem.h"
#include "kernels/kv_copy.h"
#include "radix_index.h"
#include "ssd_io.h"
#include "transfer_group.h"
#include "bindings_common.h"
#include "native_log.h"

namespace py = pybind11;
using namespace fkv;

void init_kernel_bindings(py::module_& m);     // bindings_kernels.cpp
void init_layerwise_bindings(py::module_& m);  // bindings_layerwise.cpp
void init_dist_bindings(py::module_& m);       // bindings_dist.cpp

PYBIND11_MODULE(_C, m) {
  m.doc() = "flexkv_b200 native core (sm_100a kernels + C++ control plane)";
  m.attr("MAX_GPU_PTRS") = kMaxGpuPtrs;

  // ------------------------------------------------- transfer-graph scheduler
  py::class_<GraphScheduler>(m, "GraphScheduler")
      .def(py::init<>())
      .def("submit", [](GraphScheduler& g, int64_t graph_id, std::vector<int64_t> op_ids, std::vector<int32_t> flags,
                        std::vector<std::pair<int64_t, int64_t>> edges) {
             return g.submit(graph_id, op_ids, flags, edges);
           }, py::arg("graph_id"), py::arg("op_ids"), py::arg("flags"), py::arg("edges"))
      .def("set_fanout", &GraphScheduler::set_fanout)
      .def("op_done", [](GraphScheduler& g, int64_t graph_id, int64_t op_id, bool ok, double ms, int64_t bytes) {
             SchedDone r = g.op_done(graph_id, op_id, ok, ms, bytes);
             // (accepted, op finished, op success, ms, bytes, graph finished, graph failed, ready op ids)
             return py::make_tuple(r.accepted, r.op_finished, r.op_success, r.ms, r.bytes, r.graph_finished,
                                   r.graph_failed, r.ready);
           }, py::arg("graph_id"), py::arg("op_id"), py::arg("success"), py::arg("ms") = 0.0, py::arg("bytes") = 0)
      .def("requeue", &GraphScheduler::requeue)
      .def("take_ready", &GraphScheduler::take_ready)
      .def("wait", [](GraphScheduler& g, double timeout_s) {
             std::vector<SchedCompletion> v;
             {
               py::gil_scoped_release rel;
               v = g.wait(timeout_s);
             }
             py::list out;
             for (const auto& c : v) out.append(py::make_tuple(c.graph_id, c.op_id, c.success, c.ms, c.bytes));
             return out;
           }, py::arg("timeout_s"))
      .def("completion_fd", &GraphScheduler::completion_fd)
      .def("has_graph", &GraphScheduler::has_graph)
      .def("graphs_in_flight", &GraphScheduler::graphs_in_flight)
      .def("stats", [](GraphScheduler& g) {
             auto s = g.stats();
             py::dict d;
             d["ops"] = s.ops; d["failed_ops"] = s.failed_ops; d["graphs"] = s.graphs; d["failed_graphs"] = s.failed_graphs;
             return d;
           });
  m.attr("SCHED_OP_INSTANT") = (int)GraphScheduler::kInstant;

  // ------------------------------------------------- native logging / counters
  m.def("configure_cpp_metrics", [](bool enabled) { configure_metrics(enabled); }, py::arg("enabled"));
  m.def("reset_cpp_metrics", [] { reset_metrics(); });
  m.def("cpp_metrics_snapshot", [] {
    py::dict ops, blocks;
    auto& c = cache_counters();
    for (int i = 0; i < kNumCacheOps; ++i) {
      ops[kCacheOpNames[i]] = c.ops[i].load();
      blocks[kCacheOpNames[i]] = c.blocks[i].load();
    }
    py::dict d;
    d["enabled"] = metrics_enabled();
    d["ops"] = ops;
    d["blocks"] = blocks;
    return d;
  });
  m.def("start_cpp_metrics_exposer", [](int port, const std::string& addr) {
    py::gil_scoped_release nogil;
    return metrics_exposer_start(port, addr);
  }, py::arg("port"), py::arg("bind_addr") = "0.0.0.0");
  m.def("stop_cpp_metrics_exposer", [] { py::gil_scoped_release nogil; metrics_exposer_stop(); });
  m.def("cpp_metrics_exposer_port", [] { return metrics_exposer_port(); });
  m.def("cpp_metrics_text", [] { return metrics_text(); });
  m.def("set_log_level", [](const std::string& name) { set_log_level(name); });
  m.def("get_log_level", [] { return (int)log_level(); });
  m.def("set_log_prefix", [](const std::string& p) { set_log_prefix(p); });
  m.def("native_log", [](int level, const std::string& msg) {
    FKV_LOG((LogLevel)level, "%s", msg.c_str());
  });
  m.def("native_log_recent", [](size_t n) { return log_recent(n); }, py::arg("max_lines") = 64);

  // ---------------------------------------------------------------- hashing
  m.def("xxh64", [](py::buffer b, uint64_t seed) {
    py::buffer_info info = b.request();
    return XXH64::hash(info.ptr, (size_t)(info.size * info.itemsize), seed);
  }, py::arg("data"), py::arg("seed") = 0);

  m.def("gen_hashes", [](I64Array tokens, int tokens_per_block, py::object ns) {
    if (tokens_per_block <= 0) throw std::invalid_argument("tokens_per_block must be positive");
    const int64_t n = (int64_t)tokens.size();
    I64Array nsa;
    const int64_t* nsp = nullptr;
    int64_t nsl = 0;
    if (!ns.is_none()) { nsa = ns.cast<I64Array>(); nsp = nsa.data(); nsl = (int64_t)nsa.size(); }
    py::array_t<uint64_t> out((py::ssize_t)(n / tokens_per_block));
    {
      const int64_t* tp = tokens.data();
      uint64_t* op = out.mutable_data();
      py::gil_scoped_release rel;
      gen_block_hashes(tp, n, tokens_per_block, nsp, nsl, op);
    }
    return out;
  }, py::arg("token_ids"), py::arg("tokens_per_block"), py::arg("namespace_prefix") = py::none());

  m.def("gen_hashes_batch", [](std::vector<I64Array> seqs, int tokens_per_block, py::object ns, int threads) {
    if (tokens_per_block <= 0) throw std::invalid_argument("tokens_per_block must be positive");
    I64Array nsa;
    const int64_t* nsp = nullptr;
    int64_t nsl = 0;
    if (!ns.is_none()) { nsa = ns.cast<I64Array>(); nsp = nsa.data(); nsl = (int64_t)nsa.size(); }
    const int64_t n = (int64_t)seqs.size();
    // hash straight from the callers' arrays into the result arrays: no flattening copies
    std::vector<const int64_t*> in((size_t)n);
    std::vector<int64_t> len((size_t)n);
    std::vector<uint64_t*> out((size_t)n);
    py::list res;
    for (int64_t i = 0; i < n; ++i) {
      in[(size_t)i] = seqs[(size_t)i].data();
      len[(size_t)i] = (int64_t)seqs[(size_t)i].size();
      py::array_t<uint64_t> a((py::ssize_t)(len[(size_t)i] / tokens_per_block));
      out[(size_t)i] = a.mutable_data();
      res.append(a);
    }
    {
      py::gil_scoped_release rel;
      gen_block_hashes_ptrs(in.data(), len.data(), n, tokens_per_block, nsp, nsl, out.data(), threads);
    }
    return res;
  }, py::arg("seqs"), py::arg("tokens_per_block"), py::arg("namespace_prefix") = py::none(), py::arg("threads") = 4);

  // ---------------------------------------------------------------- radix index
  py::class_<PyMatch>(m, "MatchResult")
      .def_property_readonly("num_ready_matched_blocks", [](const PyMatch& p) { return p.r.num_ready_matched; })
      .def_property_readonly("num_matched_blocks", [](const PyMatch& p) { return p.r.num_matched; })
      .def_property_readonly("last_node_matched_length", [](const PyMatch& p) { return p.r.last_node_matched_length; })
      .def_property_readonly("last_ready_node", [](const PyMatch& p) { return handle_to_py(p.r.last_ready_node); })
      .def_property_readonly("last_node", [](const PyMatch& p) { return handle_to_py(p.r.last_node); })
      .def_property_readonly("physical_blocks", [](const PyMatch& p) { return to_array(p.r.physical_blocks); })
      .def_property_readonly("last_swa_node", [](const PyMatch& p) { return handle_to_py(p.r.last_swa_node); })
      .def_property_readonly("swa_hit_blocks", [](const PyMatch& p) { return p.r.swa_hit_blocks; })
      .def_property_readonly("swa_slot", [](const PyMatch& p) { return p.r.swa_slot; });

  py::class_<RadixIndex>(m, "RadixIndex")
      .def(py::init([](int tpb, int64_t max_blocks, const std::string& policy, double reward, uint32_t slru) {
             return new RadixIndex(tpb, max_blocks, parse_policy(policy), reward, slru);
           }),
           py::arg("tokens_per_block"), py::arg("max_num_blocks") = 0, py::arg("eviction_policy") = "lru",
           py::arg("hit_reward_seconds") = 0.0, py::arg("slru_threshold") = 2)
      .def("match_prefix", [](RadixIndex& t, U64Array hashes, int64_t n, bool update) {
             if (n < 0 || n > (int64_t)hashes.size()) n = (int64_t)hashes.size();
             PyMatch pm;
             pm.r = t.match_prefix(hashes.data(), n, update);
             return pm;
           }, py::arg("block_hashes"), py::arg("num_blocks") = -1, py::arg("update_cache_info") = true)
      .def("insert", [](RadixIndex& t, I64Array physical, U64Array hashes, int64_t num_insert, bool ready,
                        py::object match) {
             const MatchResult* mr = nullptr;
             PyMatch pm;
             if (!match.is_none()) { pm = match.cast<PyMatch>(); mr = &pm.r; }
             if (num_insert < 0) num_insert = (int64_t)hashes.size();
             return handle_to_py(t.insert(physical.data(), (int64_t)physical.size(), hashes.data(),
                                          (int64_t)hashes.size(), num_insert, ready, mr));
           }, py::arg("physical_block_ids"), py::arg("block_hashes"), py::arg("num_insert_blocks") = -1,
           py::arg("is_ready") = true, py::arg("match_result") = py::none())
      .def("evict", [](RadixIndex& t, int64_t n) {
             EvictResult r = t.evict(n);
             return py::make_tuple(to_array(r.blocks), to_array(r.hashes));
           })
      .def("set_swa", [](RadixIndex& t, py::object h, int32_t slot) { t.set_swa(handle_from_py(h), slot); })
      .def("has_swa", [](RadixIndex& t, py::object h) { return t.has_swa(handle_from_py(h)); })
      .def("swa_slot", [](RadixIndex& t, py::object h) { return t.swa_slot(handle_from_py(h)); })
      .def("swa_lock_cnt", [](RadixIndex& t, py::object h) { return t.swa_lock_cnt(handle_from_py(h)); })
      .def("lock_swa", [](RadixIndex& t, py::object h) { t.lock_swa(handle_from_py(h)); })
      .def("unlock_swa", [](RadixIndex& t, py::object h) { t.unlock_swa(handle_from_py(h)); })
      .def("evict_swa", [](RadixIndex& t, int64_t n) {
             std::vector<int64_t> blocks;
             std::vector<uint64_t> hashes;
             int64_t freed = t.evict_swa(n, &blocks, &hashes);
             return py::make_tuple(to_array(blocks), to_array(hashes), freed);
           })
      .def("drain_freed_swa_slots", [](RadixIndex& t) { return to_array(t.drain_freed_swa_slots()); })
      .def("total_swa_slots", &RadixIndex::total_swa_slots)
      .def("lock", [](RadixIndex& t, py::object h) { t.lock(handle_from_py(h)); })
      .def("unlock", [](RadixIndex& t, py::object h) { t.unlock(handle_from_py(h)); })
      .def("set_ready", [](RadixIndex& t, py::object h, bool ready, int64_t len) {
             t.set_ready(handle_from_py(h), ready, len);
           }, py::arg("node"), py::arg("ready") = true, py::arg("ready_length") = -1)
      .def("remove_unready_leaf", [](RadixIndex& t, py::object h) {
             return to_array(t.remove_unready_leaf(handle_from_py(h)));
           })
      .def("truncate_unready_leaf", [](RadixIndex& t, py::object h, int64_t keep) {
             return to_array(t.truncate_unready_leaf(handle_from_py(h), keep));
           })
      .def("reset", [](RadixIndex& t) { return to_array(t.reset()); })
      .def("export_ready", [](RadixIndex& t) {
             IndexSnapshot s = t.export_ready();
             return py::make_tuple(to_array(s.parents), to_array(s.sizes), to_array(s.hashes), to_array(s.blocks));
           })
      .def("import_snapshot", [](RadixIndex& t, py::array_t<int32_t, py::array::c_style | py::array::forcecast> parents,
                                 I64Array sizes, U64Array hashes, I64Array blocks) {
             IndexSnapshot s;
             s.parents.assign(parents.data(), parents.data() + parents.size());
             s.sizes.assign(sizes.data(), sizes.data() + sizes.size());
             s.hashes.assign(hashes.data(), hashes.data() + hashes.size());
             s.blocks.assign(blocks.data(), blocks.data() + blocks.size());
             return t.import_snapshot(s);
           })
      .def("alive", [](RadixIndex& t, py::object h) { return t.alive(handle_from_py(h)); })
      .def("is_root", [](RadixIndex& t, py::object h) { return t.is_root(handle_from_py(h)); })
      .def("root", [](RadixIndex& t) { return handle_to_py(t.root_handle()); })
      .def("node_size", [](RadixIndex& t, py::object h) { return t.node_size(handle_from_py(h)); })
      .def("node_ready", [](RadixIndex& t, py::object h) { return t.node_ready(handle_from_py(h)); })
      .def("node_lock_cnt", [](RadixIndex& t, py::object h) { return t.node_lock_cnt(handle_from_py(h)); })
      .def("node_parent", [](RadixIndex& t, py::object h) { return handle_to_py(t.node_parent(handle_from_py(h))); })
      .def("node_is_leaf", [](RadixIndex& t, py::object h) { return t.node_is_leaf(handle_from_py(h)); })
      .def("node_hit_count", [](RadixIndex& t, py::object h) { return t.node_hit_count(handle_from_py(h)); })
      .def("total_cached_blocks", &RadixIndex::total_cached_blocks)
      .def("total_ready_blocks", &RadixIndex::total_ready_blocks)
      .def("num_nodes", &RadixIndex::num_nodes)
      .def("num_leaves", &RadixIndex::num_leaves)
      .def("num_evictable_blocks", &RadixIndex::num_evictable_blocks)
      .def("is_empty", &RadixIndex::is_empty)
      .def("set_clock_override", &RadixIndex::set_clock_override)
      .def("set_policy", [](RadixIndex& t, const std::string& p) { t.set_policy(parse_policy(p)); })
      .def("stats", [](RadixIndex& t) {
        py::dict d;
        d["hit"] = t.stat_hit; d["match"] = t.stat_match; d["miss"] = t.stat_miss;
        d["insert_blocks"] = t.stat_insert_blocks; d["evict_blocks"] = t.stat_evict_blocks;
        return d;
      });

  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int64_t>())
      .def("allocate", [](BlockPool& p, int64_t n, bool strict) { return to_array(p.allocate(n, strict)); },
           py::arg("num"), py::arg("strict") = true)
      .def("recycle", [](BlockPool& p, I64Array ids) { p.recycle(ids.data(), (int64_t)ids.size()); })
      .def("reserve", [](BlockPool& p, I64Array ids) { p.reserve(ids.data(), (int64_t)ids.size()); })
      .def("reset", &BlockPool::reset)
      .def_property_readonly("num_free", &BlockPool::num_free)
      .def_property_readonly("num_total", &BlockPool::num_total)
      .def_property_readonly("num_used", &BlockPool::num_used)
      .def("is_free", &BlockPool::is_free);

  // ---------------------------------------------------------------- host memory
  py::class_<HostRegion>(m, "HostRegion", py::buffer_protocol())
      .def_property_readonly("ptr", [](const HostRegion& r) { return (uint64_t)(uintptr_t)r.ptr; })
      .def_readonly("bytes", &HostRegion::bytes)
      .def_readonly("map_bytes", &HostRegion::map_bytes)
      .def_readonly("hugepage", &HostRegion::hugepage)
      .def_readonly("file_backed", &HostRegion::file_backed)
      .def_readonly("registered", &HostRegion::registered)
      .def("register", [](HostRegion& r, size_t chunk) { py::gil_scoped_release rel; host_region_register(r, chunk); },
           py::arg("chunk_bytes") = 0)
      .def("unregister", [](HostRegion& r) { host_region_unregister(r); })
      .def("free", [](HostRegion& r) { host_region_free(r); })
      .def_buffer([](HostRegion& r) {
        return py::buffer_info(r.ptr, 1, py::format_descriptor<uint8_t>::format(), 1, {(py::ssize_t)r.bytes}, {1});
      });

  m.def("host_region_alloc", [](size_t bytes, bool hugepage, size_t hugepage_bytes, int numa_node, bool populate,
                                int touch_threads, bool cuda_register, size_t register_chunk, std::string file) {
    HostAllocOptions o;
    o.hugepage = hugepage; o.hugepage_bytes = hugepage_bytes; o.numa_node = numa_node; o.populate = populate;
    o.touch_threads = touch_threads; o.cuda_register = cuda_register; o.register_chunk_bytes = register_chunk;
    o.backing_file = file;
    py::gil_scoped_release rel;
    return host_region_alloc(bytes, o);
  }, py::arg("bytes"), py::arg("hugepage") = false, py::arg("hugepage_bytes") = (size_t)(2u << 20),
     py::arg("numa_node") = -1, py::arg("populate") = true, py::arg("touch_threads") = 8,
     py::arg("cuda_register") = false, py::arg("register_chunk_bytes") = (size_t)0, py::arg("backing_file") = "");
  m.def("host_region_open", &host_region_open, py::arg("file"), py::arg("bytes"), py::arg("hugepage") = false,
        py::arg("hugepage_bytes") = (size_t)(2u << 20));
  m.def("gpu_numa_node", &gpu_numa_node);
  m.def("cuda_device_count", [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n;
  });

  // ---------------------------------------------------------------- SSD IO
  py::class_<SsdIoEngine>(m, "SsdIoEngine")
      .def(py::init<const std::vector<std::vector<std::string>>&, int64_t, int64_t, bool, bool, int, int>(),
           py::arg("files"), py::arg("block_bytes"), py::arg("blocks_per_file"), py::arg("create") = true,
           py::arg("try_direct") = true, py::arg("iouring_entries") = 512, py::arg("num_threads") = 8)
      .def("transfer", [](SsdIoEngine& e, uint64_t cpu_base, I64Array cpu_blocks, I64Array ssd_blocks, bool is_read,
                          py::dict lay, int layer_start, int num_layers) {
             if (cpu_blocks.size() != ssd_blocks.size()) throw std::invalid_argument("block id arrays differ in size");
             SsdLayout L = parse_ssd_layout(lay);
             const int64_t n = (int64_t)cpu_blocks.size();
             py::array_t<uint8_t> ok((py::ssize_t)n);
             int64_t nfail;
             {
               const int64_t* cb = cpu_blocks.data();
               const int64_t* sb = ssd_blocks.data();
               uint8_t* okp = ok.mutable_data();
               py::gil_scoped_release rel;
               nfail = e.transfer((uint8_t*)(uintptr_t)cpu_base, cb, sb, n, is_read, L, layer_start, num_layers, okp);
             }
             return py::make_tuple(nfail, ok);
           })
      .def("transfer_packed", [](SsdIoEngine& e, uint64_t cpu_base, I64Array cpu_blocks, I64Array ssd_blocks,
                                 bool is_read, py::dict geo,
                                 py::array_t<int32_t, py::array::c_style | py::array::forcecast> sizes) {
             if (cpu_blocks.size() != ssd_blocks.size()) throw std::invalid_argument("block id arrays differ in size");
             SsdIoEngine::PackedGeometry g;
             g.cpu_block_stride = geo["cpu_block_stride"].cast<int64_t>();
             g.chunk_slot_bytes = geo["chunk_slot_bytes"].cast<int64_t>();
             g.tile_slot_bytes = geo["tile_slot_bytes"].cast<int64_t>();
             g.last_tile_slot_bytes = geo["last_tile_slot_bytes"].cast<int64_t>();
             g.tiles_per_chunk = geo["tiles_per_chunk"].cast<int32_t>();
             g.entries = geo["entries"].cast<int32_t>();
             const int64_t n = (int64_t)cpu_blocks.size();
             if ((int64_t)sizes.size() != n * g.entries) throw std::invalid_argument("one row of sizes per block");
             py::array_t<uint8_t> ok((py::ssize_t)n);
             int64_t nfail;
             {
               const int64_t* cb = cpu_blocks.data();
               const int64_t* sb = ssd_blocks.data();
               const int32_t* sz = sizes.data();
               uint8_t* okp = ok.mutable_data();
               py::gil_scoped_release rel;
               nfail = e.transfer_packed((uint8_t*)(uintptr_t)cpu_base, cb, sb, n, is_read, g, sz, okp);
             }
             return py::make_tuple(nfail, ok);
           })
      .def("set_fault", [](SsdIoEngine& e, int mode, int64_t nth) { SsdFault f; f.mode = mode; f.nth = nth; e.set_fault(f); })
      .def("sync_files", &SsdIoEngine::sync_files)
      .def_property_readonly("using_iouring", &SsdIoEngine::using_iouring)
      .def_property_readonly("direct_available", &SsdIoEngine::direct_available)
      .def_property_readonly("capacity_blocks", &SsdIoEngine::capacity_blocks)
      .def_property_readonly("bytes_read", &SsdIoEngine::bytes_read)
      .def_property_readonly("bytes_written", &SsdIoEngine::bytes_written);

  // ---------------------------------------------------------------- transfer group
  py::class_<OpResult>(m, "OpResult")
      .def_readonly("status", &OpResult::status)
      .def_readonly("gpu_ms", &OpResult::gpu_ms);

  py::class_<TransferGroup>(m, "TransferGroup")
      .def(py::init([](py::list gpus, py::dict host, py::dict o) {
             std::vector<GpuSide> gs = parse_gpu_sides(gpus);
             HostSide h = parse_host_side(host);
             GroupOptions g = parse_group_options(o);
             py::gil_scoped_release rel;
             return new TransferGroup(std::move(gs), h, g);
           }))
      .def("submit", [](TransferGroup& t, I64Array gb, I64Array cb, bool h2d, int ls, int nl, int engine) {
             if (gb.size() != cb.size()) throw std::invalid_argument("block id arrays differ in size");
             const int64_t* g = gb.data();
             const int64_t* c = cb.data();
             const int64_t n = (int64_t)gb.size();
             py::gil_scoped_release rel;
             return t.submit(g, c, n, h2d, ls, nl, engine);
           }, py::arg("gpu_blocks"), py::arg("cpu_blocks"), py::arg("h2d"), py::arg("layer_start"),
           py::arg("num_layers"), py::arg("engine") = -1)
      .def("wait", [](TransferGroup& t, uint64_t ticket) { py::gil_scoped_release rel; return t.wait(ticket); })
      .def("poll", &TransferGroup::poll)
      .def("transfer", [](TransferGroup& t, I64Array gb, I64Array cb, bool h2d, int ls, int nl, int engine) {
             if (gb.size() != cb.size()) throw std::invalid_argument("block id arrays differ in size");
             const int64_t* g = gb.data();
             const int64_t* c = cb.data();
             const int64_t n = (int64_t)gb.size();
             py::gil_scoped_release rel;
             return t.transfer(g, c, n, h2d, ls, nl, engine);
           }, py::arg("gpu_blocks"), py::arg("cpu_blocks"), py::arg("h2d"), py::arg("layer_start"),
           py::arg("num_layers"), py::arg("engine") = -1)
      .def("transfer_refshape", [](TransferGroup& t, I64Array gb, I64Array cb, bool h2d, int ctas) {
             const int64_t* g = gb.data();
             const int64_t* c = cb.data();
             const int64_t n = (int64_t)gb.size();
             py::gil_scoped_release rel;
             return t.transfer_refshape(g, c, n, h2d, ctas);
           }, py::arg("gpu_blocks"), py::arg("cpu_blocks"), py::arg("h2d"), py::arg("num_ctas") = 4)
      .def("update_gpu_ptrs", &TransferGroup::update_gpu_ptrs)
      .def("set_launch", [](TransferGroup& t, bool h2d, int ctas, int tile, int engine) {
             t.set_launch(h2d, KvCopyLaunch{ctas, tile, engine});
           })
      .def_property_readonly("ce_ops", &TransferGroup::ce_ops)
      .def_property_readonly("staged_ops", &TransferGroup::staged_ops)
      .def_property_readonly("num_ranks", &TransferGroup::num_ranks);

  init_kernel_bindings(m);
  init_layerwise_bindings(m);
  init_dist_bindings(m);
}
