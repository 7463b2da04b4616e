// Python bindings of the cross-node index (dist_index.h).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "bindings_common.h"
#include "dist_index.h"
#include "redis_meta_channel.h"
#include "resp_client.h"

namespace py = pybind11;
using namespace fkv;

namespace {

// A channel implemented in Python (e.g. the registry client). Calls may arrive from the
// native refresh threads, so every call takes the GIL.
class PyMetaChannel : public MetaChannel {
 public:
  explicit PyMetaChannel(py::object impl) : impl_(std::move(impl)) {}
  ~PyMetaChannel() override {
    py::gil_scoped_acquire g;
    impl_ = py::object();
  }
  static py::list to_rows(const std::vector<BlockMeta>& metas) {
    py::list rows;
    for (const BlockMeta& m : metas) rows.append(py::make_tuple(m.ph, m.pb, m.nid, m.hash, m.lt, m.state));
    return rows;
  }
  void publish(uint32_t nid, const std::vector<BlockMeta>& metas) override {
    py::gil_scoped_acquire g;
    impl_.attr("publish")(nid, to_rows(metas));
  }
  void remove(uint32_t nid, const std::vector<uint64_t>& hashes) override {
    py::gil_scoped_acquire g;
    impl_.attr("remove")(nid, hashes);
  }
  std::vector<uint32_t> list_nodes() override {
    py::gil_scoped_acquire g;
    return impl_.attr("list_nodes")().cast<std::vector<uint32_t>>();
  }
  std::vector<BlockMeta> load(uint32_t nid) override {
    py::gil_scoped_acquire g;
    std::vector<BlockMeta> out;
    for (auto row : impl_.attr("load")(nid)) {
      py::tuple t = row.cast<py::tuple>();
      BlockMeta m;
      m.ph = t[0].cast<uint64_t>();
      m.pb = t[1].cast<int64_t>();
      m.nid = t[2].cast<uint32_t>();
      m.hash = t[3].cast<uint64_t>();
      m.lt = t[4].cast<int64_t>();
      m.state = t[5].cast<int>();
      out.push_back(m);
    }
    return out;
  }
  void clear_node(uint32_t nid) override {
    py::gil_scoped_acquire g;
    impl_.attr("clear_node")(nid);
  }

 private:
  py::object impl_;
};

std::shared_ptr<MetaChannel> channel_from_py(const py::object& o) {
  if (o.is_none()) return nullptr;
  if (py::isinstance<InProcMetaChannel>(o)) return o.cast<std::shared_ptr<InProcMetaChannel>>();
  if (py::isinstance<RedisMetaChannel>(o)) return o.cast<std::shared_ptr<RedisMetaChannel>>();
  return std::make_shared<PyMetaChannel>(o);
}

template <typename T>
std::shared_ptr<T> gil_free_delete(T* p) {
  // the destructor joins a thread that may be waiting for the GIL
  return std::shared_ptr<T>(p, [](T* q) {
    py::gil_scoped_release rel;
    delete q;
  });
}

}  // namespace

namespace {

py::object resp_to_py(const RespValue& v) {
  switch (v.type) {
    case RespValue::kNil: return py::none();
    case RespValue::kString: return py::str(v.str);
    case RespValue::kInteger: return py::int_(v.integer);
    case RespValue::kBulk: return py::bytes(v.str);
    case RespValue::kArray: {
      py::list l;
      for (const auto& it : v.items) l.append(resp_to_py(it));
      return std::move(l);
    }
    case RespValue::kError: break;
  }
  throw std::runtime_error("redis error reply: " + v.str);
}

std::vector<std::string> resp_args(const py::sequence& seq) {
  std::vector<std::string> out;
  for (auto a : seq) {
    if (py::isinstance<py::bytes>(a)) out.push_back(a.cast<std::string>());
    else out.push_back(py::str(a).cast<std::string>());
  }
  return out;
}

}  // namespace

void init_dist_bindings(py::module_& m) {
  m.def("wall_clock_ms", &wall_clock_ms);

  // Redis wire protocol (an IO failure is a ConnectionError, an error reply a RuntimeError)
  py::register_exception<RespIoError>(m, "RespIoError", PyExc_ConnectionError);
  py::class_<RespClient>(m, "RespClient")
      .def(py::init<std::string, int, int, std::string, int>(), py::arg("host"), py::arg("port"),
           py::arg("timeout_ms") = 3000, py::arg("password") = "", py::arg("db") = 0)
      .def("command", [](RespClient& c, py::args args) {
        auto a = resp_args(args);
        RespValue v;
        {
          py::gil_scoped_release nogil;
          v = c.command(a);
        }
        return resp_to_py(v);
      })
      .def("pipeline", [](RespClient& c, py::list cmds) {
        std::vector<std::vector<std::string>> cs;
        for (auto one : cmds) cs.push_back(resp_args(one.cast<py::sequence>()));
        std::vector<RespValue> vs;
        {
          py::gil_scoped_release nogil;
          vs = c.pipeline(cs);
        }
        py::list out;
        for (const auto& v : vs) out.append(resp_to_py(v));
        return out;
      })
      .def("close", &RespClient::close)
      .def("connected", &RespClient::connected)
      .def_static("encode", [](py::args args) { return py::bytes(RespClient::encode(resp_args(args))); })
      .def_static("parse", [](py::bytes data) -> py::object {
        std::string s = data;
        size_t pos = 0;
        RespValue v;
        if (!RespClient::parse(s, pos, v)) return py::none();
        return py::make_tuple(resp_to_py(v), pos);
      });

  // block records in a Redis server, spoken to from native code (no interpreter lock on the refresh path)
  py::class_<RedisMetaChannel, std::shared_ptr<RedisMetaChannel>>(m, "RedisMetaChannel")
      .def(py::init([](const std::string& host, int port, const std::string& kind, int timeout_ms,
                       const std::string& password, int db) {
             return std::make_shared<RedisMetaChannel>(host, port, kind, timeout_ms, password, db);
           }), py::arg("host"), py::arg("port"), py::arg("kind") = "CPUB", py::arg("timeout_ms") = 3000,
           py::arg("password") = "", py::arg("db") = 0)
      .def("publish", [](RedisMetaChannel& c, uint32_t nid, py::list rows) {
        std::vector<BlockMeta> v;
        for (auto row : rows) {
          py::tuple t = row.cast<py::tuple>();
          BlockMeta b;
          b.ph = t[0].cast<uint64_t>(); b.pb = t[1].cast<int64_t>(); b.nid = t[2].cast<uint32_t>();
          b.hash = t[3].cast<uint64_t>(); b.lt = t[4].cast<int64_t>(); b.state = t[5].cast<int>();
          v.push_back(b);
        }
        py::gil_scoped_release nogil;
        c.publish(nid, v);
      })
      .def("remove", [](RedisMetaChannel& c, uint32_t nid, std::vector<uint64_t> hashes) {
        py::gil_scoped_release nogil;
        c.remove(nid, hashes);
      })
      .def("list_nodes", [](RedisMetaChannel& c) {
        py::gil_scoped_release nogil;
        return c.list_nodes();
      })
      .def("load", [](RedisMetaChannel& c, uint32_t nid) {
        std::vector<BlockMeta> v;
        {
          py::gil_scoped_release nogil;
          v = c.load(nid);
        }
        return PyMetaChannel::to_rows(v);
      })
      .def("clear_node", [](RedisMetaChannel& c, uint32_t nid) {
        py::gil_scoped_release nogil;
        c.clear_node(nid);
      });

  py::class_<InProcMetaChannel, std::shared_ptr<InProcMetaChannel>>(m, "InProcMetaChannel")
      .def(py::init([] { return std::make_shared<InProcMetaChannel>(); }))
      .def_static("named", &InProcMetaChannel::named)
      .def("publish", [](InProcMetaChannel& c, uint32_t nid, py::list rows) {
        std::vector<BlockMeta> v;
        for (auto row : rows) {
          py::tuple t = row.cast<py::tuple>();
          BlockMeta b;
          b.ph = t[0].cast<uint64_t>(); b.pb = t[1].cast<int64_t>(); b.nid = t[2].cast<uint32_t>();
          b.hash = t[3].cast<uint64_t>(); b.lt = t[4].cast<int64_t>(); b.state = t[5].cast<int>();
          v.push_back(b);
        }
        c.publish(nid, v);
      })
      .def("remove", &InProcMetaChannel::remove)
      .def("list_nodes", &InProcMetaChannel::list_nodes)
      .def("load", [](InProcMetaChannel& c, uint32_t nid) { return PyMetaChannel::to_rows(c.load(nid)); })
      .def("clear_node", &InProcMetaChannel::clear_node)
      .def("total_records", &InProcMetaChannel::total_records);

  py::class_<LocalRadixTree, std::shared_ptr<LocalRadixTree>>(m, "LocalRadixTree")
      .def(py::init([](uint32_t nid, int tpb, int64_t max_blocks, const std::string& policy, double reward,
                       py::object channel, int64_t lease_ttl_ms, int64_t renew_margin_ms, int64_t refresh_ms,
                       int64_t safety_ttl_ms, bool start_thread) {
             LeaseOptions o;
             o.lease_ttl_ms = lease_ttl_ms;
             o.renew_margin_ms = renew_margin_ms;
             o.refresh_interval_ms = refresh_ms;
             o.safety_ttl_ms = safety_ttl_ms;
             return gil_free_delete(new LocalRadixTree(nid, tpb, max_blocks, parse_policy(policy), reward,
                                                       channel_from_py(channel), o, start_thread));
           }),
           py::arg("node_id"), py::arg("tokens_per_block"), py::arg("max_num_blocks") = 0,
           py::arg("eviction_policy") = "lru", py::arg("hit_reward_seconds") = 0.0, py::arg("channel") = py::none(),
           py::arg("lease_ttl_ms") = 10000, py::arg("renew_margin_ms") = 4000, py::arg("refresh_interval_ms") = 100,
           py::arg("safety_ttl_ms") = 100, py::arg("start_thread") = true)
      .def("match_prefix", [](LocalRadixTree& t, U64Array hashes, int64_t n, bool update) {
             if (n < 0 || n > (int64_t)hashes.size()) n = (int64_t)hashes.size();
             PyMatch pm;
             pm.r = t.match_prefix(hashes.data(), n, update);
             return pm;
           }, py::arg("block_hashes"), py::arg("num_blocks") = -1, py::arg("update_cache_info") = true)
      .def("insert", [](LocalRadixTree& t, I64Array physical, U64Array hashes, int64_t num_insert, bool ready,
                        py::object match) {
             const MatchResult* mr = nullptr;
             PyMatch pm;
             if (!match.is_none()) { pm = match.cast<PyMatch>(); mr = &pm.r; }
             if (num_insert < 0) num_insert = (int64_t)hashes.size();
             return handle_to_py(t.insert(physical.data(), (int64_t)physical.size(), hashes.data(),
                                          (int64_t)hashes.size(), num_insert, ready, mr));
           }, py::arg("physical_block_ids"), py::arg("block_hashes"), py::arg("num_insert_blocks") = -1,
           py::arg("is_ready") = true, py::arg("match_result") = py::none())
      .def("evict", [](LocalRadixTree& t, int64_t n) {
             EvictResult r = t.evict(n);
             return py::make_tuple(to_array(r.blocks), to_array(r.hashes));
           })
      .def("lock", [](LocalRadixTree& t, py::object h) { t.lock(handle_from_py(h)); })
      .def("unlock", [](LocalRadixTree& t, py::object h) { t.unlock(handle_from_py(h)); })
      .def("set_ready", [](LocalRadixTree& t, py::object h, bool ready, int64_t len) {
             t.set_ready(handle_from_py(h), ready, len);
           }, py::arg("node"), py::arg("ready") = true, py::arg("ready_length") = -1)
      .def("remove_unready_leaf", [](LocalRadixTree& t, py::object h) {
             return to_array(t.remove_unready_leaf(handle_from_py(h)));
           })
      .def("truncate_unready_leaf", [](LocalRadixTree& t, py::object h, int64_t keep) {
             return to_array(t.truncate_unready_leaf(handle_from_py(h), keep));
           })
      .def("reset", [](LocalRadixTree& t) {
             std::vector<int64_t> v;
             { py::gil_scoped_release rel; v = t.reset(); }
             return to_array(v);
           })
      .def("total_cached_blocks", &LocalRadixTree::total_cached_blocks)
      .def("num_evictable_blocks", &LocalRadixTree::num_evictable_blocks)
      .def("refresh_once", [](LocalRadixTree& t, int64_t now_ms) {
             py::gil_scoped_release rel;
             t.refresh_once(now_ms);
           }, py::arg("now_ms") = -1)
      .def("set_clock_override_ms", &LocalRadixTree::set_clock_override_ms)
      .def("shutdown", [](LocalRadixTree& t) { py::gil_scoped_release rel; t.shutdown(); })
      .def_property_readonly("node_id", &LocalRadixTree::node_id)
      .def("stats", [](LocalRadixTree& t) {
             LocalTreeStats s = t.stats();
             py::dict d;
             d["published"] = s.published;
             d["renewed"] = s.renewed;
             d["withdrawn"] = s.withdrawn;
             d["marked_about_to_evict"] = s.marked_about_to_evict;
             d["refreshes"] = s.refreshes;
             return d;
           })
      // node accessors used by the Python cache engine
      .def("alive", [](LocalRadixTree& t, py::object h) { return t.raw_index().alive(handle_from_py(h)); })
      .def("is_root", [](LocalRadixTree& t, py::object h) { return t.raw_index().is_root(handle_from_py(h)); })
      .def("root", [](LocalRadixTree& t) { return handle_to_py(t.raw_index().root_handle()); })
      .def("node_size", [](LocalRadixTree& t, py::object h) { return t.raw_index().node_size(handle_from_py(h)); })
      .def("node_ready", [](LocalRadixTree& t, py::object h) { return t.raw_index().node_ready(handle_from_py(h)); })
      .def("node_lock_cnt", [](LocalRadixTree& t, py::object h) { return t.raw_index().node_lock_cnt(handle_from_py(h)); })
      .def("node_parent", [](LocalRadixTree& t, py::object h) {
             return handle_to_py(t.raw_index().node_parent(handle_from_py(h)));
           })
      .def("node_is_leaf", [](LocalRadixTree& t, py::object h) { return t.raw_index().node_is_leaf(handle_from_py(h)); });

  py::class_<DistributedRadixTree, std::shared_ptr<DistributedRadixTree>>(m, "DistributedRadixTree")
      .def(py::init([](uint32_t self_nid, py::object channel, int64_t refresh_ms, int64_t safety_ms, bool start_thread) {
             return gil_free_delete(new DistributedRadixTree(self_nid, channel_from_py(channel), refresh_ms, safety_ms,
                                                             start_thread));
           }),
           py::arg("node_id"), py::arg("channel"), py::arg("refresh_interval_ms") = 100,
           py::arg("safety_ttl_ms") = 100, py::arg("start_thread") = true)
      .def("refresh_once", [](DistributedRadixTree& t) { py::gil_scoped_release rel; t.refresh_once(); })
      .def("match_prefix", [](DistributedRadixTree& t, U64Array hashes, int64_t n, int64_t now_ms) {
             if (n < 0 || n > (int64_t)hashes.size()) n = (int64_t)hashes.size();
             RemoteMatch r = t.match_prefix(hashes.data(), n, now_ms);
             return py::make_tuple(r.num_matched, to_array(r.physical_blocks), to_array(r.node_ids));
           }, py::arg("block_hashes"), py::arg("num_blocks") = -1, py::arg("now_ms") = -1)
      .def("set_clock_override_ms", &DistributedRadixTree::set_clock_override_ms)
      .def("shutdown", [](DistributedRadixTree& t) { py::gil_scoped_release rel; t.shutdown(); })
      .def_property_readonly("generation", &DistributedRadixTree::generation)
      .def("num_remote_blocks", &DistributedRadixTree::num_remote_blocks);
}
