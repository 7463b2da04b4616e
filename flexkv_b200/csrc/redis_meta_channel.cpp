#include "redis_meta_channel.h"

#include <algorithm>
#include <cinttypes>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>

namespace fkv {
namespace {

void throw_on_error(const RespValue& v, const char* what) {
  if (v.type == RespValue::kError) throw std::runtime_error(std::string("redis ") + what + ": " + v.str);
}

// field -> value pairs of an HGETALL reply
bool field(const RespValue& flat, const char* name, std::string& out) {
  for (size_t i = 0; i + 1 < flat.items.size(); i += 2)
    if (flat.items[i].str == name) {
      out = flat.items[i + 1].str;
      return true;
    }
  return false;
}

}  // namespace

RedisMetaChannel::RedisMetaChannel(std::string host, int port, std::string kind, int timeout_ms, std::string password,
                                   int db)
    : kind_(std::move(kind)), client_(std::move(host), port, timeout_ms, std::move(password), db) {}

std::string RedisMetaChannel::key(uint32_t nid, uint64_t hash) const {
  char buf[64];
  std::snprintf(buf, sizeof(buf), ":block:%u:%016" PRIx64, nid, hash);
  return kind_ + buf;
}

std::vector<std::string> RedisMetaChannel::scan(const std::string& prefix) {
  std::vector<std::string> keys;
  std::string cursor = "0";
  do {
    RespValue v = client_.command({"SCAN", cursor, "MATCH", prefix + "*", "COUNT", "1000"});
    throw_on_error(v, "SCAN");
    if (v.type != RespValue::kArray || v.items.size() != 2) throw std::runtime_error("redis SCAN: unexpected reply");
    cursor = v.items[0].type == RespValue::kInteger ? std::to_string(v.items[0].integer) : v.items[0].str;
    for (const auto& k : v.items[1].items) keys.push_back(k.str);
  } while (cursor != "0");
  std::sort(keys.begin(), keys.end());
  keys.erase(std::unique(keys.begin(), keys.end()), keys.end());     // SCAN may return a key twice
  return keys;
}

void RedisMetaChannel::publish(uint32_t nid, const std::vector<BlockMeta>& metas) {
  if (metas.empty()) return;
  std::vector<std::vector<std::string>> cmds;
  cmds.reserve(metas.size());
  for (const BlockMeta& b : metas)
    cmds.push_back({"HSET", key(nid, b.hash), "ph", std::to_string(b.ph), "pb", std::to_string(b.pb), "nid",
                    std::to_string(b.nid), "hash", std::to_string(b.hash), "lt", std::to_string(b.lt), "state",
                    std::to_string(b.state)});
  for (const RespValue& v : client_.pipeline(cmds)) throw_on_error(v, "HSET");
}

void RedisMetaChannel::remove(uint32_t nid, const std::vector<uint64_t>& hashes) {
  for (size_t i = 0; i < hashes.size(); i += 512) {
    std::vector<std::string> cmd{"DEL"};
    for (size_t j = i; j < std::min(hashes.size(), i + 512); ++j) cmd.push_back(key(nid, hashes[j]));
    throw_on_error(client_.command(cmd), "DEL");
  }
}

std::vector<uint32_t> RedisMetaChannel::list_nodes() {
  std::vector<std::string> keys = scan("node:");
  std::vector<std::vector<std::string>> cmds;
  for (const auto& k : keys) cmds.push_back({"HGETALL", k});
  std::vector<uint32_t> out;
  if (cmds.empty()) return out;
  for (const RespValue& v : client_.pipeline(cmds)) {
    throw_on_error(v, "HGETALL");
    std::string status, id;
    if (field(v, "status", status) && status == "active" && field(v, "node_id", id))
      out.push_back((uint32_t)std::strtoul(id.c_str(), nullptr, 10));
  }
  std::sort(out.begin(), out.end());
  return out;
}

std::vector<BlockMeta> RedisMetaChannel::load(uint32_t nid) {
  std::vector<std::string> keys = scan(kind_ + ":block:" + std::to_string(nid) + ":");
  std::vector<std::vector<std::string>> cmds;
  for (const auto& k : keys) cmds.push_back({"HGETALL", k});
  std::vector<BlockMeta> out;
  if (cmds.empty()) return out;
  for (const RespValue& v : client_.pipeline(cmds)) {
    throw_on_error(v, "HGETALL");
    std::string ph, pb, n, h, lt, st;
    if (!(field(v, "ph", ph) && field(v, "pb", pb) && field(v, "nid", n) && field(v, "hash", h) &&
          field(v, "lt", lt) && field(v, "state", st)))
      continue;                                   // deleted since the scan, or not a block record
    BlockMeta b;
    b.ph = std::strtoull(ph.c_str(), nullptr, 10);
    b.pb = std::strtoll(pb.c_str(), nullptr, 10);
    b.nid = (uint32_t)std::strtoul(n.c_str(), nullptr, 10);
    b.hash = std::strtoull(h.c_str(), nullptr, 10);
    b.lt = std::strtoll(lt.c_str(), nullptr, 10);
    b.state = (int)std::strtol(st.c_str(), nullptr, 10);
    out.push_back(b);
  }
  return out;
}

void RedisMetaChannel::clear_node(uint32_t nid) {
  std::vector<std::string> keys = scan(kind_ + ":block:" + std::to_string(nid) + ":");
  for (size_t i = 0; i < keys.size(); i += 512) {
    std::vector<std::string> cmd{"DEL"};
    for (size_t j = i; j < std::min(keys.size(), i + 512); ++j) cmd.push_back(keys[j]);
    throw_on_error(client_.command(cmd), "DEL");
  }
}

}  // namespace fkv
