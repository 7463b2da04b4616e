// Block records of the cross-node index in a Redis server, written and read from native code.
//
// Same key schema as the Python RegistryMetaChannel and as the reference (csrc/dist/redis_meta_channel.cpp:
// 198-215): one hash per published block, key "<kind>:block:<node id>:<block hash, 16 hex digits>", fields
// ph, pb, nid, hash, lt, state as decimal strings; live nodes are the "node:<id>" hashes with status "active".
// The lease-aware tree and the remote view call the channel from their own refresh threads, so a native
// channel keeps that path free of the interpreter lock. Commands touching many keys are pipelined.
#pragma once
#include <memory>
#include <string>

#include "dist_index.h"
#include "resp_client.h"

namespace fkv {

class RedisMetaChannel : public MetaChannel {
 public:
  RedisMetaChannel(std::string host, int port, std::string kind = "CPUB", int timeout_ms = 3000,
                   std::string password = "", int db = 0);
  void publish(uint32_t nid, const std::vector<BlockMeta>& metas) override;
  void remove(uint32_t nid, const std::vector<uint64_t>& hashes) override;
  std::vector<uint32_t> list_nodes() override;
  std::vector<BlockMeta> load(uint32_t nid) override;
  void clear_node(uint32_t nid) override;

 private:
  std::string key(uint32_t nid, uint64_t hash) const;
  std::vector<std::string> scan(const std::string& prefix);
  std::string kind_;
  RespClient client_;
};

}  // namespace fkv
