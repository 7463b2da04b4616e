// Cross-node prefix index: every node publishes which blocks its host tier holds,
// with a lease, and keeps a read-only picture of what the other nodes hold.
//
// Roles follow the reference's distributed radix trees (csrc/dist/local_radix_tree.cpp:193-245,
// 351-454; csrc/dist/distributed_radix_tree.cpp:119-204,272-416; csrc/dist/block_meta.h:9-16):
//   * LocalRadixTree  = the tier's RadixIndex plus a lease per published block and a refresh
//     step that, in priority order, withdraws evicted blocks, announces blocks about to be
//     evicted, publishes new blocks and renews leases;
//   * DistributedRadixTree = a refresh step that rebuilds a read-only reference index from
//     every other node's published blocks and swaps it in as a new generation;
//   * MetaChannel = where the block records live. The reference talks to Redis
//     (csrc/dist/redis_meta_channel.h:58-133); here the channel is an interface with an
//     in-process registry (several nodes in one process, used by single-box deployments
//     and tests) and a trampoline so that a channel written in Python (the registry
//     client) can be plugged in.
// Because block hashes are cumulative (hash i covers tokens [0, (i+1)*tokens_per_block)),
// the reference index does not need tree edges: a block matches when its hash is present
// and its recorded parent hash equals the previous block's hash.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "radix_index.h"

namespace fkv {

enum LeaseState : int { LEASE_NORMAL = 0, LEASE_ABOUT_TO_EVICT = 1, LEASE_EVICTED = 2 };

struct BlockMeta {
  uint64_t ph = 0;    // parent block hash (0 for the first block of a sequence)
  int64_t pb = 0;     // physical block id in the owner's host pool
  uint32_t nid = 0;   // owner node
  uint64_t hash = 0;  // cumulative block hash
  int64_t lt = 0;     // lease expiry, milliseconds on the shared clock
  int state = LEASE_NORMAL;
};

class MetaChannel {
 public:
  virtual ~MetaChannel() = default;
  virtual void publish(uint32_t nid, const std::vector<BlockMeta>& metas) = 0;  // insert or overwrite by hash
  virtual void remove(uint32_t nid, const std::vector<uint64_t>& hashes) = 0;
  virtual std::vector<uint32_t> list_nodes() = 0;
  virtual std::vector<BlockMeta> load(uint32_t nid) = 0;
  virtual void clear_node(uint32_t nid) = 0;
};

class InProcMetaChannel : public MetaChannel {
 public:
  // process-wide registry by name, so that several managers in one process share a channel
  static std::shared_ptr<InProcMetaChannel> named(const std::string& name);
  void publish(uint32_t nid, const std::vector<BlockMeta>& metas) override;
  void remove(uint32_t nid, const std::vector<uint64_t>& hashes) override;
  std::vector<uint32_t> list_nodes() override;
  std::vector<BlockMeta> load(uint32_t nid) override;
  void clear_node(uint32_t nid) override;
  size_t total_records();

 private:
  std::mutex mu_;
  std::unordered_map<uint32_t, std::unordered_map<uint64_t, BlockMeta>> nodes_;
};

int64_t wall_clock_ms();

struct LeaseOptions {
  int64_t lease_ttl_ms = 10000;     // a published block stays readable this long after each renewal
  int64_t renew_margin_ms = 4000;   // renew when less than this is left
  int64_t refresh_interval_ms = 100;
  int64_t safety_ttl_ms = 100;      // readers ignore blocks closer than this to expiry
};

struct LocalTreeStats {
  uint64_t published = 0, renewed = 0, withdrawn = 0, marked_about_to_evict = 0, refreshes = 0;
};

class LocalRadixTree {
 public:
  LocalRadixTree(uint32_t nid, int tokens_per_block, int64_t max_num_blocks, EvictPolicy policy,
                 double hit_reward_seconds, std::shared_ptr<MetaChannel> channel, LeaseOptions opt,
                 bool start_thread);
  ~LocalRadixTree();
  void shutdown();   // stops the refresh thread; idempotent

  MatchResult match_prefix(const uint64_t* hashes, int64_t n, bool update_cache_info);
  NodeHandle insert(const int64_t* physical, int64_t num_physical, const uint64_t* hashes, int64_t n,
                    int64_t num_insert, bool ready, const MatchResult* match);
  // Frees what no peer can still be reading; what is held back by a lease is marked
  // ABOUT_TO_EVICT (no further renewals) and becomes evictable once its lease ran out.
  EvictResult evict(int64_t num_blocks);
  void lock(NodeHandle h);
  void unlock(NodeHandle h);
  void set_ready(NodeHandle h, bool ready, int64_t ready_length);
  std::vector<int64_t> remove_unready_leaf(NodeHandle h);
  std::vector<int64_t> truncate_unready_leaf(NodeHandle h, int64_t keep);
  std::vector<int64_t> reset();
  int64_t total_cached_blocks();
  int64_t num_evictable_blocks();

  // One pass of the refresh thread; `now_ms < 0` reads the wall clock.
  void refresh_once(int64_t now_ms = -1);
  void set_clock_override_ms(int64_t ms) { clock_override_ms_ = ms; }
  LocalTreeStats stats();
  uint32_t node_id() const { return nid_; }
  RadixIndex& raw_index() { return index_; }  // callers hold no other reference across threads

 private:
  struct Lease {
    uint64_t ph;
    int64_t pb;
    int64_t lt = 0;
    int state = LEASE_NORMAL;
    bool published = false;
    bool dirty = true;  // needs (re)publication
  };
  int64_t now_ms() const;
  void track_ready_locked(NodeHandle h, int64_t ready_length);
  void thread_main();

  uint32_t nid_;
  RadixIndex index_;
  std::shared_ptr<MetaChannel> channel_;
  LeaseOptions opt_;
  std::mutex mu_;
  std::unordered_map<uint64_t, Lease> leases_;
  std::vector<uint64_t> pending_remove_;
  LocalTreeStats stats_;
  int64_t clock_override_ms_ = -1;
  std::atomic<bool> stop_{false};
  std::condition_variable cv_;
  std::thread th_;
};

struct RemoteMatch {
  int64_t num_matched = 0;
  std::vector<int64_t> physical_blocks;
  std::vector<uint32_t> node_ids;
};

class DistributedRadixTree {
 public:
  DistributedRadixTree(uint32_t self_nid, std::shared_ptr<MetaChannel> channel, int64_t refresh_interval_ms,
                       int64_t safety_ttl_ms, bool start_thread);
  ~DistributedRadixTree();
  void shutdown();
  // Rebuilds the reference index from every other node (nearest node id first: on a
  // duplicate hash the nearest owner wins) and publishes it as a new generation.
  void refresh_once();
  RemoteMatch match_prefix(const uint64_t* hashes, int64_t n, int64_t now_ms = -1);
  uint64_t generation() const { return generation_.load(); }
  int64_t num_remote_blocks();
  void set_clock_override_ms(int64_t ms) { clock_override_ms_ = ms; }

 private:
  using RefIndex = std::unordered_map<uint64_t, BlockMeta>;
  void thread_main();
  uint32_t self_;
  std::shared_ptr<MetaChannel> channel_;
  int64_t refresh_ms_, safety_ms_;
  std::mutex mu_;                             // guards the pointer swap only
  std::shared_ptr<const RefIndex> current_;   // readers copy the pointer and match without the lock
  std::atomic<uint64_t> generation_{0};
  int64_t clock_override_ms_ = -1;
  std::atomic<bool> stop_{false};
  std::mutex sleep_mu_;
  std::condition_variable cv_;
  std::thread th_;
};

}  // namespace fkv
