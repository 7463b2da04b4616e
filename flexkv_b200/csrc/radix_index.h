// Prefix index of one cache tier: a compressed radix tree over cumulative
// block hashes, with readiness, lock counts and pluggable eviction order.
//
// Behavioural counterpart of the reference's CRadixTreeIndex / CRadixNode
// (csrc/radix_tree.h:21-257, csrc/radix_tree.cpp:260-839) and its eviction
// comparators (csrc/eviction_strategy.cpp:36-134). The structure here is a
// slab of nodes addressed by generation-tagged 64-bit handles, so a stale
// handle (node freed, merged away or re-used since the match) is detected in
// O(1) instead of by walking parent links.
#pragma once
#include <cstdint>
#include <functional>
#include <list>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace fkv {

enum class EvictPolicy : int { LRU = 0, LFU = 1, FIFO = 2, MRU = 3, FILO = 4, SLRU = 5 };
EvictPolicy parse_policy(const std::string& s);

using NodeHandle = uint64_t;
static constexpr NodeHandle kNullHandle = ~0ULL;

struct MatchResult {
  int64_t num_ready_matched = 0;        // contiguous ready prefix, in blocks
  int64_t num_matched = 0;              // matched prefix ready or not
  int64_t last_node_matched_length = 0; // blocks matched inside last_node
  NodeHandle last_ready_node = kNullHandle;
  NodeHandle last_node = kNullHandle;   // deepest node with a match (root if none)
  std::vector<int64_t> physical_blocks; // size num_matched
  // sliding-window state: deepest fully matched ready node that carries a window snapshot
  NodeHandle last_swa_node = kNullHandle;
  int64_t swa_hit_blocks = 0;           // prefix length (blocks) that snapshot covers
  int32_t swa_slot = -1;
};

struct EvictResult {
  std::vector<int64_t> blocks;
  std::vector<uint64_t> hashes;
};

// Flat image of the ready part of an index, parents before children: node i hangs below
// node parents[i] (-1 = the root) and owns sizes[i] consecutive entries of hashes / blocks.
struct IndexSnapshot {
  std::vector<int32_t> parents;
  std::vector<int64_t> sizes;
  std::vector<uint64_t> hashes;
  std::vector<int64_t> blocks;
};

class RadixIndex {
 public:
  RadixIndex(int tokens_per_block, int64_t max_num_blocks, EvictPolicy policy,
             double hit_reward_seconds = 0.0, uint32_t slru_threshold = 2);

  // count_stats=false for lookups the index makes on its own behalf (inside insert).
  MatchResult match_prefix(const uint64_t* hashes, int64_t n, bool update_cache_info, bool count_stats = true);

  // Adds hashes[num_matched:num_insert) with the given physical blocks below
  // the match point. `match` may be null (the call re-matches). Throws
  // std::runtime_error on a stale match (nothing is mutated, the caller keeps
  // its blocks). Returns kNullHandle when there is nothing to add.
  NodeHandle insert(const int64_t* physical, int64_t num_physical, const uint64_t* hashes, int64_t n,
                    int64_t num_insert, bool ready, const MatchResult* match);

  EvictResult evict(int64_t num_blocks);

  // Optional veto consulted for every eviction candidate: return true to keep the node
  // (used by the lease layer: blocks a peer may still be reading must stay). The callback
  // sees the node's block hashes and must not call back into the index.
  using EvictVeto = std::function<bool(const uint64_t* hashes, size_t n)>;
  void set_evict_veto(EvictVeto v) { veto_ = std::move(v); }
  // Hash lists of leaves that only the veto keeps alive, in eviction order, until they
  // cover at least min_blocks blocks (no cascading to parents).
  std::vector<std::vector<uint64_t>> vetoed_leaves(int64_t min_blocks) const;
  // ---- sliding-window snapshots mounted on nodes --------------------------------
  // A node carries at most one snapshot, valid at its trailing block (the window state
  // after the node's last token). Snapshots are a subset of full KV: freeing a node's
  // blocks frees its slot; a split leaves the snapshot on the suffix half. Slots that
  // the index gave up are buffered until drain_freed_swa_slots()
  // (reference: csrc/radix_tree.h:32-46, csrc/radix_tree.cpp:541-582).
  void set_swa(NodeHandle h, int32_t slot);
  bool has_swa(NodeHandle h) const;
  int32_t swa_slot(NodeHandle h) const;
  int swa_lock_cnt(NodeHandle h) const;
  void lock_swa(NodeHandle h);     // takes a full lock as well: full locks >= window locks
  void unlock_swa(NodeHandle h);
  // Frees up to n snapshots, least recently used first. Interior nodes and fully locked
  // leaves only lose the snapshot; an unlocked ready leaf is deleted whole (its blocks
  // are returned). Returns the number of snapshots freed.
  int64_t evict_swa(int64_t n, std::vector<int64_t>* freed_full_blocks, std::vector<uint64_t>* freed_hashes);
  std::vector<int32_t> drain_freed_swa_slots();
  int64_t total_swa_slots() const { return (int64_t)swa_lru_.size(); }

  const std::vector<uint64_t>& node_hashes(NodeHandle h) const;
  const std::vector<int64_t>& node_blocks(NodeHandle h) const;

  void lock(NodeHandle h);
  void unlock(NodeHandle h);
  // marks `h` and as many ancestors as needed to cover ready_length blocks
  void set_ready(NodeHandle h, bool ready, int64_t ready_length);
  // detaches h when it is still an unready, unlocked leaf; returns its blocks
  std::vector<int64_t> remove_unready_leaf(NodeHandle h);
  // keeps the first `keep` blocks of an unready, unlocked leaf and returns the rest (keep <= 0 removes it)
  std::vector<int64_t> truncate_unready_leaf(NodeHandle h, int64_t keep);
  std::vector<int64_t> reset();  // returns every physical block that was indexed

  // Warm restart of a tier whose bytes outlive the process (SSD files, a shared mount):
  // export_ready() lists every ready node (subtrees below an unready node are left out,
  // their data was still in flight); import_snapshot() rebuilds them in an empty index and
  // returns the number of blocks restored. A malformed image (forward parent, size mismatch,
  // block id out of range or listed twice) throws std::invalid_argument and leaves the index empty.
  IndexSnapshot export_ready() const;
  int64_t import_snapshot(const IndexSnapshot& snap);

  bool alive(NodeHandle h) const;
  bool is_root(NodeHandle h) const { return h == root_handle(); }
  NodeHandle root_handle() const { return make_handle(0); }
  int64_t node_size(NodeHandle h) const;
  bool node_ready(NodeHandle h) const;
  int node_lock_cnt(NodeHandle h) const;
  NodeHandle node_parent(NodeHandle h) const;
  bool node_is_leaf(NodeHandle h) const;
  uint32_t node_hit_count(NodeHandle h) const;

  int64_t total_cached_blocks() const { return total_blocks_; }
  int64_t total_ready_blocks() const;
  int64_t num_nodes() const { return live_nodes_; }
  int64_t num_leaves() const { return (int64_t)leaves_.size(); }
  int64_t num_evictable_blocks() const;
  int tokens_per_block() const { return tokens_per_block_; }
  bool is_empty() const { return live_nodes_ == 1; }

  // test hook: a fixed clock in microseconds (negative = wall clock)
  void set_clock_override(int64_t us) { clock_override_us_ = us; }
  void set_policy(EvictPolicy p) { policy_ = p; }

  // counters (cumulative): hit = full match, match = partial, miss = none
  uint64_t stat_hit = 0, stat_match = 0, stat_miss = 0, stat_insert_blocks = 0, stat_evict_blocks = 0;

 private:
  struct Node {
    std::vector<uint64_t> hashes;
    std::vector<int64_t> blocks;
    std::unique_ptr<std::unordered_map<uint64_t, int32_t>> children;
    int32_t parent = -1;
    uint32_t gen = 0;
    int32_t lock_cnt = 0;
    uint32_t hit_count = 0;
    bool ready = false;
    bool live = false;
    int64_t grace_us = 0, last_access_us = 0, creation_us = 0;
    uint64_t serial = 0;  // allocation order, the deterministic eviction tie-break
    int32_t swa_slot = -1;
    int32_t swa_lock = 0;
    bool on_swa_lru = false;
    std::list<int32_t>::iterator swa_it;
    size_t size() const { return hashes.size(); }
    bool leaf() const { return !children || children->empty(); }
  };

  NodeHandle make_handle(int32_t idx) const { return ((uint64_t)nodes_[idx].gen << 32) | (uint32_t)idx; }
  int32_t resolve(NodeHandle h) const;           // -1 if stale
  int32_t resolve_or_throw(NodeHandle h) const;
  int32_t alloc_node();
  void free_node(int32_t idx);
  int64_t now_us() const;
  void touch(Node& n, int64_t now);
  int32_t find_child(const Node& n, uint64_t head) const;
  void add_child(int32_t parent, int32_t child);
  void remove_child(int32_t parent, uint64_t head);
  int32_t split(int32_t idx, int64_t prefix_len);  // returns the new prefix node
  bool evictable(int32_t idx) const;
  bool evictable_ignoring_veto(int32_t idx) const;
  bool evict_before(const Node& a, const Node& b) const;  // a leaves before b
  void validate_insert_target(const uint64_t* hashes, int64_t n, int64_t num_insert, const MatchResult& m,
                              int32_t idx) const;

  int tokens_per_block_;
  int64_t max_num_blocks_;
  EvictPolicy policy_;
  int64_t hit_reward_us_;
  uint32_t slru_threshold_;
  int64_t clock_override_us_ = -1;

  std::vector<Node> nodes_;
  std::vector<int32_t> free_slots_;
  std::unordered_set<int32_t> leaves_;
  int64_t total_blocks_ = 0;
  int64_t live_nodes_ = 0;
  uint64_t next_serial_ = 0;
  EvictVeto veto_;
  void drop_swa(int32_t idx);           // frees the node's snapshot, if any
  // Once window snapshots are in use, a leaf without one serves no window-aware request. After a deletion
  // the ancestors that became such leaves (evictable, no snapshot) are deleted too; their blocks and hashes are
  // appended to the output, beyond what the caller asked for. Returns the first ancestor that stays
  // (reference: flexkv/cache/radixtree.py:726-749).
  int32_t prune_snapshotless_leaves(int32_t idx, std::vector<int64_t>* blocks, std::vector<uint64_t>* hashes);
  bool swa_armed_ = false;              // a snapshot was mounted at least once; survives reset()
  void swa_touch(int32_t idx);          // moves the node to the recently-used end
  std::list<int32_t> swa_lru_;          // front = least recently used
  std::vector<int32_t> freed_swa_;
};

// Fixed-capacity id pool with duplicate / double-free detection
// (reference behaviour: flexkv/cache/mempool.py:26-56).
class BlockPool {
 public:
  explicit BlockPool(int64_t num_blocks);
  // returns fewer than n ids only when strict == false and the pool is short
  std::vector<int64_t> allocate(int64_t n, bool strict);
  void recycle(const int64_t* ids, int64_t n);
  // takes these specific free ids out of the pool (blocks restored from a saved index);
  // throws and changes nothing when one is out of range, listed twice or already in use
  void reserve(const int64_t* ids, int64_t n);
  void reset();
  int64_t num_free() const { return (int64_t)free_.size(); }
  int64_t num_total() const { return total_; }
  int64_t num_used() const { return total_ - (int64_t)free_.size(); }
  bool is_free(int64_t id) const { return id >= 0 && id < total_ && !used_[id]; }

 private:
  int64_t total_;
  std::vector<int64_t> free_;   // stack, lowest id on top after reset
  std::vector<uint8_t> used_;
};

}  // namespace fkv
