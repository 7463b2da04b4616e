#include "radix_index.h"
#include "native_log.h"

#include <algorithm>
#include <chrono>
#include <queue>
#include <unordered_set>

namespace fkv {

EvictPolicy parse_policy(const std::string& s) {
  std::string t;
  for (char c : s) t.push_back((char)std::tolower((unsigned char)c));
  if (t == "lru") return EvictPolicy::LRU;
  if (t == "lfu") return EvictPolicy::LFU;
  if (t == "fifo") return EvictPolicy::FIFO;
  if (t == "mru") return EvictPolicy::MRU;
  if (t == "filo") return EvictPolicy::FILO;
  if (t == "slru") return EvictPolicy::SLRU;
  throw std::invalid_argument("unknown eviction policy: " + s);
}

RadixIndex::RadixIndex(int tokens_per_block, int64_t max_num_blocks, EvictPolicy policy,
                       double hit_reward_seconds, uint32_t slru_threshold)
    : tokens_per_block_(tokens_per_block), max_num_blocks_(max_num_blocks), policy_(policy),
      hit_reward_us_((int64_t)(hit_reward_seconds * 1e6)), slru_threshold_(slru_threshold) {
  if (tokens_per_block <= 0 || (tokens_per_block & (tokens_per_block - 1)) != 0)
    throw std::invalid_argument("tokens_per_block must be a power of two");
  nodes_.reserve(1024);
  int32_t r = alloc_node();  // root, index 0
  nodes_[r].ready = true;
  nodes_[r].parent = -1;
}

int64_t RadixIndex::now_us() const {
  if (clock_override_us_ >= 0) return clock_override_us_;
  using namespace std::chrono;
  return duration_cast<microseconds>(system_clock::now().time_since_epoch()).count();
}

int32_t RadixIndex::alloc_node() {
  int32_t idx;
  if (!free_slots_.empty()) {
    idx = free_slots_.back();
    free_slots_.pop_back();
  } else {
    idx = (int32_t)nodes_.size();
    nodes_.emplace_back();
  }
  Node& n = nodes_[idx];
  n.live = true;
  n.lock_cnt = 0;
  n.hit_count = 0;
  n.ready = false;
  n.parent = -1;
  n.swa_slot = -1;
  n.swa_lock = 0;
  n.on_swa_lru = false;
  int64_t t = now_us();
  n.grace_us = n.last_access_us = n.creation_us = t;
  n.serial = ++next_serial_;
  ++live_nodes_;
  return idx;
}

void RadixIndex::free_node(int32_t idx) {
  drop_swa(idx);
  Node& n = nodes_[idx];
  n.live = false;
  ++n.gen;  // invalidates every outstanding handle
  n.hashes.clear();
  n.hashes.shrink_to_fit();
  n.blocks.clear();
  n.blocks.shrink_to_fit();
  n.children.reset();
  leaves_.erase(idx);
  free_slots_.push_back(idx);
  --live_nodes_;
}

int32_t RadixIndex::resolve(NodeHandle h) const {
  if (h == kNullHandle) return -1;
  uint32_t idx = (uint32_t)(h & 0xffffffffu);
  uint32_t gen = (uint32_t)(h >> 32);
  if (idx >= nodes_.size()) return -1;
  const Node& n = nodes_[idx];
  if (!n.live || n.gen != gen) return -1;
  return (int32_t)idx;
}

int32_t RadixIndex::resolve_or_throw(NodeHandle h) const {
  int32_t i = resolve(h);
  if (i < 0) throw std::runtime_error("radix index: stale or null node handle");
  return i;
}

bool RadixIndex::alive(NodeHandle h) const { return resolve(h) >= 0; }
int64_t RadixIndex::node_size(NodeHandle h) const { return (int64_t)nodes_[resolve_or_throw(h)].size(); }
bool RadixIndex::node_ready(NodeHandle h) const { return nodes_[resolve_or_throw(h)].ready; }
int RadixIndex::node_lock_cnt(NodeHandle h) const { return nodes_[resolve_or_throw(h)].lock_cnt; }
bool RadixIndex::node_is_leaf(NodeHandle h) const { return nodes_[resolve_or_throw(h)].leaf(); }
uint32_t RadixIndex::node_hit_count(NodeHandle h) const { return nodes_[resolve_or_throw(h)].hit_count; }
NodeHandle RadixIndex::node_parent(NodeHandle h) const {
  int32_t p = nodes_[resolve_or_throw(h)].parent;
  return p < 0 ? kNullHandle : make_handle(p);
}

void RadixIndex::touch(Node& n, int64_t now) {
  n.last_access_us = now;
  n.grace_us = std::max(n.grace_us, now) + hit_reward_us_;
  if (n.hit_count != 0xffffffffu) ++n.hit_count;
}

int32_t RadixIndex::find_child(const Node& n, uint64_t head) const {
  if (!n.children) return -1;
  auto it = n.children->find(head);
  return it == n.children->end() ? -1 : it->second;
}

void RadixIndex::add_child(int32_t parent, int32_t child) {
  Node& p = nodes_[parent];
  if (!p.children) p.children = std::make_unique<std::unordered_map<uint64_t, int32_t>>();
  (*p.children)[nodes_[child].hashes.front()] = child;
  nodes_[child].parent = parent;
  leaves_.erase(parent);
}

void RadixIndex::remove_child(int32_t parent, uint64_t head) {
  Node& p = nodes_[parent];
  if (p.children) p.children->erase(head);
  if (p.leaf() && parent != 0) leaves_.insert(parent);
}

MatchResult RadixIndex::match_prefix(const uint64_t* hashes, int64_t n, bool update_cache_info, bool count_stats) {
  MatchResult r;
  r.last_node = root_handle();
  r.last_ready_node = root_handle();
  if (n > 0) r.physical_blocks.reserve((size_t)n);
  int64_t now = update_cache_info ? now_us() : 0;
  int32_t cur = 0;
  int64_t prefix = 0;
  bool ready_chain = true;
  while (prefix < n) {
    int32_t c = find_child(nodes_[cur], hashes[prefix]);
    if (c < 0) break;
    Node& node = nodes_[c];
    int64_t span = std::min<int64_t>((int64_t)node.size(), n - prefix);
    int64_t m;
    // hashes are cumulative, so "position i matches" is monotone in i: a match
    // at the end of the span implies the whole span.
    if (node.hashes[span - 1] == hashes[prefix + span - 1]) {
      m = span;
    } else {
      int64_t lo = 1, hi = span - 1;  // head already matched through the child key
      while (lo < hi) {
        int64_t mid = (lo + hi + 1) >> 1;
        if (node.hashes[mid - 1] == hashes[prefix + mid - 1]) lo = mid; else hi = mid - 1;
      }
      m = lo;
    }
    if (update_cache_info) touch(node, now);
    r.physical_blocks.insert(r.physical_blocks.end(), node.blocks.begin(), node.blocks.begin() + m);
    prefix += m;
    r.last_node = make_handle(c);
    r.last_node_matched_length = m;
    if (ready_chain && node.ready) {
      r.num_ready_matched = prefix;
      r.last_ready_node = make_handle(c);
      // a snapshot sits at the node's trailing block: only a fully matched node exposes it
      if (node.swa_slot >= 0 && m == (int64_t)node.size()) {
        r.last_swa_node = make_handle(c);
        r.swa_hit_blocks = prefix;
        r.swa_slot = node.swa_slot;
        if (update_cache_info) swa_touch(c);
      }
    } else {
      ready_chain = false;
    }
    if (m < (int64_t)node.size()) break;
    cur = c;
  }
  r.num_matched = prefix;
  if (n > 0 && count_stats) {
    if (prefix == n) ++stat_hit; else if (prefix > 0) ++stat_match; else ++stat_miss;
    count_cache_op(prefix == n ? kOpHit : (prefix > 0 ? kOpMatch : kOpMiss), (uint64_t)(prefix > 0 ? prefix : n));
  }
  return r;
}

int32_t RadixIndex::split(int32_t idx, int64_t prefix_len) {
  // The existing node keeps the suffix (so handles held by lockers keep
  // pointing at the deepest part of the path); a new node takes the prefix
  // and is spliced in as the parent.
  int32_t pre = alloc_node();
  Node& node = nodes_[idx];
  Node& p = nodes_[pre];
  int32_t parent = node.parent;
  uint64_t old_head = node.hashes.front();
  p.hashes.assign(node.hashes.begin(), node.hashes.begin() + prefix_len);
  p.blocks.assign(node.blocks.begin(), node.blocks.begin() + prefix_len);
  node.hashes.erase(node.hashes.begin(), node.hashes.begin() + prefix_len);
  node.blocks.erase(node.blocks.begin(), node.blocks.begin() + prefix_len);
  p.ready = node.ready;
  p.hit_count = node.hit_count;
  p.grace_us = node.grace_us;
  p.last_access_us = node.last_access_us;
  p.creation_us = node.creation_us;
  p.parent = parent;
  // re-key: parent -> pre -> node
  (*nodes_[parent].children)[old_head] = pre;
  p.children = std::make_unique<std::unordered_map<uint64_t, int32_t>>();
  (*p.children)[node.hashes.front()] = idx;
  node.parent = pre;
  return pre;
}

void RadixIndex::validate_insert_target(const uint64_t* hashes, int64_t n, int64_t num_insert,
                                        const MatchResult& m, int32_t idx) const {
  auto stale = [](const char* why) {
    throw std::runtime_error(std::string("radix index insert: stale match result; rematch (") + why + ")");
  };
  if (idx < 0) stale("node no longer exists");
  const Node& node = nodes_[idx];
  if (m.num_matched < 0 || m.num_matched > n) stale("matched length out of range");
  if (idx == 0) {
    if (m.num_matched != 0) stale("root cannot carry a match");
    if (num_insert > 0 && find_child(node, hashes[0]) >= 0) stale("first block appeared meanwhile");
    return;
  }
  int64_t ml = m.last_node_matched_length;
  if (ml <= 0 || ml > (int64_t)node.size() || ml > m.num_matched) stale("matched span out of range");
  if (node.parent < 0) stale("detached node");
  if (find_child(nodes_[node.parent], node.hashes.front()) != idx) stale("node not under its parent");
  if (node.hashes[ml - 1] != hashes[m.num_matched - 1] || node.hashes[0] != hashes[m.num_matched - ml])
    stale("matched span changed");
  if (num_insert > m.num_matched) {
    if (ml < (int64_t)node.size()) {
      if (node.hashes[ml] == hashes[m.num_matched]) stale("split point does not diverge");
    } else if (find_child(node, hashes[m.num_matched]) >= 0) {
      stale("target child exists");
    }
  }
}

NodeHandle RadixIndex::insert(const int64_t* physical, int64_t num_physical, const uint64_t* hashes, int64_t n,
                              int64_t num_insert, bool ready, const MatchResult* match) {
  if (num_insert < 0) num_insert = n;
  if (num_insert > n) throw std::invalid_argument("radix index insert: num_insert exceeds hash count");
  MatchResult local;
  if (match == nullptr) {
    local = match_prefix(hashes, num_insert, false, false);
    match = &local;
  }
  if (num_insert <= match->num_matched) return kNullHandle;
  if (num_physical != num_insert - match->num_matched)
    throw std::invalid_argument("radix index insert: physical block count != num_insert - num_matched");
  int32_t idx = resolve(match->last_node);
  validate_insert_target(hashes, n, num_insert, *match, idx);
  if (total_blocks_ + num_physical > max_num_blocks_ && max_num_blocks_ > 0)
    throw std::runtime_error("radix index insert: capacity exceeded");

  int32_t parent = idx;
  if (idx != 0 && match->last_node_matched_length < (int64_t)nodes_[idx].size())
    parent = split(idx, match->last_node_matched_length);

  int32_t nn = alloc_node();
  Node& node = nodes_[nn];
  node.hashes.assign(hashes + match->num_matched, hashes + num_insert);
  node.blocks.assign(physical, physical + num_physical);
  node.ready = ready;
  add_child(parent, nn);
  leaves_.insert(nn);
  total_blocks_ += num_physical;
  stat_insert_blocks += (uint64_t)num_physical;
  count_cache_op(kOpInsert, (uint64_t)num_physical);
  return make_handle(nn);
}

bool RadixIndex::evictable_ignoring_veto(int32_t idx) const {
  if (idx == 0) return false;
  const Node& n = nodes_[idx];
  return n.live && n.leaf() && n.lock_cnt == 0 && n.ready;
}

bool RadixIndex::evictable(int32_t idx) const {
  if (!evictable_ignoring_veto(idx)) return false;
  const Node& n = nodes_[idx];
  return !veto_ || !veto_(n.hashes.data(), n.hashes.size());
}

std::vector<std::vector<uint64_t>> RadixIndex::vetoed_leaves(int64_t min_blocks) const {
  std::vector<int32_t> cand;
  if (!veto_) return {};
  for (int32_t l : leaves_)
    if (evictable_ignoring_veto(l) && !evictable(l)) cand.push_back(l);
  std::sort(cand.begin(), cand.end(), [this](int32_t x, int32_t y) {
    const Node& a = nodes_[x];
    const Node& b = nodes_[y];
    if (evict_before(a, b)) return true;
    if (evict_before(b, a)) return false;
    return a.serial < b.serial;
  });
  std::vector<std::vector<uint64_t>> out;
  int64_t got = 0;
  for (int32_t idx : cand) {
    if (got >= min_blocks) break;
    out.push_back(nodes_[idx].hashes);
    got += (int64_t)nodes_[idx].size();
  }
  return out;
}

const std::vector<uint64_t>& RadixIndex::node_hashes(NodeHandle h) const { return nodes_[resolve_or_throw(h)].hashes; }
const std::vector<int64_t>& RadixIndex::node_blocks(NodeHandle h) const { return nodes_[resolve_or_throw(h)].blocks; }

bool RadixIndex::evict_before(const Node& a, const Node& b) const {
  switch (policy_) {
    case EvictPolicy::LRU: return a.grace_us < b.grace_us;
    case EvictPolicy::MRU: return a.grace_us > b.grace_us;
    case EvictPolicy::FIFO: return a.creation_us < b.creation_us;
    case EvictPolicy::FILO: return a.creation_us > b.creation_us;
    case EvictPolicy::LFU:
      if (a.hit_count != b.hit_count) return a.hit_count < b.hit_count;
      return a.last_access_us < b.last_access_us;
    case EvictPolicy::SLRU: {
      bool pa = a.hit_count >= slru_threshold_, pb = b.hit_count >= slru_threshold_;
      if (pa != pb) return !pa;  // probationary segment leaves first
      return a.last_access_us < b.last_access_us;
    }
  }
  return false;
}

EvictResult RadixIndex::evict(int64_t num_blocks) {
  EvictResult out;
  if (num_blocks <= 0) return out;
  auto later = [this](int32_t x, int32_t y) {  // max-heap comparator: top = evicted first
    const Node& a = nodes_[x];
    const Node& b = nodes_[y];
    if (evict_before(b, a)) return true;
    if (evict_before(a, b)) return false;
    return a.serial > b.serial;  // deterministic tie-break: older allocation leaves first
  };
  std::priority_queue<int32_t, std::vector<int32_t>, decltype(later)> heap(later);
  for (int32_t l : leaves_)
    if (evictable(l)) heap.push(l);
  int64_t need = num_blocks;
  while (need > 0 && !heap.empty()) {
    int32_t idx = heap.top();
    heap.pop();
    Node& node = nodes_[idx];
    int64_t sz = (int64_t)node.size();
    if (sz > need) {
      // partial shrink: drop the tail, the node stays a leaf; its snapshot described the dropped tail
      drop_swa(idx);
      out.blocks.insert(out.blocks.end(), node.blocks.end() - need, node.blocks.end());
      out.hashes.insert(out.hashes.end(), node.hashes.end() - need, node.hashes.end());
      node.blocks.resize((size_t)(sz - need));
      node.hashes.resize((size_t)(sz - need));
      total_blocks_ -= need;
      need = 0;
      break;
    }
    out.blocks.insert(out.blocks.end(), node.blocks.begin(), node.blocks.end());
    out.hashes.insert(out.hashes.end(), node.hashes.begin(), node.hashes.end());
    total_blocks_ -= sz;
    need -= sz;
    int32_t parent = node.parent;
    uint64_t head = node.hashes.front();
    free_node(idx);
    remove_child(parent, head);
    parent = prune_snapshotless_leaves(parent, &out.blocks, &out.hashes);
    if (evictable(parent)) heap.push(parent);
  }
  stat_evict_blocks += (uint64_t)out.blocks.size();
  if (!out.blocks.empty()) count_cache_op(kOpEvict, (uint64_t)out.blocks.size());
  return out;
}

int32_t RadixIndex::prune_snapshotless_leaves(int32_t idx, std::vector<int64_t>* blocks,
                                             std::vector<uint64_t>* hashes) {
  if (!swa_armed_) return idx;
  while (idx > 0 && nodes_[idx].swa_slot < 0 && evictable(idx)) {
    Node& n = nodes_[idx];
    if (blocks) blocks->insert(blocks->end(), n.blocks.begin(), n.blocks.end());
    if (hashes) hashes->insert(hashes->end(), n.hashes.begin(), n.hashes.end());
    total_blocks_ -= (int64_t)n.size();
    const int32_t parent = n.parent;
    const uint64_t head = n.hashes.front();
    free_node(idx);
    remove_child(parent, head);
    idx = parent;
  }
  return idx;
}

void RadixIndex::lock(NodeHandle h) { ++nodes_[resolve_or_throw(h)].lock_cnt; }

void RadixIndex::unlock(NodeHandle h) {
  Node& n = nodes_[resolve_or_throw(h)];
  if (n.lock_cnt <= 0) throw std::runtime_error("radix index: unlock of an unlocked node");
  --n.lock_cnt;
}

void RadixIndex::set_ready(NodeHandle h, bool ready, int64_t ready_length) {
  int32_t idx = resolve_or_throw(h);
  int64_t covered = 0;
  while (idx > 0) {
    Node& n = nodes_[idx];
    n.ready = ready;
    covered += (int64_t)n.size();
    if (ready_length < 0 || covered >= ready_length) break;
    idx = n.parent;
  }
}

std::vector<int64_t> RadixIndex::remove_unready_leaf(NodeHandle h) {
  std::vector<int64_t> out;
  int32_t idx = resolve(h);
  if (idx <= 0) return out;
  Node& n = nodes_[idx];
  if (!n.leaf() || n.ready || n.lock_cnt > 0) return out;
  out = n.blocks;
  total_blocks_ -= (int64_t)n.size();
  int32_t parent = n.parent;
  uint64_t head = n.hashes.front();
  free_node(idx);
  remove_child(parent, head);
  return out;
}

std::vector<int64_t> RadixIndex::truncate_unready_leaf(NodeHandle h, int64_t keep) {
  if (keep <= 0) return remove_unready_leaf(h);
  std::vector<int64_t> out;
  int32_t idx = resolve(h);
  if (idx <= 0) return out;
  Node& n = nodes_[idx];
  if (!n.leaf() || n.ready || n.lock_cnt > 0 || keep >= (int64_t)n.size()) return out;
  out.assign(n.blocks.begin() + keep, n.blocks.end());
  n.blocks.resize((size_t)keep);
  n.hashes.resize((size_t)keep);
  total_blocks_ -= (int64_t)out.size();
  return out;
}

std::vector<int64_t> RadixIndex::reset() {
  std::vector<int64_t> all;
  all.reserve((size_t)total_blocks_);
  for (size_t i = 1; i < nodes_.size(); ++i) {
    Node& n = nodes_[i];
    if (!n.live) continue;
    all.insert(all.end(), n.blocks.begin(), n.blocks.end());
    free_node((int32_t)i);
  }
  nodes_[0].children.reset();
  leaves_.clear();
  swa_lru_.clear();
  freed_swa_.clear();  // the owner re-arms its slot pool as a whole on reset
  total_blocks_ = 0;
  return all;
}

// ---- warm restart ---------------------------------------------------------------

IndexSnapshot RadixIndex::export_ready() const {
  IndexSnapshot snap;
  snap.hashes.reserve((size_t)total_blocks_);
  snap.blocks.reserve((size_t)total_blocks_);
  snap.parents.reserve((size_t)live_nodes_);
  snap.sizes.reserve((size_t)live_nodes_);
  // explicit stack of (node, position of its parent in the image); children in key order
  // so that the image of a given tree is deterministic
  std::vector<std::pair<int32_t, int32_t>> stack;
  auto push_children = [&](const Node& n, int32_t pos) {
    if (!n.children) return;
    std::vector<std::pair<uint64_t, int32_t>> kids(n.children->begin(), n.children->end());
    std::sort(kids.begin(), kids.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
    for (const auto& kv : kids) stack.emplace_back(kv.second, pos);
  };
  push_children(nodes_[0], -1);
  while (!stack.empty()) {
    auto [idx, parent_pos] = stack.back();
    stack.pop_back();
    const Node& n = nodes_[idx];
    if (!n.live || !n.ready) continue;
    int32_t pos = (int32_t)snap.parents.size();
    snap.parents.push_back(parent_pos);
    snap.sizes.push_back((int64_t)n.size());
    snap.hashes.insert(snap.hashes.end(), n.hashes.begin(), n.hashes.end());
    snap.blocks.insert(snap.blocks.end(), n.blocks.begin(), n.blocks.end());
    push_children(n, pos);
  }
  return snap;
}

int64_t RadixIndex::import_snapshot(const IndexSnapshot& snap) {
  if (!is_empty()) throw std::invalid_argument("radix index import: the index is not empty");
  const size_t nn = snap.parents.size();
  if (snap.sizes.size() != nn) throw std::invalid_argument("radix index import: parents / sizes differ in length");
  int64_t total = 0;
  for (size_t i = 0; i < nn; ++i) {
    if (snap.sizes[i] <= 0) throw std::invalid_argument("radix index import: empty node");
    if (snap.parents[i] < -1 || snap.parents[i] >= (int32_t)i)
      throw std::invalid_argument("radix index import: a node is listed before its parent");
    total += snap.sizes[i];
  }
  if ((int64_t)snap.hashes.size() != total || (int64_t)snap.blocks.size() != total)
    throw std::invalid_argument("radix index import: hashes / blocks do not cover the nodes");
  if (max_num_blocks_ > 0 && total > max_num_blocks_)
    throw std::invalid_argument("radix index import: more blocks than this index may hold");
  {
    std::vector<uint8_t> seen((size_t)std::max<int64_t>(max_num_blocks_, 0), 0);
    std::unordered_set<int64_t> seen_sparse;
    for (int64_t b : snap.blocks) {
      if (b < 0 || (max_num_blocks_ > 0 && b >= max_num_blocks_))
        throw std::invalid_argument("radix index import: block id out of range");
      bool dup = max_num_blocks_ > 0 ? seen[(size_t)b]++ != 0 : !seen_sparse.insert(b).second;
      if (dup) throw std::invalid_argument("radix index import: a block id is listed twice");
    }
  }
  // replay as inserts: the image is in pre-order, so the path of the node being added is
  // the path of the previous one cut back to the common ancestor
  std::vector<uint64_t> path;
  std::vector<std::pair<int32_t, size_t>> open;  // (position in the image, path length with that node)
  std::vector<size_t> offset(nn + 1, 0);
  for (size_t i = 0; i < nn; ++i) offset[i + 1] = offset[i] + (size_t)snap.sizes[i];
  try {
    for (size_t i = 0; i < nn; ++i) {
      while (!open.empty() && open.back().first != snap.parents[i]) open.pop_back();
      if (open.empty() && snap.parents[i] != -1)
        throw std::invalid_argument("radix index import: the image is not in pre-order");
      path.resize(open.empty() ? 0 : open.back().second);
      path.insert(path.end(), snap.hashes.begin() + (ptrdiff_t)offset[i], snap.hashes.begin() + (ptrdiff_t)offset[i + 1]);
      NodeHandle h = insert(snap.blocks.data() + offset[i], snap.sizes[i], path.data(), (int64_t)path.size(),
                            (int64_t)path.size(), true, nullptr);
      if (h == kNullHandle) throw std::invalid_argument("radix index import: two nodes share a path");
      open.emplace_back((int32_t)i, path.size());
    }
  } catch (...) {
    reset();
    throw;
  }
  return total;
}

// ---- sliding-window snapshots ---------------------------------------------------

void RadixIndex::drop_swa(int32_t idx) {
  Node& n = nodes_[idx];
  if (n.swa_slot >= 0) freed_swa_.push_back(n.swa_slot);
  n.swa_slot = -1;
  n.swa_lock = 0;
  if (n.on_swa_lru) {
    swa_lru_.erase(n.swa_it);
    n.on_swa_lru = false;
  }
}

void RadixIndex::swa_touch(int32_t idx) {
  Node& n = nodes_[idx];
  if (n.on_swa_lru) swa_lru_.erase(n.swa_it);
  swa_lru_.push_back(idx);
  n.swa_it = std::prev(swa_lru_.end());
  n.on_swa_lru = true;
}

void RadixIndex::set_swa(NodeHandle h, int32_t slot) {
  int32_t idx = resolve_or_throw(h);
  if (idx == 0) throw std::invalid_argument("radix index: the root carries no window snapshot");
  if (slot < 0) throw std::invalid_argument("radix index: negative snapshot slot");
  Node& n = nodes_[idx];
  if (n.swa_slot >= 0 && n.swa_slot != slot) freed_swa_.push_back(n.swa_slot);
  n.swa_slot = slot;
  swa_armed_ = true;
  swa_touch(idx);
}

bool RadixIndex::has_swa(NodeHandle h) const {
  int32_t idx = resolve(h);
  return idx > 0 && nodes_[idx].swa_slot >= 0;
}
int32_t RadixIndex::swa_slot(NodeHandle h) const { return nodes_[resolve_or_throw(h)].swa_slot; }
int RadixIndex::swa_lock_cnt(NodeHandle h) const { return nodes_[resolve_or_throw(h)].swa_lock; }

void RadixIndex::lock_swa(NodeHandle h) {
  Node& n = nodes_[resolve_or_throw(h)];
  if (n.swa_slot < 0) throw std::runtime_error("radix index: node has no window snapshot to lock");
  ++n.lock_cnt;
  ++n.swa_lock;
}

void RadixIndex::unlock_swa(NodeHandle h) {
  int32_t idx = resolve(h);
  if (idx < 0) return;
  Node& n = nodes_[idx];
  if (n.swa_lock > 0) --n.swa_lock;
  if (n.lock_cnt > 0) --n.lock_cnt;
}

int64_t RadixIndex::evict_swa(int64_t want, std::vector<int64_t>* freed_full, std::vector<uint64_t>* freed_hashes) {
  int64_t freed = 0;
  for (auto it = swa_lru_.begin(); it != swa_lru_.end() && freed < want;) {
    int32_t idx = *it;
    ++it;  // the entry may be erased below
    Node& n = nodes_[idx];
    if (n.swa_lock > 0) continue;
    if (n.leaf() && n.lock_cnt == 0 && n.ready && (!veto_ || !veto_(n.hashes.data(), n.hashes.size()))) {
      // a leaf is only worth keeping for its snapshot: delete it whole
      if (freed_full) freed_full->insert(freed_full->end(), n.blocks.begin(), n.blocks.end());
      if (freed_hashes) freed_hashes->insert(freed_hashes->end(), n.hashes.begin(), n.hashes.end());
      total_blocks_ -= (int64_t)n.size();
      stat_evict_blocks += n.size();
      int32_t parent = n.parent;
      uint64_t head = n.hashes.front();
      free_node(idx);  // drops the snapshot too
      remove_child(parent, head);
      if (freed_full) {     // without a place to report the blocks nothing more is deleted
        const size_t before = freed_full->size();
        prune_snapshotless_leaves(parent, freed_full, freed_hashes);
        stat_evict_blocks += freed_full->size() - before;
      }
    } else {
      drop_swa(idx);
    }
    ++freed;
  }
  return freed;
}

std::vector<int32_t> RadixIndex::drain_freed_swa_slots() {
  std::vector<int32_t> out;
  out.swap(freed_swa_);
  return out;
}

int64_t RadixIndex::total_ready_blocks() const {
  int64_t t = 0;
  for (size_t i = 1; i < nodes_.size(); ++i)
    if (nodes_[i].live && nodes_[i].ready) t += (int64_t)nodes_[i].size();
  return t;
}

int64_t RadixIndex::num_evictable_blocks() const {
  // upper bound reachable by repeated leaf eviction: every unlocked, ready
  // node whose whole subtree is also unlocked and ready
  std::vector<int8_t> ok(nodes_.size(), -1);
  int64_t total = 0;
  // process children before parents: iterate by repeated passes over leaves upward
  std::vector<int32_t> order;
  order.reserve(nodes_.size());
  std::vector<int32_t> stack{0};
  while (!stack.empty()) {
    int32_t i = stack.back();
    stack.pop_back();
    order.push_back(i);
    if (nodes_[i].children)
      for (auto& kv : *nodes_[i].children) stack.push_back(kv.second);
  }
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    int32_t i = *it;
    const Node& n = nodes_[i];
    bool good = i != 0 && n.lock_cnt == 0 && n.ready;
    if (n.children)
      for (auto& kv : *n.children) good = good && ok[kv.second] == 1;
    ok[i] = good ? 1 : 0;
    if (good) total += (int64_t)n.size();
  }
  return total;
}

// ---------------------------------------------------------------- BlockPool

BlockPool::BlockPool(int64_t num_blocks) : total_(num_blocks) {
  if (num_blocks < 0) throw std::invalid_argument("BlockPool: negative size");
  reset();
}

void BlockPool::reset() {
  used_.assign((size_t)total_, 0);
  free_.resize((size_t)total_);
  for (int64_t i = 0; i < total_; ++i) free_[(size_t)i] = total_ - 1 - i;
}

std::vector<int64_t> BlockPool::allocate(int64_t n, bool strict) {
  if (n < 0) throw std::invalid_argument("BlockPool: negative allocation");
  if (n > (int64_t)free_.size()) {
    if (strict) throw std::runtime_error("BlockPool: not enough free blocks");
    n = (int64_t)free_.size();
  }
  std::vector<int64_t> out((size_t)n);
  for (int64_t i = 0; i < n; ++i) {
    int64_t id = free_.back();
    free_.pop_back();
    used_[(size_t)id] = 1;
    out[(size_t)i] = id;
  }
  // Ascending ids: blocks freed together (an evicted sequence) come back as runs of neighbours, and a request
  // whose host blocks lie in a row can be moved with large copies instead of one per block.
  std::sort(out.begin(), out.end());
  return out;
}

void BlockPool::reserve(const int64_t* ids, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    int64_t id = ids[i];
    bool in_range = id >= 0 && id < total_;
    if (!in_range || used_[(size_t)id]) {
      for (int64_t j = 0; j < i; ++j) used_[(size_t)ids[j]] = 0;  // roll back
      if (!in_range) throw std::out_of_range("BlockPool: block id out of range");
      throw std::runtime_error("BlockPool: block already in use or listed twice");
    }
    used_[(size_t)id] = 1;
  }
  if (n == 0) return;
  size_t w = 0;
  for (size_t r = 0; r < free_.size(); ++r)
    if (!used_[(size_t)free_[r]]) free_[w++] = free_[r];
  free_.resize(w);
}

void BlockPool::recycle(const int64_t* ids, int64_t n) {
  // validate first so that a bad call changes nothing
  for (int64_t i = 0; i < n; ++i) {
    int64_t id = ids[i];
    bool in_range = id >= 0 && id < total_;
    if (!in_range || !used_[(size_t)id]) {
      for (int64_t j = 0; j < i; ++j) used_[(size_t)ids[j]] = 1;  // roll back
      if (!in_range) throw std::out_of_range("BlockPool: block id out of range");
      throw std::runtime_error("BlockPool: double free or duplicate id");
    }
    used_[(size_t)id] = 0;  // marks duplicates inside this call too
  }
  for (int64_t i = 0; i < n; ++i) free_.push_back(ids[i]);
}

}  // namespace fkv
