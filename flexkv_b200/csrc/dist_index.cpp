#include "dist_index.h"

#include <algorithm>
#include <chrono>
#include <map>

#include "native_log.h"

namespace fkv {

int64_t wall_clock_ms() {
  using namespace std::chrono;
  return duration_cast<milliseconds>(system_clock::now().time_since_epoch()).count();
}

// ------------------------------------------------------------------ in-process channel

std::shared_ptr<InProcMetaChannel> InProcMetaChannel::named(const std::string& name) {
  static std::mutex mu;
  static std::map<std::string, std::weak_ptr<InProcMetaChannel>> table;
  std::lock_guard<std::mutex> g(mu);
  auto sp = table[name].lock();
  if (!sp) {
    sp = std::make_shared<InProcMetaChannel>();
    table[name] = sp;
  }
  return sp;
}

void InProcMetaChannel::publish(uint32_t nid, const std::vector<BlockMeta>& metas) {
  std::lock_guard<std::mutex> g(mu_);
  auto& m = nodes_[nid];
  for (const BlockMeta& b : metas) m[b.hash] = b;
}

void InProcMetaChannel::remove(uint32_t nid, const std::vector<uint64_t>& hashes) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = nodes_.find(nid);
  if (it == nodes_.end()) return;
  for (uint64_t h : hashes) it->second.erase(h);
}

std::vector<uint32_t> InProcMetaChannel::list_nodes() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<uint32_t> out;
  for (auto& kv : nodes_) out.push_back(kv.first);
  std::sort(out.begin(), out.end());
  return out;
}

std::vector<BlockMeta> InProcMetaChannel::load(uint32_t nid) {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<BlockMeta> out;
  auto it = nodes_.find(nid);
  if (it == nodes_.end()) return out;
  out.reserve(it->second.size());
  for (auto& kv : it->second) out.push_back(kv.second);
  return out;
}

void InProcMetaChannel::clear_node(uint32_t nid) {
  std::lock_guard<std::mutex> g(mu_);
  nodes_.erase(nid);
}

size_t InProcMetaChannel::total_records() {
  std::lock_guard<std::mutex> g(mu_);
  size_t n = 0;
  for (auto& kv : nodes_) n += kv.second.size();
  return n;
}

// ------------------------------------------------------------------ local tree

LocalRadixTree::LocalRadixTree(uint32_t nid, int tokens_per_block, int64_t max_num_blocks, EvictPolicy policy,
                               double hit_reward_seconds, std::shared_ptr<MetaChannel> channel, LeaseOptions opt,
                               bool start_thread)
    : nid_(nid), index_(tokens_per_block, max_num_blocks, policy, hit_reward_seconds), channel_(std::move(channel)),
      opt_(opt) {
  // Called by the index with mu_ already held (every index call goes through this class).
  index_.set_evict_veto([this](const uint64_t* hashes, size_t n) {
    const int64_t now = now_ms();
    for (size_t i = 0; i < n; ++i) {
      auto it = leases_.find(hashes[i]);
      if (it != leases_.end() && it->second.published && it->second.lt > now) return true;
    }
    return false;
  });
  if (start_thread) th_ = std::thread([this] { thread_main(); });
}

void LocalRadixTree::shutdown() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (th_.joinable()) th_.join();
}

LocalRadixTree::~LocalRadixTree() {
  shutdown();
  // a node that goes away withdraws what it published
  try {
    if (channel_) channel_->clear_node(nid_);
  } catch (...) {
  }
}

int64_t LocalRadixTree::now_ms() const { return clock_override_ms_ >= 0 ? clock_override_ms_ : wall_clock_ms(); }

MatchResult LocalRadixTree::match_prefix(const uint64_t* hashes, int64_t n, bool update) {
  std::lock_guard<std::mutex> g(mu_);
  return index_.match_prefix(hashes, n, update);
}

void LocalRadixTree::track_ready_locked(NodeHandle h, int64_t ready_length) {
  // walk up from h until ready_length blocks are covered (ready_length < 0: this node only)
  int64_t left = ready_length < 0 ? index_.node_size(h) : ready_length;
  NodeHandle cur = h;
  while (left > 0 && !index_.is_root(cur) && index_.alive(cur)) {
    const auto& hs = index_.node_hashes(cur);
    const auto& bs = index_.node_blocks(cur);
    NodeHandle parent = index_.node_parent(cur);
    uint64_t before = 0;
    if (!index_.is_root(parent)) before = index_.node_hashes(parent).back();
    for (size_t i = 0; i < hs.size(); ++i) {
      auto it = leases_.find(hs[i]);
      if (it == leases_.end()) {
        Lease l;
        l.ph = i == 0 ? before : hs[i - 1];
        l.pb = bs[i];
        leases_.emplace(hs[i], l);
      } else if (it->second.pb != bs[i]) {
        it->second.pb = bs[i];
        it->second.dirty = true;
      }
    }
    left -= (int64_t)hs.size();
    cur = parent;
  }
}

NodeHandle LocalRadixTree::insert(const int64_t* physical, int64_t num_physical, const uint64_t* hashes, int64_t n,
                                  int64_t num_insert, bool ready, const MatchResult* match) {
  std::lock_guard<std::mutex> g(mu_);
  NodeHandle h = index_.insert(physical, num_physical, hashes, n, num_insert, ready, match);
  if (h != kNullHandle && ready) track_ready_locked(h, -1);
  return h;
}

void LocalRadixTree::set_ready(NodeHandle h, bool ready, int64_t ready_length) {
  std::lock_guard<std::mutex> g(mu_);
  index_.set_ready(h, ready, ready_length);
  if (ready) track_ready_locked(h, ready_length);
}

EvictResult LocalRadixTree::evict(int64_t num_blocks) {
  std::lock_guard<std::mutex> g(mu_);
  EvictResult r = index_.evict(num_blocks);
  for (uint64_t h : r.hashes) {
    auto it = leases_.find(h);
    if (it == leases_.end()) continue;
    if (it->second.published) pending_remove_.push_back(h);
    leases_.erase(it);
  }
  int64_t missing = num_blocks - (int64_t)r.blocks.size();
  if (missing > 0) {
    for (auto& hs : index_.vetoed_leaves(missing)) {
      for (uint64_t h : hs) {
        auto it = leases_.find(h);
        if (it != leases_.end() && it->second.state == LEASE_NORMAL) {
          it->second.state = LEASE_ABOUT_TO_EVICT;
          it->second.dirty = true;
          ++stats_.marked_about_to_evict;
        }
      }
    }
  }
  return r;
}

void LocalRadixTree::lock(NodeHandle h) {
  std::lock_guard<std::mutex> g(mu_);
  index_.lock(h);
}
void LocalRadixTree::unlock(NodeHandle h) {
  std::lock_guard<std::mutex> g(mu_);
  index_.unlock(h);
}
std::vector<int64_t> LocalRadixTree::remove_unready_leaf(NodeHandle h) {
  std::lock_guard<std::mutex> g(mu_);
  return index_.remove_unready_leaf(h);
}
std::vector<int64_t> LocalRadixTree::truncate_unready_leaf(NodeHandle h, int64_t keep) {
  std::lock_guard<std::mutex> g(mu_);
  return index_.truncate_unready_leaf(h, keep);
}
std::vector<int64_t> LocalRadixTree::reset() {
  std::vector<int64_t> out;
  {
    std::lock_guard<std::mutex> g(mu_);
    out = index_.reset();
    leases_.clear();
    pending_remove_.clear();
  }
  if (channel_) channel_->clear_node(nid_);
  return out;
}
int64_t LocalRadixTree::total_cached_blocks() {
  std::lock_guard<std::mutex> g(mu_);
  return index_.total_cached_blocks();
}
int64_t LocalRadixTree::num_evictable_blocks() {
  std::lock_guard<std::mutex> g(mu_);
  return index_.num_evictable_blocks();
}
LocalTreeStats LocalRadixTree::stats() {
  std::lock_guard<std::mutex> g(mu_);
  return stats_;
}

void LocalRadixTree::refresh_once(int64_t now) {
  std::vector<uint64_t> removes;
  std::vector<BlockMeta> announce, fresh, renew;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (now < 0) now = now_ms();
    removes.swap(pending_remove_);
    for (auto& kv : leases_) {
      Lease& l = kv.second;
      BlockMeta m;
      m.ph = l.ph; m.pb = l.pb; m.nid = nid_; m.hash = kv.first; m.state = l.state;
      if (l.state == LEASE_ABOUT_TO_EVICT) {
        if (l.dirty && l.published) { m.lt = l.lt; announce.push_back(m); }
        l.dirty = false;
        continue;
      }
      if (!l.published) {
        l.lt = now + opt_.lease_ttl_ms;
        m.lt = l.lt;
        l.published = true;
        l.dirty = false;
        fresh.push_back(m);
      } else if (l.dirty || l.lt - now < opt_.renew_margin_ms) {
        l.lt = now + opt_.lease_ttl_ms;
        m.lt = l.lt;
        l.dirty = false;
        renew.push_back(m);
      }
    }
    stats_.withdrawn += removes.size();
    stats_.published += fresh.size();
    stats_.renewed += renew.size();
    ++stats_.refreshes;
  }
  if (!channel_) return;
  // priority order: withdraw, announce imminent evictions, publish, renew
  if (!removes.empty()) channel_->remove(nid_, removes);
  if (!announce.empty()) channel_->publish(nid_, announce);
  if (!fresh.empty()) channel_->publish(nid_, fresh);
  if (!renew.empty()) channel_->publish(nid_, renew);
}

void LocalRadixTree::thread_main() {
  std::unique_lock<std::mutex> lk(mu_);
  int64_t backoff_ms = 0;   // grows while the channel keeps failing (registry down), so the log is not flooded
  while (!stop_) {
    cv_.wait_for(lk, std::chrono::milliseconds(opt_.refresh_interval_ms + backoff_ms));
    if (stop_) break;
    lk.unlock();
    try {
      refresh_once(-1);
      backoff_ms = 0;
    } catch (const std::exception& e) {
      if (backoff_ms == 0) FKV_WARN("local index refresh failed: %s", e.what());
      backoff_ms = std::min<int64_t>(5000, std::max<int64_t>(100, backoff_ms * 2));
    }
    lk.lock();
  }
}

// ------------------------------------------------------------------ distributed view

DistributedRadixTree::DistributedRadixTree(uint32_t self_nid, std::shared_ptr<MetaChannel> channel,
                                           int64_t refresh_interval_ms, int64_t safety_ttl_ms, bool start_thread)
    : self_(self_nid), channel_(std::move(channel)), refresh_ms_(refresh_interval_ms), safety_ms_(safety_ttl_ms),
      current_(std::make_shared<const RefIndex>()) {
  if (start_thread) th_ = std::thread([this] { thread_main(); });
}

void DistributedRadixTree::shutdown() {
  {
    std::lock_guard<std::mutex> g(sleep_mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (th_.joinable()) th_.join();
}

DistributedRadixTree::~DistributedRadixTree() { shutdown(); }

void DistributedRadixTree::refresh_once() {
  if (!channel_) return;
  std::vector<uint32_t> nodes = channel_->list_nodes();
  nodes.erase(std::remove(nodes.begin(), nodes.end(), self_), nodes.end());
  std::sort(nodes.begin(), nodes.end(), [this](uint32_t a, uint32_t b) {
    auto d = [this](uint32_t x) { return x > self_ ? x - self_ : self_ - x; };
    return d(a) != d(b) ? d(a) < d(b) : a < b;
  });
  auto next = std::make_shared<RefIndex>();
  for (uint32_t nid : nodes)
    for (const BlockMeta& m : channel_->load(nid))
      if (m.state == LEASE_NORMAL) next->emplace(m.hash, m);  // nearest owner inserted first wins
  {
    std::lock_guard<std::mutex> g(mu_);
    current_ = std::move(next);
  }
  generation_.fetch_add(1);
}

RemoteMatch DistributedRadixTree::match_prefix(const uint64_t* hashes, int64_t n, int64_t now) {
  std::shared_ptr<const RefIndex> idx;
  {
    std::lock_guard<std::mutex> g(mu_);
    idx = current_;
  }
  if (now < 0) now = clock_override_ms_ >= 0 ? clock_override_ms_ : wall_clock_ms();
  RemoteMatch r;
  for (int64_t i = 0; i < n; ++i) {
    auto it = idx->find(hashes[i]);
    if (it == idx->end()) break;
    const BlockMeta& m = it->second;
    if (m.lt - now <= safety_ms_) break;
    if (m.ph != (i == 0 ? 0 : hashes[i - 1])) break;
    r.physical_blocks.push_back(m.pb);
    r.node_ids.push_back(m.nid);
  }
  r.num_matched = (int64_t)r.physical_blocks.size();
  return r;
}

int64_t DistributedRadixTree::num_remote_blocks() {
  std::lock_guard<std::mutex> g(mu_);
  return (int64_t)current_->size();
}

void DistributedRadixTree::thread_main() {
  std::unique_lock<std::mutex> lk(sleep_mu_);
  int64_t backoff_ms = 0;
  while (!stop_) {
    cv_.wait_for(lk, std::chrono::milliseconds(refresh_ms_ + backoff_ms));
    if (stop_) break;
    lk.unlock();
    try {
      refresh_once();
      backoff_ms = 0;
    } catch (const std::exception& e) {
      if (backoff_ms == 0) FKV_WARN("distributed index refresh failed: %s", e.what());
      backoff_ms = std::min<int64_t>(5000, std::max<int64_t>(100, backoff_ms * 2));
      // a view that cannot be refreshed must not keep offering blocks whose leases it cannot see renewed:
      // entries simply age out through the lease check in match_prefix
    }
    lk.lock();
  }
}

}  // namespace fkv
