// Stand-alone stress of the C++ control plane, built by tests/test_native_sanitizers.py with
// -fsanitize=address,undefined (memory errors, UB) and with -fsanitize=thread (data races).
// No Python, no CUDA: radix index, block pool, hasher, lease-aware tree and peer view, transfer-graph scheduler.
#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "dist_index.h"
#include "graph_scheduler.h"
#include "hasher.h"
#include "radix_index.h"

using namespace fkv;

#define CHECK(c)                                                          \
  do {                                                                    \
    if (!(c)) {                                                           \
      std::fprintf(stderr, "CHECK failed: %s (%s:%d)\n", #c, __FILE__, __LINE__); \
      std::exit(2);                                                       \
    }                                                                     \
  } while (0)

static std::vector<uint64_t> make_hashes(std::mt19937_64& rng, const std::vector<std::vector<uint64_t>>& seen, int len) {
  std::vector<uint64_t> h;
  if (!seen.empty() && (rng() & 1)) {  // share a prefix with an earlier sequence
    const auto& base = seen[rng() % seen.size()];
    size_t k = 1 + rng() % base.size();
    h.assign(base.begin(), base.begin() + (long)std::min<size_t>(k, (size_t)len));
  }
  while ((int)h.size() < len) h.push_back(rng() | 1);
  return h;
}

static void single_thread_index(uint64_t seed) {
  std::mt19937_64 rng(seed);
  const int64_t cap = 512;
  RadixIndex idx(16, cap, EvictPolicy::LRU, 0.0);
  BlockPool pool(cap);
  std::vector<std::vector<uint64_t>> seen;
  std::vector<NodeHandle> locked;
  int32_t next_slot = 0;
  for (int it = 0; it < 4000; ++it) {
    int op = (int)(rng() % 10);
    if (op < 5) {
      auto h = make_hashes(rng, seen, 1 + (int)(rng() % 24));
      MatchResult m = idx.match_prefix(h.data(), (int64_t)h.size(), true);
      CHECK(m.num_matched <= (int64_t)h.size());
      CHECK((int64_t)m.physical_blocks.size() == m.num_matched);
      int64_t need = (int64_t)h.size() - m.num_matched;
      if (need == 0) continue;
      if (pool.num_free() < need) {
        // as the planner does: the matched node is locked while room is made, so that the eviction (which may
        // take ancestors left without a snapshot along) cannot delete what the insert is about to extend
        const bool guard = m.num_matched > 0;
        if (guard) idx.lock(m.last_node);
        EvictResult ev = idx.evict(need - pool.num_free());
        if (guard) idx.unlock(m.last_node);
        pool.recycle(ev.blocks.data(), (int64_t)ev.blocks.size());
        for (int32_t s : idx.drain_freed_swa_slots()) CHECK(s >= 0);
      }
      if (pool.num_free() < need) continue;
      auto blocks = pool.allocate(need, true);
      bool ready = (rng() % 8) != 0;
      NodeHandle n = idx.insert(blocks.data(), need, h.data(), (int64_t)h.size(), (int64_t)h.size(), ready, &m);
      CHECK(n != kNullHandle);
      if (!ready) {
        if (rng() & 1) idx.set_ready(n, true, need);
        else {
          auto back = idx.remove_unready_leaf(n);
          CHECK((int64_t)back.size() == need);
          pool.recycle(back.data(), need);
        }
      } else if ((rng() % 4) == 0) {
        idx.set_swa(n, next_slot++);
      }
      seen.push_back(h);
      if (seen.size() > 64) seen.erase(seen.begin());
    } else if (op < 7 && !seen.empty()) {
      const auto& h = seen[rng() % seen.size()];
      MatchResult m = idx.match_prefix(h.data(), (int64_t)h.size(), true);
      if (m.num_matched > 0 && locked.size() < 8) {
        idx.lock(m.last_node);
        locked.push_back(m.last_node);
      }
    } else if (op < 8 && !locked.empty()) {
      idx.unlock(locked.back());
      locked.pop_back();
    } else if (op == 8) {
      EvictResult ev = idx.evict(1 + (int64_t)(rng() % 32));
      pool.recycle(ev.blocks.data(), (int64_t)ev.blocks.size());
    } else {
      std::vector<int64_t> fb;
      std::vector<uint64_t> fh;
      idx.evict_swa(1 + (int64_t)(rng() % 3), &fb, &fh);
      pool.recycle(fb.data(), (int64_t)fb.size());
    }
    CHECK(idx.total_cached_blocks() == pool.num_used());
    CHECK(idx.total_cached_blocks() <= cap);
    if (it % 500 == 499) {
      // warm-restart image: a second index and pool rebuilt from it agree with the first
      IndexSnapshot snap = idx.export_ready();
      RadixIndex copy(16, cap, EvictPolicy::LRU, 0.0);
      BlockPool pool2(cap);
      CHECK(copy.import_snapshot(snap) == idx.total_ready_blocks());
      pool2.reserve(snap.blocks.data(), (int64_t)snap.blocks.size());
      CHECK(pool2.num_used() == copy.total_cached_blocks());
      for (const auto& h : seen) {
        MatchResult a = idx.match_prefix(h.data(), (int64_t)h.size(), false, false);
        MatchResult b = copy.match_prefix(h.data(), (int64_t)h.size(), false, false);
        CHECK(b.num_matched == b.num_ready_matched);
        CHECK(b.num_ready_matched >= a.num_ready_matched);  // ready nodes below an unready gap cannot exist
        CHECK(b.num_ready_matched == a.num_ready_matched);
        for (int64_t k = 0; k < b.num_matched; ++k) CHECK(a.physical_blocks[(size_t)k] == b.physical_blocks[(size_t)k]);
      }
      IndexSnapshot again = copy.export_ready();
      CHECK(again.parents == snap.parents && again.sizes == snap.sizes && again.hashes == snap.hashes &&
            again.blocks == snap.blocks);
    }
  }
  for (NodeHandle h : locked) idx.unlock(h);
  auto all = idx.reset();
  pool.recycle(all.data(), (int64_t)all.size());
  CHECK(pool.num_used() == 0);
}

static void hashing() {
  std::vector<int64_t> tok(4096);
  for (size_t i = 0; i < tok.size(); ++i) tok[i] = (int64_t)(i * 2654435761u);
  std::vector<uint64_t> a(256), b(256);
  gen_block_hashes(tok.data(), (int64_t)tok.size(), 16, nullptr, 0, a.data());
  const int64_t* seqs[1] = {tok.data()};
  int64_t lens[1] = {(int64_t)tok.size()};
  uint64_t* outs[1] = {b.data()};
  gen_block_hashes_ptrs(seqs, lens, 1, 16, nullptr, 0, outs, 4);
  CHECK(a == b);
  CHECK(a[0] != a[1]);
}

static void threaded_leases() {
  auto ch = std::make_shared<InProcMetaChannel>();
  LeaseOptions opt;
  opt.lease_ttl_ms = 40;
  opt.renew_margin_ms = 30;
  opt.refresh_interval_ms = 1;
  opt.safety_ttl_ms = 2;
  LocalRadixTree a(1, 16, 4096, EvictPolicy::LRU, 0.0, ch, opt, true);
  LocalRadixTree b(2, 16, 4096, EvictPolicy::LRU, 0.0, ch, opt, true);
  DistributedRadixTree view(3, ch, 1, 2, true);
  std::atomic<bool> stop{false};
  std::atomic<int64_t> remote_hits{0};
  auto writer = [&](LocalRadixTree* t, uint64_t seed) {
    std::mt19937_64 rng(seed);
    int64_t next_block = 0;
    for (int it = 0; it < 600; ++it) {
      std::vector<uint64_t> h(1 + rng() % 6);
      uint64_t base = (rng() % 64) * 1000 + 1;
      for (size_t i = 0; i < h.size(); ++i) h[i] = base + i;
      MatchResult m = t->match_prefix(h.data(), (int64_t)h.size(), true);
      int64_t need = (int64_t)h.size() - m.num_matched;
      if (need > 0) {
        std::vector<int64_t> blocks((size_t)need);
        for (auto& x : blocks) x = next_block++;
        try {
          t->insert(blocks.data(), need, h.data(), (int64_t)h.size(), (int64_t)h.size(), true, &m);
        } catch (const std::exception&) {
        }
      }
      if ((it % 7) == 0) t->evict(8);
      if ((it % 97) == 0) std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
  };
  auto reader = [&] {
    std::mt19937_64 rng(99);
    while (!stop.load()) {
      uint64_t base = (rng() % 64) * 1000 + 1;
      uint64_t h[3] = {base, base + 1, base + 2};
      RemoteMatch r = view.match_prefix(h, 3);
      CHECK(r.num_matched >= 0 && r.num_matched <= 3);
      for (uint32_t nid : r.node_ids) CHECK(nid == 1 || nid == 2);
      remote_hits += r.num_matched;
    }
  };
  std::thread w1(writer, &a, 1), w2(writer, &b, 2), r1(reader), r2(reader);
  w1.join();
  w2.join();
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  stop = true;
  r1.join();
  r2.join();
  CHECK(remote_hits.load() > 0);
  CHECK(a.stats().published > 0 && b.stats().published > 0);
  a.shutdown();
  b.shutdown();
  view.shutdown();
}

// Random DAGs submitted from several threads, executed by several "worker" threads that report through
// op_done (some ops fail, some are fanned out to two executors, some are requeued once), completions drained
// by a waiter: every graph must finish exactly once, no op may run twice or after its graph failed for good,
// and nothing may be left behind.
static void threaded_scheduler() {
  GraphScheduler sched;
  struct Item { int64_t g, op; };
  std::mutex qmu;
  std::condition_variable qcv;
  std::deque<Item> queue;
  std::atomic<bool> stop{false};
  std::atomic<int64_t> ran{0}, graph_records{0}, op_records{0}, failed_graphs{0};
  constexpr int kSubmitters = 3, kGraphsEach = 150, kWorkers = 4;
  std::vector<std::atomic<int>> runs((size_t)kSubmitters * kGraphsEach * 16);
  for (auto& r : runs) r = 0;
  auto push = [&](int64_t g, const std::vector<int64_t>& ops) {
    std::lock_guard<std::mutex> lk(qmu);
    for (int64_t o : ops) queue.push_back({g, o});
    qcv.notify_all();
  };
  auto worker = [&](uint64_t seed) {
    std::mt19937_64 rng(seed);
    for (;;) {
      Item it;
      {
        std::unique_lock<std::mutex> lk(qmu);
        qcv.wait(lk, [&] { return stop.load() || !queue.empty(); });
        if (queue.empty()) return;
        it = queue.front();
        queue.pop_front();
      }
      const size_t slot = (size_t)it.g * 16 + (size_t)it.op;
      if ((rng() % 23) == 0 && runs[slot].load() == 0) {     // could not start: back to the ready set, once
        runs[slot] = -1;
        CHECK(sched.requeue(it.g, it.op));
        push(it.g, sched.take_ready(it.g));
        continue;
      }
      const int before = runs[slot].exchange(1);
      CHECK(before <= 0);                                     // handed out once (after at most one requeue)
      ++ran;
      const bool two = (rng() % 5) == 0;
      if (two) sched.set_fanout(it.g, it.op, 2);
      const bool ok = (rng() % 17) != 0;
      SchedDone d = sched.op_done(it.g, it.op, ok, 0.1, 100);
      CHECK(d.accepted);
      if (two) {
        CHECK(!d.op_finished);
        d = sched.op_done(it.g, it.op, true, 0.2, 100);
        CHECK(d.accepted && d.op_finished && d.op_success == ok && d.bytes == 200);
      }
      push(it.g, d.ready);
    }
  };
  auto submitter = [&](int who) {
    std::mt19937_64 rng(1000 + (uint64_t)who);
    for (int k = 0; k < kGraphsEach; ++k) {
      const int64_t g = (int64_t)who * kGraphsEach + k;
      const int n = 1 + (int)(rng() % 12);
      std::vector<int64_t> ids((size_t)n);
      std::vector<int32_t> flags((size_t)n, 0);
      std::vector<std::pair<int64_t, int64_t>> edges;
      for (int i = 0; i < n; ++i) {
        ids[(size_t)i] = i;
        if ((rng() % 9) == 0) flags[(size_t)i] = GraphScheduler::kInstant;
        for (int j = 0; j < i; ++j)
          if ((rng() % 4) == 0) edges.emplace_back(i, j);     // successor i depends on j < i: acyclic
      }
      push(g, sched.submit(g, ids, flags, edges));
    }
  };
  auto waiter = [&] {
    const int64_t want = (int64_t)kSubmitters * kGraphsEach;
    while (graph_records.load() < want) {
      for (const SchedCompletion& c : sched.wait(0.05)) {
        if (c.op_id < 0) {
          ++graph_records;
          if (!c.success) ++failed_graphs;
        } else {
          ++op_records;
        }
      }
    }
  };
  std::vector<std::thread> th;
  for (int w = 0; w < kWorkers; ++w) th.emplace_back(worker, 7 + (uint64_t)w);
  std::thread wt(waiter);
  std::vector<std::thread> subs;
  for (int s = 0; s < kSubmitters; ++s) subs.emplace_back(submitter, s);
  for (auto& t : subs) t.join();
  wt.join();
  stop = true;
  qcv.notify_all();
  for (auto& t : th) t.join();
  CHECK(graph_records.load() == (int64_t)kSubmitters * kGraphsEach);
  CHECK(sched.graphs_in_flight() == 0);
  const GraphScheduler::Stats st = sched.stats();
  CHECK(st.graphs == graph_records.load() && st.failed_graphs == failed_graphs.load() && failed_graphs.load() > 0);
  CHECK(op_records.load() >= ran.load());                     // instant ops have records but were never run
  CHECK(sched.wait(0.0).empty());
}

int main(int argc, char** argv) {
  const bool threads_only = argc > 1 && std::string(argv[1]) == "threads";
  if (!threads_only) {
    for (uint64_t s = 1; s <= 6; ++s) single_thread_index(s);
    hashing();
  }
  threaded_leases();
  threaded_scheduler();
  std::printf("OK\n");
  return 0;
}
