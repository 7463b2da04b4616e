#include "graph_scheduler.h"

#include <sys/eventfd.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <stdexcept>

namespace fkv {

std::vector<int64_t> GraphScheduler::submit(int64_t graph_id, const std::vector<int64_t>& op_ids,
                                            const std::vector<int32_t>& flags,
                                            const std::vector<std::pair<int64_t, int64_t>>& edges) {
  if (flags.size() != op_ids.size()) throw std::invalid_argument("GraphScheduler: one flag word per op");
  Graph g;
  g.ops.resize(op_ids.size());
  for (size_t i = 0; i < op_ids.size(); ++i) {
    g.ops[i].id = op_ids[i];
    g.ops[i].flags = flags[i];
    if (!g.index.emplace(op_ids[i], (int32_t)i).second) throw std::invalid_argument("GraphScheduler: duplicate op id");
  }
  for (const auto& e : edges) {
    auto s = g.index.find(e.first), p = g.index.find(e.second);
    if (s == g.index.end() || p == g.index.end()) throw std::invalid_argument("GraphScheduler: edge names an unknown op");
    if (s->second == p->second) throw std::invalid_argument("GraphScheduler: an op cannot depend on itself");
    g.ops[(size_t)p->second].succ.push_back(s->second);
    g.ops[(size_t)s->second].npred++;
  }
  g.unfinished = (int)g.ops.size();

  std::vector<int64_t> ready;
  std::lock_guard<std::mutex> lk(mu_);
  if (graphs_.count(graph_id)) throw std::invalid_argument("GraphScheduler: graph id already in flight");
  Graph& gr = graphs_.emplace(graph_id, std::move(g)).first->second;
  stats_.graphs++;
  // roots, in ascending id order (the order of a Python set walk is not a contract; ids are)
  std::vector<int32_t> roots;
  for (int32_t i = 0; i < (int32_t)gr.ops.size(); ++i)
    if (gr.ops[(size_t)i].npred == 0) roots.push_back(i);
  std::sort(roots.begin(), roots.end(), [&](int32_t a, int32_t b) { return gr.ops[(size_t)a].id < gr.ops[(size_t)b].id; });
  for (int32_t i : roots) {
    Op& op = gr.ops[(size_t)i];
    if (op.st != St::PENDING) continue;     // already completed as the instant successor of an earlier root
    if (op.flags & kInstant) {
      op.st = St::RUNNING;
      gr.running++;
      complete_locked(graph_id, gr, i, true, ready);
    } else {
      op.st = St::RUNNING;
      gr.running++;
      ready.push_back(op.id);
    }
  }
  maybe_finish_locked(graph_id, gr);
  cv_.notify_all();
  std::sort(ready.begin(), ready.end());
  return ready;
}

void GraphScheduler::complete_locked(int64_t gid, Graph& g, int32_t i, bool success, std::vector<int64_t>& ready) {
  Op& op = g.ops[(size_t)i];
  op.st = success ? St::DONE : St::FAILED;
  g.running--;
  g.unfinished--;
  stats_.ops++;
  if (!success) {
    stats_.failed_ops++;
    g.failed = true;
  }
  done_.push_back(SchedCompletion{gid, op.id, success, op.ms, op.bytes});
  signal_locked();
  if (!success || g.failed) return;      // a failed graph hands out nothing more
  for (int32_t s : op.succ) {
    Op& so = g.ops[(size_t)s];
    if (--so.npred > 0 || so.st != St::PENDING) continue;
    so.st = St::RUNNING;
    g.running++;
    if (so.flags & kInstant) complete_locked(gid, g, s, true, ready);
    else ready.push_back(so.id);
  }
}

bool GraphScheduler::maybe_finish_locked(int64_t gid, Graph& g) {
  const bool finished = g.unfinished == 0 || (g.failed && g.running == 0);
  if (!finished) return false;
  if (g.failed) stats_.failed_graphs++;
  done_.push_back(SchedCompletion{gid, -1, !g.failed, 0.0, 0});
  signal_locked();
  graphs_.erase(gid);
  cv_.notify_all();
  return true;
}

void GraphScheduler::set_fanout(int64_t graph_id, int64_t op_id, int n) {
  std::lock_guard<std::mutex> lk(mu_);
  auto git = graphs_.find(graph_id);
  if (git == graphs_.end()) return;
  auto it = git->second.index.find(op_id);
  if (it == git->second.index.end()) return;
  git->second.ops[(size_t)it->second].fanout = std::max(1, n);
}

SchedDone GraphScheduler::op_done(int64_t graph_id, int64_t op_id, bool success, double ms, int64_t bytes) {
  SchedDone r;
  std::lock_guard<std::mutex> lk(mu_);
  auto git = graphs_.find(graph_id);
  if (git == graphs_.end()) return r;
  Graph& g = git->second;
  auto it = g.index.find(op_id);
  if (it == g.index.end()) return r;
  Op& op = g.ops[(size_t)it->second];
  if (op.st != St::RUNNING) return r;
  r.accepted = true;
  op.all_ok = op.all_ok && success;
  op.ms = std::max(op.ms, ms);
  op.bytes += bytes;
  if (++op.reported < op.fanout) return r;
  r.op_finished = true;
  r.op_success = op.all_ok;
  r.ms = op.ms;
  r.bytes = op.bytes;
  complete_locked(graph_id, g, it->second, op.all_ok, r.ready);
  std::sort(r.ready.begin(), r.ready.end());
  r.graph_failed = g.failed;
  r.graph_finished = maybe_finish_locked(graph_id, g);
  cv_.notify_all();
  return r;
}

bool GraphScheduler::requeue(int64_t graph_id, int64_t op_id) {
  std::lock_guard<std::mutex> lk(mu_);
  auto git = graphs_.find(graph_id);
  if (git == graphs_.end()) return false;
  auto it = git->second.index.find(op_id);
  if (it == git->second.index.end()) return false;
  Op& op = git->second.ops[(size_t)it->second];
  if (op.st != St::RUNNING || op.reported > 0) return false;
  op.st = St::READY;
  git->second.running--;
  return true;
}

std::vector<int64_t> GraphScheduler::take_ready(int64_t graph_id) {
  std::vector<int64_t> out;
  std::lock_guard<std::mutex> lk(mu_);
  auto git = graphs_.find(graph_id);
  if (git == graphs_.end()) return out;
  Graph& g = git->second;
  if (g.failed) {
    // parked ops of a graph that failed meanwhile are dropped: they count as never started
    for (Op& op : g.ops)
      if (op.st == St::READY) { op.st = St::FAILED; g.unfinished--; }
    maybe_finish_locked(graph_id, g);
    return out;
  }
  for (Op& op : g.ops)
    if (op.st == St::READY) {
      op.st = St::RUNNING;
      g.running++;
      out.push_back(op.id);
    }
  std::sort(out.begin(), out.end());
  return out;
}

std::vector<SchedCompletion> GraphScheduler::wait(double timeout_s) {
  std::vector<SchedCompletion> out;
  std::unique_lock<std::mutex> lk(mu_);
  if (done_.empty() && timeout_s != 0.0) {
    if (timeout_s < 0) cv_.wait(lk, [&] { return !done_.empty(); });
    else cv_.wait_for(lk, std::chrono::duration<double>(timeout_s), [&] { return !done_.empty(); });
  }
  out.assign(done_.begin(), done_.end());
  done_.clear();
  if (event_fd_ >= 0) {       // nothing is waiting any more: the descriptor stops being readable
    uint64_t v;
    while (::read(event_fd_, &v, sizeof(v)) == (ssize_t)sizeof(v)) {
    }
  }
  return out;
}

void GraphScheduler::signal_locked() {
  if (event_fd_ < 0) return;
  const uint64_t one = 1;
  (void)!::write(event_fd_, &one, sizeof(one));
}

int GraphScheduler::completion_fd() {
  std::lock_guard<std::mutex> lk(mu_);
  if (event_fd_ < 0) {
    event_fd_ = ::eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    if (event_fd_ >= 0 && !done_.empty()) signal_locked();
  }
  return event_fd_;
}

GraphScheduler::~GraphScheduler() {
  if (event_fd_ >= 0) ::close(event_fd_);
}

bool GraphScheduler::has_graph(int64_t graph_id) {
  std::lock_guard<std::mutex> lk(mu_);
  return graphs_.count(graph_id) != 0;
}

int64_t GraphScheduler::graphs_in_flight() {
  std::lock_guard<std::mutex> lk(mu_);
  return (int64_t)graphs_.size();
}

GraphScheduler::Stats GraphScheduler::stats() {
  std::lock_guard<std::mutex> lk(mu_);
  return stats_;
}

}  // namespace fkv
