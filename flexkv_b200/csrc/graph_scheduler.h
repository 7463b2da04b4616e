// Transfer-graph scheduler: which op of a graph may run next, dependency release, failure drain,
// fan-out joins and the completion queue.
//
// A transfer graph is a small DAG of ops (D2H -> H2DISK, DISK2H -> H2D, ...). The planner builds it
// in Python; from submission on, its state lives here:
//   * ready set: ops whose predecessors have all completed and that were not handed out yet;
//   * release: completing an op hands out the successors it was the last predecessor of;
//   * fan-out join: an op sent to several executors (one per pipeline stage) completes when the last
//     of them reports, success = all of them, bytes summed, time = max;
//   * failure drain: after the first failed op a graph hands out nothing more, the ops in flight
//     finish, and the graph is reported once, as failed;
//   * completion queue: one record per finished op and one per finished graph, popped by the task
//     layer with a blocking, GIL-free wait.
// Every method may be called from any thread (submitters, executor threads).
// Reference behaviour: flexkv/transfer/transfer_engine.py:1115-1286 (scheduler loop), :1320-1378
// (failure drain, failed_graph), :1445-1492 (pending_count fan-out), flexkv/transfer/scheduler.py:7-97.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace fkv {

struct SchedCompletion {
  int64_t graph_id = 0;
  int64_t op_id = -1;        // -1: the record closes the graph
  bool success = true;
  double ms = 0.0;           // device or IO time of the op (max over its executors)
  int64_t bytes = 0;
};

struct SchedDone {
  bool accepted = false;            // false: unknown graph/op, or a report for an op that is not running
  bool op_finished = false;         // the last executor of the op reported
  bool op_success = true;
  double ms = 0.0;
  int64_t bytes = 0;
  bool graph_finished = false;
  bool graph_failed = false;
  std::vector<int64_t> ready;       // ops released by this completion, to be dispatched now
};

class GraphScheduler {
 public:
  enum OpFlag : int32_t { kInstant = 1 };   // completes as soon as it is ready (virtual or empty op)

  // Registers a graph. `edges` holds (successor op id, predecessor op id) pairs. Ops flagged kInstant are
  // completed on the spot (a completion record each, successors released). Returns the ops to dispatch now,
  // in ascending id order. Throws on a duplicate graph id, an unknown op in an edge, or a cycle-free check
  // failure (an op depending on itself).
  std::vector<int64_t> submit(int64_t graph_id, const std::vector<int64_t>& op_ids, const std::vector<int32_t>& flags,
                              const std::vector<std::pair<int64_t, int64_t>>& edges);

  // The op was handed to `n` executors (default 1); call before the first of them can report.
  void set_fanout(int64_t graph_id, int64_t op_id, int n);

  // One executor of a running op reports.
  SchedDone op_done(int64_t graph_id, int64_t op_id, bool success, double ms, int64_t bytes);

  // An op that was handed out but could not be started (its GPU memory is suspended) goes back to the ready
  // set; take_ready() hands it out again.
  bool requeue(int64_t graph_id, int64_t op_id);
  std::vector<int64_t> take_ready(int64_t graph_id);

  // Completion records so far; blocks up to timeout_s for the first one (timeout_s < 0: no limit, 0: poll).
  std::vector<SchedCompletion> wait(double timeout_s);

  // A descriptor that is readable exactly while completion records are waiting (an eventfd, created on the first
  // call, owned by the scheduler): an event loop that also serves sockets polls it instead of calling wait()
  // on a timer. -1 when the descriptor cannot be created.
  int completion_fd();
  ~GraphScheduler();

  bool has_graph(int64_t graph_id);
  int64_t graphs_in_flight();
  struct Stats { int64_t ops = 0, failed_ops = 0, graphs = 0, failed_graphs = 0; };
  Stats stats();

 private:
  enum class St : uint8_t { PENDING, READY, RUNNING, DONE, FAILED };
  struct Op {
    int64_t id;
    int32_t flags;
    St st = St::PENDING;
    int npred = 0;
    int fanout = 1, reported = 0;
    bool all_ok = true;
    double ms = 0.0;
    int64_t bytes = 0;
    std::vector<int32_t> succ;    // indices into Graph::ops
  };
  struct Graph {
    std::vector<Op> ops;
    std::unordered_map<int64_t, int32_t> index;
    int unfinished = 0, running = 0;
    bool failed = false;
  };

  // completes op `i` of `g` (success path or failure), pushes its record, releases successors into `ready`;
  // instant successors are completed recursively
  void complete_locked(int64_t gid, Graph& g, int32_t i, bool success, std::vector<int64_t>& ready);
  bool maybe_finish_locked(int64_t gid, Graph& g);

  std::mutex mu_;
  std::condition_variable cv_;
  std::unordered_map<int64_t, Graph> graphs_;
  std::deque<SchedCompletion> done_;
  int event_fd_ = -1;
  void signal_locked();     // after a push to done_
  Stats stats_;
};

}  // namespace fkv
