// Layer-by-layer restore with per-layer completion signals.
//
// A restore first brings any SSD-resident blocks into the host pool (all
// layers), then copies host -> GPU one layer batch at a time on a
// highest-priority stream per GPU, so that the model's layer l can start as
// soon as its KV has landed while layers l+1.. are still in flight
// (reference behaviour: csrc/layerwise.cpp:944-1311, eventfd table
// [counters][tp][layers] :537-544, host-callback notification :105-137,
// polling notification :36-68).
//
// Each layer batch is one copy kernel whose last CTA publishes the restore's
// epoch to a device flag (for consumer kernels and CUDA-event waits on the same
// GPU) and to a mapped host flag. Three ways reach another process's eventfd:
//   hostfunc : cudaLaunchHostFunc after the kernel writes the eventfd
//   polling  : a host thread polls cudaEventQuery on per-layer events
//   flag     : a host thread polls the mapped host flag the kernel wrote
// Every rank signals its own eventfd as soon as its own copy is done.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "ssd_io.h"
#include "transfer_group.h"

namespace fkv {

enum class NotifyMode : int { HOSTFUNC = 0, POLLING = 1, FLAG = 2 };
NotifyMode parse_notify_mode(const std::string& s);

struct LayerwiseOptions {
  GroupOptions group;
  NotifyMode notify = NotifyMode::HOSTFUNC;
  int num_counters = 3;       // independent flag / eventfd sets (restores in flight)
  int layers_per_batch = 1;   // 0 = ONE launch for all layers, flags published per layer from inside the kernel;
                              // -1 = decide per restore: fused up to fused_max_bytes, else one launch per layer
  int64_t fused_max_bytes = 64ll << 20;
  bool create_eventfds = true;
  // Host pool kept in the lossless bf16 codec's packed form (uniform caches only): the restore then runs the
  // unpacking kernel, layer by layer with the same per-layer flags, and reads only the packed bytes from the host.
  // size_table: mapped uint32 table of the pool; rank r starts size_table_rank_entries * r entries in and is told
  // the table holds size_table_layers layers per block (see transfer/compression/size_table.py).
  uint32_t* size_table = nullptr;
  int size_table_layers = 0;
  int64_t size_table_rank_entries = 0;
  int codec_pipelines = 64;   // 128-thread tile pipelines of the unpacking kernel (two per SM)
};

struct LayerwiseResult {
  int status = 0;
  uint32_t epoch = 0;                // the value this restore published to its counter's flags
  float total_ms = 0.f;              // first launch to last completion, max over ranks (CUDA events)
  float disk_ms = 0.f;               // host wall time of the SSD -> host stage
  std::vector<float> layer_done_ms;  // per layer, time since first launch (rank 0)
};

// Caches made of several layer groups with different KV shapes (an indexer beside the main
// cache, compressed-KV groups): every group has its own tensors, chunk size and place inside
// the byte-flat host block, and a model layer is complete when each of its members
// (group, layer inside the group) has landed
// (reference behaviour: csrc/layerwise.cpp:1313-1682, layer_members[orig] = [(group, local_layer)]).
struct LayerMember {
  int group;
  int local_layer;
};
struct LayerwiseMemberGroup {
  std::vector<GpuSide> gpus;   // one per rank, same rank order in every group
  HostSide host;               // strides of this group inside the host block; `base` already at the group's offset
  GroupOptions group;          // num_layers / kv_dim / chunk_bytes / cpu_tp_stride / shared_kv of this group
};

class LayerwiseGroup {
 public:
  LayerwiseGroup(std::vector<GpuSide> gpus, HostSide host, LayerwiseOptions opt);
  // Multi-group form: `members[l]` lists what model layer l consists of (may be empty: the layer is
  // signalled at once, in order). opt.group supplies the launch shapes and max_blocks_per_op; its
  // num_layers is replaced by members.size(). One launch per member, flags from the layer's last one.
  LayerwiseGroup(std::vector<LayerwiseMemberGroup> groups, std::vector<std::vector<LayerMember>> members,
                 HostSide host_block, LayerwiseOptions opt);
  ~LayerwiseGroup();

  // blocking; `ssd` may be null when nothing comes from disk
  LayerwiseResult restore(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, int counter_id,
                          SsdIoEngine* ssd, const SsdLayout* ssd_layout, const int64_t* ssd_src,
                          const int64_t* cpu_dst, int64_t n_disk);

  // eventfd of (counter, rank, layer); -1 when eventfds are disabled
  int eventfd_of(int counter, int rank, int layer) const;
  std::vector<int> eventfds_flat() const { return eventfds_; }
  // installs a caller-owned eventfd (e.g. received from the engine over a UNIX
  // socket); the group takes a dup() of it
  void set_eventfd(int counter, int rank, int layer, int fd);
  uint64_t device_flags_ptr(int rank, int counter) const;  // uint32[num_layers] in device memory
  uint64_t host_flags_ptr(int rank, int counter) const;    // uint32[num_layers] in mapped host memory
  uint32_t epoch_of(int counter);
  // Reserves and returns the epoch that the NEXT restore() on `counter` will publish. A consumer that wants to
  // queue its waits before (or while) the restore is issued calls this first and hands the value to
  // stream_wait_layer; restore() then publishes exactly that epoch. Without a reservation restore() takes the
  // next epoch itself and returns it in LayerwiseResult::epoch.
  uint32_t begin_restore(int counter);
  // Blocks (on the host, up to timeout_ms) until every rank has QUEUED all launches of the restore that publishes
  // `epoch` on `counter`, or until that restore has failed. True when queued. A consumer calls this between
  // begin_restore() and its stream_wait_layer() calls: a stream wait that reaches the GPU ahead of the producer's
  // launch can share a hardware queue with it and then nothing behind the wait, the producer included, ever runs.
  bool wait_launched(int counter, uint32_t epoch, int timeout_ms);
  // Makes `stream` (a CUDA stream of rank's device) wait until layer `layer` of the restore that publishes
  // `epoch` on `counter` has landed (a stream-ordered wait on the device flag, value >= epoch). `epoch` 0
  // means "the newest epoch handed out for this counter", which is only right once that restore has been
  // started or reserved. Queue it only once wait_launched() has returned true (see there). A failed restore
  // releases the waiters too; whether the data is usable is told by
  // counter_status() / the restore's result, never by the flag alone.
  cudaError_t stream_wait_layer(int rank, int counter, int layer, cudaStream_t stream, uint32_t epoch = 0);
  // 0 while the newest restore on `counter` is running or has succeeded, else its failure status
  int counter_status(int counter) const { return counter_status_[(size_t)counter].load(std::memory_order_acquire); }
  int num_ranks() const { return (int)gpus_.size(); }
  // new tensor addresses after the engine re-created its cache; call with no restore in flight
  void update_gpu_ptrs(int rank, const std::vector<uint64_t>& ptrs);
  void update_group_gpu_ptrs(int group, int rank, const std::vector<uint64_t>& ptrs);   // multi-group form
  bool multi_group() const { return !mgroups_.empty(); }
  int num_layers() const { return opt_.group.num_layers; }
  int num_counters() const { return opt_.num_counters; }

 private:
  struct Job {
    int64_t n;
    int counter;
    uint32_t epoch;
    int fail_status = 0;        // non-zero: nothing is copied, the waiters are released with this failure
    const int64_t* gpu_blocks;  // in the id ring
    const int64_t* cpu_blocks;
  };
  struct Rank {
    std::thread th;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Job> q;
    bool ready = false;
    std::string init_error;
    cudaStream_t stream = nullptr;
    cudaStream_t notify_stream = nullptr;   // carries host callbacks so the copy stream never blocks on them
    uint32_t* dev_flags = nullptr;      // [counters][layers]
    uint32_t* host_flags = nullptr;     // mapped, [counters][layers]
    uint32_t* done_counter = nullptr;   // device scratch, one word per layer, zero between launches
    int64_t* dev_ids = nullptr;         // [2][max_blocks] device copy of a job's block ids (gpu ids, then host ids):
                                        // id reads from mapped host memory would queue behind the bulk reads on the link
    int32_t* status = nullptr;          // mapped, kStatusWords
    std::vector<cudaEvent_t> layer_ev;  // [counters][layers]
    cudaEvent_t ev_begin = nullptr;
    // result of the last job
    int res_status = 0;
    float res_ms = 0.f;
    std::vector<float> res_layer_ms;
    bool done = false;
  };
  struct HostFnArg {
    LayerwiseGroup* self;
    int rank, counter, layer_lo, layer_hi;
  };

  void start_ranks();
  void rank_main(int r);
  void run_job(int r, const Job& j);
  void run_job_members(int r, const Job& j);
  cudaError_t stage_ids(Rank& rk, const Job& j, const int64_t*& gpu_ids, const int64_t*& cpu_ids);
  void notify(int rank, int counter, int layer_lo, int layer_hi);
  // failure path of a job: records the status for counter_status(), then publishes the epoch to the flags of
  // layers [from_layer, L) from the host and fires their eventfds (one unit each, as for a good layer: the
  // eventfds are semaphores, so the failure is told by counter_status() and the restore's result, not by a value)
  void release_waiters(int r, const Job& j, int from_layer, int status);
  static bool status_words_set(const volatile int32_t* words);
  static void CUDART_CB host_fn(void* arg);

  std::vector<GpuSide> gpus_;
  HostSide host_;
  std::vector<LayerwiseMemberGroup> mgroups_;            // empty for the uniform form
  std::vector<std::vector<LayerMember>> members_;        // [model layer]
  LayerwiseOptions opt_;
  std::vector<std::unique_ptr<Rank>> ranks_;
  std::atomic<bool> stop_{false};
  std::vector<int> eventfds_;       // [counters][ranks][layers]
  std::vector<uint32_t> epochs_;    // per counter, guarded by epoch_mu_
  std::vector<uint8_t> reserved_;   // per counter: begin_restore() handed the next epoch out already
  std::mutex epoch_mu_;
  std::unique_ptr<std::atomic<int>[]> counter_status_;
  std::mutex launched_mu_;
  std::condition_variable launched_cv_;
  std::vector<uint32_t> launched_;  // [counters][ranks]: newest epoch whose launches are all queued (or that failed)
  void mark_launched(int r, const Job& j);
  int64_t* id_ring_ = nullptr;      // [2][max_blocks], mapped pinned
  std::mutex api_mu_;               // one restore at a time per group
  std::mutex done_mu_;
  std::condition_variable done_cv_;
  std::vector<std::unique_ptr<HostFnArg>> fn_args_;
};

}  // namespace fkv
