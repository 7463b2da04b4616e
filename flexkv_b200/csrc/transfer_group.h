// GPU<->host transfer executor for one tensor-parallel group.
//
// One persistent host thread, CUDA stream and mapped status word per GPU of
// the group; an op (a list of gpu/cpu block-id pairs, a direction and a layer
// range) is fanned out to every rank and joined. Block ids are written once
// into a mapped pinned ring that all GPUs read directly, so an op costs one
// kernel launch per GPU and no staging copies. Shared-KV (MLA) write modes
// and the per-rank placement inside a host block follow the reference
// (csrc/tp_transfer_thread_group.cpp:199-381; flexkv/transfer/worker.py:1196-1204).
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "ce_copy.h"
#include "kernels/kv_copy.h"

namespace fkv {

struct GpuSide {
  int device = 0;
  std::vector<uint64_t> ptrs;
  int idx_layer_mul = 1, idx_kv_mul = 0;
  int64_t layer_stride = 0, kv_stride = 0, block_stride = 0;
  int64_t num_blocks = 0;
};

struct HostSide {
  uint64_t base = 0;
  int64_t layer_stride = 0, kv_stride = 0, block_stride = 0;
  int64_t num_blocks = 0;
};

enum class SharedKvMode : int { SHARDED = 0, ALL_WRITE = 1, RANK0_ONLY = 2, LAYER_PARALLEL = 3, RANK_ROTATE = 4 };
SharedKvMode parse_shared_kv_mode(const std::string& s);

struct GroupOptions {
  int num_layers = 1;
  int kv_dim = 2;
  int64_t chunk_bytes = 0;       // bytes one rank moves per (layer, kv, block)
  int64_t cpu_tp_stride = 0;     // byte offset of rank r inside the host chunk/block = r * cpu_tp_stride
  bool shared_kv = false;        // every rank holds identical KV (MLA, num_kv_heads == 1)
  SharedKvMode shared_mode = SharedKvMode::SHARDED;
  KvCopyLaunch h2d{16, 16384, 0};
  KvCopyLaunch d2h{16, 16384, 0};
  int ring_slots = 8;
  int64_t max_blocks_per_op = 1 << 16;
  bool high_priority_stream = false;
  CePolicy ce_policy;
  int64_t ce_staging_blocks = 32;   // blocks per staging buffer of the gather + large-copy route (0 = route off);
                                    // two buffers of this size are allocated per GPU the first time the route runs
};

// Engine selectors of an op (KvCopyLaunch::engine or a per-op override).
constexpr int kEngineTma = 0, kEngineSimt = 1, kEngineCe = 2, kEngineAuto = 3, kEngineRefshape = 9;

struct OpResult {
  int status = 0;        // OR of KvCopyStatus bits over ranks; negative = CUDA error code
  float gpu_ms = 0.f;    // max over ranks, CUDA events on the launching stream
};

// Fills the addressing part of a launch for rank `r` of `n_ranks` (shared by the
// transfer group and the layerwise group). `skip` is set when the rank has
// nothing to do under the shared-KV write mode.
void fill_kv_params(const GpuSide& gs, const HostSide& host, const GroupOptions& opt, int r, int n_ranks,
                    const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d, int layer_start,
                    int num_layers, uint64_t rotate, KvCopyParams& p, bool& skip);

class TransferGroup {
 public:
  TransferGroup(std::vector<GpuSide> gpus, HostSide host, GroupOptions opt);
  ~TransferGroup();

  // asynchronous: returns a ticket to pass to wait()
  uint64_t submit(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d, int layer_start,
                  int num_layers, int engine_override = -1);
  OpResult wait(uint64_t ticket);
  bool poll(uint64_t ticket);
  OpResult transfer(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d, int layer_start,
                    int num_layers, int engine_override = -1) {
    return wait(submit(gpu_blocks, cpu_blocks, n, h2d, layer_start, num_layers, engine_override));
  }
  // baseline shape for timing comparisons (4 CTAs x 1024 threads, warp per chunk)
  OpResult transfer_refshape(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d, int num_ctas);

  void update_gpu_ptrs(int rank, const std::vector<uint64_t>& ptrs);  // sleep/wake re-registration
  void set_launch(bool h2d, KvCopyLaunch cfg);
  int num_ranks() const { return (int)gpus_.size(); }
  uint64_t ce_ops() const { return ce_ops_.load(); }   // ops that went through the copy engines
  uint64_t staged_ops() const { return staged_ops_.load(); }   // of which through the staging area
  const GroupOptions& options() const { return opt_; }

 private:
  struct Task {
    uint64_t ticket;
    int slot;          // ring slot holding the ids
    int64_t n;
    bool h2d;
    int layer_start, num_layers;
    int engine;        // -1 default, else one of the kEngine* selectors
    int refshape_ctas;
    uint64_t rotate;   // op counter for RANK_ROTATE
  };
  struct Rank {
    std::thread th;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Task> q;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int32_t* status = nullptr;  // mapped pinned word
    CeStaging staging;          // device staging of the gather + large-copy route (allocated on first use)
    bool ready = false;
    std::string init_error;
  };
  struct Pending {
    int remaining;
    OpResult res;
    int slot;
  };

  void rank_main(int r);
  void fill_params(int r, const Task& t, KvCopyParams& p, bool& skip) const;
  void finish(uint64_t ticket, int status, float ms);

  std::vector<GpuSide> gpus_;
  HostSide host_;
  GroupOptions opt_;
  std::vector<std::unique_ptr<Rank>> ranks_;
  std::atomic<bool> stop_{false};

  int64_t* id_ring_ = nullptr;  // [ring_slots][2][max_blocks_per_op], mapped pinned, portable
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<int> free_slots_;
  std::unordered_map<uint64_t, Pending> pending_;
  uint64_t next_ticket_ = 1;
  uint64_t op_counter_ = 0;
  std::atomic<uint64_t> ce_ops_{0}, staged_ops_{0};
  mutable std::mutex ptr_mu_;
};

}  // namespace fkv
