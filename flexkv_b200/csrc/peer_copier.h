// GPU<->GPU prefix pull over NVLink peer memory.
//
// When a prefix a rank needs already sits in another rank's paged KV cache, the
// destination GPU pulls the blocks straight out of the owner's HBM: the copy
// kernel runs on the destination, its bulk loads target the peer's tensors
// (plain, non-multicast bulk copies over NVLink), its stores target the local
// paged cache, and source and destination layouts are addressed independently
// so the two engines need not share a layout. There is no counterpart in the
// reference, whose only cross-instance path is host-to-host RDMA.
#pragma once
#include <cstdint>
#include <memory>
#include <mutex>
#include <vector>

#include <cuda_runtime.h>

#include "transfer_group.h"

namespace fkv {

class PeerCopier {
 public:
  // ranks[i] describes rank i's registered KV cache (device, tensors, strides)
  PeerCopier(std::vector<GpuSide> ranks, int num_layers, int kv_dim, int64_t chunk_bytes, KvCopyLaunch launch,
             int64_t max_blocks_per_op);
  ~PeerCopier();

  // dst_rank's blocks dst_blocks[i] <- src_rank's blocks src_blocks[i]; blocking
  OpResult pull(int dst_rank, int src_rank, const int64_t* dst_blocks, const int64_t* src_blocks, int64_t n,
                int layer_start, int num_layers);
  bool can_access(int dst_rank, int src_rank);
  int num_ranks() const { return (int)ranks_.size(); }
  void update_gpu_ptrs(int rank, const std::vector<uint64_t>& ptrs);  // with no pull in flight for that rank

 private:
  struct PerDst {
    std::mutex mu;
    bool init = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int64_t* ids = nullptr;      // mapped pinned [2][max_blocks]
    int32_t* status = nullptr;   // mapped pinned [kStatusWords]
    std::vector<int> peer_ok;    // -1 unknown, 0 no, 1 enabled
  };
  void ensure_init(int dst_rank);

  std::vector<GpuSide> ranks_;
  int num_layers_, kv_dim_;
  int64_t chunk_bytes_;
  KvCopyLaunch launch_;
  int64_t max_blocks_;
  std::vector<std::unique_ptr<PerDst>> dst_;
};

}  // namespace fkv
