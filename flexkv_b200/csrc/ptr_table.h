// Tensor-pointer tables of registrations that do not fit the launch parameters.
//
// KvCopyParams carries up to kMaxGpuPtrs tensor pointers by value. A registration with more tensors (K and V
// tensors of a model deeper than 128 layers, several layer groups in one list) keeps its table in memory of
// its own: one copy on the device that runs the kernel, one on the host for argument checks and copy-engine
// planning. Tables are cached by (device, contents): an op looks its table up, a re-registration with new
// addresses adds an entry. Entries live until the process exits; each is 8 bytes per tensor.
#pragma once
#include <cstdint>
#include <vector>

#include "kernels/kv_copy.h"

namespace fkv {

struct PtrTable {
  const uint64_t* host = nullptr;   // stable host copy
  const uint64_t* exec = nullptr;   // what the executing side reads: device memory, or `host` for CPU execution
  int32_t n = 0;
};

// `device` >= 0: the table is also uploaded to that device (the current device is restored); -1: host only.
// Throws std::invalid_argument beyond kMaxGpuPtrsExt entries and std::runtime_error when the upload fails.
PtrTable ptr_table_get(const std::vector<uint64_t>& ptrs, int device);

// Fills the gpu-side table of `p` from `ptrs`: inline up to kMaxGpuPtrs entries, through the cache beyond.
void kv_set_gpu_table(KvCopyParams& p, const std::vector<uint64_t>& ptrs, int device);
// The same for the second table (a peer's tensors, or the multicast twins of the fan-out kernel); does not
// touch c_use_table or the index multipliers.
void kv_set_c_table(KvCopyParams& p, const std::vector<uint64_t>& ptrs, int device);

int64_t ptr_table_cache_size();

}  // namespace fkv
