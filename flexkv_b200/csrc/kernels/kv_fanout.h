// Restore with NVSwitch fan-out: one rank reads a host block over PCIe once and
// `multimem.st` replicates every 16 bytes into the same offset of every rank's
// KV cache bound to the multicast object. For KV that is identical on all ranks
// of a tensor-parallel group (MLA latent cache, num_kv_heads == 1) this replaces
// N independent host reads (what the reference does: every rank re-reads the
// same host bytes, csrc/layerwise.cpp:1142-1165) by one.
//
// The destination caches must be carved out of one symmetric allocation per
// rank: multicast address = local address + mc_delta.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "kv_copy.h"

namespace fkv {

struct KvFanoutParams {
  KvCopyParams base;    // host -> local GPU addressing (h2d = 1); done_counter = device scratch word
  int64_t mc_delta;     // multicast address of a local address a: a + mc_delta
                        // When base.num_c_ptrs > 0 the delta is not used: base.c_ptrs[i] is the multicast address
                        // of tensor gpu_ptrs[i], so the tensors may come from several symmetric allocations
                        // (one multicast object each), e.g. segments kept under a few GiB
  uint32_t* mc_flag;    // multicast address of a per-rank flag word, set to base.epoch after the data; may be null
};

cudaError_t launch_kv_fanout(const KvFanoutParams& p, int num_ctas, int tile_bytes, cudaStream_t stream);

}  // namespace fkv
