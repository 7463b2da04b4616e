// Batched block-key generation on the GPU: cumulative streaming XXH64 (seed 0) over int64
// token ids, one digest per block, bit-identical to the host hasher (hasher.h; reference
// behaviour csrc/hash.cpp:47-66). For callers whose token ids already live on the device
// (an engine that keeps its prompts in HBM) or that hash thousands of long sequences at once;
// for a single request the host hasher (about 12 us per 8K tokens) is faster than any launch.
#pragma once
#include <cstdint>

#include <cuda_runtime.h>

namespace fkv {

// tokens: all sequences back to back; offsets[n+1] (in tokens) and out_offsets[n+1] (in blocks)
// are device- or mapped-host-readable. ns_prefix (ns_len int64 values, may be null) is fed
// before every sequence. One quad of threads hashes one sequence.
cudaError_t launch_kv_block_hashes(const int64_t* tokens, const int64_t* offsets, int64_t num_seqs, int tokens_per_block,
                                   const int64_t* ns_prefix, int64_t ns_len, uint64_t* out, const int64_t* out_offsets,
                                   cudaStream_t stream);

}  // namespace fkv
