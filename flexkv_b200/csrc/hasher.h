// Block-key generation: cumulative streaming XXH64 over int64 token ids.
// hash[i] covers tokens [0, (i+1)*tokens_per_block) preceded by the optional
// namespace prefix (one int64 per UTF-8 byte of "\0".join(namespace));
// reference behaviour: csrc/hash.cpp:47-66, flexkv/common/block.py:11-20,82-90.
#pragma once
#include <cstdint>
#include <vector>

#include "xxh64.h"

namespace fkv {

// Writes floor(num_tokens / tokens_per_block) keys into out.
inline int64_t gen_block_hashes(const int64_t* tokens, int64_t num_tokens, int tokens_per_block,
                                const int64_t* ns_prefix, int64_t ns_len, uint64_t* out) {
  XXH64 st(0);
  if (ns_len > 0) st.update(ns_prefix, (size_t)ns_len * sizeof(int64_t));
  const int64_t nb = num_tokens / tokens_per_block;
  const size_t bytes = (size_t)tokens_per_block * sizeof(int64_t);
  for (int64_t i = 0; i < nb; ++i) {
    st.update(tokens + i * tokens_per_block, bytes);
    out[i] = st.digest();
  }
  return nb;
}

// Many sequences at once on a small thread team (offsets has n+1 entries into
// tokens; out_offsets has n+1 entries into out).
void gen_block_hashes_batch(const int64_t* tokens, const int64_t* offsets, int64_t n, int tokens_per_block,
                            const int64_t* ns_prefix, int64_t ns_len, uint64_t* out, const int64_t* out_offsets,
                            int num_threads);
// Same, over separately stored sequences and result buffers (no flattening).
void gen_block_hashes_ptrs(const int64_t* const* seqs, const int64_t* lens, int64_t n, int tokens_per_block,
                           const int64_t* ns_prefix, int64_t ns_len, uint64_t* const* outs, int num_threads);

}  // namespace fkv
