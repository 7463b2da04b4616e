#include "hasher.h"

#include <algorithm>
#include <atomic>
#include <thread>

namespace fkv {

void gen_block_hashes_batch(const int64_t* tokens, const int64_t* offsets, int64_t n, int tokens_per_block,
                            const int64_t* ns_prefix, int64_t ns_len, uint64_t* out, const int64_t* out_offsets,
                            int num_threads) {
  auto one = [&](int64_t i) {
    gen_block_hashes(tokens + offsets[i], offsets[i + 1] - offsets[i], tokens_per_block, ns_prefix, ns_len,
                     out + out_offsets[i]);
  };
  // a thread is worth starting for a few hundred microseconds of hashing (about 256K tokens)
  const int64_t total_tokens = offsets[n] - offsets[0];
  num_threads = (int)std::max<int64_t>(1, std::min<int64_t>({(int64_t)num_threads, n, total_tokens / 262144 + 1}));
  if (num_threads == 1) {
    for (int64_t i = 0; i < n; ++i) one(i);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> team;
  for (int t = 0; t < num_threads; ++t)
    team.emplace_back([&] {
      for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) one(i);
    });
  for (auto& th : team) th.join();
}

void gen_block_hashes_ptrs(const int64_t* const* seqs, const int64_t* lens, int64_t n, int tokens_per_block,
                           const int64_t* ns_prefix, int64_t ns_len, uint64_t* const* outs, int num_threads) {
  int64_t total_tokens = 0;
  for (int64_t i = 0; i < n; ++i) total_tokens += lens[i];
  auto one = [&](int64_t i) { gen_block_hashes(seqs[i], lens[i], tokens_per_block, ns_prefix, ns_len, outs[i]); };
  num_threads = (int)std::max<int64_t>(1, std::min<int64_t>({(int64_t)num_threads, n, total_tokens / 262144 + 1}));
  if (num_threads == 1) {
    for (int64_t i = 0; i < n; ++i) one(i);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> team;
  for (int t = 0; t < num_threads; ++t)
    team.emplace_back([&] {
      for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) one(i);
    });
  for (auto& th : team) th.join();
}

}  // namespace fkv
