// CPU restatement of the paged KV gather/scatter addressing (kernels/kv_copy.h).
// It is the byte-exact oracle for the CUDA kernels and the data plane of
// GPU-less deployments and tests, where the "GPU" side is a host-resident
// stand-in for the engine's paged cache.
#include <algorithm>
#include <atomic>
#include <cstring>
#include <thread>
#include <vector>

#include "kernels/kv_copy.h"

namespace fkv {

int host_kv_copy(const KvCopyParams& p, int num_threads) {
  if (p.num_pairs <= 0 || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return 0;
  if (!kv_copy_tables_ok(p)) return KV_ERR_BAD_ARGS;
  std::atomic<int> err{0};
  std::atomic<int64_t> next{0};
  const int64_t total = (int64_t)p.num_pairs * p.num_layers;
  auto work = [&] {
    for (int64_t w = next.fetch_add(1); w < total; w = next.fetch_add(1)) {
      const int64_t pair = w / p.num_layers;
      const int layer = p.layer_start + (int)(w % p.num_layers);
      const int64_t g = p.gpu_blocks[pair], c = p.cpu_blocks[pair];
      if (p.gpu_num_blocks > 0 && (g < 0 || g >= p.gpu_num_blocks)) { err |= KV_ERR_GPU_BLOCK_RANGE; continue; }
      if (p.cpu_num_blocks > 0 && (c < 0 || c >= p.cpu_num_blocks)) { err |= KV_ERR_CPU_BLOCK_RANGE; continue; }
      for (int kv = 0; kv < p.kv_dim; ++kv) {
        uint8_t* ga = reinterpret_cast<uint8_t*>(p.gpu_ptrs[layer * p.idx_layer_mul + kv * p.idx_kv_mul] +
                                                 layer * p.g_layer_stride + kv * p.g_kv_stride +
                                                 g * p.g_block_stride + p.g_off);
        const uint64_t cbase =
            p.c_use_table ? p.c_ptrs[layer * p.c_idx_layer_mul + kv * p.c_idx_kv_mul] : p.cpu_base;
        uint8_t* ca = reinterpret_cast<uint8_t*>(cbase + layer * p.c_layer_stride + kv * p.c_kv_stride +
                                                 c * p.c_block_stride + p.c_off);
        if (p.h2d) std::memcpy(ga, ca, (size_t)p.chunk_bytes);
        else std::memcpy(ca, ga, (size_t)p.chunk_bytes);
      }
    }
  };
  num_threads = (int)std::max<int64_t>(1, std::min<int64_t>(num_threads, total / 64 + 1));
  if (num_threads == 1) work();
  else {
    std::vector<std::thread> team;
    for (int t = 0; t < num_threads; ++t) team.emplace_back(work);
    for (auto& th : team) th.join();
  }
  return err.load();
}

}  // namespace fkv
