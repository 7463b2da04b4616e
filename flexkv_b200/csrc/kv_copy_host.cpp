// CPU restatement of the paged KV gather/scatter addressing (kernels/kv_copy.h).
// It is the byte-exact oracle for the CUDA kernels and the data plane of
// GPU-less deployments and tests, where the "GPU" side is a host-resident
// stand-in for the engine's paged cache.
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "kernels/kv_copy.h"

namespace fkv {

namespace {

// Persistent helpers for the CPU data plane: an op borrows up to `n - 1` of them and runs the
// same work function on its own thread too, so a request never pays for thread creation
// (the reference keeps a per-thread CopyPool for its CPU gather/scatter: csrc/ce_transfer.cu:523-641).
class CopyPool {
 public:
  CopyPool() {
    const unsigned hw = std::max(2u, std::thread::hardware_concurrency());
    const int n = (int)std::min(16u, hw) - 1;
    for (int i = 0; i < n; ++i) threads_.emplace_back([this] { loop(); });
  }
  ~CopyPool() {
    { std::lock_guard<std::mutex> g(mu_); stop_ = true; }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  int size() const { return (int)threads_.size() + 1; }
  // runs `fn` on min(n, size()) threads in total and returns when all of them are done
  void run(int n, const std::function<void()>& fn) {
    const int helpers = std::max(0, std::min(n, size()) - 1);
    if (helpers == 0) { fn(); return; }
    std::unique_lock<std::mutex> op(op_mu_);     // one parallel op at a time; others wait their turn
    {
      std::lock_guard<std::mutex> g(mu_);
      fn_ = &fn;
      tickets_ = helpers;
      running_ = helpers;
    }
    cv_.notify_all();
    fn();
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [&] { return running_ == 0; });
    fn_ = nullptr;
  }

 private:
  void loop() {
    for (;;) {
      const std::function<void()>* fn;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || tickets_ > 0; });
        if (stop_) return;
        --tickets_;
        fn = fn_;
      }
      (*fn)();
      {
        std::lock_guard<std::mutex> g(mu_);
        if (--running_ == 0) done_cv_.notify_all();
      }
    }
  }
  std::vector<std::thread> threads_;
  std::mutex mu_, op_mu_;
  std::condition_variable cv_, done_cv_;
  const std::function<void()>* fn_ = nullptr;
  int tickets_ = 0, running_ = 0;
  bool stop_ = false;
};

CopyPool& copy_pool() {
  static CopyPool* pool = new CopyPool();   // lives until exit: no join at static destruction after fork/exit races
  return *pool;
}

}  // namespace

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
        uint8_t* ga = reinterpret_cast<uint8_t*>(kv_gpu_tensor(p, layer * p.idx_layer_mul + kv * p.idx_kv_mul) +
                                                 layer * p.g_layer_stride + kv * p.g_kv_stride +
                                                 g * p.g_block_stride + p.g_off);
        const uint64_t cbase =
            p.c_use_table ? kv_c_tensor(p, layer * p.c_idx_layer_mul + kv * p.c_idx_kv_mul) : p.cpu_base;
        uint8_t* ca = reinterpret_cast<uint8_t*>(cbase + layer * p.c_layer_stride + kv * p.c_kv_stride +
                                                 c * p.c_block_stride + p.c_off);
        if (p.h2d) std::memcpy(ga, ca, (size_t)p.chunk_bytes);
        else std::memcpy(ca, ga, (size_t)p.chunk_bytes);
      }
    }
  };
  // one helper per 512 KiB of payload, the caller's thread included; small ops run inline
  const int64_t bytes = total * p.kv_dim * p.chunk_bytes;
  const int want = (int)std::max<int64_t>(1, std::min<int64_t>(num_threads, bytes / (512 << 10)));
  copy_pool().run(want, work);
  return err.load();
}

}  // namespace fkv
