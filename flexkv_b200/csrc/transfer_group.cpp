#include "transfer_group.h"

#include <climits>

#include "ce_copy.h"
#include "ptr_table.h"

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace fkv {

SharedKvMode parse_shared_kv_mode(const std::string& s) {
  if (s == "sharded") return SharedKvMode::SHARDED;
  if (s == "all_write") return SharedKvMode::ALL_WRITE;
  if (s == "rank0_only") return SharedKvMode::RANK0_ONLY;
  if (s == "layer_parallel") return SharedKvMode::LAYER_PARALLEL;
  if (s == "rank_rotate") return SharedKvMode::RANK_ROTATE;
  throw std::invalid_argument("unknown kv_shared_across_ranks_mode: " + s);
}

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

static constexpr int kInflight = 4;

TransferGroup::TransferGroup(std::vector<GpuSide> gpus, HostSide host, GroupOptions opt)
    : gpus_(std::move(gpus)), host_(host), opt_(opt) {
  if (gpus_.empty()) throw std::invalid_argument("TransferGroup: no GPUs");
  for (auto& g : gpus_)
    if ((int)g.ptrs.size() > kMaxGpuPtrsExt) throw std::invalid_argument("TransferGroup: too many GPU tensors per rank");
  if (opt_.shared_kv && opt_.shared_mode == SharedKvMode::SHARDED && (opt_.chunk_bytes % (int64_t)gpus_.size()) != 0)
    throw std::invalid_argument("TransferGroup: sharded shared-KV mode needs chunk_bytes divisible by the group size");
  check(cudaSetDevice(gpus_[0].device), "cudaSetDevice");
  const size_t ring_bytes = (size_t)opt_.ring_slots * 2 * (size_t)opt_.max_blocks_per_op * sizeof(int64_t);
  check(cudaHostAlloc((void**)&id_ring_, ring_bytes, cudaHostAllocPortable | cudaHostAllocMapped),
        "cudaHostAlloc(id ring)");
  for (int s = 0; s < opt_.ring_slots; ++s) free_slots_.push_back(s);
  for (size_t r = 0; r < gpus_.size(); ++r) ranks_.emplace_back(new Rank());
  for (size_t r = 0; r < gpus_.size(); ++r) ranks_[r]->th = std::thread([this, r] { rank_main((int)r); });
  for (auto& rk : ranks_) {
    std::unique_lock<std::mutex> lk(rk->mu);
    rk->cv.wait(lk, [&] { return rk->ready; });
    if (!rk->init_error.empty()) {
      std::string msg = rk->init_error;
      lk.unlock();
      stop_ = true;
      for (auto& x : ranks_) { x->cv.notify_all(); if (x->th.joinable()) x->th.join(); }
      cudaFreeHost(id_ring_);
      throw std::runtime_error("TransferGroup: " + msg);
    }
  }
}

TransferGroup::~TransferGroup() {
  stop_ = true;
  for (auto& rk : ranks_) {
    { std::lock_guard<std::mutex> g(rk->mu); }
    rk->cv.notify_all();
  }
  for (auto& rk : ranks_) if (rk->th.joinable()) rk->th.join();
  if (id_ring_) cudaFreeHost(id_ring_);
}

void TransferGroup::update_gpu_ptrs(int rank, const std::vector<uint64_t>& ptrs) {
  if ((int)ptrs.size() > kMaxGpuPtrsExt) throw std::invalid_argument("too many GPU tensors");
  std::lock_guard<std::mutex> g(ptr_mu_);
  gpus_.at((size_t)rank).ptrs = ptrs;
}

void TransferGroup::set_launch(bool h2d, KvCopyLaunch cfg) {
  std::lock_guard<std::mutex> g(ptr_mu_);
  (h2d ? opt_.h2d : opt_.d2h) = cfg;
}

void fill_kv_params(const GpuSide& gs, const HostSide& host, const GroupOptions& opt, int r, int N,
                    const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d, int layer_start,
                    int num_layers, uint64_t rotate, KvCopyParams& p, bool& skip) {
  std::memset(&p, 0, sizeof(p));
  kv_set_gpu_table(p, gs.ptrs, gs.device);
  p.idx_layer_mul = gs.idx_layer_mul;
  p.idx_kv_mul = gs.idx_kv_mul;
  p.g_layer_stride = gs.layer_stride;
  p.g_kv_stride = gs.kv_stride;
  p.g_block_stride = gs.block_stride;
  p.cpu_base = host.base;
  p.c_layer_stride = host.layer_stride;
  p.c_kv_stride = host.kv_stride;
  p.c_block_stride = host.block_stride;
  p.gpu_blocks = gpu_blocks;
  p.cpu_blocks = cpu_blocks;
  p.num_pairs = (int32_t)n;
  p.layer_start = layer_start;
  p.num_layers = num_layers;
  p.kv_dim = opt.kv_dim;
  p.chunk_bytes = opt.chunk_bytes;
  p.gpu_num_blocks = gs.num_blocks;
  p.cpu_num_blocks = host.num_blocks;
  p.h2d = h2d ? 1 : 0;
  skip = false;
  if (!opt.shared_kv) {
    p.c_off = (int64_t)r * opt.cpu_tp_stride;
    return;
  }
  if (h2d || N == 1) return;  // every rank restores the full chunk
  switch (opt.shared_mode) {
    case SharedKvMode::SHARDED:
      p.chunk_bytes = opt.chunk_bytes / N;
      p.g_off = p.c_off = (int64_t)r * p.chunk_bytes;
      break;
    case SharedKvMode::ALL_WRITE: break;
    case SharedKvMode::RANK0_ONLY: skip = r != 0; break;
    case SharedKvMode::RANK_ROTATE: skip = (int)(rotate % (uint64_t)N) != r; break;
    case SharedKvMode::LAYER_PARALLEL: {
      const int per = (num_layers + N - 1) / N;
      const int lo = std::min(num_layers, r * per), hi = std::min(num_layers, (r + 1) * per);
      p.layer_start = layer_start + lo;
      p.num_layers = hi - lo;
      skip = hi <= lo;
      break;
    }
  }
}

void TransferGroup::fill_params(int r, const Task& t, KvCopyParams& p, bool& skip) const {
  std::lock_guard<std::mutex> g(ptr_mu_);
  fill_kv_params(gpus_[(size_t)r], host_, opt_, r, (int)gpus_.size(),
                 id_ring_ + ((size_t)t.slot * 2 + 0) * (size_t)opt_.max_blocks_per_op,
                 id_ring_ + ((size_t)t.slot * 2 + 1) * (size_t)opt_.max_blocks_per_op, t.n, t.h2d, t.layer_start,
                 t.num_layers, t.rotate, p, skip);
}

void TransferGroup::rank_main(int r) {
  Rank& rk = *ranks_[(size_t)r];
  cudaEvent_t ev0[kInflight], ev1[kInflight];
  try {
    check(cudaSetDevice(gpus_[(size_t)r].device), "cudaSetDevice");
    int lo = 0, hi = 0;
    check(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
    check(cudaStreamCreateWithPriority(&rk.stream, cudaStreamNonBlocking, opt_.high_priority_stream ? hi : lo),
          "cudaStreamCreateWithPriority");
    for (int i = 0; i < kInflight; ++i) {
      check(cudaEventCreate(&ev0[i]), "cudaEventCreate");
      check(cudaEventCreate(&ev1[i]), "cudaEventCreate");
    }
    check(cudaHostAlloc((void**)&rk.status, kInflight * kStatusWords * sizeof(int32_t),
                        cudaHostAllocPortable | cudaHostAllocMapped),
          "cudaHostAlloc(status)");
    for (int i = 0; i < kInflight * kStatusWords; ++i) rk.status[i] = 0;
  } catch (const std::exception& e) {
    std::lock_guard<std::mutex> g(rk.mu);
    rk.init_error = e.what();
    rk.ready = true;
    rk.cv.notify_all();
    return;
  }
  {
    std::lock_guard<std::mutex> g(rk.mu);
    rk.ready = true;
  }
  rk.cv.notify_all();

  std::vector<Task> batch;
  for (;;) {
    batch.clear();
    {
      std::unique_lock<std::mutex> lk(rk.mu);
      rk.cv.wait(lk, [&] { return stop_.load() || !rk.q.empty(); });
      if (rk.q.empty() && stop_.load()) break;
      while (!rk.q.empty() && (int)batch.size() < kInflight) {
        batch.push_back(rk.q.front());
        rk.q.pop_front();
      }
    }
    // launch everything that is queued, then retire in order: consecutive ops overlap their launch latency
    int launched[kInflight];
    cudaError_t lerr[kInflight];
    for (size_t i = 0; i < batch.size(); ++i) {
      const Task& t = batch[i];
      KvCopyParams p;
      bool skip = false;
      fill_params(r, t, p, skip);
      p.status = rk.status + i * kStatusWords;
      launched[i] = skip ? 0 : 1;
      lerr[i] = cudaSuccess;
      if (skip) continue;
      cudaEventRecord(ev0[i], rk.stream);
      if (t.engine == kEngineRefshape) {
        lerr[i] = launch_kv_copy_refshape(p, t.refshape_ctas, rk.stream);
      } else {
        KvCopyLaunch cfg = t.h2d ? opt_.h2d : opt_.d2h;
        if (t.engine >= 0) cfg.engine = t.engine;
        bool done = false;
        if (cfg.engine == kEngineCe || cfg.engine == kEngineAuto) {
          // the id ring is mapped pinned memory: the same pointers are readable here
          CeAnalysis a = ce_analyze(p.gpu_blocks, p.cpu_blocks, p.num_pairs, p.gpu_num_blocks, p.cpu_num_blocks);
          CePath path = ce_choose(a, p, cfg.engine == kEngineCe ? CePolicy{INT64_MAX, 0} : opt_.ce_policy);
          if (path != CePath::KERNEL) {
            lerr[i] = ce_copy(p, a, path, rk.stream);
            for (int b = 0; b < kStatusWords; ++b)
              if (a.status & (1 << b)) p.status[b] = 1;
            ce_ops_.fetch_add(1, std::memory_order_relaxed);
            done = true;
          } else if (opt_.ce_staging_blocks > 0 && p.c_block_stride > 0) {
            // scattered GPU pages, host blocks in a row: gather into device staging, one large copy per piece
            const int64_t min_run = std::max<int64_t>(1, (opt_.ce_policy.min_bytes_per_copy + p.c_block_stride - 1) /
                                                             p.c_block_stride);
            std::vector<CeHostRun> runs;
            if ((int)gpus_.size() == 1 &&
                ce_host_runs(p, p.gpu_blocks, p.cpu_blocks, p.num_pairs, opt_.num_layers, min_run, runs)) {
              KvCopyLaunch kcfg = cfg;
              kcfg.engine = 0;
              lerr[i] = ce_copy_staged(p, runs, rk.staging, opt_.ce_staging_blocks, kcfg, rk.stream);
              ce_ops_.fetch_add(1, std::memory_order_relaxed);
              staged_ops_.fetch_add(1, std::memory_order_relaxed);
              done = true;
            }
          }
        }
        if (!done) {
          if (cfg.engine >= kEngineCe) cfg.engine = 0;
          lerr[i] = launch_kv_copy(p, cfg, rk.stream);
        }
      }
      cudaEventRecord(ev1[i], rk.stream);
    }
    for (size_t i = 0; i < batch.size(); ++i) {
      int status = 0;
      float ms = 0.f;
      if (launched[i]) {
        cudaError_t e = lerr[i];
        if (e == cudaSuccess) e = cudaEventSynchronize(ev1[i]);
        if (e == cudaSuccess) {
          cudaEventElapsedTime(&ms, ev0[i], ev1[i]);
          status = collect_status(rk.status + i * kStatusWords);
        } else {
          (void)cudaGetLastError();
          status = -(int)e;
        }
      }
      finish(batch[i].ticket, status, ms);
    }
  }
  ce_staging_free(rk.staging);
  for (int i = 0; i < kInflight; ++i) { cudaEventDestroy(ev0[i]); cudaEventDestroy(ev1[i]); }
  if (rk.status) cudaFreeHost(rk.status);
  if (rk.stream) cudaStreamDestroy(rk.stream);
}

void TransferGroup::finish(uint64_t ticket, int status, float ms) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = pending_.find(ticket);
  if (it == pending_.end()) return;
  Pending& pd = it->second;
  if (status < 0) pd.res.status = status;
  else if (pd.res.status >= 0) pd.res.status |= status;
  pd.res.gpu_ms = std::max(pd.res.gpu_ms, ms);
  if (--pd.remaining == 0) {
    if (pd.slot >= 0) free_slots_.push_back(pd.slot);
    pd.slot = -1;
    cv_.notify_all();
  }
}

uint64_t TransferGroup::submit(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d,
                               int layer_start, int num_layers, int engine_override) {
  if (n > opt_.max_blocks_per_op) throw std::invalid_argument("TransferGroup: op exceeds max_blocks_per_op");
  if (layer_start < 0 || num_layers < 0 || layer_start + num_layers > opt_.num_layers)
    throw std::invalid_argument("TransferGroup: layer range out of bounds");
  Task t;
  {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !free_slots_.empty(); });
    t.slot = free_slots_.back();
    free_slots_.pop_back();
    t.ticket = next_ticket_++;
    t.rotate = op_counter_++;
    Pending pd;
    pd.remaining = (int)ranks_.size();
    pd.slot = t.slot;
    pending_[t.ticket] = pd;
  }
  int64_t* gdst = id_ring_ + ((size_t)t.slot * 2 + 0) * (size_t)opt_.max_blocks_per_op;
  int64_t* cdst = id_ring_ + ((size_t)t.slot * 2 + 1) * (size_t)opt_.max_blocks_per_op;
  if (n > 0) {
    std::memcpy(gdst, gpu_blocks, (size_t)n * sizeof(int64_t));
    std::memcpy(cdst, cpu_blocks, (size_t)n * sizeof(int64_t));
  }
  t.n = n;
  t.h2d = h2d;
  t.layer_start = layer_start;
  t.num_layers = num_layers;
  t.engine = engine_override;
  t.refshape_ctas = 4;
  for (auto& rk : ranks_) {
    { std::lock_guard<std::mutex> g(rk->mu); rk->q.push_back(t); }
    rk->cv.notify_one();
  }
  return t.ticket;
}

bool TransferGroup::poll(uint64_t ticket) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = pending_.find(ticket);
  return it == pending_.end() || it->second.remaining == 0;
}

OpResult TransferGroup::wait(uint64_t ticket) {
  std::unique_lock<std::mutex> lk(mu_);
  auto it = pending_.find(ticket);
  if (it == pending_.end()) throw std::invalid_argument("TransferGroup: unknown ticket");
  cv_.wait(lk, [&] { return it->second.remaining == 0; });
  OpResult r = it->second.res;
  pending_.erase(it);
  return r;
}

OpResult TransferGroup::transfer_refshape(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, bool h2d,
                                          int num_ctas) {
  if (n > opt_.max_blocks_per_op) throw std::invalid_argument("TransferGroup: op exceeds max_blocks_per_op");
  Task t;
  {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !free_slots_.empty(); });
    t.slot = free_slots_.back();
    free_slots_.pop_back();
    t.ticket = next_ticket_++;
    t.rotate = op_counter_++;
    Pending pd;
    pd.remaining = (int)ranks_.size();
    pd.slot = t.slot;
    pending_[t.ticket] = pd;
  }
  std::memcpy(id_ring_ + ((size_t)t.slot * 2 + 0) * (size_t)opt_.max_blocks_per_op, gpu_blocks, (size_t)n * 8);
  std::memcpy(id_ring_ + ((size_t)t.slot * 2 + 1) * (size_t)opt_.max_blocks_per_op, cpu_blocks, (size_t)n * 8);
  t.n = n; t.h2d = h2d; t.layer_start = 0; t.num_layers = opt_.num_layers; t.engine = kEngineRefshape; t.refshape_ctas = num_ctas;
  for (auto& rk : ranks_) {
    { std::lock_guard<std::mutex> g(rk->mu); rk->q.push_back(t); }
    rk->cv.notify_one();
  }
  return wait(t.ticket);
}

}  // namespace fkv
