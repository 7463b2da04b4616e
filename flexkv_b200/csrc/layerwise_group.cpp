#include "layerwise_group.h"

#include "kernels/kv_compress.h"

#include <cuda.h>

#include <sys/eventfd.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <stdexcept>

namespace fkv {

NotifyMode parse_notify_mode(const std::string& s) {
  if (s == "hostfunc") return NotifyMode::HOSTFUNC;
  if (s == "polling") return NotifyMode::POLLING;
  if (s == "flag") return NotifyMode::FLAG;
  throw std::invalid_argument("unknown layerwise notify mode: " + s);
}

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

// cuStreamWaitValue32 through the runtime's driver-entry lookup (no link against libcuda)
typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
static StreamWaitValue32Fn stream_wait_value32() {
  static StreamWaitValue32Fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<StreamWaitValue32Fn>(p);
  }();
  return fn;
}

LayerwiseGroup::LayerwiseGroup(std::vector<GpuSide> gpus, HostSide host, LayerwiseOptions opt)
    : gpus_(std::move(gpus)), host_(host), opt_(opt) {
  start_ranks();
}

LayerwiseGroup::LayerwiseGroup(std::vector<LayerwiseMemberGroup> groups, std::vector<std::vector<LayerMember>> members,
                               HostSide host_block, LayerwiseOptions opt)
    : host_(host_block), mgroups_(std::move(groups)), members_(std::move(members)), opt_(opt) {
  if (mgroups_.empty() || members_.empty()) throw std::invalid_argument("LayerwiseGroup: no layer groups or no layers");
  const size_t R = mgroups_[0].gpus.size();
  for (const auto& g : mgroups_) {
    if (g.gpus.size() != R || R == 0) throw std::invalid_argument("LayerwiseGroup: every group needs one GPU side per rank");
    for (size_t r = 0; r < R; ++r)
      if (g.gpus[r].device != mgroups_[0].gpus[r].device)
        throw std::invalid_argument("LayerwiseGroup: a rank's groups live on different devices");
  }
  std::vector<std::vector<uint8_t>> seen;
  for (const auto& g : mgroups_) seen.emplace_back((size_t)g.group.num_layers, 0);
  for (const auto& layer : members_)
    for (const LayerMember& m : layer) {
      if (m.group < 0 || m.group >= (int)mgroups_.size() || m.local_layer < 0 ||
          m.local_layer >= mgroups_[(size_t)m.group].group.num_layers)
        throw std::invalid_argument("LayerwiseGroup: layer member out of range");
      if (seen[(size_t)m.group][(size_t)m.local_layer]++)
        throw std::invalid_argument("LayerwiseGroup: a group layer is a member of two model layers");
    }
  for (size_t g = 0; g < seen.size(); ++g)
    for (uint8_t s : seen[g])
      if (!s) throw std::invalid_argument("LayerwiseGroup: a group layer belongs to no model layer and would never be restored");
  gpus_ = mgroups_[0].gpus;                 // devices and rank count
  opt_.group.num_layers = (int)members_.size();
  opt_.layers_per_batch = 1;                // one model layer per signal; members are separate launches
  start_ranks();
}

void LayerwiseGroup::start_ranks() {
  if (gpus_.empty()) throw std::invalid_argument("LayerwiseGroup: no GPUs");
  if (opt_.num_counters < 1 || opt_.layers_per_batch < -1) throw std::invalid_argument("LayerwiseGroup: bad options");
  const int L = opt_.group.num_layers, R = (int)gpus_.size(), C = opt_.num_counters;
  epochs_.assign((size_t)C, 0);
  reserved_.assign((size_t)C, 0);
  launched_.assign((size_t)C * gpus_.size(), 0);
  counter_status_.reset(new std::atomic<int>[(size_t)C]);
  for (int i = 0; i < C; ++i) counter_status_[(size_t)i].store(0);
  if (opt_.create_eventfds) {
    eventfds_.assign((size_t)C * R * L, -1);
    for (auto& fd : eventfds_) {
      fd = eventfd(0, EFD_NONBLOCK | EFD_SEMAPHORE);
      if (fd < 0) throw std::runtime_error(std::string("eventfd: ") + strerror(errno));
    }
  }
  check(cudaSetDevice(gpus_[0].device), "cudaSetDevice");
  check(cudaHostAlloc((void**)&id_ring_, 2 * (size_t)opt_.group.max_blocks_per_op * sizeof(int64_t),
                      cudaHostAllocPortable | cudaHostAllocMapped),
        "cudaHostAlloc(id ring)");
  const int lpb = opt_.layers_per_batch > 0 ? opt_.layers_per_batch : (opt_.layers_per_batch < 0 ? 1 : L);
  const int batches = (L + lpb - 1) / lpb;
  for (int r = 0; r < R; ++r)
    for (int c = 0; c < C; ++c)
      for (int b = 0; b < batches; ++b) {
        auto a = std::make_unique<HostFnArg>();
        a->self = this; a->rank = r; a->counter = c;
        a->layer_lo = b * lpb;
        a->layer_hi = std::min(L, a->layer_lo + lpb);
        fn_args_.push_back(std::move(a));
      }
  for (int r = 0; r < R; ++r) ranks_.emplace_back(new Rank());
  for (int r = 0; r < R; ++r) ranks_[(size_t)r]->th = std::thread([this, r] { rank_main(r); });
  for (auto& rk : ranks_) {
    std::unique_lock<std::mutex> lk(rk->mu);
    rk->cv.wait(lk, [&] { return rk->ready; });
    if (!rk->init_error.empty()) {
      std::string msg = rk->init_error;
      lk.unlock();
      stop_ = true;
      for (auto& x : ranks_) { x->cv.notify_all(); if (x->th.joinable()) x->th.join(); }
      throw std::runtime_error("LayerwiseGroup: " + msg);
    }
  }
}

LayerwiseGroup::~LayerwiseGroup() {
  stop_ = true;
  for (auto& rk : ranks_) {
    { std::lock_guard<std::mutex> g(rk->mu); }
    rk->cv.notify_all();
  }
  for (auto& rk : ranks_) if (rk->th.joinable()) rk->th.join();
  for (int fd : eventfds_) if (fd >= 0) close(fd);
  if (id_ring_) cudaFreeHost(id_ring_);
}

int LayerwiseGroup::eventfd_of(int counter, int rank, int layer) const {
  if (eventfds_.empty()) return -1;
  const int L = opt_.group.num_layers, R = (int)gpus_.size();
  return eventfds_[((size_t)counter * R + rank) * L + layer];
}

void LayerwiseGroup::set_eventfd(int counter, int rank, int layer, int fd) {
  const int L = opt_.group.num_layers, R = (int)gpus_.size(), C = opt_.num_counters;
  if (counter < 0 || counter >= C || rank < 0 || rank >= R || layer < 0 || layer >= L)
    throw std::out_of_range("LayerwiseGroup::set_eventfd: index out of range");
  std::lock_guard<std::mutex> api(api_mu_);
  if (eventfds_.empty()) eventfds_.assign((size_t)C * R * L, -1);
  int& slot = eventfds_[((size_t)counter * R + rank) * L + layer];
  if (slot >= 0) close(slot);
  slot = dup(fd);
  if (slot < 0) throw std::runtime_error(std::string("dup(eventfd): ") + strerror(errno));
}

uint64_t LayerwiseGroup::device_flags_ptr(int rank, int counter) const {
  return (uint64_t)(uintptr_t)(ranks_.at((size_t)rank)->dev_flags + (size_t)counter * opt_.group.num_layers);
}
uint64_t LayerwiseGroup::host_flags_ptr(int rank, int counter) const {
  return (uint64_t)(uintptr_t)(ranks_.at((size_t)rank)->host_flags + (size_t)counter * opt_.group.num_layers);
}

uint32_t LayerwiseGroup::epoch_of(int counter) {
  std::lock_guard<std::mutex> g(epoch_mu_);
  return epochs_.at((size_t)counter);
}

uint32_t LayerwiseGroup::begin_restore(int counter) {
  if (counter < 0 || counter >= opt_.num_counters) throw std::invalid_argument("LayerwiseGroup: bad counter id");
  std::lock_guard<std::mutex> g(epoch_mu_);
  if (!reserved_[(size_t)counter]) {
    reserved_[(size_t)counter] = 1;
    ++epochs_[(size_t)counter];
  }
  return epochs_[(size_t)counter];
}

void LayerwiseGroup::mark_launched(int r, const Job& j) {
  {
    std::lock_guard<std::mutex> g(launched_mu_);
    launched_[(size_t)j.counter * gpus_.size() + (size_t)r] = j.epoch;
  }
  launched_cv_.notify_all();
}

bool LayerwiseGroup::wait_launched(int counter, uint32_t epoch, int timeout_ms) {
  if (counter < 0 || counter >= opt_.num_counters) throw std::invalid_argument("LayerwiseGroup: bad counter id");
  std::unique_lock<std::mutex> lk(launched_mu_);
  const size_t R = gpus_.size();
  return launched_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] {
    for (size_t r = 0; r < R; ++r)
      if ((int32_t)(launched_[(size_t)counter * R + r] - epoch) < 0) return false;
    return true;
  });
}

cudaError_t LayerwiseGroup::stream_wait_layer(int rank, int counter, int layer, cudaStream_t stream, uint32_t epoch) {
  Rank& rk = *ranks_.at((size_t)rank);
  if (counter < 0 || counter >= opt_.num_counters || layer < 0 || layer >= opt_.group.num_layers)
    return cudaErrorInvalidValue;
  if (epoch == 0) {
    std::lock_guard<std::mutex> g(epoch_mu_);
    epoch = epochs_[(size_t)counter];
  }
  // Every launch form publishes the device flag, so the wait is on the flag's value: an event wait would bind to
  // whatever record of the per-layer event was last queued, i.e. to the previous restore when the consumer runs ahead.
  StreamWaitValue32Fn fn = stream_wait_value32();
  if (fn == nullptr) return cudaErrorNotSupported;
  uint32_t* flag = rk.dev_flags + (size_t)counter * opt_.group.num_layers + layer;
  const CUresult r = fn((CUstream)stream, (CUdeviceptr)(uintptr_t)flag, epoch, CU_STREAM_WAIT_VALUE_GEQ);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorUnknown;
}

void LayerwiseGroup::notify(int rank, int counter, int layer_lo, int layer_hi) {
  if (eventfds_.empty()) return;
  const uint64_t v = 1;
  for (int l = layer_lo; l < layer_hi; ++l) {
    const int fd = eventfd_of(counter, rank, l);
    if (fd >= 0) { ssize_t w = write(fd, &v, sizeof(v)); (void)w; }
  }
}

bool LayerwiseGroup::status_words_set(const volatile int32_t* words) {
  for (int b = 0; b < kStatusWords; ++b)
    if (words[b]) return true;
  return false;
}

void LayerwiseGroup::release_waiters(int r, const Job& j, int from_layer, int status) {
  Rank& rk = *ranks_[(size_t)r];
  const int L = opt_.group.num_layers;
  counter_status_[(size_t)j.counter].store(status ? status : -1, std::memory_order_release);
  mark_launched(r, j);      // nothing more will be queued for this epoch
  if (from_layer >= L) return;
  uint32_t* hflags = rk.host_flags + (size_t)j.counter * L;
  for (int l = from_layer; l < L; ++l) __atomic_store_n(hflags + l, j.epoch, __ATOMIC_RELEASE);
  // device flags from the host, on the side stream: the copy stream may hold the failed work
  if (rk.dev_flags != nullptr && rk.notify_stream != nullptr) {
    cudaError_t e = cudaMemcpyAsync(rk.dev_flags + (size_t)j.counter * L + from_layer, hflags + from_layer,
                                    (size_t)(L - from_layer) * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                    rk.notify_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rk.notify_stream);
    if (e != cudaSuccess) (void)cudaGetLastError();
  }
  notify(r, j.counter, from_layer, L);
}

void CUDART_CB LayerwiseGroup::host_fn(void* arg) {
  auto* a = static_cast<HostFnArg*>(arg);
  // a kernel that gave up has written its status words before it released the layers it did not restore:
  // make the failure visible to whoever this wake-up releases
  if (status_words_set(a->self->ranks_[(size_t)a->rank]->status))
    a->self->counter_status_[(size_t)a->counter].store(-1, std::memory_order_release);
  a->self->notify(a->rank, a->counter, a->layer_lo, a->layer_hi);
}

void LayerwiseGroup::rank_main(int r) {
  Rank& rk = *ranks_[(size_t)r];
  const int L = opt_.group.num_layers, C = opt_.num_counters;
  try {
    check(cudaSetDevice(gpus_[(size_t)r].device), "cudaSetDevice");
    int lo = 0, hi = 0;
    check(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
    check(cudaStreamCreateWithPriority(&rk.stream, cudaStreamNonBlocking, hi), "cudaStreamCreateWithPriority");
    check(cudaStreamCreateWithFlags(&rk.notify_stream, cudaStreamNonBlocking), "cudaStreamCreate(notify)");
    check(cudaMalloc((void**)&rk.dev_flags, (size_t)C * L * sizeof(uint32_t)), "cudaMalloc(flags)");
    check(cudaMemset(rk.dev_flags, 0, (size_t)C * L * sizeof(uint32_t)), "cudaMemset(flags)");
    check(cudaMalloc((void**)&rk.done_counter, (size_t)L * sizeof(uint32_t)), "cudaMalloc(counter)");
    check(cudaMemset(rk.done_counter, 0, (size_t)L * sizeof(uint32_t)), "cudaMemset(counter)");
    check(cudaMalloc((void**)&rk.dev_ids, 2 * (size_t)opt_.group.max_blocks_per_op * sizeof(int64_t)), "cudaMalloc(ids)");
    check(cudaHostAlloc((void**)&rk.host_flags, (size_t)C * L * sizeof(uint32_t),
                        cudaHostAllocPortable | cudaHostAllocMapped), "cudaHostAlloc(flags)");
    std::memset(rk.host_flags, 0, (size_t)C * L * sizeof(uint32_t));
    check(cudaHostAlloc((void**)&rk.status, kStatusWords * sizeof(int32_t),
                        cudaHostAllocPortable | cudaHostAllocMapped), "cudaHostAlloc(status)");
    std::memset(rk.status, 0, kStatusWords * sizeof(int32_t));
    rk.layer_ev.resize((size_t)C * L);
    for (auto& e : rk.layer_ev) check(cudaEventCreate(&e), "cudaEventCreate");
    check(cudaEventCreate(&rk.ev_begin), "cudaEventCreate");
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  } catch (const std::exception& e) {
    std::lock_guard<std::mutex> g(rk.mu);
    rk.init_error = e.what();
    rk.ready = true;
    rk.cv.notify_all();
    return;
  }
  { std::lock_guard<std::mutex> g(rk.mu); rk.ready = true; }
  rk.cv.notify_all();
  for (;;) {
    Job j;
    {
      std::unique_lock<std::mutex> lk(rk.mu);
      rk.cv.wait(lk, [&] { return stop_.load() || !rk.q.empty(); });
      if (rk.q.empty() && stop_.load()) break;
      j = rk.q.front();
      rk.q.pop_front();
    }
    run_job(r, j);
    { std::lock_guard<std::mutex> g(done_mu_); rk.done = true; }
    done_cv_.notify_all();
  }
  for (auto& e : rk.layer_ev) cudaEventDestroy(e);
  if (rk.ev_begin) cudaEventDestroy(rk.ev_begin);
  if (rk.dev_flags) cudaFree(rk.dev_flags);
  if (rk.done_counter) cudaFree(rk.done_counter);
  if (rk.dev_ids) cudaFree(rk.dev_ids);
  if (rk.host_flags) cudaFreeHost(rk.host_flags);
  if (rk.status) cudaFreeHost(rk.status);
  if (rk.stream) cudaStreamDestroy(rk.stream);
  if (rk.notify_stream) cudaStreamDestroy(rk.notify_stream);
}

void LayerwiseGroup::update_gpu_ptrs(int rank, const std::vector<uint64_t>& ptrs) {
  if ((int)ptrs.size() > kMaxGpuPtrsExt) throw std::invalid_argument("too many GPU tensors");
  std::lock_guard<std::mutex> api(api_mu_);
  gpus_.at((size_t)rank).ptrs = ptrs;
}

void LayerwiseGroup::update_group_gpu_ptrs(int group, int rank, const std::vector<uint64_t>& ptrs) {
  if ((int)ptrs.size() > kMaxGpuPtrsExt) throw std::invalid_argument("too many GPU tensors");
  std::lock_guard<std::mutex> api(api_mu_);
  mgroups_.at((size_t)group).gpus.at((size_t)rank).ptrs = ptrs;
}

// Copies a job's block ids from the mapped host ring into device memory, in stream order before the launches
// that read them. A layer-major walk touches a new 32-id window every few tiles; fetched from host memory each of
// those reads would wait behind the bulk reads already queued on the link.
cudaError_t LayerwiseGroup::stage_ids(Rank& rk, const Job& j, const int64_t*& gpu_ids, const int64_t*& cpu_ids) {
  if (j.n <= 0 || rk.dev_ids == nullptr) return cudaSuccess;
  const size_t half = (size_t)opt_.group.max_blocks_per_op;
  cudaError_t err = cudaMemcpyAsync(rk.dev_ids, j.gpu_blocks, (size_t)j.n * sizeof(int64_t), cudaMemcpyHostToDevice,
                                    rk.stream);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(rk.dev_ids + half, j.cpu_blocks, (size_t)j.n * sizeof(int64_t), cudaMemcpyHostToDevice,
                          rk.stream);
  if (err == cudaSuccess) {
    gpu_ids = rk.dev_ids;
    cpu_ids = rk.dev_ids + half;
  }
  return err;
}

// Multi-group restore of one rank: model layer by model layer, one launch per member; the last
// member's launch carries the completion signal of the model layer (same stream, so the earlier
// members have landed when its last CTA publishes the flag).
void LayerwiseGroup::run_job_members(int r, const Job& j) {
  Rank& rk = *ranks_[(size_t)r];
  const int L = (int)members_.size(), R = (int)gpus_.size();
  rk.res_status = 0;
  rk.res_layer_ms.assign((size_t)L, 0.f);
  if (j.fail_status) {
    release_waiters(r, j, 0, j.fail_status);
    rk.res_status = j.fail_status;
    rk.res_ms = 0.f;
    return;
  }
  int queued_upto = 0, notified_upto = 0;   // layers whose signal is queued on the side stream / already sent
  cudaEvent_t* ev = rk.layer_ev.data() + (size_t)j.counter * L;
  uint32_t* hflags = rk.host_flags + (size_t)j.counter * L;
  uint32_t* dflags = rk.dev_flags + (size_t)j.counter * L;
  cudaError_t err = cudaEventRecord(rk.ev_begin, rk.stream);
  const int64_t* gpu_ids = j.gpu_blocks;
  const int64_t* cpu_ids = j.cpu_blocks;
  if (err == cudaSuccess) err = stage_ids(rk, j, gpu_ids, cpu_ids);
  for (int l = 0; l < L && err == cudaSuccess; ++l) {
    const auto& ms = members_[(size_t)l];
    bool signalled = false;
    for (size_t k = 0; k < ms.size() && err == cudaSuccess && j.n > 0; ++k) {
      const LayerwiseMemberGroup& g = mgroups_[(size_t)ms[k].group];
      KvCopyParams p;
      bool skip = false;
      fill_kv_params(g.gpus[(size_t)r], g.host, g.group, r, R, gpu_ids, cpu_ids, j.n, true,
                     ms[k].local_layer, 1, 0, p, skip);
      p.status = rk.status;
      if (k + 1 == ms.size()) {
        // the kernel publishes flag word [layer_start]: bias the arrays so that this is model layer l
        const intptr_t bias = ((intptr_t)l - (intptr_t)ms[k].local_layer) * (intptr_t)sizeof(uint32_t);
        p.done_counter = rk.done_counter;
        p.dev_flags = reinterpret_cast<uint32_t*>((intptr_t)dflags + bias);
        p.host_flags = reinterpret_cast<uint32_t*>((intptr_t)hflags + bias);
        p.epoch = j.epoch;
        signalled = true;
      }
      err = launch_kv_copy(p, opt_.group.h2d, rk.stream);
    }
    if (!signalled && err == cudaSuccess) {
      // a layer without members, or an empty restore: publish from the host, in stream order
      hflags[l] = j.epoch;
      err = cudaMemcpyAsync(dflags + l, hflags + l, sizeof(uint32_t), cudaMemcpyHostToDevice, rk.stream);
    }
    if (err == cudaSuccess) err = cudaEventRecord(ev[l], rk.stream);
    if (err == cudaSuccess && opt_.notify == NotifyMode::HOSTFUNC) {
      HostFnArg* a = fn_args_[((size_t)r * opt_.num_counters + j.counter) * L + l].get();
      err = cudaStreamWaitEvent(rk.notify_stream, ev[l], 0);
      if (err == cudaSuccess) err = cudaLaunchHostFunc(rk.notify_stream, host_fn, a);
      if (err == cudaSuccess) queued_upto = l + 1;
    }
  }
  bool kernel_failed = false;
  mark_launched(r, j);      // every launch of this rank is queued: consumers may queue their stream waits now
  if (err == cudaSuccess && opt_.notify != NotifyMode::HOSTFUNC) {
    const auto t0 = std::chrono::steady_clock::now();
    for (int l = 0; l < L && err == cudaSuccess && !kernel_failed; ++l) {
      for (;;) {
        // events in both modes: a host-published flag of an empty layer is set before the stream reaches it
        cudaError_t q = cudaEventQuery(ev[l]);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) { err = q; break; }
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(120)) { err = cudaErrorTimeout; break; }
      }
      if (err != cudaSuccess) break;
      // a kernel that gave up has written its status words before the flags of the layers it did not restore
      if (status_words_set(rk.status)) { kernel_failed = true; break; }
      notify(r, j.counter, l, l + 1);
      notified_upto = l + 1;
    }
  }
  if (err == cudaSuccess) err = cudaStreamSynchronize(rk.stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(rk.notify_stream);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    (void)cudaStreamSynchronize(rk.notify_stream);   // callbacks already queued run first
    (void)cudaGetLastError();
    rk.res_status = -(int)err;
    rk.res_ms = 0.f;
    release_waiters(r, j, std::max(queued_upto, notified_upto), rk.res_status);
    return;
  }
  rk.res_status = collect_status(rk.status);
  if (rk.res_status != 0) {
    release_waiters(r, j, std::max(queued_upto, notified_upto), rk.res_status);
    rk.res_ms = 0.f;
    return;
  }
  counter_status_[(size_t)j.counter].store(0, std::memory_order_release);
  for (int l = 0; l < L; ++l) cudaEventElapsedTime(&rk.res_layer_ms[(size_t)l], rk.ev_begin, ev[l]);
  rk.res_ms = rk.res_layer_ms[(size_t)L - 1];
}

void LayerwiseGroup::run_job(int r, const Job& j) {
  if (!mgroups_.empty()) {
    run_job_members(r, j);
    return;
  }
  Rank& rk = *ranks_[(size_t)r];
  const int L = opt_.group.num_layers, R = (int)gpus_.size();
  // adaptive mode: a fused launch saves L-1 launches and wins at every size once the grid has
  // enough single-warp CTAs to keep the link busy (measured on B200, 2 MiB / 32 MiB / 320 MiB:
  // 8 CTAs 0.165 / 1.03 / 8.32 ms fused against 0.217 / 1.31 / 8.87 ms per layer; 4 CTAs 0.119 /
  // 1.11 / 10.9 against 0.21 / 1.33 / 8.93). Narrow grids keep one launch per layer above fused_max_bytes.
  const int64_t job_bytes = j.n * (int64_t)L * opt_.group.kv_dim * opt_.group.chunk_bytes;
  const bool wide_grid = opt_.group.h2d.num_ctas >= 8;
  const bool fused = opt_.layers_per_batch == 0 ||
                     (opt_.layers_per_batch < 0 && (wide_grid || job_bytes <= opt_.fused_max_bytes));
  const int B = fused ? L : (opt_.layers_per_batch > 0 ? opt_.layers_per_batch : 1);
  const int batches = (L + B - 1) / B;
  const auto t_begin = std::chrono::steady_clock::now();
  rk.res_status = 0;
  rk.res_layer_ms.assign((size_t)L, 0.f);
  if (j.fail_status) {
    release_waiters(r, j, 0, j.fail_status);
    rk.res_status = j.fail_status;
    rk.res_ms = 0.f;
    return;
  }
  int queued_upto = 0, notified_upto = 0;   // layers whose signal is queued on the side stream / already sent
  bool kernel_failed = false;
  cudaEvent_t* ev = rk.layer_ev.data() + (size_t)j.counter * L;
  uint32_t* hflags = rk.host_flags + (size_t)j.counter * L;
  cudaError_t err = cudaEventRecord(rk.ev_begin, rk.stream);
  const int64_t* gpu_ids = j.gpu_blocks;
  const int64_t* cpu_ids = j.cpu_blocks;
  if (err == cudaSuccess) err = stage_ids(rk, j, gpu_ids, cpu_ids);
  for (int b = 0; b < batches && err == cudaSuccess; ++b) {
    const int l0 = b * B, l1 = std::min(L, l0 + B);
    KvCopyParams p;
    bool skip = false;
    fill_kv_params(gpus_[(size_t)r], host_, opt_.group, r, R, gpu_ids, cpu_ids, j.n, true, l0, l1 - l0, 0,
                   p, skip);
    p.status = rk.status;
    p.done_counter = rk.done_counter;
    p.dev_flags = rk.dev_flags + (size_t)j.counter * L;
    p.host_flags = hflags;
    p.epoch = j.epoch;
    p.layer_major = fused ? 1 : 0;
    if (j.n > 0) {
      if (opt_.size_table != nullptr)
        err = launch_kv_compress_bf16(p, opt_.size_table + (int64_t)r * opt_.size_table_rank_entries,
                                      opt_.size_table_layers, opt_.codec_pipelines, rk.stream);
      else
        err = launch_kv_copy(p, opt_.group.h2d, rk.stream);
    } else {
      // nothing to restore: publish the flags from the host so waiters are released at once
      for (int l = l0; l < l1; ++l) hflags[l] = j.epoch;
      err = cudaMemcpyAsync(rk.dev_flags + (size_t)j.counter * L + l0, hflags + l0, (size_t)(l1 - l0) * 4,
                            cudaMemcpyHostToDevice, rk.stream);
    }
    for (int l = l0; l < l1 && err == cudaSuccess; ++l) err = cudaEventRecord(ev[l], rk.stream);
    if (err == cudaSuccess && opt_.notify == NotifyMode::HOSTFUNC && !fused) {
      // the callback runs on a side stream behind the layer's event, so the copy stream never waits for the host
      HostFnArg* a = fn_args_[((size_t)r * opt_.num_counters + j.counter) * batches + b].get();
      err = cudaStreamWaitEvent(rk.notify_stream, ev[l1 - 1], 0);
      if (err == cudaSuccess) err = cudaLaunchHostFunc(rk.notify_stream, host_fn, a);
      if (err == cudaSuccess) queued_upto = l1;
    }
  }
  mark_launched(r, j);      // every launch of this rank is queued: consumers may queue their stream waits now
  if (err == cudaSuccess && (opt_.notify != NotifyMode::HOSTFUNC || fused)) {
    // retire in order from this thread; a fused launch is watched layer by layer through the mapped flags
    const auto t0 = std::chrono::steady_clock::now();
    const int units = fused ? L : batches;
    for (int b = 0; b < units; ++b) {
      const int l0 = fused ? b : b * B, l1 = fused ? b + 1 : std::min(L, l0 + B);
      for (;;) {
        bool ready;
        if (opt_.notify == NotifyMode::POLLING && !fused) {
          cudaError_t q = cudaEventQuery(ev[l1 - 1]);
          if (q != cudaSuccess && q != cudaErrorNotReady) { err = q; break; }
          ready = q == cudaSuccess;
        } else {
          ready = __atomic_load_n(hflags + l1 - 1, __ATOMIC_ACQUIRE) == j.epoch;
        }
        if (ready) break;
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(120)) { err = cudaErrorTimeout; break; }
      }
      if (err != cudaSuccess) break;
      // a kernel that gave up has written its status words before the flags of the layers it did not restore
      if (status_words_set(rk.status)) { kernel_failed = true; break; }
      notify(r, j.counter, l0, l1);
      notified_upto = l1;
      if (fused)
        rk.res_layer_ms[(size_t)l0] =
            std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t_begin).count();
    }
  }
  (void)kernel_failed;
  if (err == cudaSuccess) err = cudaStreamSynchronize(rk.stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(rk.notify_stream);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    (void)cudaStreamSynchronize(rk.notify_stream);   // callbacks already queued run first
    (void)cudaGetLastError();
    rk.res_status = -(int)err;
    rk.res_ms = 0.f;
    release_waiters(r, j, std::max(queued_upto, notified_upto), rk.res_status);
    return;
  }
  rk.res_status = collect_status(rk.status);
  if (rk.res_status != 0) {
    // the data of some layers is not what was asked for: whoever is still waiting is released with the failure
    release_waiters(r, j, std::max(queued_upto, notified_upto), rk.res_status);
    rk.res_ms = 0.f;
    return;
  }
  counter_status_[(size_t)j.counter].store(0, std::memory_order_release);
  if (!fused) {
    for (int l = 0; l < L; ++l) cudaEventElapsedTime(&rk.res_layer_ms[(size_t)l], rk.ev_begin, ev[l]);
    rk.res_ms = rk.res_layer_ms[(size_t)L - 1];
  } else {
    cudaEventElapsedTime(&rk.res_ms, rk.ev_begin, ev[L - 1]);   // whole launch, CUDA events
  }
}

LayerwiseResult LayerwiseGroup::restore(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n,
                                        int counter_id, SsdIoEngine* ssd, const SsdLayout* ssd_layout,
                                        const int64_t* ssd_src, const int64_t* cpu_dst, int64_t n_disk) {
  if (counter_id < 0 || counter_id >= opt_.num_counters) throw std::invalid_argument("LayerwiseGroup: bad counter id");
  if (n > opt_.group.max_blocks_per_op) throw std::invalid_argument("LayerwiseGroup: op exceeds max_blocks_per_op");
  std::lock_guard<std::mutex> api(api_mu_);
  LayerwiseResult res;
  Job j;
  j.counter = counter_id;
  {
    std::lock_guard<std::mutex> g(epoch_mu_);
    if (reserved_[(size_t)counter_id]) reserved_[(size_t)counter_id] = 0;
    else ++epochs_[(size_t)counter_id];
    j.epoch = epochs_[(size_t)counter_id];
  }
  res.epoch = j.epoch;
  counter_status_[(size_t)counter_id].store(0, std::memory_order_release);
  if (n_disk > 0) {
    if (ssd == nullptr || ssd_layout == nullptr) throw std::invalid_argument("LayerwiseGroup: disk blocks without an SSD engine");
    const auto t0 = std::chrono::steady_clock::now();
    std::vector<uint8_t> ok((size_t)n_disk, 0);
    const int64_t nfail = ssd->transfer(reinterpret_cast<uint8_t*>(host_.base), cpu_dst, ssd_src, n_disk, true,
                                        *ssd_layout, 0, ssd_layout->num_layers_total, ok.data());
    res.disk_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (nfail > 0) j.fail_status = 1 << 29;   // disk stage failed: nothing is copied, every waiter is released
  }
  if (n > 0 && !j.fail_status) {
    std::memcpy(id_ring_, gpu_blocks, (size_t)n * sizeof(int64_t));
    std::memcpy(id_ring_ + opt_.group.max_blocks_per_op, cpu_blocks, (size_t)n * sizeof(int64_t));
  }
  j.n = n;
  j.gpu_blocks = id_ring_;
  j.cpu_blocks = id_ring_ + opt_.group.max_blocks_per_op;
  {
    std::lock_guard<std::mutex> g(done_mu_);
    for (auto& rk : ranks_) rk->done = false;
  }
  for (auto& rk : ranks_) {
    { std::lock_guard<std::mutex> g(rk->mu); rk->q.push_back(j); }
    rk->cv.notify_one();
  }
  {
    std::unique_lock<std::mutex> lk(done_mu_);
    done_cv_.wait(lk, [&] {
      for (auto& rk : ranks_) if (!rk->done) return false;
      return true;
    });
  }
  for (auto& rk : ranks_) {
    if (rk->res_status < 0) res.status = rk->res_status;
    else if (res.status >= 0) res.status |= rk->res_status;
    res.total_ms = std::max(res.total_ms, rk->res_ms);
  }
  res.layer_done_ms = ranks_[0]->res_layer_ms;
  return res;
}

}  // namespace fkv
