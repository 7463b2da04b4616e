#include "peer_copier.h"
#include "ptr_table.h"

#include <cstring>
#include <stdexcept>

namespace fkv {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

PeerCopier::PeerCopier(std::vector<GpuSide> ranks, int num_layers, int kv_dim, int64_t chunk_bytes,
                       KvCopyLaunch launch, int64_t max_blocks_per_op)
    : ranks_(std::move(ranks)), num_layers_(num_layers), kv_dim_(kv_dim), chunk_bytes_(chunk_bytes), launch_(launch),
      max_blocks_(max_blocks_per_op) {
  if (ranks_.empty()) throw std::invalid_argument("PeerCopier: no ranks");
  for (size_t i = 0; i < ranks_.size(); ++i) {
    dst_.emplace_back(new PerDst());
    dst_.back()->peer_ok.assign(ranks_.size(), -1);
  }
}

PeerCopier::~PeerCopier() {
  for (size_t i = 0; i < dst_.size(); ++i) {
    PerDst& d = *dst_[i];
    if (!d.init) continue;
    cudaSetDevice(ranks_[i].device);
    if (d.ev0) cudaEventDestroy(d.ev0);
    if (d.ev1) cudaEventDestroy(d.ev1);
    if (d.stream) cudaStreamDestroy(d.stream);
    if (d.ids) cudaFreeHost(d.ids);
    if (d.status) cudaFreeHost(d.status);
  }
}

void PeerCopier::ensure_init(int r) {
  PerDst& d = *dst_[(size_t)r];
  if (d.init) return;
  check(cudaSetDevice(ranks_[(size_t)r].device), "cudaSetDevice");
  check(cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking), "cudaStreamCreate");
  check(cudaEventCreate(&d.ev0), "cudaEventCreate");
  check(cudaEventCreate(&d.ev1), "cudaEventCreate");
  check(cudaHostAlloc((void**)&d.ids, 2 * (size_t)max_blocks_ * sizeof(int64_t),
                      cudaHostAllocPortable | cudaHostAllocMapped), "cudaHostAlloc(ids)");
  check(cudaHostAlloc((void**)&d.status, kStatusWords * sizeof(int32_t),
                      cudaHostAllocPortable | cudaHostAllocMapped), "cudaHostAlloc(status)");
  std::memset(d.status, 0, kStatusWords * sizeof(int32_t));
  d.init = true;
}

bool PeerCopier::can_access(int dst_rank, int src_rank) {
  PerDst& d = *dst_.at((size_t)dst_rank);
  std::lock_guard<std::mutex> g(d.mu);
  int& ok = d.peer_ok.at((size_t)src_rank);
  if (ok >= 0) return ok == 1;
  const int ddev = ranks_[(size_t)dst_rank].device, sdev = ranks_[(size_t)src_rank].device;
  if (ddev == sdev) { ok = 1; return true; }
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, ddev, sdev) != cudaSuccess || !can) {
    (void)cudaGetLastError();
    ok = 0;
    return false;
  }
  check(cudaSetDevice(ddev), "cudaSetDevice");
  cudaError_t e = cudaDeviceEnablePeerAccess(sdev, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    ok = 0;
    return false;
  }
  (void)cudaGetLastError();
  ok = 1;
  return true;
}

void PeerCopier::update_gpu_ptrs(int rank, const std::vector<uint64_t>& ptrs) {
  if ((int)ptrs.size() > kMaxGpuPtrsExt) throw std::invalid_argument("too many GPU tensors");
  ranks_.at((size_t)rank).ptrs = ptrs;
}

OpResult PeerCopier::pull(int dst_rank, int src_rank, const int64_t* dst_blocks, const int64_t* src_blocks, int64_t n,
                          int layer_start, int num_layers) {
  OpResult res;
  if (n <= 0) return res;
  if (n > max_blocks_) throw std::invalid_argument("PeerCopier: op exceeds max_blocks_per_op");
  if (layer_start < 0 || num_layers < 0 || layer_start + num_layers > num_layers_)
    throw std::invalid_argument("PeerCopier: layer range out of bounds");
  if (!can_access(dst_rank, src_rank)) throw std::runtime_error("PeerCopier: no peer access between the two GPUs");
  PerDst& d = *dst_.at((size_t)dst_rank);
  std::lock_guard<std::mutex> g(d.mu);
  ensure_init(dst_rank);
  const GpuSide& dg = ranks_[(size_t)dst_rank];
  const GpuSide& sg = ranks_[(size_t)src_rank];
  check(cudaSetDevice(dg.device), "cudaSetDevice");
  std::memcpy(d.ids, dst_blocks, (size_t)n * sizeof(int64_t));
  std::memcpy(d.ids + max_blocks_, src_blocks, (size_t)n * sizeof(int64_t));
  KvCopyParams p;
  std::memset(&p, 0, sizeof(p));
  // "gpu" side = local destination, "cpu" side = the peer's tensors; direction = peer -> local
  kv_set_gpu_table(p, dg.ptrs, dg.device);
  p.idx_layer_mul = dg.idx_layer_mul; p.idx_kv_mul = dg.idx_kv_mul;
  p.g_layer_stride = dg.layer_stride; p.g_kv_stride = dg.kv_stride; p.g_block_stride = dg.block_stride;
  kv_set_c_table(p, sg.ptrs, dg.device);      // the peer's addresses, read by the kernel on the local device
  p.c_use_table = 1;
  p.c_idx_layer_mul = sg.idx_layer_mul; p.c_idx_kv_mul = sg.idx_kv_mul;
  p.c_layer_stride = sg.layer_stride; p.c_kv_stride = sg.kv_stride; p.c_block_stride = sg.block_stride;
  p.gpu_blocks = d.ids;
  p.cpu_blocks = d.ids + max_blocks_;
  p.num_pairs = (int32_t)n;
  p.layer_start = layer_start; p.num_layers = num_layers; p.kv_dim = kv_dim_;
  p.chunk_bytes = chunk_bytes_;
  p.gpu_num_blocks = dg.num_blocks; p.cpu_num_blocks = sg.num_blocks;
  p.status = d.status;
  p.h2d = 1;
  cudaEventRecord(d.ev0, d.stream);
  cudaError_t e = launch_kv_copy(p, launch_, d.stream);
  cudaEventRecord(d.ev1, d.stream);
  if (e == cudaSuccess) e = cudaEventSynchronize(d.ev1);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    res.status = -(int)e;
    return res;
  }
  cudaEventElapsedTime(&res.gpu_ms, d.ev0, d.ev1);
  res.status = collect_status(d.status);
  return res;
}

}  // namespace fkv
