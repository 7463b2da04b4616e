// See kv_copy_noalloc.h. The scratch of the layer-major copy kernel (one
// completion counter per layer) lives in a file-scope device array here, so the
// entry point never allocates.
#include "kv_copy_noalloc.h"
#include "layer_sync.h"

#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda_runtime.h>

#include "kv_copy.h"

namespace {

// Per-layer completion counters of the copy kernel. Every GPU that loads this
// library holds its own copy of the array until the process exits.
static __device__ __align__(256) uint32_t g_layer_counters[FKV_NOALLOC_MAX_LAYERS];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
uint32_t* g_counters_on_device[kMaxDevices];   // device address of g_layer_counters, per device; null = not set up

void set_error(char* buf, int len, const char* msg) {
  if (buf && len > 0) snprintf(buf, (size_t)len, "%s", msg);
}

// In host code the name g_layer_counters is only a stand-in for the symbol, not
// an address a kernel can use: the device address has to be asked for, once per
// device, while that device is current.
cudaError_t counters_for_current_device(uint32_t** out, int* device_out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(g_setup_mu);
  if (g_counters_on_device[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_layer_counters);
    if (e != cudaSuccess) return e;
    g_counters_on_device[dev] = static_cast<uint32_t*>(p);
  }
  *out = g_counters_on_device[dev];
  *device_out = dev;
  return cudaSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int fkv_layerwise_copy_noalloc(const FkvNoAllocArgs* a, void* stream_v, char* errbuf, int errbuf_len) {
  if (a == nullptr) { set_error(errbuf, errbuf_len, "null argument block"); return -1; }
  if (a->num_layers <= 0 || a->num_layers > FKV_NOALLOC_MAX_LAYERS) {
    char msg[160];
    snprintf(msg, sizeof(msg), "num_layers = %d is outside 1..%d, the capacity of the built-in scratch array",
             a->num_layers, FKV_NOALLOC_MAX_LAYERS);
    set_error(errbuf, errbuf_len, msg);
    return -1;
  }
  if (a->num_gpu_ptrs <= 0 || a->num_gpu_ptrs > FKV_NOALLOC_MAX_PTRS || a->gpu_ptrs == nullptr) {
    set_error(errbuf, errbuf_len, "gpu_ptrs must hold between 1 and 256 tensor addresses");
    return -1;
  }
  if (a->num_pairs < 0 || a->kv_dim <= 0 || a->chunk_bytes <= 0 || (a->num_pairs > 0 && (!a->gpu_blocks || !a->cpu_blocks))) {
    set_error(errbuf, errbuf_len, "bad work description (pairs, kv_dim, chunk_bytes or block id arrays)");
    return -1;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // Every argument check comes before the first CUDA call, so a rejected call has queued nothing.
  fkv::KvCopyParams p;
  std::memset(&p, 0, sizeof(p));
  for (int i = 0; i < a->num_gpu_ptrs; ++i) p.gpu_ptrs[i] = a->gpu_ptrs[i];
  p.num_gpu_ptrs = a->num_gpu_ptrs;
  p.idx_layer_mul = a->idx_layer_mul;
  p.idx_kv_mul = a->idx_kv_mul;
  p.g_layer_stride = a->g_layer_stride;
  p.g_kv_stride = a->g_kv_stride;
  p.g_block_stride = a->g_block_stride;
  p.cpu_base = a->cpu_base;
  p.c_layer_stride = a->c_layer_stride;
  p.c_kv_stride = a->c_kv_stride;
  p.c_block_stride = a->c_block_stride;
  p.c_off = a->c_off;
  p.gpu_blocks = a->gpu_blocks;
  p.cpu_blocks = a->cpu_blocks;
  p.num_pairs = a->num_pairs;
  p.layer_start = 0;
  p.num_layers = a->num_layers;
  p.kv_dim = a->kv_dim;
  p.chunk_bytes = a->chunk_bytes;
  p.gpu_num_blocks = a->gpu_num_blocks;
  p.cpu_num_blocks = a->cpu_num_blocks;
  p.status = a->status;
  p.h2d = 1;
  p.dev_flags = a->dev_flags;
  p.host_flags = a->host_flags;
  p.epoch = a->epoch;
  p.layer_major = 1;
  if (!fkv::kv_copy_tables_ok(p)) {
    char msg[200];
    snprintf(msg, sizeof(msg), "tensor table too short or holed: layer %d, kv plane %d index entry %lld of %d "
             "(idx_layer_mul %d, idx_kv_mul %d), and every addressed entry must be non-null",
             a->num_layers - 1, a->kv_dim - 1,
             (long long)(a->num_layers - 1) * a->idx_layer_mul + (long long)(a->kv_dim - 1) * a->idx_kv_mul,
             a->num_gpu_ptrs, a->idx_layer_mul, a->idx_kv_mul);
    set_error(errbuf, errbuf_len, msg);
    return -1;
  }
  if (!fkv::kv_copy_tma_eligible(p)) {
    set_error(errbuf, errbuf_len, "addresses, strides and chunk_bytes must be multiples of 16 bytes");
    return -1;
  }
  cudaError_t e;
  if (a->num_pairs == 0) {
    // nothing to copy: release whoever waits on the layer flags, in stream order, as the ordinary path does
    e = cudaSuccess;
    if (a->dev_flags) e = fkv::launch_set_flags(a->dev_flags, a->num_layers, a->epoch, stream);
    if (e == cudaSuccess && a->host_flags) e = fkv::launch_set_flags(a->host_flags, a->num_layers, a->epoch, stream);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      set_error(errbuf, errbuf_len, cudaGetErrorString(e));
      return (int)e;
    }
    return 0;
  }
  uint32_t* counters = nullptr;
  int dev = -1;
  e = counters_for_current_device(&counters, &dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error(errbuf, errbuf_len, cudaGetErrorString(e));
    return (int)e;
  }
  // the array keeps whatever the previous call left: start from zero
  e = cudaMemsetAsync(counters, 0, (size_t)a->num_layers * sizeof(uint32_t), stream);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error(errbuf, errbuf_len, cudaGetErrorString(e));
    return (int)e;
  }
  p.done_counter = counters;
  fkv::KvCopyLaunch cfg{a->num_ctas > 0 ? a->num_ctas : 8, a->tile_bytes > 0 ? a->tile_bytes : 16384, 0};
  e = fkv::launch_kv_copy(p, cfg, stream);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error(errbuf, errbuf_len, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
