#include "ptr_table.h"

#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

namespace fkv {

namespace {
struct Entry {
  std::unique_ptr<uint64_t[]> host;
  uint64_t* dev = nullptr;
};
std::mutex g_mu;
std::map<std::pair<int, std::vector<uint64_t>>, Entry>& cache() {
  static auto* m = new std::map<std::pair<int, std::vector<uint64_t>>, Entry>();   // never destroyed: kernels may be in flight at exit
  return *m;
}
}  // namespace

PtrTable ptr_table_get(const std::vector<uint64_t>& ptrs, int device) {
  if (ptrs.empty() || (int64_t)ptrs.size() > kMaxGpuPtrsExt)
    throw std::invalid_argument("tensor table: " + std::to_string(ptrs.size()) + " entries (1.." +
                                std::to_string(kMaxGpuPtrsExt) + " supported)");
  std::lock_guard<std::mutex> g(g_mu);
  auto key = std::make_pair(device, ptrs);
  auto it = cache().find(key);
  if (it == cache().end()) {
    Entry e;
    e.host.reset(new uint64_t[ptrs.size()]);
    for (size_t i = 0; i < ptrs.size(); ++i) e.host[i] = ptrs[i];
    if (device >= 0) {
      int prev = -1;
      cudaError_t err = cudaGetDevice(&prev);
      if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
      if (err == cudaSuccess) err = cudaMalloc((void**)&e.dev, ptrs.size() * sizeof(uint64_t));
      if (err == cudaSuccess)
        err = cudaMemcpy(e.dev, e.host.get(), ptrs.size() * sizeof(uint64_t), cudaMemcpyHostToDevice);
      if (prev >= 0 && prev != device) (void)cudaSetDevice(prev);
      if (err != cudaSuccess) {
        (void)cudaGetLastError();
        if (e.dev) (void)cudaFree(e.dev);
        throw std::runtime_error(std::string("tensor table upload: ") + cudaGetErrorString(err));
      }
    }
    it = cache().emplace(std::move(key), std::move(e)).first;
  }
  PtrTable t;
  t.host = it->second.host.get();
  t.exec = device >= 0 ? it->second.dev : it->second.host.get();
  t.n = (int32_t)ptrs.size();
  return t;
}

void kv_set_gpu_table(KvCopyParams& p, const std::vector<uint64_t>& ptrs, int device) {
  p.num_gpu_ptrs = (int32_t)ptrs.size();
  p.gpu_ptrs_ext = p.gpu_ptrs_ext_host = nullptr;
  if ((int)ptrs.size() <= kMaxGpuPtrs) {
    for (size_t i = 0; i < ptrs.size(); ++i) p.gpu_ptrs[i] = ptrs[i];
    return;
  }
  const PtrTable t = ptr_table_get(ptrs, device);
  p.gpu_ptrs_ext = t.exec;
  p.gpu_ptrs_ext_host = t.host;
}

void kv_set_c_table(KvCopyParams& p, const std::vector<uint64_t>& ptrs, int device) {
  p.num_c_ptrs = (int32_t)ptrs.size();
  p.c_ptrs_ext = p.c_ptrs_ext_host = nullptr;
  if ((int)ptrs.size() <= kMaxGpuPtrs) {
    for (size_t i = 0; i < ptrs.size(); ++i) p.c_ptrs[i] = ptrs[i];
    return;
  }
  const PtrTable t = ptr_table_get(ptrs, device);
  p.c_ptrs_ext = t.exec;
  p.c_ptrs_ext_host = t.host;
}

int64_t ptr_table_cache_size() {
  std::lock_guard<std::mutex> g(g_mu);
  return (int64_t)cache().size();
}

}  // namespace fkv
