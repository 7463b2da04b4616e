// CUDA IPC export/import of device allocations, so that engine worker processes
// can hand their paged KV tensors to the process that runs the data plane
// (reference: flexkv/common/memory_handle.py:466-545, mode "cuda_ipc").
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>
#include <string>

#include "ipc.h"

namespace fkv {

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

static GetAddressRangeFn get_address_range() {
  static GetAddressRangeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<GetAddressRangeFn>(p);
  }();
  return fn;
}

IpcExport ipc_export(uint64_t ptr) {
  IpcExport out;
  GetAddressRangeFn fn = get_address_range();
  if (!fn) throw std::runtime_error("cuMemGetAddressRange is unavailable");
  CUdeviceptr base = 0;
  size_t size = 0;
  if (fn(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) throw std::runtime_error("not a device allocation");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  out.handle.assign(reinterpret_cast<const char*>(&h), sizeof(h));
  out.offset = ptr - (uint64_t)base;
  out.alloc_bytes = size;
  return out;
}

uint64_t ipc_import(const std::string& handle, int device) {
  if (handle.size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  cudaError_t e = cudaSetDevice(device);
  void* p = nullptr;
  if (e == cudaSuccess) e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
  }
  return (uint64_t)(uintptr_t)p;
}

void ipc_close(uint64_t base_ptr, int device) {
  if (cudaSetDevice(device) == cudaSuccess) (void)cudaIpcCloseMemHandle((void*)(uintptr_t)base_ptr);
  (void)cudaGetLastError();
}

}  // namespace fkv
