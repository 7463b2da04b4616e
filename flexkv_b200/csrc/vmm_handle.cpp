#include "vmm_handle.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>

namespace fkv {
namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
    (void)cudaGetLastError();
    p = nullptr;
  }
  return reinterpret_cast<Fn>(p);
}

using RetainFn = CUresult (*)(CUmemGenericAllocationHandle*, void*);
using ReleaseFn = CUresult (*)(CUmemGenericAllocationHandle);
using ExportFn = CUresult (*)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
using ImportFn = CUresult (*)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
using ReserveFn = CUresult (*)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
using MapFn = CUresult (*)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
using SetAccessFn = CUresult (*)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
using UnmapFn = CUresult (*)(CUdeviceptr, size_t);
using AddressFreeFn = CUresult (*)(CUdeviceptr, size_t);
using CreateFn = CUresult (*)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
using GranularityFn = CUresult (*)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
using PointerAttrFn = CUresult (*)(void*, CUpointer_attribute, CUdeviceptr);
using PropsFromHandleFn = CUresult (*)(CUmemAllocationProp*, CUmemGenericAllocationHandle);

struct Driver {
  RetainFn retain = driver_fn<RetainFn>("cuMemRetainAllocationHandle");
  ReleaseFn release = driver_fn<ReleaseFn>("cuMemRelease");
  ExportFn export_handle = driver_fn<ExportFn>("cuMemExportToShareableHandle");
  ImportFn import_handle = driver_fn<ImportFn>("cuMemImportFromShareableHandle");
  ReserveFn reserve = driver_fn<ReserveFn>("cuMemAddressReserve");
  MapFn map = driver_fn<MapFn>("cuMemMap");
  SetAccessFn set_access = driver_fn<SetAccessFn>("cuMemSetAccess");
  UnmapFn unmap = driver_fn<UnmapFn>("cuMemUnmap");
  AddressFreeFn address_free = driver_fn<AddressFreeFn>("cuMemAddressFree");
  CreateFn create = driver_fn<CreateFn>("cuMemCreate");
  GranularityFn granularity = driver_fn<GranularityFn>("cuMemGetAllocationGranularity");
  PointerAttrFn pointer_attr = driver_fn<PointerAttrFn>("cuPointerGetAttribute");
  PropsFromHandleFn props_from_handle = driver_fn<PropsFromHandleFn>("cuMemGetAllocationPropertiesFromHandle");
  bool ok() const {
    return retain && release && export_handle && import_handle && reserve && map && set_access && unmap &&
           address_free && create && granularity && pointer_attr && props_from_handle;
  }
};

const Driver& driver() {
  static Driver d;
  if (!d.ok()) throw std::runtime_error("the CUDA driver's virtual-memory entry points are unavailable");
  return d;
}

void check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string(what) + " failed with driver error " + std::to_string((int)r));
}

void ensure_context(int device) {
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaFree(nullptr);   // creates the primary context if this thread has none
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  }
}

CUmemAllocationProp device_prop(int device, unsigned handle_types) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = (CUmemAllocationHandleType)handle_types;
  return prop;
}

// reserves a range, maps `handle` into it and opens it for `device`; releases `handle` either way
VmmMapping map_handle(const Driver& d, CUmemGenericAllocationHandle handle, uint64_t size, int device) {
  CUmemAllocationProp prop = device_prop(device, 0);
  size_t gran = 0;
  CUresult r = d.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  CUdeviceptr va = 0;
  if (r == CUDA_SUCCESS) r = d.reserve(&va, (size_t)size, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    d.release(handle);
    check(r, "cuMemAddressReserve");
  }
  r = d.map(va, (size_t)size, 0, handle, 0);
  if (r != CUDA_SUCCESS) {
    d.address_free(va, (size_t)size);
    d.release(handle);
    check(r, "cuMemMap");
  }
  // the mapping keeps the physical memory alive from here on
  d.release(handle);
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.set_access(va, (size_t)size, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.unmap(va, (size_t)size);
    d.address_free(va, (size_t)size);
    check(r, "cuMemSetAccess");
  }
  return VmmMapping{(uint64_t)va, size};
}

}  // namespace

bool vmm_is_vmm_pointer(uint64_t device_ptr) {
  const Driver& d = driver();
  CUmemGenericAllocationHandle h = 0;
  if (d.retain(&h, (void*)(uintptr_t)device_ptr) != CUDA_SUCCESS) return false;
  d.release(h);
  return true;
}

VmmExport vmm_export(uint64_t device_ptr, bool prefer_fabric) {
  const Driver& d = driver();
  VmmExport out;
  CUdeviceptr base = 0;
  size_t size = 0;
  check(d.pointer_attr(&base, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, (CUdeviceptr)device_ptr),
        "cuPointerGetAttribute(RANGE_START_ADDR)");
  check(d.pointer_attr(&size, CU_POINTER_ATTRIBUTE_RANGE_SIZE, (CUdeviceptr)device_ptr),
        "cuPointerGetAttribute(RANGE_SIZE)");
  CUmemGenericAllocationHandle h = 0;
  check(d.retain(&h, (void*)(uintptr_t)device_ptr), "cuMemRetainAllocationHandle (not a cuMemCreate allocation?)");
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  CUresult r = d.props_from_handle(&prop, h);
  const unsigned allowed = r == CUDA_SUCCESS ? (unsigned)prop.requestedHandleTypes : 0u;
  out.base = (uint64_t)base;
  out.size = (uint64_t)size;
  out.offset = device_ptr - (uint64_t)base;
  if (prefer_fabric && (allowed & (unsigned)CU_MEM_HANDLE_TYPE_FABRIC)) {
    CUmemFabricHandle fh;
    std::memset(&fh, 0, sizeof(fh));
    if (d.export_handle(&fh, h, CU_MEM_HANDLE_TYPE_FABRIC, 0) == CUDA_SUCCESS) {
      out.kind = VmmHandleKind::FABRIC;
      out.fabric.assign(reinterpret_cast<const char*>(&fh), sizeof(fh));
    }
  }
  if (out.kind == VmmHandleKind::NONE && (allowed & (unsigned)CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR)) {
    int fd = -1;
    r = d.export_handle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r == CUDA_SUCCESS && fd >= 0) {
      out.kind = VmmHandleKind::POSIX_FD;
      out.fd = fd;
    }
  }
  d.release(h);
  if (out.kind == VmmHandleKind::NONE)
    throw std::runtime_error("the allocation was not created with a shareable handle type (POSIX fd or fabric); "
                             "requestedHandleTypes=" + std::to_string(allowed));
  return out;
}

VmmMapping vmm_import_fd(int fd, uint64_t size, int device) {
  const Driver& d = driver();
  ensure_context(device);
  CUmemGenericAllocationHandle h = 0;
  check(d.import_handle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle(posix fd)");
  return map_handle(d, h, size, device);
}

VmmMapping vmm_import_fabric(const std::string& fabric, uint64_t size, int device) {
  const Driver& d = driver();
  ensure_context(device);
  if (fabric.size() != sizeof(CUmemFabricHandle)) throw std::invalid_argument("bad fabric handle size");
  CUmemFabricHandle fh;
  std::memcpy(&fh, fabric.data(), sizeof(fh));
  CUmemGenericAllocationHandle h = 0;
  check(d.import_handle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC), "cuMemImportFromShareableHandle(fabric)");
  return map_handle(d, h, size, device);
}

void vmm_unmap(uint64_t va, uint64_t size) {
  if (!va) return;
  const Driver& d = driver();
  d.unmap((CUdeviceptr)va, (size_t)size);
  d.address_free((CUdeviceptr)va, (size_t)size);
}

VmmMapping vmm_alloc(uint64_t bytes, int device, bool fabric) {
  const Driver& d = driver();
  ensure_context(device);
  unsigned types = (unsigned)CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemAllocationProp prop = device_prop(device, types | (fabric ? (unsigned)CU_MEM_HANDLE_TYPE_FABRIC : 0u));
  size_t gran = 0;
  CUresult r = d.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  if (r != CUDA_SUCCESS && fabric) {          // no fabric on this platform: fd only
    prop = device_prop(device, types);
    r = d.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  }
  check(r, "cuMemGetAllocationGranularity");
  const uint64_t size = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h = 0;
  r = d.create(&h, (size_t)size, &prop, 0);
  if (r != CUDA_SUCCESS && (prop.requestedHandleTypes & CU_MEM_HANDLE_TYPE_FABRIC)) {
    prop = device_prop(device, types);
    r = d.create(&h, (size_t)size, &prop, 0);
  }
  check(r, "cuMemCreate");
  return map_handle(d, h, size, device);
}

void vmm_free(uint64_t va, uint64_t size) { vmm_unmap(va, size); }

}  // namespace fkv
