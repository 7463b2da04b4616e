#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace fkv {

struct HostAllocOptions {
  bool hugepage = false;
  size_t hugepage_bytes = 2u << 20;
  int numa_node = -1;              // preferred node, -1 = leave to the kernel
  bool populate = true;            // touch every page at allocation time
  int touch_threads = 8;
  bool cuda_register = false;      // cudaHostRegister(PORTABLE | MAPPED)
  size_t register_chunk_bytes = 0; // 0 = one registration
  std::string backing_file;        // hugetlbfs or shm file for cross-process pools
};

struct HostRegion {
  void* ptr = nullptr;
  size_t bytes = 0;      // usable bytes
  size_t map_bytes = 0;  // mapped length (page-rounded)
  bool hugepage = false;
  bool file_backed = false;
  bool registered = false;
  size_t register_chunk = 0;
};

HostRegion host_region_alloc(size_t bytes, const HostAllocOptions& opt);
HostRegion host_region_open(const std::string& file, size_t bytes, bool hugepage, size_t hugepage_bytes);
void host_region_register(HostRegion& r, size_t chunk_bytes);
void host_region_unregister(HostRegion& r);
void host_region_free(HostRegion& r);
int gpu_numa_node(int device);  // -1 when unknown

}  // namespace fkv
