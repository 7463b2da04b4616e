// Host block pools: anonymous or file-backed (hugetlbfs / shm) mappings,
// NUMA placement next to the owning GPU, parallel first touch, and chunked
// cudaHostRegister(PORTABLE|MAPPED) so that copy kernels can address the pool
// directly (reference behaviour: flexkv/storage/allocator.py:190-590,
// flexkv/transfer/host_buffer.py:66-98,180-202).
#include "host_mem.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#ifndef MAP_HUGE_SHIFT
#define MAP_HUGE_SHIFT 26
#endif
#ifndef MPOL_BIND
#define MPOL_BIND 2
#endif
#ifndef MPOL_PREFERRED
#define MPOL_PREFERRED 1
#endif

namespace fkv {

static int log2_u64(uint64_t v) {
  int r = 0;
  while (v > 1) { v >>= 1; ++r; }
  return r;
}

static void bind_to_numa(void* p, size_t bytes, int node) {
  if (node < 0 || node >= 1024) return;
  unsigned long mask[16] = {0};
  mask[node / (8 * sizeof(unsigned long))] |= 1UL << (node % (8 * sizeof(unsigned long)));
  // preferred, not strict: a full node must not make the allocation fail
  (void)syscall(SYS_mbind, p, bytes, MPOL_PREFERRED, mask, sizeof(mask) * 8, 0);
}

static void first_touch(uint8_t* base, size_t bytes, size_t page, int threads) {
  threads = std::max(1, threads);
  std::vector<std::thread> team;
  const size_t per = ((bytes / threads + page - 1) / page) * page;
  for (int t = 0; t < threads; ++t) {
    const size_t lo = std::min(bytes, per * t), hi = std::min(bytes, per * (t + 1));
    if (lo >= hi) break;
    team.emplace_back([=] {
      for (size_t off = lo; off < hi; off += page) reinterpret_cast<volatile uint8_t*>(base)[off] = 0;
    });
  }
  for (auto& th : team) th.join();
}

HostRegion host_region_alloc(size_t bytes, const HostAllocOptions& opt) {
  if (bytes == 0) throw std::invalid_argument("host_region_alloc: zero bytes");
  HostRegion r;
  r.bytes = bytes;
  size_t page = 4096;
  void* p = MAP_FAILED;
  if (!opt.backing_file.empty()) {
    // file-backed (hugetlbfs file or /dev/shm) so other processes can map the same pool
    int fd = open(opt.backing_file.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("host_region_alloc: open " + opt.backing_file + ": " + strerror(errno));
    size_t len = bytes;
    if (opt.hugepage) {
      page = opt.hugepage_bytes;
      len = (bytes + page - 1) / page * page;
    }
    if (ftruncate(fd, (off_t)len) != 0) {
      int e = errno; close(fd);
      throw std::runtime_error(std::string("host_region_alloc: ftruncate: ") + strerror(e));
    }
    p = mmap(nullptr, len, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) throw std::runtime_error(std::string("host_region_alloc: mmap(file): ") + strerror(errno));
    r.map_bytes = len;
    r.hugepage = opt.hugepage;
    r.file_backed = true;
  } else {
    if (opt.hugepage) {
      page = opt.hugepage_bytes;
      const size_t len = (bytes + page - 1) / page * page;
      int flags = MAP_PRIVATE | MAP_ANONYMOUS | MAP_HUGETLB | (log2_u64(page) << MAP_HUGE_SHIFT);
      p = mmap(nullptr, len, PROT_READ | PROT_WRITE, flags, -1, 0);
      if (p != MAP_FAILED) { r.map_bytes = len; r.hugepage = true; }
    }
    if (p == MAP_FAILED) {
      // no reserved huge pages (or not requested): fall back to normal pages,
      // asking for transparent huge pages where the kernel offers them
      page = 4096;
      const size_t len = (bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
      p = mmap(nullptr, len, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
      if (p == MAP_FAILED) throw std::runtime_error(std::string("host_region_alloc: mmap: ") + strerror(errno));
      (void)madvise(p, len, MADV_HUGEPAGE);
      r.map_bytes = len;
      r.hugepage = false;
    }
  }
  r.ptr = p;
  bind_to_numa(p, r.map_bytes, opt.numa_node);
  if (opt.populate) first_touch(static_cast<uint8_t*>(p), r.map_bytes, page, opt.touch_threads);
  if (opt.cuda_register) {
    try {
      host_region_register(r, opt.register_chunk_bytes);
    } catch (...) {
      munmap(p, r.map_bytes);
      throw;
    }
  }
  return r;
}

HostRegion host_region_open(const std::string& file, size_t bytes, bool hugepage, size_t hugepage_bytes) {
  HostRegion r;
  int fd = open(file.c_str(), O_RDWR);
  if (fd < 0) throw std::runtime_error("host_region_open: open " + file + ": " + strerror(errno));
  size_t len = bytes;
  if (hugepage) len = (bytes + hugepage_bytes - 1) / hugepage_bytes * hugepage_bytes;
  void* p = mmap(nullptr, len, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) throw std::runtime_error(std::string("host_region_open: mmap: ") + strerror(errno));
  r.ptr = p; r.bytes = bytes; r.map_bytes = len; r.hugepage = hugepage; r.file_backed = true;
  return r;
}

void host_region_register(HostRegion& r, size_t chunk_bytes) {
  if (r.registered) return;
  uint8_t* base = static_cast<uint8_t*>(r.ptr);
  if (chunk_bytes == 0) chunk_bytes = r.map_bytes;
  size_t done = 0;
  while (done < r.map_bytes) {
    const size_t n = std::min(chunk_bytes, r.map_bytes - done);
    cudaError_t e = cudaHostRegister(base + done, n, cudaHostRegisterPortable | cudaHostRegisterMapped);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      for (size_t off = 0; off < done; off += chunk_bytes) cudaHostUnregister(base + off);
      throw std::runtime_error(std::string("cudaHostRegister failed: ") + cudaGetErrorString(e));
    }
    done += n;
  }
  r.registered = true;
  r.register_chunk = chunk_bytes;
}

void host_region_unregister(HostRegion& r) {
  if (!r.registered) return;
  uint8_t* base = static_cast<uint8_t*>(r.ptr);
  for (size_t off = 0; off < r.map_bytes; off += r.register_chunk) (void)cudaHostUnregister(base + off);
  r.registered = false;
}

void host_region_free(HostRegion& r) {
  if (!r.ptr) return;
  host_region_unregister(r);
  munmap(r.ptr, r.map_bytes);
  r.ptr = nullptr;
}

int gpu_numa_node(int device) {
  char busid[32] = {0};
  if (cudaDeviceGetPCIBusId(busid, sizeof(busid), device) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  std::string s(busid);
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
  std::ifstream f("/sys/bus/pci/devices/" + s + "/numa_node");
  int node = -1;
  if (f) f >> node;
  return node;
}

}  // namespace fkv
