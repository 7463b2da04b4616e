// Sharing of device memory that was allocated with the CUDA virtual-memory API
// (cuMemCreate + cuMemMap): such memory has no legacy IPC handle, so an engine that
// builds its KV cache this way (sleep-mode allocators that unmap and remap physical
// memory under a stable address) is reached through a shareable handle of the
// physical allocation instead: a fabric handle (64 opaque bytes that travel in any
// message) where the platform offers one, else a POSIX file descriptor that the
// exporter hands over on a UNIX socket
// (reference behaviour: flexkv/common/memory_handle.py:466-545,600-700,800-900,
// modes "vmm_fabric" / "vmm_posix_fd").
//
// Every driver entry point is looked up through the runtime, so the module links
// against nothing but cudart; on a box without a driver the calls throw.
#pragma once
#include <cstdint>
#include <string>

namespace fkv {

enum class VmmHandleKind : int { NONE = 0, POSIX_FD = 1, FABRIC = 2 };

struct VmmExport {
  VmmHandleKind kind = VmmHandleKind::NONE;
  int fd = -1;             // POSIX_FD: owned by the caller (close it when the export is dropped)
  std::string fabric;      // FABRIC: 64 opaque bytes
  uint64_t base = 0;       // start of the mapped range that holds the pointer
  uint64_t size = 0;       // bytes of that range (= bytes of the physical allocation)
  uint64_t offset = 0;     // of the exported pointer inside the range
};

struct VmmMapping {
  uint64_t va = 0;
  uint64_t size = 0;
};

// True when `device_ptr` lies in memory mapped from a cuMemCreate allocation.
bool vmm_is_vmm_pointer(uint64_t device_ptr);

// Exports the physical allocation behind `device_ptr`. The allocation must have been created
// with the matching requestedHandleTypes; fabric is tried first when `prefer_fabric`.
VmmExport vmm_export(uint64_t device_ptr, bool prefer_fabric);

// Maps an exported allocation read-write on `device` and returns the new range. `fd` is not
// consumed (the caller closes it); `fabric` is the 64-byte handle.
VmmMapping vmm_import_fd(int fd, uint64_t size, int device);
VmmMapping vmm_import_fabric(const std::string& fabric, uint64_t size, int device);
void vmm_unmap(uint64_t va, uint64_t size);

// A mapped allocation of at least `bytes` on `device` that can be exported as a POSIX fd
// (and as a fabric handle when `fabric` and the platform allows it); for engines' stand-ins
// in tests and for callers that want an exportable cache. Freed with vmm_free.
VmmMapping vmm_alloc(uint64_t bytes, int device, bool fabric);
void vmm_free(uint64_t va, uint64_t size);

}  // namespace fkv
