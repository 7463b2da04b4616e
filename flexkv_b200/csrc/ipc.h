#pragma once
#include <cstdint>
#include <string>

namespace fkv {

struct IpcExport {
  std::string handle;     // 64 opaque bytes
  uint64_t offset = 0;    // of the exported pointer inside its allocation
  uint64_t alloc_bytes = 0;
};

IpcExport ipc_export(uint64_t device_ptr);
uint64_t ipc_import(const std::string& handle, int device);   // returns the allocation's base address here
void ipc_close(uint64_t base_ptr, int device);

}  // namespace fkv
