// SSD <-> GPU direct path through cuFile (GPUDirect Storage), loaded with dlopen
// so the package has no hard dependency on libcufile. A block is read from its
// cache file straight into a device bounce buffer; the paged-layout scatter is
// then the ordinary copy kernel with the bounce buffer as its flat side
// (reference: csrc/gds/gds_manager.cpp:13-573,596-795; its separate
// layout_transform kernel, csrc/gds/layout_transform.cu:25-113, is not needed).
// File geometry is the SSD tier's (ssd_io.h).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace fkv {

class GdsEngine {
 public:
  GdsEngine(const std::vector<std::vector<std::string>>& files, int64_t block_bytes, int64_t blocks_per_file,
            int num_threads);
  ~GdsEngine();

  bool available() const { return available_; }
  const std::string& why_unavailable() const { return why_; }

  // Registers a device buffer for direct DMA (optional; unregistered buffers are staged by cuFile).
  bool register_buffer(uint64_t dev_ptr, size_t bytes);
  void deregister_buffer(uint64_t dev_ptr);

  // For block i: file(ssd_blocks[i]) + slice_off .. + slice_bytes  <->  dev_base + dev_offsets[i]
  // Returns the number of failed blocks; ok[i] tells which moved completely.
  int64_t transfer(uint64_t dev_base, const int64_t* dev_offsets, const int64_t* ssd_blocks, int64_t n, bool is_read,
                   int64_t slice_off, int64_t slice_bytes, uint8_t* ok);

 private:
  void locate(int64_t ssd_block, int& fd_index, int64_t& base_off) const;
  struct Api;
  Api* api_ = nullptr;
  bool available_ = false;
  std::string why_;
  int64_t block_bytes_, blocks_per_file_, num_devices_, files_per_device_;
  int num_threads_;
  std::vector<int> fds_;
  std::vector<void*> handles_;
};

}  // namespace fkv
