// SSD tier IO: block-addressed reads/writes between a host block pool and a
// set of pre-sized files spread over one or more devices, through io_uring
// (raw syscalls, no liburing) with a pread/pwrite thread team as fallback.
//
// File geometry and addressing follow the reference's block format so that
// cache files are interchangeable (csrc/transfer_ssd.cpp:22-44,67-118,336-352;
// flexkv/storage/allocator.py:615-647):
//   global ssd block id -> device = id % num_devices, in_dev = id / num_devices
//   in_dev -> file = in_dev % files_per_device, slot = in_dev / files_per_device
//   byte offset = slot*block_bytes + layer*ssd_layer_stride + kv*ssd_kv_stride
// O_DIRECT is used only when address, offset and length are all 4 KiB multiples.
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace fkv {

struct IoReq {
  int fd_index;       // index into the engine's file table
  int64_t file_off;
  uint8_t* mem;
  int64_t len;
  int32_t block_slot; // index of the originating block in the call (for per-block results)
};

struct SsdFault {       // host-side fault injection for tests
  int mode = 0;         // 0 none, 1 = fail the nth IO with EIO, 2 = make the nth IO short once, 3 = fail every IO
  int64_t nth = 0;
};

struct SsdLayout {      // strides in bytes
  int64_t cpu_layer_stride, cpu_kv_stride, cpu_block_stride;
  int64_t ssd_layer_stride, ssd_kv_stride, ssd_block_stride;
  int64_t chunk_bytes;
  int32_t num_layers_total, kv_dim;
  bool block_first;     // both sides BLOCKFIRST: one contiguous run per block and layer range
};

class IoUring;  // defined in ssd_io.cpp

class SsdIoEngine {
 public:
  // files[d] = paths on device d (all devices must have the same count)
  SsdIoEngine(const std::vector<std::vector<std::string>>& files, int64_t block_bytes, int64_t blocks_per_file,
              bool create, bool try_direct, int iouring_entries, int num_threads);
  ~SsdIoEngine();

  // Moves blocks; `ok[i]` tells whether block i moved completely. Returns the
  // number of failed blocks.
  int64_t transfer(uint8_t* cpu_base, const int64_t* cpu_blocks, const int64_t* ssd_blocks, int64_t n, bool is_read,
                   const SsdLayout& lay, int layer_start, int num_layers, uint8_t* ok);

  // Packed form for host pools kept in the lossless codec's format: a host block is a grid of fixed tile
  // slots of which only the first sizes[i] bytes are in use. A write gathers the used bytes of a block's tiles
  // back to back (row order of the size table) and writes that run, rounded up to 4 KiB, at the start of the
  // block's SSD slot; a read fetches the run and scatters the tiles back into their slots. The SSD slot keeps
  // its size (block ids map to the same offsets), what shrinks are the bytes that cross the SSD interface.
  // `sizes` holds n rows of `geo.entries` int32 (host table rows for a write, SSD table rows for a read); a row
  // with an entry that is 0, not a multiple of 16 or larger than its tile's slot fails that block.
  // (reference: csrc/compression/common/packed_ssd.cpp:64-250, one 512-aligned IO per block.)
  struct PackedGeometry {
    int64_t cpu_block_stride;   // bytes between host blocks
    int64_t chunk_slot_bytes;   // host slot of one chunk
    int64_t tile_slot_bytes;    // slot of a full tile; tile t of a chunk starts t * tile_slot_bytes into the chunk slot
    int32_t tiles_per_chunk;
    int32_t entries;            // tiles per block = chunks per block * tiles_per_chunk
    int64_t last_tile_slot_bytes;   // slot of the last tile of a chunk (shorter when the chunk is not a whole number of tiles)
  };
  int64_t transfer_packed(uint8_t* cpu_base, const int64_t* cpu_blocks, const int64_t* ssd_blocks, int64_t n,
                          bool is_read, const PackedGeometry& geo, const int32_t* sizes, uint8_t* ok);

  bool using_iouring() const { return ring_ != nullptr; }
  bool direct_available() const { return direct_ok_; }
  int num_devices() const { return (int)num_devices_; }
  int files_per_device() const { return (int)files_per_device_; }
  int64_t capacity_blocks() const { return blocks_per_file_ * files_per_device_ * num_devices_; }
  void set_fault(const SsdFault& f) { fault_ = f; fault_counter_ = 0; }
  uint64_t bytes_read() const { return bytes_read_; }
  uint64_t bytes_written() const { return bytes_written_; }
  void sync_files();

 private:
  void locate(int64_t ssd_block, int& fd_index, int64_t& base_off) const;
  void run_iouring(std::vector<IoReq>& reqs, bool is_read, bool direct, std::vector<uint8_t>& failed);
  void run_threads(std::vector<IoReq>& reqs, bool is_read, bool direct, std::vector<uint8_t>& failed);
  bool inject(int64_t& len, int& err);

  int64_t block_bytes_, blocks_per_file_;
  int64_t num_devices_, files_per_device_;
  std::vector<int> fds_buffered_, fds_direct_;
  bool direct_ok_ = false;
  int num_threads_;
  std::unique_ptr<IoUring> ring_;
  std::mutex mu_;
  SsdFault fault_;
  std::atomic<int64_t> fault_counter_{0};
  std::atomic<uint64_t> bytes_read_{0}, bytes_written_{0};
  uint8_t* staging_ = nullptr;      // packed IO: page-aligned gather/scatter area, kPackedBatch blocks
  std::mutex staging_mu_;
};

}  // namespace fkv
