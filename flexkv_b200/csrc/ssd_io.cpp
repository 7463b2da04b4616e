#include "ssd_io.h"

#include <fcntl.h>
#include <linux/io_uring.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace fkv {

// ------------------------------------------------------------------ io_uring
class IoUring {
 public:
  explicit IoUring(unsigned entries) {
    struct io_uring_params p;
    std::memset(&p, 0, sizeof(p));
    fd_ = (int)syscall(__NR_io_uring_setup, entries, &p);
    if (fd_ < 0) throw std::runtime_error(std::string("io_uring_setup: ") + strerror(errno));
    sq_entries_ = p.sq_entries;
    size_t sq_sz = p.sq_off.array + p.sq_entries * sizeof(unsigned);
    size_t cq_sz = p.cq_off.cqes + p.cq_entries * sizeof(struct io_uring_cqe);
    const bool single = (p.features & IORING_FEAT_SINGLE_MMAP) != 0;
    if (single) sq_sz = cq_sz = std::max(sq_sz, cq_sz);
    sq_ptr_ = mmap(nullptr, sq_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd_, IORING_OFF_SQ_RING);
    if (sq_ptr_ == MAP_FAILED) { close(fd_); throw std::runtime_error("io_uring: mmap sq ring failed"); }
    sq_sz_ = sq_sz;
    if (single) {
      cq_ptr_ = sq_ptr_;
      cq_sz_ = 0;
    } else {
      cq_ptr_ = mmap(nullptr, cq_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd_, IORING_OFF_CQ_RING);
      if (cq_ptr_ == MAP_FAILED) { munmap(sq_ptr_, sq_sz_); close(fd_); throw std::runtime_error("io_uring: mmap cq ring failed"); }
      cq_sz_ = cq_sz;
    }
    sqes_sz_ = p.sq_entries * sizeof(struct io_uring_sqe);
    sqes_ = (struct io_uring_sqe*)mmap(nullptr, sqes_sz_, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd_,
                                       IORING_OFF_SQES);
    if (sqes_ == MAP_FAILED) {
      munmap(sq_ptr_, sq_sz_);
      if (cq_sz_) munmap(cq_ptr_, cq_sz_);
      close(fd_);
      throw std::runtime_error("io_uring: mmap sqes failed");
    }
    auto sq = (uint8_t*)sq_ptr_;
    sq_head_ = (unsigned*)(sq + p.sq_off.head);
    sq_tail_ = (unsigned*)(sq + p.sq_off.tail);
    sq_mask_ = *(unsigned*)(sq + p.sq_off.ring_mask);
    sq_array_ = (unsigned*)(sq + p.sq_off.array);
    auto cq = (uint8_t*)cq_ptr_;
    cq_head_ = (unsigned*)(cq + p.cq_off.head);
    cq_tail_ = (unsigned*)(cq + p.cq_off.tail);
    cq_mask_ = *(unsigned*)(cq + p.cq_off.ring_mask);
    cqes_ = (struct io_uring_cqe*)(cq + p.cq_off.cqes);
  }
  ~IoUring() {
    munmap(sqes_, sqes_sz_);
    if (cq_sz_) munmap(cq_ptr_, cq_sz_);
    munmap(sq_ptr_, sq_sz_);
    close(fd_);
  }
  unsigned capacity() const { return sq_entries_; }

  // queue one read/write; returns false when the submission ring is full
  bool prep(bool is_read, int fd, void* buf, unsigned len, int64_t off, uint64_t user) {
    unsigned tail = *sq_tail_;
    unsigned head = __atomic_load_n(sq_head_, __ATOMIC_ACQUIRE);
    if (tail - head >= sq_entries_) return false;
    unsigned idx = tail & sq_mask_;
    struct io_uring_sqe* e = &sqes_[idx];
    std::memset(e, 0, sizeof(*e));
    e->opcode = is_read ? IORING_OP_READ : IORING_OP_WRITE;
    e->fd = fd;
    e->addr = (uint64_t)(uintptr_t)buf;
    e->len = len;
    e->off = (uint64_t)off;
    e->user_data = user;
    sq_array_[idx] = idx;
    __atomic_store_n(sq_tail_, tail + 1, __ATOMIC_RELEASE);
    ++pending_submit_;
    return true;
  }
  // submit everything queued and wait for at least `min_complete` completions
  int submit_and_wait(unsigned min_complete) {
    for (;;) {
      int r = (int)syscall(__NR_io_uring_enter, fd_, pending_submit_, min_complete,
                           min_complete ? IORING_ENTER_GETEVENTS : 0, nullptr, 0);
      if (r >= 0) { pending_submit_ -= (unsigned)r; return r; }
      if (errno == EINTR) continue;
      return -errno;
    }
  }
  template <typename F>
  unsigned reap(F&& f) {
    unsigned head = *cq_head_;
    unsigned n = 0;
    while (head != __atomic_load_n(cq_tail_, __ATOMIC_ACQUIRE)) {
      struct io_uring_cqe* c = &cqes_[head & cq_mask_];
      f(c->user_data, c->res);
      ++head;
      ++n;
    }
    __atomic_store_n(cq_head_, head, __ATOMIC_RELEASE);
    return n;
  }

 private:
  int fd_ = -1;
  unsigned sq_entries_ = 0, pending_submit_ = 0;
  void *sq_ptr_ = nullptr, *cq_ptr_ = nullptr;
  size_t sq_sz_ = 0, cq_sz_ = 0, sqes_sz_ = 0;
  struct io_uring_sqe* sqes_ = nullptr;
  unsigned *sq_head_, *sq_tail_, sq_mask_, *sq_array_;
  unsigned *cq_head_, *cq_tail_, cq_mask_;
  struct io_uring_cqe* cqes_;
};

// ------------------------------------------------------------------ engine

static constexpr int64_t kDirectAlign = 4096;

SsdIoEngine::SsdIoEngine(const std::vector<std::vector<std::string>>& files, int64_t block_bytes,
                         int64_t blocks_per_file, bool create, bool try_direct, int iouring_entries, int num_threads)
    : block_bytes_(block_bytes), blocks_per_file_(blocks_per_file), num_threads_(std::max(1, num_threads)) {
  if (files.empty() || files[0].empty()) throw std::invalid_argument("SsdIoEngine: no files");
  num_devices_ = (int64_t)files.size();
  files_per_device_ = (int64_t)files[0].size();
  for (auto& d : files)
    if ((int64_t)d.size() != files_per_device_) throw std::invalid_argument("SsdIoEngine: uneven file counts");
  direct_ok_ = try_direct;
  for (auto& d : files)
    for (auto& path : d) {
      int flags = O_RDWR | (create ? O_CREAT : 0);
      int fd = open(path.c_str(), flags, 0600);
      if (fd < 0) throw std::runtime_error("SsdIoEngine: open " + path + ": " + strerror(errno));
      if (create) {
        const off_t want = (off_t)(block_bytes_ * blocks_per_file_);
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size != want) {
          if (ftruncate(fd, want) != 0) {
            int e = errno; close(fd);
            throw std::runtime_error("SsdIoEngine: ftruncate " + path + ": " + strerror(e));
          }
        }
      }
      fds_buffered_.push_back(fd);
      int dfd = -1;
      if (try_direct) dfd = open(path.c_str(), O_RDWR | O_DIRECT);
      if (dfd < 0) direct_ok_ = false;
      fds_direct_.push_back(dfd);
    }
  if (iouring_entries > 0) {
    try {
      ring_ = std::make_unique<IoUring>((unsigned)iouring_entries);
    } catch (const std::exception&) {
      ring_.reset();  // kernel or sandbox without io_uring: thread team takes over
    }
  }
}

SsdIoEngine::~SsdIoEngine() {
  for (int fd : fds_buffered_) if (fd >= 0) close(fd);
  for (int fd : fds_direct_) if (fd >= 0) close(fd);
  if (staging_) free(staging_);
}

void SsdIoEngine::sync_files() {
  for (int fd : fds_buffered_) if (fd >= 0) (void)fdatasync(fd);
}

void SsdIoEngine::locate(int64_t ssd_block, int& fd_index, int64_t& base_off) const {
  const int64_t dev = ssd_block % num_devices_;
  const int64_t in_dev = ssd_block / num_devices_;
  const int64_t file = in_dev % files_per_device_;
  const int64_t slot = in_dev / files_per_device_;
  fd_index = (int)(dev * files_per_device_ + file);
  base_off = slot * block_bytes_;
}

bool SsdIoEngine::inject(int64_t& len, int& err) {
  if (fault_.mode == 0) return false;
  const int64_t k = fault_counter_.fetch_add(1);
  if (fault_.mode == 3) { err = EIO; return true; }
  if (k != fault_.nth) return false;
  if (fault_.mode == 1) { err = EIO; return true; }
  if (fault_.mode == 2 && len > 512) { len = (len / 2) & ~int64_t(511); err = 0; return true; }
  return false;
}

void SsdIoEngine::run_threads(std::vector<IoReq>& reqs, bool is_read, bool direct, std::vector<uint8_t>& failed) {
  std::atomic<size_t> next{0};
  auto work = [&] {
    for (size_t i = next.fetch_add(1); i < reqs.size(); i = next.fetch_add(1)) {
      IoReq& r = reqs[i];
      const int fd = direct ? fds_direct_[r.fd_index] : fds_buffered_[r.fd_index];
      int64_t done = 0;
      while (done < r.len) {
        int64_t want = r.len - done;
        int ferr = 0;
        ssize_t n;
        if (inject(want, ferr) && ferr) { n = -1; errno = ferr; }
        else n = is_read ? pread(fd, r.mem + done, (size_t)want, r.file_off + done)
                         : pwrite(fd, r.mem + done, (size_t)want, r.file_off + done);
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) { failed[(size_t)r.block_slot] = 1; break; }
        done += n;
      }
    }
  };
  const int nt = (int)std::min<size_t>((size_t)num_threads_, reqs.size());
  if (nt <= 1) { work(); return; }
  std::vector<std::thread> team;
  for (int t = 0; t < nt; ++t) team.emplace_back(work);
  for (auto& th : team) th.join();
}

void SsdIoEngine::run_iouring(std::vector<IoReq>& reqs, bool is_read, bool direct, std::vector<uint8_t>& failed) {
  // progress[i] = bytes already moved for request i (short IOs are re-queued)
  std::vector<int64_t> progress(reqs.size(), 0);
  std::vector<int64_t> issued_len(reqs.size(), 0);
  std::vector<size_t> retry;
  size_t next = 0, inflight = 0;
  const unsigned cap = ring_->capacity();
  constexpr int64_t kMaxIo = 1 << 30;
  auto queue = [&](size_t i) -> bool {
    IoReq& r = reqs[i];
    int64_t want = std::min(r.len - progress[i], kMaxIo);
    int ferr = 0;
    if (inject(want, ferr) && ferr) { failed[(size_t)r.block_slot] = 1; return true; }
    const int fd = direct ? fds_direct_[r.fd_index] : fds_buffered_[r.fd_index];
    if (!ring_->prep(is_read, fd, r.mem + progress[i], (unsigned)want, r.file_off + progress[i], (uint64_t)i))
      return false;
    issued_len[i] = want;
    ++inflight;
    return true;
  };
  while (next < reqs.size() || !retry.empty() || inflight > 0) {
    while (inflight < cap && (!retry.empty() || next < reqs.size())) {
      size_t i;
      bool from_retry = !retry.empty();
      if (from_retry) i = retry.back(); else i = next;
      if (!queue(i)) break;
      if (from_retry) retry.pop_back(); else ++next;
    }
    if (inflight == 0) continue;
    int r = ring_->submit_and_wait(1);
    if (r < 0) {
      // ring broke: fail what is left rather than spin
      for (size_t i = 0; i < reqs.size(); ++i)
        if (progress[i] < reqs[i].len) failed[(size_t)reqs[i].block_slot] = 1;
      return;
    }
    ring_->reap([&](uint64_t user, int32_t res) {
      --inflight;
      const size_t i = (size_t)user;
      if (res <= 0) { failed[(size_t)reqs[i].block_slot] = 1; return; }
      progress[i] += res;
      if (progress[i] < reqs[i].len && !failed[(size_t)reqs[i].block_slot]) retry.push_back(i);
    });
  }
}

int64_t SsdIoEngine::transfer(uint8_t* cpu_base, const int64_t* cpu_blocks, const int64_t* ssd_blocks, int64_t n,
                              bool is_read, const SsdLayout& lay, int layer_start, int num_layers, uint8_t* ok) {
  if (n <= 0) return 0;
  std::vector<IoReq> reqs;
  std::vector<uint8_t> failed((size_t)n, 0);
  const int64_t cap = capacity_blocks();
  for (int64_t i = 0; i < n; ++i) {
    if (ssd_blocks[i] < 0 || ssd_blocks[i] >= cap || cpu_blocks[i] < 0) { failed[(size_t)i] = 1; continue; }
    int fdi; int64_t base;
    locate(ssd_blocks[i], fdi, base);
    if (lay.block_first) {
      // one run per block: [layer_start, layer_start+num_layers) x all kv planes
      IoReq r;
      r.fd_index = fdi;
      r.file_off = base + (int64_t)layer_start * lay.ssd_layer_stride;
      r.mem = cpu_base + cpu_blocks[i] * lay.cpu_block_stride + (int64_t)layer_start * lay.cpu_layer_stride;
      r.len = (int64_t)num_layers * lay.cpu_layer_stride;
      r.block_slot = (int32_t)i;
      reqs.push_back(r);
    } else {
      for (int l = layer_start; l < layer_start + num_layers; ++l)
        for (int kv = 0; kv < lay.kv_dim; ++kv) {
          IoReq r;
          r.fd_index = fdi;
          r.file_off = base + (int64_t)l * lay.ssd_layer_stride + (int64_t)kv * lay.ssd_kv_stride;
          r.mem = cpu_base + cpu_blocks[i] * lay.cpu_block_stride + (int64_t)l * lay.cpu_layer_stride +
                  (int64_t)kv * lay.cpu_kv_stride;
          r.len = lay.chunk_bytes;
          r.block_slot = (int32_t)i;
          reqs.push_back(r);
        }
    }
  }
  // ascending (file, offset) order, then merge neighbours that are contiguous on both sides
  std::sort(reqs.begin(), reqs.end(), [](const IoReq& a, const IoReq& b) {
    return a.fd_index != b.fd_index ? a.fd_index < b.fd_index : a.file_off < b.file_off;
  });
  bool direct = direct_ok_;
  for (auto& r : reqs)
    if ((r.file_off % kDirectAlign) || (r.len % kDirectAlign) || ((uintptr_t)r.mem % kDirectAlign)) { direct = false; break; }
  std::vector<IoReq> merged;
  merged.reserve(reqs.size());
  for (auto& r : reqs) {
    if (!merged.empty()) {
      IoReq& m = merged.back();
      // merging across blocks would blur per-block results, so only chunks of one block are fused
      if (m.fd_index == r.fd_index && m.block_slot == r.block_slot && m.file_off + m.len == r.file_off &&
          m.mem + m.len == r.mem) {
        m.len += r.len;
        continue;
      }
    }
    merged.push_back(r);
  }
  {
    std::lock_guard<std::mutex> g(mu_);  // the ring is single-issuer
    if (ring_) run_iouring(merged, is_read, direct, failed);
    else run_threads(merged, is_read, direct, failed);
  }
  int64_t nfail = 0, bytes = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (ok) ok[i] = failed[(size_t)i] ? 0 : 1;
    nfail += failed[(size_t)i];
  }
  for (auto& r : merged) if (!failed[(size_t)r.block_slot]) bytes += r.len;
  (is_read ? bytes_read_ : bytes_written_) += (uint64_t)bytes;
  return nfail;
}

// ---------------------------------------------------------------- packed blocks

static constexpr int64_t kPackedBatch = 32;   // blocks gathered per round of IO

int64_t SsdIoEngine::transfer_packed(uint8_t* cpu_base, const int64_t* cpu_blocks, const int64_t* ssd_blocks, int64_t n,
                                     bool is_read, const PackedGeometry& geo, const int32_t* sizes, uint8_t* ok) {
  if (n <= 0) return 0;
  if (geo.entries <= 0 || geo.tiles_per_chunk <= 0 || geo.entries % geo.tiles_per_chunk != 0)
    throw std::invalid_argument("SsdIoEngine::transfer_packed: bad geometry");
  std::lock_guard<std::mutex> sg(staging_mu_);
  if (staging_ == nullptr) {
    void* p = nullptr;
    if (posix_memalign(&p, (size_t)kDirectAlign, (size_t)(kPackedBatch * block_bytes_ + kDirectAlign)) != 0)
      throw std::runtime_error("SsdIoEngine: no memory for the packed staging area");
    staging_ = static_cast<uint8_t*>(p);
  }
  const int64_t cap = capacity_blocks();
  std::vector<uint8_t> failed((size_t)n, 0);
  std::vector<int64_t> total((size_t)n, 0);
  // validate the rows and size every block's run
  for (int64_t i = 0; i < n; ++i) {
    if (ssd_blocks[i] < 0 || ssd_blocks[i] >= cap || cpu_blocks[i] < 0) { failed[(size_t)i] = 1; continue; }
    const int32_t* row = sizes + i * geo.entries;
    int64_t sum = 0;
    for (int32_t e = 0; e < geo.entries; ++e) {
      const bool last = (e % geo.tiles_per_chunk) == geo.tiles_per_chunk - 1;
      const int64_t slot = last ? geo.last_tile_slot_bytes : geo.tile_slot_bytes;
      if (row[e] <= 0 || (row[e] & 15) || row[e] > slot) { failed[(size_t)i] = 1; break; }
      sum += row[e];
    }
    if (!failed[(size_t)i] && sum > block_bytes_) failed[(size_t)i] = 1;
    total[(size_t)i] = sum;
  }
  auto tile_ptr = [&](int64_t cpu_block, int32_t e) {
    return cpu_base + cpu_block * geo.cpu_block_stride + (int64_t)(e / geo.tiles_per_chunk) * geo.chunk_slot_bytes +
           (int64_t)(e % geo.tiles_per_chunk) * geo.tile_slot_bytes;
  };
  int64_t moved = 0;
  for (int64_t lo = 0; lo < n; lo += kPackedBatch) {
    const int64_t hi = std::min(n, lo + kPackedBatch);
    std::vector<IoReq> reqs;
    for (int64_t i = lo; i < hi; ++i) {
      if (failed[(size_t)i]) continue;
      uint8_t* st = staging_ + (i - lo) * block_bytes_;
      const int64_t len = std::min(block_bytes_, (total[(size_t)i] + kDirectAlign - 1) / kDirectAlign * kDirectAlign);
      if (!is_read) {
        const int32_t* row = sizes + i * geo.entries;
        int64_t off = 0;
        for (int32_t e = 0; e < geo.entries; ++e) {
          std::memcpy(st + off, tile_ptr(cpu_blocks[i], e), (size_t)row[e]);
          off += row[e];
        }
        std::memset(st + off, 0, (size_t)(len - off));
      }
      int fdi; int64_t base;
      locate(ssd_blocks[i], fdi, base);
      IoReq r;
      r.fd_index = fdi;
      r.file_off = base;
      r.mem = st;
      r.len = len;
      r.block_slot = (int32_t)i;
      reqs.push_back(r);
    }
    if (reqs.empty()) continue;
    bool direct = direct_ok_;
    for (auto& r : reqs)
      if ((r.file_off % kDirectAlign) || (r.len % kDirectAlign) || ((uintptr_t)r.mem % kDirectAlign)) { direct = false; break; }
    std::sort(reqs.begin(), reqs.end(), [](const IoReq& a, const IoReq& b) {
      return a.fd_index != b.fd_index ? a.fd_index < b.fd_index : a.file_off < b.file_off;
    });
    {
      std::lock_guard<std::mutex> g(mu_);
      if (ring_) run_iouring(reqs, is_read, direct, failed);
      else run_threads(reqs, is_read, direct, failed);
    }
    for (auto& r : reqs) {
      const int64_t i = r.block_slot;
      if (failed[(size_t)i]) continue;
      moved += r.len;
      if (is_read) {
        const int32_t* row = sizes + i * geo.entries;
        const uint8_t* st = r.mem;
        int64_t off = 0;
        for (int32_t e = 0; e < geo.entries; ++e) {
          std::memcpy(tile_ptr(cpu_blocks[i], e), st + off, (size_t)row[e]);
          off += row[e];
        }
      }
    }
  }
  int64_t nfail = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (ok) ok[i] = failed[(size_t)i] ? 0 : 1;
    nfail += failed[(size_t)i];
  }
  (is_read ? bytes_read_ : bytes_written_) += (uint64_t)moved;
  return nfail;
}

}  // namespace fkv
