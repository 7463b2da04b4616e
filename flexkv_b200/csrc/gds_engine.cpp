#include "gds_engine.h"

#include <cufile.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace fkv {

struct GdsEngine::Api {
  void* lib = nullptr;
  CUfileError_t (*DriverOpen)() = nullptr;
  CUfileError_t (*DriverClose)() = nullptr;
  CUfileError_t (*HandleRegister)(CUfileHandle_t*, CUfileDescr_t*) = nullptr;
  void (*HandleDeregister)(CUfileHandle_t) = nullptr;
  CUfileError_t (*BufRegister)(const void*, size_t, int) = nullptr;
  CUfileError_t (*BufDeregister)(const void*) = nullptr;
  ssize_t (*Read)(CUfileHandle_t, void*, size_t, off_t, off_t) = nullptr;
  ssize_t (*Write)(CUfileHandle_t, const void*, size_t, off_t, off_t) = nullptr;
  bool driver_open = false;
};

template <typename F>
static bool sym(void* lib, const char* name, F& out) {
  out = reinterpret_cast<F>(dlsym(lib, name));
  return out != nullptr;
}

GdsEngine::GdsEngine(const std::vector<std::vector<std::string>>& files, int64_t block_bytes, int64_t blocks_per_file,
                     int num_threads)
    : block_bytes_(block_bytes), blocks_per_file_(blocks_per_file), num_threads_(num_threads > 0 ? num_threads : 4) {
  if (files.empty() || files[0].empty()) throw std::invalid_argument("GdsEngine: no files");
  num_devices_ = (int64_t)files.size();
  files_per_device_ = (int64_t)files[0].size();
  api_ = new Api();
  const char* names[] = {"libcufile.so.0", "libcufile.so", "/usr/local/cuda/lib64/libcufile.so.0"};
  for (const char* n : names) {
    api_->lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (api_->lib) break;
  }
  if (!api_->lib) { why_ = "libcufile not found"; return; }
  bool ok = sym(api_->lib, "cuFileDriverOpen", api_->DriverOpen) &&
            sym(api_->lib, "cuFileHandleRegister", api_->HandleRegister) &&
            sym(api_->lib, "cuFileHandleDeregister", api_->HandleDeregister) &&
            sym(api_->lib, "cuFileBufRegister", api_->BufRegister) &&
            sym(api_->lib, "cuFileBufDeregister", api_->BufDeregister) && sym(api_->lib, "cuFileRead", api_->Read) &&
            sym(api_->lib, "cuFileWrite", api_->Write);
  if (!sym(api_->lib, "cuFileDriverClose_v2", api_->DriverClose)) sym(api_->lib, "cuFileDriverClose", api_->DriverClose);
  if (!ok) { why_ = "libcufile lacks required symbols"; return; }
  CUfileError_t st = api_->DriverOpen();
  if (st.err != CU_FILE_SUCCESS) { why_ = "cuFileDriverOpen failed (" + std::to_string((int)st.err) + ")"; return; }
  api_->driver_open = true;
  for (auto& d : files)
    for (auto& path : d) {
      int fd = open(path.c_str(), O_RDWR | O_DIRECT);
      if (fd < 0) { why_ = "open O_DIRECT failed for " + path + ": " + strerror(errno); return; }
      fds_.push_back(fd);
      CUfileDescr_t descr;
      std::memset(&descr, 0, sizeof(descr));
      descr.handle.fd = fd;
      descr.type = CU_FILE_HANDLE_TYPE_OPAQUE_FD;
      CUfileHandle_t h = nullptr;
      st = api_->HandleRegister(&h, &descr);
      if (st.err != CU_FILE_SUCCESS) { why_ = "cuFileHandleRegister failed (" + std::to_string((int)st.err) + ")"; return; }
      handles_.push_back(h);
    }
  available_ = true;
}

GdsEngine::~GdsEngine() {
  if (api_) {
    for (void* h : handles_) if (h && api_->HandleDeregister) api_->HandleDeregister(h);
    for (int fd : fds_) if (fd >= 0) close(fd);
    if (api_->driver_open && api_->DriverClose) api_->DriverClose();
    // the library stays loaded: unloading it under a live CUDA context is not worth the risk
    delete api_;
  }
}

bool GdsEngine::register_buffer(uint64_t dev_ptr, size_t bytes) {
  if (!available_) return false;
  return api_->BufRegister((const void*)(uintptr_t)dev_ptr, bytes, 0).err == CU_FILE_SUCCESS;
}

void GdsEngine::deregister_buffer(uint64_t dev_ptr) {
  if (available_) (void)api_->BufDeregister((const void*)(uintptr_t)dev_ptr);
}

void GdsEngine::locate(int64_t ssd_block, int& fd_index, int64_t& base_off) const {
  const int64_t dev = ssd_block % num_devices_, in_dev = ssd_block / num_devices_;
  fd_index = (int)(dev * files_per_device_ + in_dev % files_per_device_);
  base_off = (in_dev / files_per_device_) * block_bytes_;
}

int64_t GdsEngine::transfer(uint64_t dev_base, const int64_t* dev_offsets, const int64_t* ssd_blocks, int64_t n,
                            bool is_read, int64_t slice_off, int64_t slice_bytes, uint8_t* ok) {
  if (!available_) throw std::runtime_error("GdsEngine unavailable: " + why_);
  const int64_t cap = blocks_per_file_ * files_per_device_ * num_devices_;
  std::atomic<int64_t> next{0}, nfail{0};
  auto work = [&] {
    for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) {
      bool good = ssd_blocks[i] >= 0 && ssd_blocks[i] < cap && slice_off + slice_bytes <= block_bytes_;
      if (good) {
        int fdi; int64_t base;
        locate(ssd_blocks[i], fdi, base);
        int64_t done = 0;
        while (done < slice_bytes) {
          ssize_t r = is_read ? api_->Read(handles_[(size_t)fdi], (void*)(uintptr_t)dev_base, (size_t)(slice_bytes - done),
                                           (off_t)(base + slice_off + done), (off_t)(dev_offsets[i] + done))
                              : api_->Write(handles_[(size_t)fdi], (const void*)(uintptr_t)dev_base,
                                            (size_t)(slice_bytes - done), (off_t)(base + slice_off + done),
                                            (off_t)(dev_offsets[i] + done));
          if (r <= 0) { good = false; break; }
          done += r;
        }
      }
      if (ok) ok[i] = good ? 1 : 0;
      if (!good) ++nfail;
    }
  };
  const int nt = (int)std::min<int64_t>(num_threads_, n);
  if (nt <= 1) work();
  else {
    std::vector<std::thread> team;
    for (int t = 0; t < nt; ++t) team.emplace_back(work);
    for (auto& th : team) th.join();
  }
  return nfail.load();
}

}  // namespace fkv
