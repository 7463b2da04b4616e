#include "ce_copy.h"

#include <algorithm>

namespace fkv {

CeAnalysis ce_analyze(const int64_t* g, const int64_t* c, int64_t n, int64_t gpu_num_blocks,
                      int64_t cpu_num_blocks) {
  CeAnalysis a;
  for (int64_t i = 0; i < n; ++i) {
    if (gpu_num_blocks > 0 && (g[i] < 0 || g[i] >= gpu_num_blocks)) { a.status |= KV_ERR_GPU_BLOCK_RANGE; continue; }
    if (cpu_num_blocks > 0 && (c[i] < 0 || c[i] >= cpu_num_blocks)) { a.status |= KV_ERR_CPU_BLOCK_RANGE; continue; }
    ++a.num_blocks;
    if (!a.runs.empty()) {
      CeRun& r = a.runs.back();
      if (g[i] == r.gpu_block + r.len && c[i] == r.cpu_block + r.len) {
        ++r.len;
        continue;
      }
    }
    a.runs.push_back(CeRun{g[i], c[i], 1});
  }
  for (const CeRun& r : a.runs) a.longest = std::max(a.longest, r.len);
  return a;
}

namespace {

// True when a whole block (all layers of the op, all kv) is one contiguous span with
// the same internal geometry on both sides, so a run of blocks is a single 1-D copy.
bool block_geometry_matches(const KvCopyParams& p) {
  if (p.idx_layer_mul != 0 || p.idx_kv_mul != 0 || p.c_use_table) return false;
  if (p.g_layer_stride != p.c_layer_stride || p.g_kv_stride != p.c_kv_stride) return false;
  if (p.g_block_stride != p.c_block_stride) return false;
  const int64_t kv_span = (p.kv_dim > 1) ? p.g_kv_stride : p.chunk_bytes;
  if (p.kv_dim > 1 && p.g_kv_stride != p.chunk_bytes) return false;
  const int64_t layer_span = kv_span * p.kv_dim;
  if (p.num_layers > 1 && p.g_layer_stride != layer_span) return false;
  // consecutive blocks must abut, otherwise a run is not one span
  return p.g_block_stride == layer_span * p.num_layers && p.layer_start == 0;
}

inline uint64_t gpu_addr(const KvCopyParams& p, int layer, int kv, int64_t block) {
  return kv_gpu_tensor(p, layer * p.idx_layer_mul + kv * p.idx_kv_mul) + (uint64_t)(layer * p.g_layer_stride) +
         (uint64_t)(kv * p.g_kv_stride) + (uint64_t)(block * p.g_block_stride) + (uint64_t)p.g_off;
}
inline uint64_t cpu_addr(const KvCopyParams& p, int layer, int kv, int64_t block) {
  const uint64_t base = p.c_use_table ? kv_c_tensor(p, layer * p.c_idx_layer_mul + kv * p.c_idx_kv_mul) : p.cpu_base;
  return base + (uint64_t)(layer * p.c_layer_stride) + (uint64_t)(kv * p.c_kv_stride) +
         (uint64_t)(block * p.c_block_stride) + (uint64_t)p.c_off;
}

}  // namespace

int64_t ce_num_copies(const CeAnalysis& a, const KvCopyParams& p, CePath path) {
  if (path == CePath::CONTIG_BLOCKS) return (int64_t)a.runs.size();
  if (path == CePath::SEGMENT_2D) return (int64_t)a.runs.size() * p.num_layers * p.kv_dim;
  return 0;
}

CePath ce_choose(const CeAnalysis& a, const KvCopyParams& p, const CePolicy& pol) {
  if (a.runs.empty() || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return CePath::KERNEL;
  const int64_t total_bytes = a.num_blocks * p.num_layers * p.kv_dim * p.chunk_bytes;
  const CePath candidates[2] = {CePath::CONTIG_BLOCKS, CePath::SEGMENT_2D};
  for (CePath path : candidates) {
    if (path == CePath::CONTIG_BLOCKS && !block_geometry_matches(p)) continue;
    const int64_t copies = ce_num_copies(a, p, path);
    if (copies <= pol.max_copies && total_bytes / copies >= pol.min_bytes_per_copy) return path;
  }
  return CePath::KERNEL;
}

cudaError_t ce_copy(const KvCopyParams& p, const CeAnalysis& a, CePath path, cudaStream_t stream) {
  const cudaMemcpyKind kind = p.h2d ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
  for (const CeRun& r : a.runs) {
    if (path == CePath::CONTIG_BLOCKS) {
      void* ga = reinterpret_cast<void*>(gpu_addr(p, p.layer_start, 0, r.gpu_block));
      void* ca = reinterpret_cast<void*>(cpu_addr(p, p.layer_start, 0, r.cpu_block));
      const size_t bytes = (size_t)(r.len * p.g_block_stride);
      cudaError_t e = p.h2d ? cudaMemcpyAsync(ga, ca, bytes, kind, stream) : cudaMemcpyAsync(ca, ga, bytes, kind, stream);
      if (e != cudaSuccess) return e;
      continue;
    }
    for (int l = 0; l < p.num_layers; ++l) {
      const int layer = p.layer_start + l;
      for (int kv = 0; kv < p.kv_dim; ++kv) {
        void* ga = reinterpret_cast<void*>(gpu_addr(p, layer, kv, r.gpu_block));
        void* ca = reinterpret_cast<void*>(cpu_addr(p, layer, kv, r.cpu_block));
        cudaError_t e;
        if (r.len == 1 || (p.g_block_stride == p.chunk_bytes && p.c_block_stride == p.chunk_bytes)) {
          const size_t bytes = (size_t)(r.len * p.chunk_bytes);
          e = p.h2d ? cudaMemcpyAsync(ga, ca, bytes, kind, stream) : cudaMemcpyAsync(ca, ga, bytes, kind, stream);
        } else if (p.h2d) {
          e = cudaMemcpy2DAsync(ga, (size_t)p.g_block_stride, ca, (size_t)p.c_block_stride, (size_t)p.chunk_bytes,
                                (size_t)r.len, kind, stream);
        } else {
          e = cudaMemcpy2DAsync(ca, (size_t)p.c_block_stride, ga, (size_t)p.g_block_stride, (size_t)p.chunk_bytes,
                                (size_t)r.len, kind, stream);
        }
        if (e != cudaSuccess) return e;
      }
    }
  }
  return cudaSuccess;
}

// ---------------------------------------------------------------- staged route

void ce_staging_free(CeStaging& st) {
  for (int b = 0; b < 2; ++b) {
    if (st.buf[b]) cudaFree(st.buf[b]);
    if (st.kernel_done[b]) cudaEventDestroy(st.kernel_done[b]);
    if (st.copy_done[b]) cudaEventDestroy(st.copy_done[b]);
    st.buf[b] = nullptr;
    st.kernel_done[b] = st.copy_done[b] = nullptr;
  }
  if (st.iota) cudaFree(st.iota);
  if (st.copy_stream) cudaStreamDestroy(st.copy_stream);
  st.iota = nullptr;
  st.copy_stream = nullptr;
  st.blocks = 0;
}

bool ce_host_runs(const KvCopyParams& p, const int64_t* g, const int64_t* c, int64_t n, int total_layers,
                  int64_t min_run, std::vector<CeHostRun>& runs) {
  runs.clear();
  if (n <= 0 || p.c_use_table || p.layer_start != 0 || p.num_layers != total_layers || p.c_off != 0) return false;
  if (p.c_kv_stride != p.chunk_bytes || p.c_layer_stride != p.chunk_bytes * p.kv_dim ||
      p.c_block_stride != p.c_layer_stride * p.num_layers)
    return false;                                          // host blocks do not abut in [layer][kv][chunk] order
  for (int64_t i = 0; i < n; ++i) {
    if (p.gpu_num_blocks > 0 && (g[i] < 0 || g[i] >= p.gpu_num_blocks)) return false;
    if (p.cpu_num_blocks > 0 && (c[i] < 0 || c[i] >= p.cpu_num_blocks)) return false;
    if (!runs.empty() && c[i] == runs.back().cpu_block + runs.back().len) {
      ++runs.back().len;
      continue;
    }
    if (!runs.empty() && runs.back().len < min_run) return false;
    runs.push_back(CeHostRun{i, c[i], 1});
  }
  return runs.back().len >= min_run;
}

static cudaError_t staging_prepare(CeStaging& st, int64_t blocks, int64_t block_bytes) {
  if (st.blocks >= blocks && st.block_bytes == block_bytes) return cudaSuccess;
  ce_staging_free(st);
  cudaError_t e = cudaSuccess;
  for (int b = 0; b < 2 && e == cudaSuccess; ++b) {
    e = cudaMalloc((void**)&st.buf[b], (size_t)(blocks * block_bytes));
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&st.kernel_done[b], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&st.copy_done[b], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaMalloc((void**)&st.iota, (size_t)blocks * sizeof(int64_t));
  if (e == cudaSuccess) {
    std::vector<int64_t> ids((size_t)blocks);
    for (int64_t i = 0; i < blocks; ++i) ids[(size_t)i] = i;
    e = cudaMemcpy(st.iota, ids.data(), ids.size() * sizeof(int64_t), cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&st.copy_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    ce_staging_free(st);
    return e;
  }
  st.blocks = blocks;
  st.block_bytes = block_bytes;
  st.used[0] = st.used[1] = false;
  return cudaSuccess;
}

cudaError_t ce_copy_staged(const KvCopyParams& p, const std::vector<CeHostRun>& runs, CeStaging& st,
                           int64_t staging_blocks, const KvCopyLaunch& cfg, cudaStream_t stream) {
  const int64_t block_bytes = p.c_block_stride;
  cudaError_t e = staging_prepare(st, staging_blocks, block_bytes);
  if (e != cudaSuccess) return e;
  int k = 0;
  for (const CeHostRun& r : runs) {
    for (int64_t lo = 0; lo < r.len; lo += st.blocks, ++k) {
      const int b = k & 1;
      const int64_t m = std::min(st.blocks, r.len - lo);
      uint8_t* host = reinterpret_cast<uint8_t*>(p.cpu_base) + (r.cpu_block + lo) * block_bytes;
      KvCopyParams q = p;            // the staging buffer plays the host side, in host block format
      q.cpu_base = reinterpret_cast<uint64_t>(st.buf[b]);
      q.gpu_blocks = p.gpu_blocks + r.first + lo;
      q.cpu_blocks = st.iota;
      q.num_pairs = (int32_t)m;
      q.cpu_num_blocks = st.blocks;
      q.done_counter = nullptr;
      q.dev_flags = q.host_flags = nullptr;
      q.layer_major = 0;
      if (!p.h2d) {
        // gather on `stream` once the previous copy out of this buffer is done, then one large copy
        if (st.used[b]) e = cudaStreamWaitEvent(stream, st.copy_done[b], 0);
        if (e == cudaSuccess) e = launch_kv_copy(q, cfg, stream);
        if (e == cudaSuccess) e = cudaEventRecord(st.kernel_done[b], stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(st.copy_stream, st.kernel_done[b], 0);
        if (e == cudaSuccess)
          e = cudaMemcpyAsync(host, st.buf[b], (size_t)(m * block_bytes), cudaMemcpyDeviceToHost, st.copy_stream);
        if (e == cudaSuccess) e = cudaEventRecord(st.copy_done[b], st.copy_stream);
      } else {
        // one large copy in once the previous scatter out of this buffer is done, then the scatter kernel
        if (st.used[b]) e = cudaStreamWaitEvent(st.copy_stream, st.kernel_done[b], 0);
        if (e == cudaSuccess)
          e = cudaMemcpyAsync(st.buf[b], host, (size_t)(m * block_bytes), cudaMemcpyHostToDevice, st.copy_stream);
        if (e == cudaSuccess) e = cudaEventRecord(st.copy_done[b], st.copy_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, st.copy_done[b], 0);
        if (e == cudaSuccess) e = launch_kv_copy(q, cfg, stream);
        if (e == cudaSuccess) e = cudaEventRecord(st.kernel_done[b], stream);
      }
      if (e != cudaSuccess) return e;
      st.used[b] = true;
    }
  }
  // the caller's stream ends after the last copies
  for (int b = 0; b < 2 && e == cudaSuccess; ++b)
    if (st.used[b]) e = cudaStreamWaitEvent(stream, st.copy_done[b], 0);
  return e;
}

}  // namespace fkv
