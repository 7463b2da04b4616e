// Paged KV gather/scatter between a GPU block table and a host block pool.
//
// One launch moves, for every (gpu_block, cpu_block) pair, every layer in
// [layer_start, layer_start + num_layers) and every kv plane, one contiguous
// chunk of `chunk_bytes`. The two sides are addressed independently, which is
// what converts between the engine's paged layout and the host block format:
//
//   gpu = gpu_ptrs[layer*idx_layer_mul + kv*idx_kv_mul]
//         + layer*g_layer_stride + kv*g_kv_stride + gpu_block*g_block_stride + g_off
//   cpu = cpu_base + layer*c_layer_stride + kv*c_kv_stride + cpu_block*c_block_stride + c_off
//         (cpu_base is replaced by a second tensor table for GPU<->GPU moves, see c_ptrs)
//
// vLLM (one tensor per layer):      idx_layer_mul=1, idx_kv_mul=0, g_layer_stride=0
// TensorRT-LLM (one tensor):        idx_*=0, all three g_* strides set
// SGLang (K tensors then V tensors):idx_layer_mul=1, idx_kv_mul=num_layers, g_kv_stride=g_layer_stride=0
// (reference addressing rules: csrc/gtensor_handler.cuh:43-67).
//
// The block-id arrays may live in mapped pinned host memory: the kernels read
// them directly, so an op needs no staging copy before the launch.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace fkv {

constexpr int kMaxGpuPtrs = 256;      // tensor pointers carried inside the launch parameters
constexpr int kMaxGpuPtrsExt = 16384; // tensor pointers in a table of its own (gpu_ptrs_ext), for larger registrations

#if defined(__CUDACC__)
#define FKV_HD __host__ __device__ __forceinline__
#else
#define FKV_HD inline
#endif
constexpr int kStatusWords = 8;   // status arrays hold one int32 per KvCopyStatus bit

enum KvCopyStatus : int {
  KV_OK = 0,
  KV_ERR_GPU_BLOCK_RANGE = 1,   // a gpu block id outside [0, gpu_num_blocks)
  KV_ERR_CPU_BLOCK_RANGE = 2,   // a cpu block id outside [0, cpu_num_blocks)
  KV_ERR_WAIT_EXPIRED = 4,      // a bounded wait on a bulk copy ran out
  KV_ERR_BAD_ARGS = 8,
  KV_ERR_PAYLOAD_OVERFLOW = 16, // compressed payload larger than its slot
  KV_ERR_PEER_WAIT_EXPIRED = 32,
};

struct KvCopyParams {
  uint64_t gpu_ptrs[kMaxGpuPtrs];
  int32_t idx_layer_mul;
  int32_t idx_kv_mul;
  int64_t g_layer_stride, g_kv_stride, g_block_stride, g_off;
  uint64_t cpu_base;
  int64_t c_layer_stride, c_kv_stride, c_block_stride, c_off;
  // The "cpu" side may itself be a table of tensors (a peer GPU's paged cache
  // reached over NVLink): when c_use_table is set its base is
  // c_ptrs[layer*c_idx_layer_mul + kv*c_idx_kv_mul] instead of cpu_base.
  uint64_t c_ptrs[kMaxGpuPtrs];
  int32_t c_use_table, c_idx_layer_mul, c_idx_kv_mul;
  // how many leading entries of gpu_ptrs / c_ptrs the caller filled: every launch path rejects a call whose
  // largest table index (last layer, last kv plane) is not below these counts
  int32_t num_gpu_ptrs, num_c_ptrs, pad0_;
  // A registration of more than kMaxGpuPtrs tensors (K and V tensors of a model deeper than 128 layers) keeps
  // its table outside the parameters: `*_ext` is the table as the executing side reads it (device memory for a
  // kernel, host memory for host_kv_copy), `*_ext_host` the same entries readable by the launching host code
  // (argument checks, copy-engine planning). Null: the inline arrays above are the table.
  const uint64_t* gpu_ptrs_ext;
  const uint64_t* gpu_ptrs_ext_host;
  const uint64_t* c_ptrs_ext;
  const uint64_t* c_ptrs_ext_host;
  const int64_t* gpu_blocks;
  const int64_t* cpu_blocks;
  int32_t num_pairs;
  int32_t layer_start, num_layers, kv_dim;
  int64_t chunk_bytes;
  int64_t gpu_num_blocks, cpu_num_blocks;  // <= 0 disables the range check
  int32_t* status;                         // device or mapped int32[kStatusWords], word b set to 1 when bit b
                                           // of KvCopyStatus occurred; may be null
  int32_t h2d;                             // 1: host -> gpu, 0: gpu -> host
  // Optional completion signal, fused into the copy: every CTA bumps
  // `done_counter` (device scratch word, zero between launches) after its last
  // store has landed; the last one resets the counter and publishes `epoch` to
  // flag words [layer_start, layer_start + num_layers) of `dev_flags` (device
  // memory, for consumer kernels on this GPU) and `host_flags` (mapped host
  // memory, for a polling host thread). All three may be null.
  //
  // With `layer_major` set (bulk engine only) the tiles are walked layer by
  // layer inside ONE launch and the signal is per layer: `done_counter` is then
  // an array of num_layers words and the flag of layer l is published as soon
  // as every CTA has drained its share of layers <= l, while later layers are
  // still in flight.
  uint32_t* done_counter;
  uint32_t* dev_flags;
  uint32_t* host_flags;
  uint32_t epoch;
  int32_t layer_major;
};

// Entry i of the two tensor tables, wherever they live. Device code reads the device view, host code the host view.
FKV_HD uint64_t kv_gpu_tensor(const KvCopyParams& p, int i) {
#if defined(__CUDA_ARCH__)
  return p.gpu_ptrs_ext ? p.gpu_ptrs_ext[i] : p.gpu_ptrs[i];
#else
  return p.gpu_ptrs_ext_host ? p.gpu_ptrs_ext_host[i] : p.gpu_ptrs[i];
#endif
}
FKV_HD uint64_t kv_c_tensor(const KvCopyParams& p, int i) {
#if defined(__CUDA_ARCH__)
  return p.c_ptrs_ext ? p.c_ptrs_ext[i] : p.c_ptrs[i];
#else
  return p.c_ptrs_ext_host ? p.c_ptrs_ext_host[i] : p.c_ptrs[i];
#endif
}

struct KvCopyLaunch {
  int32_t num_ctas;     // persistent CTAs (each one bulk-copy pipeline)
  int32_t tile_bytes;   // multiple of 16, <= 32 KiB
  int32_t engine;       // 0 = TMA bulk pipeline, 1 = SIMT vector ld/st
};

// Returns cudaSuccess or the launch error. `chunk_bytes`, all strides and
// offsets must be multiples of 16 for the TMA engine; the SIMT engine accepts
// any multiple of 4 (and single bytes through its tail path).
cudaError_t launch_kv_copy(const KvCopyParams& p, const KvCopyLaunch& cfg, cudaStream_t stream);

// Re-statement of the reference's copy kernel shape for baseline timing only:
// 4 CTAs x 1024 threads, one warp per (layer, pair), lanes move 16 bytes
// (reference: csrc/transfer.cu:95-158,176-190).
cudaError_t launch_kv_copy_refshape(const KvCopyParams& p, int num_ctas, cudaStream_t stream);

// Same addressing executed on the CPU with memcpy; every pointer (gpu_ptrs
// included) is a host address. Returns the OR of KvCopyStatus bits.
int host_kv_copy(const KvCopyParams& p, int num_threads);

// folds a status array back into a KvCopyStatus bit mask and clears it
inline int collect_status(volatile int32_t* words) {
  int m = 0;
  for (int b = 0; b < kStatusWords; ++b)
    if (words[b]) { m |= 1 << b; words[b] = 0; }
  return m;
}

// true when every address component allows 16-byte bulk copies
bool kv_copy_tma_eligible(const KvCopyParams& p);

// True when the tensor tables cover every (layer, kv) the call addresses: index multipliers and the layer
// range are non-negative, the largest index layer*idx_layer_mul + kv*idx_kv_mul is below the filled count
// (at most kMaxGpuPtrs for the inline arrays, kMaxGpuPtrsExt for a table of its own, which must come with
// its host view) and no addressed entry is null; the same for the c_ptrs table when it is in use. A short
// pointer list after a re-registration or wrong multipliers are refused here, on the host, instead of
// sending the kernel to a zero or foreign address.
inline bool kv_copy_tables_ok(const KvCopyParams& p) {
  if (p.num_layers < 0 || p.layer_start < 0 || p.kv_dim < 0) return false;
  if (p.num_layers == 0 || p.kv_dim == 0) return true;   // nothing is addressed
  auto table_ok = [&](const uint64_t* inl, const uint64_t* ext, const uint64_t* ext_host, int32_t filled,
                      int32_t lmul, int32_t kmul) {
    if ((ext == nullptr) != (ext_host == nullptr)) return false;
    const uint64_t* tbl = ext_host ? ext_host : inl;
    if (lmul < 0 || kmul < 0 || filled <= 0 || filled > (ext_host ? kMaxGpuPtrsExt : kMaxGpuPtrs)) return false;
    const int64_t last = (int64_t)(p.layer_start + p.num_layers - 1) * lmul + (int64_t)(p.kv_dim - 1) * kmul;
    if (last >= filled) return false;
    for (int32_t l = p.layer_start; l < p.layer_start + p.num_layers; ++l)
      for (int32_t k = 0; k < p.kv_dim; ++k)
        if (tbl[(int64_t)l * lmul + (int64_t)k * kmul] == 0) return false;
    return true;
  };
  if (!table_ok(p.gpu_ptrs, p.gpu_ptrs_ext, p.gpu_ptrs_ext_host, p.num_gpu_ptrs, p.idx_layer_mul, p.idx_kv_mul))
    return false;
  if (p.c_use_table &&
      !table_ok(p.c_ptrs, p.c_ptrs_ext, p.c_ptrs_ext_host, p.num_c_ptrs, p.c_idx_layer_mul, p.c_idx_kv_mul))
    return false;
  return true;
}

}  // namespace fkv
