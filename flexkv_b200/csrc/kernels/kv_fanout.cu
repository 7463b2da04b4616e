#include "kv_fanout.h"
#include "ptx_sm100.cuh"

namespace fkv {
namespace {

constexpr int kStages = 8;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = 32 * (1 + kConsumerWarps);
constexpr uint64_t kWaitBudgetNs = 2000000000ull;

__device__ __forceinline__ uint4 ld_shared_v4(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(ptx::smem_u32(p)));
  return v;
}

__device__ __forceinline__ void multimem_st_release_u32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// warp 0 streams host tiles into a shared-memory ring through the TMA unit;
// warps 1..4 drain each tile with 16-byte multimem stores
__global__ void __launch_bounds__(kThreads, 1)
kv_fanout_kernel(const __grid_constant__ KvFanoutParams fp, int tile_bytes, int tiles_per_chunk) {
  const KvCopyParams& p = fp.base;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ __align__(8) uint64_t empty[kStages];
  __shared__ uint64_t s_dst[kStages];
  __shared__ uint32_t s_bytes[kStages];
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], kConsumerWarps);
    }
    s_abort = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();

  const int32_t span = p.num_layers * p.kv_dim * tiles_per_chunk;   // tiles per pair
  const int64_t total = (int64_t)span * p.num_pairs;
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n_mine = first < total ? (total - first + step - 1) / step : 0;
  int err = 0;

  if (warp == 0) {
    // ---------------- producer
    const int32_t step_q = (int32_t)(step / span), step_r = (int32_t)(step % span);
    int32_t pair = (int32_t)(first / span), r = (int32_t)(first % span);
    int32_t cur_w = -1;
    int64_t cur_g = 0, cur_c = 0;
    for (int64_t it = 0; it < n_mine; ++it) {
      const int32_t w = pair >> 5;
      if (w != cur_w) {
        const int64_t i = ((int64_t)w << 5) + lane;
        if (i < p.num_pairs) { cur_g = __ldg(p.gpu_blocks + i); cur_c = __ldg(p.cpu_blocks + i); }
        cur_w = w;
      }
      const int64_t gblk = __shfl_sync(0xffffffffu, cur_g, pair & 31);
      const int64_t cblk = __shfl_sync(0xffffffffu, cur_c, pair & 31);
      int stop = 0;
      if (lane == 0 && *reinterpret_cast<volatile int*>(&s_abort)) stop = 1;
      if (lane == 0 && !stop) {
        const int st = (int)(it % kStages);
        const uint32_t use = (uint32_t)(it / kStages);
        // wait until the consumers released the stage (the first kStages uses start free)
        if (use > 0 && !ptx::mbar_wait_bounded(&empty[st], (use - 1) & 1u, kWaitBudgetNs)) {
          err |= KV_ERR_WAIT_EXPIRED;
          *reinterpret_cast<volatile int*>(&s_abort) = 1;
          stop = 1;
        } else {
          const int s_ = r % tiles_per_chunk, q = r / tiles_per_chunk;
          const int kv = q % p.kv_dim, layer = p.layer_start + q / p.kv_dim;
          const int64_t off = (int64_t)s_ * tile_bytes;
          const int64_t left = p.chunk_bytes - off;
          uint32_t bytes = (uint32_t)(left < tile_bytes ? left : tile_bytes);
          bool ok = true;
          if (p.gpu_num_blocks > 0 && (gblk < 0 || gblk >= p.gpu_num_blocks)) { err |= KV_ERR_GPU_BLOCK_RANGE; ok = false; }
          if (p.cpu_num_blocks > 0 && (cblk < 0 || cblk >= p.cpu_num_blocks)) { err |= KV_ERR_CPU_BLOCK_RANGE; ok = false; }
          const uint64_t g = kv_gpu_tensor(p, layer * p.idx_layer_mul + kv * p.idx_kv_mul) + layer * p.g_layer_stride +
                             kv * p.g_kv_stride + gblk * p.g_block_stride + p.g_off + off;
          const uint64_t c = p.cpu_base + layer * p.c_layer_stride + kv * p.c_kv_stride + cblk * p.c_block_stride +
                             p.c_off + off;
          // multicast twin of the local address: per-tensor table when given, else one delta for the whole cache
          const int ti = layer * p.idx_layer_mul + kv * p.idx_kv_mul;
          s_dst[st] = p.num_c_ptrs > 0 ? kv_c_tensor(p, ti) + (g - kv_gpu_tensor(p, ti)) : g + (uint64_t)fp.mc_delta;
          if (!ok) {
            // keep the barrier protocol uniform: publish an empty tile
            s_bytes[st] = 0;
            ptx::mbar_arrive(&full[st]);
          } else {
            s_bytes[st] = bytes;
            ptx::mbar_expect_tx(&full[st], bytes);
            ptx::bulk_g2s(ring + (size_t)st * tile_bytes, reinterpret_cast<const void*>(c), bytes, &full[st]);
          }
        }
      }
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (stop) break;
      pair += step_q;
      r += step_r;
      if (r >= span) { r -= span; ++pair; }
    }
  } else {
    // ---------------- consumers
    const int ctid = threadIdx.x - 32;                 // 0 .. 127
    for (int64_t it = 0; it < n_mine; ++it) {
      const int st = (int)(it % kStages);
      const uint32_t use = (uint32_t)(it / kStages);
      // every consumer thread observes the barrier itself: the completion of the phase is what
      // makes the TMA-written tile visible to that thread's shared-memory loads
      int ok = 1;
      if (*reinterpret_cast<volatile int*>(&s_abort)) ok = 0;
      else if (!ptx::mbar_wait_bounded(&full[st], use & 1u, kWaitBudgetNs)) {
        err |= KV_ERR_WAIT_EXPIRED;
        *reinterpret_cast<volatile int*>(&s_abort) = 1;
        ok = 0;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t bytes = s_bytes[st];
      uint8_t* dst = reinterpret_cast<uint8_t*>(s_dst[st]);
      const uint8_t* src = ring + (size_t)st * tile_bytes;
      const int nvec = (int)(bytes >> 4);
      for (int i = ctid; i < nvec; i += 32 * kConsumerWarps)
        ptx::multimem_st_v4(dst + (size_t)i * 16, ld_shared_v4(src + (size_t)i * 16));
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[st]);
    }
    __threadfence_system();   // this thread's multimem stores are ordered before the completion flag
  }

  __syncthreads();
  if (threadIdx.x == 0) {
    if (*reinterpret_cast<volatile int*>(&s_abort)) err |= KV_ERR_WAIT_EXPIRED;
  }
  // one reporter per warp so that no error bit is lost
  if (lane == 0 && err && p.status) {
    for (int b = 0; b < kStatusWords; ++b)
      if (err & (1 << b)) reinterpret_cast<volatile int32_t*>(p.status)[b] = 1;
  }
  if (threadIdx.x == 0 && p.done_counter) {
    __threadfence_system();
    const unsigned prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *reinterpret_cast<volatile uint32_t*>(p.done_counter) = 0;
      __threadfence_system();
      if (fp.mc_flag) multimem_st_release_u32(fp.mc_flag, p.epoch);
      if (p.host_flags) ptx::st_release_sys(p.host_flags, p.epoch);
    }
  }
}

}  // namespace

cudaError_t launch_kv_fanout(const KvFanoutParams& fp, int num_ctas, int tile_bytes, cudaStream_t stream) {
  const KvCopyParams& p = fp.base;
  if (p.num_pairs <= 0 || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return cudaSuccess;
  if (p.c_use_table) return cudaErrorInvalidValue;           // the host side is a pool, c_ptrs carries multicast bases
  if (!kv_copy_tma_eligible(p) || (fp.mc_delta & 15)) return cudaErrorInvalidValue;
  if (p.num_c_ptrs > 0) {
    if (p.num_c_ptrs != p.num_gpu_ptrs) return cudaErrorInvalidValue;
    for (int i = 0; i < p.num_c_ptrs; ++i)
      if (kv_c_tensor(p, i) == 0 || (kv_c_tensor(p, i) & 15)) return cudaErrorInvalidValue;
  }
  int tile = tile_bytes > 0 ? (tile_bytes / 16) * 16 : 16384;
  if (tile > 16384) tile = 16384;
  if (tile < 1024) tile = 1024;
  if ((int64_t)tile > p.chunk_bytes) tile = (int)p.chunk_bytes;
  const int tiles_per_chunk = (int)((p.chunk_bytes + tile - 1) / tile);
  const int64_t total = (int64_t)p.num_pairs * p.num_layers * p.kv_dim * tiles_per_chunk;
  int ctas = num_ctas > 0 ? num_ctas : 8;
  if ((int64_t)ctas > total) ctas = (int)total;
  const int smem = kStages * tile;
  cudaError_t e = cudaFuncSetAttribute(kv_fanout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  kv_fanout_kernel<<<ctas, kThreads, smem, stream>>>(fp, tile, tiles_per_chunk);
  return cudaGetLastError();
}

}  // namespace fkv
