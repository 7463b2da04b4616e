// Paged KV gather/scatter kernels (see kv_copy.h for the addressing model).
//
// Engine 0 — bulk-copy pipeline. Each persistent CTA is one warp that drives
// a ring of shared-memory stages through the TMA unit: lane 0 issues a 1-D
// bulk load (global -> shared, completion on an mbarrier) for tiles up to
// LOOKAHEAD ahead, and as each tile lands issues the matching bulk store
// (shared -> global). Either side may be mapped host memory, so the same
// pipeline does GPU->host and host->GPU with no SM load/store instructions
// on the data and no registers holding payload; the other lanes only
// prefetch block ids. Host reads need many bytes in flight to cover the PCIe
// round trip, so host->GPU runs with LOOKAHEAD = STAGES-1; GPU->host keeps
// half of the ring for queued posted writes.
//
// Engine 1 — SIMT vector copy, warp per tile, 16/8/4/1-byte lanes with an
// 8-deep unrolled load batch. It serves chunks whose size or alignment rules
// out 16-byte bulk copies (the reference needs an 8-byte path for the same
// reason: csrc/transfer.cu:34-92) and is the cross-check for engine 0.
#include "kv_copy.h"
#include "kv_signal.cuh"
#include "ptx_sm100.cuh"

namespace fkv {
namespace {

constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s per bulk-copy wait
constexpr uint64_t kSignalBudgetNs = 60000000000ull;  // signaller warp: longer than any restore, still finite

struct TileAddr {
  uint64_t gpu;
  uint64_t cpu;
  uint32_t bytes;  // 0 = skip (bad block id)
};

// Position of a tile inside the launch. Tiles are enumerated pair-major
// (pair, layer, kv, sub-tile: one host block's bytes are visited contiguously)
// or, for per-layer signalling, layer-major (layer, pair, kv, sub-tile).
struct TilePos {
  int32_t pair, layer, kv, s;
};

__device__ __forceinline__ TilePos decode_tile(const KvCopyParams& p, int32_t major, int32_t r, int tiles_per_chunk) {
  TilePos t;
  t.s = r % tiles_per_chunk;
  const int32_t q = r / tiles_per_chunk;
  if (p.layer_major) {
    t.layer = p.layer_start + major;
    t.kv = q % p.kv_dim;
    t.pair = q / p.kv_dim;
  } else {
    t.pair = major;
    t.kv = q % p.kv_dim;
    t.layer = p.layer_start + q / p.kv_dim;
  }
  return t;
}

__device__ __forceinline__ TileAddr tile_addr(const KvCopyParams& p, const TilePos& t, int64_t gblk, int64_t cblk,
                                              int tile_bytes) {
  TileAddr a;
  const int64_t off = (int64_t)t.s * tile_bytes;
  const int64_t left = p.chunk_bytes - off;
  a.bytes = (uint32_t)(left < tile_bytes ? left : tile_bytes);
  a.gpu = kv_gpu_tensor(p, t.layer * p.idx_layer_mul + t.kv * p.idx_kv_mul) + t.layer * p.g_layer_stride +
          t.kv * p.g_kv_stride + gblk * p.g_block_stride + p.g_off + off;
  const uint64_t cbase = p.c_use_table ? kv_c_tensor(p, t.layer * p.c_idx_layer_mul + t.kv * p.c_idx_kv_mul) : p.cpu_base;
  a.cpu = cbase + t.layer * p.c_layer_stride + t.kv * p.c_kv_stride + cblk * p.c_block_stride + p.c_off + off;
  return a;
}

__device__ __forceinline__ bool ids_in_range(const KvCopyParams& p, int64_t g, int64_t c, int& err) {
  bool ok = true;
  if (p.gpu_num_blocks > 0 && (g < 0 || g >= p.gpu_num_blocks)) { err |= KV_ERR_GPU_BLOCK_RANGE; ok = false; }
  if (p.cpu_num_blocks > 0 && (c < 0 || c >= p.cpu_num_blocks)) { err |= KV_ERR_CPU_BLOCK_RANGE; ok = false; }
  return ok;
}

// Layer-major launches run a second warp per CTA whose only job is the per-layer publication: fences, the
// counter atomic and the system-scope flag store issued by the copy thread itself would wait for that
// thread's loads in flight and drain the pipeline at every layer boundary. The copy thread only waits for
// its bulk stores and posts "layers [0, n) done" to a shared-memory mailbox.
template <int STAGES, int LOOKAHEAD>
__global__ void __launch_bounds__(64, 1)
kv_copy_bulk_kernel(const __grid_constant__ KvCopyParams p, int tile_bytes, int tiles_per_chunk) {
  static_assert(LOOKAHEAD >= 1 && LOOKAHEAD < STAGES, "lookahead must leave one stage for stores");
  static_assert(STAGES <= 32, "stage phases are kept in one 32-bit mask");
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[STAGES];
  __shared__ uint64_t s_dst[STAGES];
  __shared__ uint32_t s_bytes[STAGES];
  __shared__ int32_t s_layer[STAGES];   // layer-major launches: layer (relative) of the tile in the stage

  __shared__ int s_layers_done;         // mailbox: this CTA finished (stores included) layers [0, n)
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) ptx::mbar_init(&full[s], 1);
    ptx::fence_mbar_init();
    s_layers_done = 0;
  }
  __syncthreads();
  if (threadIdx.x >= 32) {
    // ---- signaller warp (present only on layer-major launches with signalling)
    if (lane != 0 || !p.layer_major || p.done_counter == nullptr) return;
    int sig = 0;
    const uint64_t t0 = ptx::globaltimer_ns();
    while (sig < p.num_layers) {
      const int d = *reinterpret_cast<volatile int*>(&s_layers_done);
      if (d > sig) {
        __threadfence_block();            // acquire side of the mailbox
        signal_layers(p, sig, d);
        sig = d;
      } else {
        if (ptx::globaltimer_ns() - t0 > kSignalBudgetNs) {   // the copy warp always posts the last layer; belt and braces
          if (p.status) report_status(p.status, KV_ERR_WAIT_EXPIRED);
          return;
        }
        __nanosleep(64);
      }
    }
    return;
  }
  const bool has_signaller = blockDim.x > 32;

  // span = tiles per major unit (a pair, or a layer when layer-major); all counts fit 32 bits
  const int32_t n_major = p.layer_major ? p.num_layers : p.num_pairs;
  const int32_t span = (p.layer_major ? p.num_pairs : p.num_layers) * p.kv_dim * tiles_per_chunk;
  const int64_t total = (int64_t)span * n_major;
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n_mine = first < total ? (total - first + step - 1) / step : 0;
  // the walk (major, r) advances by `step` tiles per iteration without divisions
  const int32_t step_q = (int32_t)(step / span), step_r = (int32_t)(step % span);
  int32_t major = (int32_t)(first / span), r = (int32_t)(first % span);

  // Block ids are fetched 32 pairs at a time, one pair per lane, and the next
  // window is requested as soon as the current one becomes active, so the
  // round trip to (possibly host-resident) id arrays is off the issue path.
  int32_t cur_w = -1;
  int64_t cur_g = 0, cur_c = 0, nxt_g = 0, nxt_c = 0;
  auto load_window = [&](int32_t w, int64_t& g, int64_t& c) {
    const int64_t i = ((int64_t)w << 5) + lane;
    if (i < p.num_pairs) {
      g = __ldg(p.gpu_blocks + i);
      c = __ldg(p.cpu_blocks + i);
    }
  };

  int err = 0;
  int dead = 0;          // set after an expired wait: stop issuing, drain, leave
  uint32_t phases = 0;   // lane 0: parity of the next completion of each stage's barrier
  int32_t signalled = 0; // lane 0, layer-major: layers [0, signalled) already reported by this CTA

  for (int64_t it = 0; it < n_mine + LOOKAHEAD && !dead; ++it) {
    const int64_t j = it - LOOKAHEAD;
    if (j >= 0 && lane == 0) {
      const int st = (int)(j % STAGES);
      const uint32_t bytes = s_bytes[st];
      if (p.layer_major && p.done_counter && s_layer[st] > signalled) {
        // first store of a later layer: everything this CTA owned in the earlier layers is committed;
        // drain those stores (the loads in flight are unaffected) and report the layers
        ptx::bulk_wait<0>();
        if (has_signaller) {
          __threadfence_block();
          *reinterpret_cast<volatile int*>(&s_layers_done) = s_layer[st];
        } else {
          signal_layers(p, signalled, s_layer[st]);
        }
        signalled = s_layer[st];
      }
      if (bytes) {
        if (ptx::mbar_wait_bounded(&full[st], (phases >> st) & 1u, kWaitBudgetNs)) {
          phases ^= 1u << st;
          ptx::bulk_s2g(reinterpret_cast<void*>(s_dst[st]), ring + (size_t)st * tile_bytes, bytes);
        } else {
          err |= KV_ERR_WAIT_EXPIRED;
        }
      }
      ptx::bulk_commit();  // one group per tile (possibly empty) keeps the wait arithmetic uniform
    }
    dead = __shfl_sync(0xffffffffu, (err & KV_ERR_WAIT_EXPIRED) ? 1 : 0, 0);
    if (dead) break;

    if (it < n_mine) {
      const TilePos t = decode_tile(p, major, r, tiles_per_chunk);
      const int32_t w = t.pair >> 5;
      if (w != cur_w) {
        if (w == cur_w + 1 && cur_w >= 0) { cur_g = nxt_g; cur_c = nxt_c; }
        else load_window(w, cur_g, cur_c);
        cur_w = w;
        load_window(w + 1, nxt_g, nxt_c);
      }
      const int64_t gblk = __shfl_sync(0xffffffffu, cur_g, t.pair & 31);
      const int64_t cblk = __shfl_sync(0xffffffffu, cur_c, t.pair & 31);
      if (lane == 0) {
        const int st = (int)(it % STAGES);
        // the stage was last used by tile it-STAGES; all but the newest
        // STAGES-LOOKAHEAD store groups must have finished reading smem
        if (it >= STAGES) ptx::bulk_wait_read<STAGES - LOOKAHEAD>();
        TileAddr a{0, 0, 0};
        if (ids_in_range(p, gblk, cblk, err)) a = tile_addr(p, t, gblk, cblk, tile_bytes);
        s_bytes[st] = a.bytes;
        s_layer[st] = major;
        if (a.bytes) {
          s_dst[st] = p.h2d ? a.gpu : a.cpu;
          ptx::mbar_expect_tx(&full[st], a.bytes);
          ptx::bulk_g2s(ring + (size_t)st * tile_bytes, reinterpret_cast<const void*>(p.h2d ? a.cpu : a.gpu),
                        a.bytes, &full[st]);
        }
      }
      major += step_q;
      r += step_r;
      if (r >= span) { r -= span; ++major; }
    }
  }
  if (lane == 0) {
    ptx::bulk_wait<0>();
    if (err && p.status) report_status(p.status, err);
    if (p.layer_major) {
      if (has_signaller) {
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&s_layers_done) = p.num_layers;   // every exit path ends here
      } else {
        signal_layers(p, signalled, p.num_layers);
      }
    } else {
      signal_done(p);
    }
  }
}

// ---------------------------------------------------------------- SIMT engine

template <typename V> struct VecIO;
template <> struct VecIO<uint4> {
  static __device__ __forceinline__ uint4 ld(const void* p) { return ptx::ld_nc_v4(p); }
  static __device__ __forceinline__ void st(void* p, const uint4& v) { ptx::st_cg_v4(p, v); }
};
template <> struct VecIO<uint2> {
  static __device__ __forceinline__ uint2 ld(const void* p) { return ptx::ld_nc_v2(p); }
  static __device__ __forceinline__ void st(void* p, const uint2& v) { ptx::st_cg_v2(p, v); }
};
template <> struct VecIO<uint32_t> {
  static __device__ __forceinline__ uint32_t ld(const void* p) { return ptx::ld_nc_u32(p); }
  static __device__ __forceinline__ void st(void* p, const uint32_t& v) { ptx::st_cg_u32(p, v); }
};
template <> struct VecIO<uint8_t> {
  static __device__ __forceinline__ uint8_t ld(const void* p) { return *reinterpret_cast<const volatile uint8_t*>(p); }
  static __device__ __forceinline__ void st(void* p, const uint8_t& v) { *reinterpret_cast<volatile uint8_t*>(p) = v; }
};

template <typename V>
__global__ void __launch_bounds__(512)
kv_copy_simt_kernel(const __grid_constant__ KvCopyParams p, int tile_bytes, int tiles_per_chunk) {
  constexpr int UNROLL = 8;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int64_t warp0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * warps_per_cta;
  const int32_t n_major = p.layer_major ? p.num_layers : p.num_pairs;
  const int32_t span = (p.layer_major ? p.num_pairs : p.num_layers) * p.kv_dim * tiles_per_chunk;
  const int64_t total = (int64_t)span * n_major;
  int err = 0;
  for (int64_t t = warp0; t < total; t += nwarps) {
    const TilePos pos = decode_tile(p, (int32_t)(t / span), (int32_t)(t % span), tiles_per_chunk);
    const int64_t gblk = __ldg(p.gpu_blocks + pos.pair);
    const int64_t cblk = __ldg(p.cpu_blocks + pos.pair);
    if (!ids_in_range(p, gblk, cblk, err)) continue;
    const TileAddr a = tile_addr(p, pos, gblk, cblk, tile_bytes);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.h2d ? a.cpu : a.gpu);
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.h2d ? a.gpu : a.cpu);
    const int nvec = (int)(a.bytes / sizeof(V));
    int i = lane;
    for (; i + 32 * (UNROLL - 1) < nvec; i += 32 * UNROLL) {
      V v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = VecIO<V>::ld(src + (size_t)(i + 32 * u) * sizeof(V));
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) VecIO<V>::st(dst + (size_t)(i + 32 * u) * sizeof(V), v[u]);
    }
    for (; i < nvec; i += 32) VecIO<V>::st(dst + (size_t)i * sizeof(V), VecIO<V>::ld(src + (size_t)i * sizeof(V)));
  }
  if (err && p.status && lane == 0) report_status(p.status, err);
  if (p.done_counter) {
    __syncthreads();
    if (threadIdx.x == 0) signal_done(p);
  }
}

// ---------------------------------------------------------------- baseline shape
// One warp per (layer, pair); inside, a loop over kv planes with 16-byte lanes.
__global__ void __launch_bounds__(1024) kv_copy_refshape_kernel(const __grid_constant__ KvCopyParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t total = (int64_t)p.num_layers * p.num_pairs;
  const int nvec = (int)(p.chunk_bytes / 16);
  for (int64_t w = warp0; w < total; w += nwarps) {
    const int layer = p.layer_start + (int)(w / p.num_pairs);
    const int64_t pair = w % p.num_pairs;
    const int64_t gblk = p.gpu_blocks[pair];
    const int64_t cblk = p.cpu_blocks[pair];
    for (int kv = 0; kv < p.kv_dim; ++kv) {
      const uint64_t g = kv_gpu_tensor(p, layer * p.idx_layer_mul + kv * p.idx_kv_mul) + layer * p.g_layer_stride +
                         kv * p.g_kv_stride + gblk * p.g_block_stride + p.g_off;
      const uint64_t c =
          p.cpu_base + layer * p.c_layer_stride + kv * p.c_kv_stride + cblk * p.c_block_stride + p.c_off;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.h2d ? c : g);
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.h2d ? g : c);
      for (int i = lane; i < nvec; i += 32) ptx::st_cg_v4(dst + (size_t)i * 16, ptx::ld_nc_v4(src + (size_t)i * 16));
    }
  }
}

template <typename K>
cudaError_t ensure_smem(K kernel, int bytes) {
  // idempotent and cheap; avoids per-device bookkeeping
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int STAGES, int LA>
cudaError_t launch_bulk(const KvCopyParams& p, int ctas, int tile_bytes, int tiles_per_chunk, cudaStream_t s) {
  const int smem = STAGES * tile_bytes;
  auto k = kv_copy_bulk_kernel<STAGES, LA>;
  cudaError_t e = ensure_smem(k, smem);
  if (e != cudaSuccess) return e;
  const int threads = (p.layer_major && p.done_counter != nullptr) ? 64 : 32;   // second warp = layer signaller
  k<<<ctas, threads, smem, s>>>(p, tile_bytes, tiles_per_chunk);
  return cudaGetLastError();
}

inline bool all_multiple(const KvCopyParams& p, int64_t m) {
  auto ok = [m](int64_t v) { return (v % m) == 0; };
  bool r = ok(p.chunk_bytes) && ok(p.g_layer_stride) && ok(p.g_kv_stride) && ok(p.g_block_stride) && ok(p.g_off) &&
           ok((int64_t)(p.cpu_base % (uint64_t)m)) && ok(p.c_layer_stride) && ok(p.c_kv_stride) &&
           ok(p.c_block_stride) && ok(p.c_off);
  const int nptr = p.idx_layer_mul == 0 && p.idx_kv_mul == 0
                       ? 1
                       : (p.layer_start + p.num_layers - 1) * p.idx_layer_mul + (p.kv_dim - 1) * p.idx_kv_mul + 1;
  for (int i = 0; i < nptr && i < p.num_gpu_ptrs; ++i) r = r && (kv_gpu_tensor(p, i) % (uint64_t)m) == 0;
  if (p.c_use_table) {
    const int nc = p.c_idx_layer_mul == 0 && p.c_idx_kv_mul == 0
                       ? 1
                       : (p.layer_start + p.num_layers - 1) * p.c_idx_layer_mul + (p.kv_dim - 1) * p.c_idx_kv_mul + 1;
    for (int i = 0; i < nc && i < p.num_c_ptrs; ++i) r = r && (kv_c_tensor(p, i) % (uint64_t)m) == 0;
  }
  return r;
}

}  // namespace

bool kv_copy_tma_eligible(const KvCopyParams& p) { return kv_copy_tables_ok(p) && all_multiple(p, 16); }

cudaError_t launch_kv_copy(const KvCopyParams& p, const KvCopyLaunch& cfg, cudaStream_t stream) {
  if (p.num_pairs <= 0 || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return cudaSuccess;
  if (!kv_copy_tables_ok(p)) return cudaErrorInvalidValue;
  int tile = cfg.tile_bytes > 0 ? cfg.tile_bytes : 16384;
  int engine = cfg.engine;
  if (engine == 0 && !all_multiple(p, 16)) engine = 1;
  if (engine == 0) {
    tile = (tile / 16) * 16;
    if (tile < 1024) tile = 1024;
    if (tile > 32768) tile = 32768;
    if ((int64_t)tile > p.chunk_bytes) tile = (int)p.chunk_bytes;
    const int tiles_per_chunk = (int)((p.chunk_bytes + tile - 1) / tile);
    const int64_t total = (int64_t)p.num_pairs * p.num_layers * p.kv_dim * tiles_per_chunk;
    int ctas = cfg.num_ctas > 0 ? cfg.num_ctas : 16;
    if ((int64_t)ctas > total) ctas = (int)total;
    // deepest ring that fits beside the static barriers (limit 227 KiB per CTA)
    const int budget = 200 * 1024;
    const int stages = budget / tile;
    if (p.h2d) {
      if (stages >= 32) return launch_bulk<32, 31>(p, ctas, tile, tiles_per_chunk, stream);
      if (stages >= 20) return launch_bulk<20, 19>(p, ctas, tile, tiles_per_chunk, stream);
      if (stages >= 12) return launch_bulk<12, 11>(p, ctas, tile, tiles_per_chunk, stream);
      if (stages >= 8) return launch_bulk<8, 7>(p, ctas, tile, tiles_per_chunk, stream);
      return launch_bulk<6, 5>(p, ctas, tile, tiles_per_chunk, stream);
    }
    if (stages >= 32) return launch_bulk<32, 16>(p, ctas, tile, tiles_per_chunk, stream);
    if (stages >= 20) return launch_bulk<20, 10>(p, ctas, tile, tiles_per_chunk, stream);
    if (stages >= 12) return launch_bulk<12, 6>(p, ctas, tile, tiles_per_chunk, stream);
    if (stages >= 8) return launch_bulk<8, 4>(p, ctas, tile, tiles_per_chunk, stream);
    return launch_bulk<6, 3>(p, ctas, tile, tiles_per_chunk, stream);
  }
  // SIMT engine
  if (tile > p.chunk_bytes) tile = (int)p.chunk_bytes;
  int vec = all_multiple(p, 16) ? 16 : all_multiple(p, 8) ? 8 : all_multiple(p, 4) ? 4 : 1;
  tile = (tile / vec) * vec;
  if (tile <= 0) tile = vec;
  const int tiles_per_chunk = (int)((p.chunk_bytes + tile - 1) / tile);
  const int64_t total = (int64_t)p.num_pairs * p.num_layers * p.kv_dim * tiles_per_chunk;
  int ctas = cfg.num_ctas > 0 ? cfg.num_ctas : 16;
  const int64_t need = (total + 15) / 16;
  if ((int64_t)ctas > need) ctas = (int)need;
  switch (vec) {
    case 16: kv_copy_simt_kernel<uint4><<<ctas, 512, 0, stream>>>(p, tile, tiles_per_chunk); break;
    case 8: kv_copy_simt_kernel<uint2><<<ctas, 512, 0, stream>>>(p, tile, tiles_per_chunk); break;
    case 4: kv_copy_simt_kernel<uint32_t><<<ctas, 512, 0, stream>>>(p, tile, tiles_per_chunk); break;
    default: kv_copy_simt_kernel<uint8_t><<<ctas, 512, 0, stream>>>(p, tile, tiles_per_chunk); break;
  }
  return cudaGetLastError();
}

cudaError_t launch_kv_copy_refshape(const KvCopyParams& p, int num_ctas, cudaStream_t stream) {
  if (p.num_pairs <= 0 || p.num_layers <= 0) return cudaSuccess;
  if (!kv_copy_tables_ok(p) || !all_multiple(p, 16)) return cudaErrorInvalidValue;
  kv_copy_refshape_kernel<<<num_ctas > 0 ? num_ctas : 4, 1024, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fkv
