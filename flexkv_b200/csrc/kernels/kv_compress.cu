#include "kv_compress.h"

#include "ptx_sm100.cuh"

namespace fkv {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kGroup = 128;
constexpr int kGroupsPerTile = kCompressTileElems / kGroup;   // 64
constexpr int kInStages = 5;
constexpr int kEpoch = 2048;                                  // tile sizes fetched per batch (decompress)
constexpr uint64_t kWaitBudgetNs = 2000000000ull;

struct __align__(16) Smem {
  uint8_t in[kInStages][kCompressTileSlot];
  uint8_t out[2][kCompressTileSlot];
};

__device__ __forceinline__ int bits_for(int range) {   // smallest w with range < 2^w
  return range == 0 ? 0 : 32 - __clz(range);
}

constexpr int kTblBatch = 32;   // size-table entries written per bulk store (128 bytes)

template <bool COMPRESS>
__global__ void __launch_bounds__(kThreads, 1)
kv_compress_kernel(const __grid_constant__ KvCopyParams p, uint32_t* __restrict__ size_table, int layers_total,
                   int tiles_per_chunk) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  __shared__ __align__(8) uint64_t full[kInStages];
  __shared__ uint64_t s_dst[kInStages];
  __shared__ uint64_t s_table_idx[kInStages];
  __shared__ __align__(128) uint32_t s_tbl[3][kTblBatch];
  __shared__ int32_t s_elems[kInStages];
  __shared__ int32_t s_w[kGroupsPerTile];
  __shared__ int32_t s_off[kGroupsPerTile + 1];
  __shared__ uint32_t s_sizes[kEpoch];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < kInStages; ++s) ptx::mbar_init(&full[s], 1);
    s_abort = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();

  const int64_t chunk_elems = p.chunk_bytes / 2;
  const int32_t span = p.num_layers * p.kv_dim * tiles_per_chunk;
  const int64_t total = (int64_t)span * p.num_pairs;
  // every CTA owns one contiguous run of tiles: consecutive tiles share their block ids (fetched
  // once per pair, possibly over PCIe) and their size-table neighbourhood
  const int64_t per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int64_t first = (int64_t)blockIdx.x * per_cta, step = 1;
  const int64_t n_mine = first < total ? (total - first < per_cta ? total - first : per_cta) : 0;
  // thread 0 keeps the ids of the pair it is working on and asks for the next pair's early
  int32_t id_pair = -1;
  int64_t id_g = 0, id_c = 0, nx_g = 0, nx_c = 0;
  auto pair_ids = [&](int32_t pair, int64_t& g, int64_t& c) {
    if (pair != id_pair) {
      if (pair == id_pair + 1 && id_pair >= 0) { id_g = nx_g; id_c = nx_c; }
      else { id_g = __ldg(p.gpu_blocks + pair); id_c = __ldg(p.cpu_blocks + pair); }
      id_pair = pair;
      if (pair + 1 < p.num_pairs) { nx_g = __ldg(p.gpu_blocks + pair + 1); nx_c = __ldg(p.cpu_blocks + pair + 1); }
    }
    g = id_g; c = id_c;
  };
  int err = 0;
  uint32_t phases = 0;

  // decodes tile `it` of this CTA; returns false for a pair whose ids are out of range
  auto locate = [&](int64_t it, uint64_t& g, uint64_t& c, uint64_t& tidx, int32_t& elems, bool cached) -> bool {
    const int64_t t = first + it * step;
    const int32_t pair = (int32_t)(t / span), r = (int32_t)(t % span);
    const int s_ = r % tiles_per_chunk, q = r / tiles_per_chunk;
    const int kv = q % p.kv_dim, layer = p.layer_start + q / p.kv_dim;
    int64_t gblk, cblk;
    if (cached) pair_ids(pair, gblk, cblk);
    else { gblk = __ldg(p.gpu_blocks + pair); cblk = __ldg(p.cpu_blocks + pair); }
    bool ok = true;
    if (p.gpu_num_blocks > 0 && (gblk < 0 || gblk >= p.gpu_num_blocks)) { err |= KV_ERR_GPU_BLOCK_RANGE; ok = false; }
    if (p.cpu_num_blocks > 0 && (cblk < 0 || cblk >= p.cpu_num_blocks)) { err |= KV_ERR_CPU_BLOCK_RANGE; ok = false; }
    const int64_t e0 = (int64_t)s_ * kCompressTileElems;
    const int64_t left = chunk_elems - e0;
    elems = (int32_t)(left < kCompressTileElems ? left : kCompressTileElems);
    g = p.gpu_ptrs[layer * p.idx_layer_mul + kv * p.idx_kv_mul] + layer * p.g_layer_stride + kv * p.g_kv_stride +
        gblk * p.g_block_stride + p.g_off + e0 * 2;
    c = p.cpu_base + layer * p.c_layer_stride + kv * p.c_kv_stride + cblk * p.c_block_stride + p.c_off +
        (int64_t)s_ * kCompressTileSlot;
    tidx = (((uint64_t)cblk * layers_total + layer) * p.kv_dim + kv) * tiles_per_chunk + s_;
    return ok;
  };

  auto issue_load = [&](int64_t it) {   // thread 0
    const int st = (int)(it % kInStages);
    uint64_t g, c, tidx;
    int32_t elems;
    const bool ok = locate(it, g, c, tidx, elems, true);
    s_table_idx[st] = tidx;
    if (!ok) {
      s_elems[st] = 0;
      ptx::mbar_arrive(&full[st]);
      return;
    }
    s_elems[st] = elems;
    if (COMPRESS) {
      s_dst[st] = c;
      ptx::mbar_expect_tx(&full[st], (uint32_t)elems * 2);
      ptx::bulk_g2s(sm.in[st], reinterpret_cast<const void*>(g), (uint32_t)elems * 2, &full[st]);
    } else {
      s_dst[st] = g;
      uint32_t sz = s_sizes[it % kEpoch];
      const uint32_t cap = 2u * (uint32_t)(elems / kGroup) + 256u * (uint32_t)(elems / kGroup);
      if (sz < 16 || sz > cap || (sz & 15u)) {   // a slot that was never written or a corrupt table entry
        err |= KV_ERR_PAYLOAD_OVERFLOW;
        s_elems[st] = 0;
        ptx::mbar_arrive(&full[st]);
        return;
      }
      ptx::mbar_expect_tx(&full[st], sz);
      ptx::bulk_g2s(sm.in[st], reinterpret_cast<const void*>(c), sz, &full[st]);
    }
  };

  // decompress: the sizes of this CTA's next kEpoch tiles are fetched by all threads at once
  auto fetch_sizes = [&](int64_t from) {
    for (int64_t it = from + tid; it < n_mine && it < from + kEpoch; it += kThreads) {
      uint64_t g, c, tidx;
      int32_t elems;
      int keep = err;
      locate(it, g, c, tidx, elems, false);
      err = keep;                      // range errors are reported once, by thread 0 at issue time
      s_sizes[it % kEpoch] = __ldg(size_table + tidx);
    }
  };

  // thread 0, compress: pending size-table entries. Three buffers in rotation: a flushed buffer is read by
  // the bulk copy of the tile's commit group, and the per-tile wait below lets one group stay in flight.
  uint64_t tbl_start = 0;
  int tbl_n = 0, tbl_buf = 0;
  auto flush_table = [&]() {
    uint32_t* dst = size_table + tbl_start;
    if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0 && (tbl_n & 3) == 0) {
      ptx::fence_proxy_async_smem();      // this thread's plain stores to s_tbl before the bulk read
      ptx::bulk_s2g(dst, s_tbl[tbl_buf], (uint32_t)tbl_n * 4);
    } else {
      for (int i = 0; i < tbl_n; ++i) dst[i] = s_tbl[tbl_buf][i];
    }
    tbl_buf = tbl_buf == 2 ? 0 : tbl_buf + 1;
    tbl_n = 0;
  };

  if (!COMPRESS) { fetch_sizes(0); __syncthreads(); }
  if (tid == 0)
    for (int64_t it = 0; it < n_mine && it < kInStages - 1; ++it) issue_load(it);

  for (int64_t it = 0; it < n_mine; ++it) {
    const int st = (int)(it % kInStages), ob = (int)(it & 1);
    if (!COMPRESS) {
      // the prefetch below reaches kInStages-1 tiles ahead: refill the size ring before it crosses into a new epoch
      const int64_t ahead = it + kInStages - 1;
      if (ahead % kEpoch == 0 && ahead > 0 && ahead < n_mine) { __syncthreads(); fetch_sizes(ahead); __syncthreads(); }
    }
    if (tid == 0) {
      if (it + kInStages - 1 < n_mine) issue_load(it + kInStages - 1);
      if (it >= 2) ptx::bulk_wait_read<1>();
    }
    __syncthreads();
    const int ok = ptx::mbar_wait_bounded(&full[st], (phases >> st) & 1u, kWaitBudgetNs) ? 1 : 0;
    phases ^= 1u << st;
    if (!__syncthreads_and(ok)) {
      if (tid == 0) s_abort = 1;
      break;
    }
    const int elems = s_elems[st];
    const int groups = elems / kGroup;
    const int hdr = (groups * 2 + 15) & ~15;
    uint32_t out_bytes = 0;
    if (COMPRESS) {
      const uint16_t* src = reinterpret_cast<const uint16_t*>(sm.in[st]);
      uint8_t* out = sm.out[ob];
      // pass 1: exponent range of every group -> header and widths
      for (int g = warp; g < groups; g += kWarps) {
        const uint2 raw = *reinterpret_cast<const uint2*>(src + g * kGroup + lane * 4);
        const int e0 = (raw.x >> 7) & 0xff, e1 = (raw.x >> 23) & 0xff, e2 = (raw.y >> 7) & 0xff, e3 = (raw.y >> 23) & 0xff;
        int emax = max(max(e0, e1), max(e2, e3)), emin = min(min(e0, e1), min(e2, e3));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          emax = max(emax, __shfl_xor_sync(0xffffffffu, emax, o));
          emin = min(emin, __shfl_xor_sync(0xffffffffu, emin, o));
        }
        if (lane == 0) {
          const int w = bits_for(emax - emin);
          s_w[g] = w;
          out[2 * g] = (uint8_t)emax;
          out[2 * g + 1] = (uint8_t)w;
        }
      }
      __syncthreads();
      if (warp == 0) {   // exclusive scan of the group sizes (two groups per lane)
        const int a = lane * 2 < groups ? kGroup + 16 * s_w[lane * 2] : 0;
        const int b = lane * 2 + 1 < groups ? kGroup + 16 * s_w[lane * 2 + 1] : 0;
        int incl = a + b;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        const int excl = incl - (a + b);
        s_off[lane * 2] = hdr + excl;
        s_off[lane * 2 + 1] = hdr + excl + a;
        if (lane == 31) s_off[kGroupsPerTile] = hdr + incl;
      }
      __syncthreads();
      // pass 2: sign|mantissa bytes and the bit planes of the exponent distances
      for (int g = warp; g < groups; g += kWarps) {
        const uint2 raw = *reinterpret_cast<const uint2*>(src + g * kGroup + lane * 4);
        const uint32_t v0 = raw.x & 0xffffu, v1 = raw.x >> 16, v2 = raw.y & 0xffffu, v3 = raw.y >> 16;
        const int emax = out[2 * g], w = s_w[g];
        uint8_t* gp = out + s_off[g];
        const uint32_t sm4 = (((v0 >> 8) & 0x80u) | (v0 & 0x7fu)) | ((((v1 >> 8) & 0x80u) | (v1 & 0x7fu)) << 8) |
                             ((((v2 >> 8) & 0x80u) | (v2 & 0x7fu)) << 16) | ((((v3 >> 8) & 0x80u) | (v3 & 0x7fu)) << 24);
        *reinterpret_cast<uint32_t*>(gp + lane * 4) = sm4;
        const int d0 = emax - (int)((v0 >> 7) & 0xff), d1 = emax - (int)((v1 >> 7) & 0xff),
                  d2 = emax - (int)((v2 >> 7) & 0xff), d3 = emax - (int)((v3 >> 7) & 0xff);
        uint32_t mine = 0;   // lane (b*4 + j) keeps the plane (b, j)
        for (int b = 0; b < w; ++b) {
          const uint32_t p0 = __ballot_sync(0xffffffffu, (d0 >> b) & 1), p1 = __ballot_sync(0xffffffffu, (d1 >> b) & 1),
                         p2 = __ballot_sync(0xffffffffu, (d2 >> b) & 1), p3 = __ballot_sync(0xffffffffu, (d3 >> b) & 1);
          if ((lane >> 2) == b) mine = (lane & 3) == 0 ? p0 : (lane & 3) == 1 ? p1 : (lane & 3) == 2 ? p2 : p3;
        }
        if (lane < 4 * w) *reinterpret_cast<uint32_t*>(gp + kGroup + lane * 4) = mine;
      }
      out_bytes = groups ? (uint32_t)s_off[groups] : 0;   // s_off[groups] = header + all group bodies
    } else {
      const uint8_t* in = sm.in[st];
      uint16_t* dst = reinterpret_cast<uint16_t*>(sm.out[ob]);
      if (tid < groups) s_w[tid] = in[2 * tid + 1] > 8 ? 8 : in[2 * tid + 1];
      __syncthreads();
      if (warp == 0) {
        const int a = lane * 2 < groups ? kGroup + 16 * s_w[lane * 2] : 0;
        const int b = lane * 2 + 1 < groups ? kGroup + 16 * s_w[lane * 2 + 1] : 0;
        int incl = a + b;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        const int excl = incl - (a + b);
        s_off[lane * 2] = hdr + excl;
        s_off[lane * 2 + 1] = hdr + excl + a;
      }
      __syncthreads();
      for (int g = warp; g < groups; g += kWarps) {
        const int emax = in[2 * g], w = s_w[g];
        const uint8_t* gp = in + s_off[g];
        const uint32_t sm4 = *reinterpret_cast<const uint32_t*>(gp + lane * 4);
        int d0 = 0, d1 = 0, d2 = 0, d3 = 0;
        for (int b = 0; b < w; ++b) {
          const uint4 pl = *reinterpret_cast<const uint4*>(gp + kGroup + b * 16);   // planes (b, 0..3), broadcast read
          d0 |= (int)((pl.x >> lane) & 1u) << b;
          d1 |= (int)((pl.y >> lane) & 1u) << b;
          d2 |= (int)((pl.z >> lane) & 1u) << b;
          d3 |= (int)((pl.w >> lane) & 1u) << b;
        }
        auto rebuild = [&](uint32_t smb, int d) -> uint32_t {
          return ((smb & 0x80u) << 8) | ((uint32_t)((emax - d) & 0xff) << 7) | (smb & 0x7fu);
        };
        uint2 o;
        o.x = rebuild(sm4 & 0xffu, d0) | (rebuild((sm4 >> 8) & 0xffu, d1) << 16);
        o.y = rebuild((sm4 >> 16) & 0xffu, d2) | (rebuild(sm4 >> 24, d3) << 16);
        *reinterpret_cast<uint2*>(dst + g * kGroup + lane * 4) = o;
      }
      out_bytes = (uint32_t)elems * 2;
    }
    ptx::fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      if (elems > 0 && out_bytes > 0) {
        ptx::bulk_s2g(reinterpret_cast<void*>(s_dst[st]), sm.out[ob], out_bytes);
        if (COMPRESS) {
          // Table entries of consecutive tiles are consecutive words: collect them and write 128 bytes
          // at a time instead of one 4-byte PCIe write per tile.
          const uint64_t tidx = s_table_idx[st];
          if (tbl_n > 0 && (tidx != tbl_start + (uint64_t)tbl_n || (tidx & (kTblBatch - 1)) == 0)) flush_table();
          if (tbl_n == 0) tbl_start = tidx;
          s_tbl[tbl_buf][tbl_n++] = out_bytes;
        }
      }
      ptx::bulk_commit();
    }
  }
  if (tid == 0) {
    if (COMPRESS && tbl_n > 0) { flush_table(); ptx::bulk_commit(); }
    ptx::bulk_wait<0>();
    if (s_abort) err |= KV_ERR_WAIT_EXPIRED;
    if (err && p.status)
      for (int b = 0; b < kStatusWords; ++b)
        if (err & (1 << b)) reinterpret_cast<volatile int32_t*>(p.status)[b] = 1;
  }
}

}  // namespace

cudaError_t launch_kv_compress_bf16(const KvCopyParams& p, uint32_t* size_table, int layers_total, int num_ctas,
                                    cudaStream_t stream) {
  if (p.num_pairs <= 0 || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return cudaSuccess;
  const int64_t chunk_elems = p.chunk_bytes / 2;
  if ((p.chunk_bytes & 1) || chunk_elems % 1024 != 0 || size_table == nullptr || !kv_copy_tma_eligible(p))
    return cudaErrorInvalidValue;
  const int tiles_per_chunk = (int)compress_tiles_per_chunk(chunk_elems);
  const int64_t total = (int64_t)p.num_pairs * p.num_layers * p.kv_dim * tiles_per_chunk;
  int ctas = num_ctas > 0 ? num_ctas : 32;
  if ((int64_t)ctas > total) ctas = (int)total;
  const int smem = (int)sizeof(Smem) + 128;
  cudaError_t e;
  if (p.h2d) {
    e = cudaFuncSetAttribute(kv_compress_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kv_compress_kernel<false><<<ctas, kThreads, smem, stream>>>(p, size_table, layers_total, tiles_per_chunk);
  } else {
    e = cudaFuncSetAttribute(kv_compress_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kv_compress_kernel<true><<<ctas, kThreads, smem, stream>>>(p, size_table, layers_total, tiles_per_chunk);
  }
  return cudaGetLastError();
}

}  // namespace fkv
