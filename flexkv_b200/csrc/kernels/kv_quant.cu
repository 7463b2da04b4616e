#include "kv_quant.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx_sm100.cuh"

namespace fkv {
namespace {

constexpr int kThreads = 128;
constexpr int kTileElems = 8192;             // 16 KiB of bf16 in, 8 KiB + 256 B out
constexpr int kInStages = 6;
constexpr uint64_t kWaitBudgetNs = 2000000000ull;

struct __align__(16) Smem {
  // pack: in = bf16 tile; unpack: in = e4m3 payload followed by its scales
  uint8_t in[kInStages][kTileElems * 2];
  uint8_t out[2][kTileElems * 2];
  float out_scales[2][kTileElems / kQuantGroup];
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <bool PACK>
__global__ void __launch_bounds__(kThreads, 1) kv_quant_fp8_kernel(const __grid_constant__ KvCopyParams p,
                                                                   int tiles_per_chunk) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  __shared__ __align__(8) uint64_t full[kInStages];
  __shared__ uint64_t s_dst[kInStages];       // destination of the tile's payload
  __shared__ uint64_t s_dst2[kInStages];      // pack: destination of the tile's scales
  __shared__ int32_t s_elems[kInStages];      // 0 = skipped tile
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
  uint32_t phases = 0;   // every thread tracks the parity of each stage's next completion

  // thread 0: address generation and all bulk copies
  auto issue_load = [&](int64_t it) {
    const int st = (int)(it % kInStages);
    const int64_t t = first + it * step;
    const int32_t pair = (int32_t)(t / span), r = (int32_t)(t % span);
    const int s_ = r % tiles_per_chunk, q = r / tiles_per_chunk;
    const int kv = q % p.kv_dim, layer = p.layer_start + q / p.kv_dim;
    int64_t gblk, cblk;
    pair_ids(pair, gblk, cblk);
    bool ok = true;
    if (p.gpu_num_blocks > 0 && (gblk < 0 || gblk >= p.gpu_num_blocks)) { err |= KV_ERR_GPU_BLOCK_RANGE; ok = false; }
    if (p.cpu_num_blocks > 0 && (cblk < 0 || cblk >= p.cpu_num_blocks)) { err |= KV_ERR_CPU_BLOCK_RANGE; ok = false; }
    const int64_t e0 = (int64_t)s_ * kTileElems;
    const int64_t left = chunk_elems - e0;
    const int32_t elems = (int32_t)(left < kTileElems ? left : kTileElems);
    const uint64_t g = kv_gpu_tensor(p, layer * p.idx_layer_mul + kv * p.idx_kv_mul) + layer * p.g_layer_stride +
                       kv * p.g_kv_stride + gblk * p.g_block_stride + p.g_off + e0 * 2;
    const uint64_t c = p.cpu_base + layer * p.c_layer_stride + kv * p.c_kv_stride + cblk * p.c_block_stride + p.c_off;
    const uint64_t c_payload = c + e0, c_scales = c + chunk_elems + (e0 / kQuantGroup) * 4;
    if (!ok) {
      s_elems[st] = 0;
      ptx::mbar_arrive(&full[st]);
      return;
    }
    s_elems[st] = elems;
    if (PACK) {
      s_dst[st] = c_payload;
      s_dst2[st] = c_scales;
      ptx::mbar_expect_tx(&full[st], (uint32_t)elems * 2);
      ptx::bulk_g2s(sm.in[st], reinterpret_cast<const void*>(g), (uint32_t)elems * 2, &full[st]);
    } else {
      s_dst[st] = g;
      const uint32_t sc_bytes = (uint32_t)(elems / kQuantGroup) * 4;
      ptx::mbar_expect_tx(&full[st], (uint32_t)elems + sc_bytes);
      ptx::bulk_g2s(sm.in[st], reinterpret_cast<const void*>(c_payload), (uint32_t)elems, &full[st]);
      ptx::bulk_g2s(sm.in[st] + kTileElems, reinterpret_cast<const void*>(c_scales), sc_bytes, &full[st]);
    }
  };

  if (tid == 0)
    for (int64_t it = 0; it < n_mine && it < kInStages - 1; ++it) issue_load(it);

  for (int64_t it = 0; it < n_mine; ++it) {
    const int st = (int)(it % kInStages), ob = (int)(it & 1);
    if (tid == 0) {
      // stage (it-1) % kInStages was drained by everyone before the barrier that ended iteration it-1
      if (it + kInStages - 1 < n_mine) issue_load(it + kInStages - 1);
      if (it >= 2) ptx::bulk_wait_read<1>();   // the store of tile it-2 has finished reading out[ob]
    }
    __syncthreads();
    int ok = ptx::mbar_wait_bounded(&full[st], (phases >> st) & 1u, kWaitBudgetNs) ? 1 : 0;
    phases ^= 1u << st;
    if (!__syncthreads_and(ok)) {
      if (tid == 0) s_abort = 1;
      break;
    }
    const int elems = s_elems[st];
    const int groups = elems / kQuantGroup;
    if (PACK) {
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(sm.in[st]);
      for (int gidx = warp; gidx < groups; gidx += kThreads / 32) {
        const uint2 raw = *reinterpret_cast<const uint2*>(src + gidx * kQuantGroup + lane * 4);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        const float x0 = __low2float(a), x1 = __high2float(a), x2 = __low2float(b), x3 = __high2float(b);
        const float amax = warp_max(fmaxf(fmaxf(fabsf(x0), fabsf(x1)), fmaxf(fabsf(x2), fabsf(x3))));
        const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
        const __nv_fp8x2_storage_t q01 =
            __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x0, scale), __fdiv_rn(x1, scale)), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t q23 =
            __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x2, scale), __fdiv_rn(x3, scale)), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint32_t*>(sm.out[ob] + gidx * kQuantGroup + lane * 4) = (uint32_t)q01 | ((uint32_t)q23 << 16);
        if (lane == 0) sm.out_scales[ob][gidx] = scale;
      }
    } else {
      const uint8_t* src = sm.in[st];
      const float* scales = reinterpret_cast<const float*>(sm.in[st] + kTileElems);
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(sm.out[ob]);
      for (int gidx = warp; gidx < groups; gidx += kThreads / 32) {
        const uint32_t q = *reinterpret_cast<const uint32_t*>(src + gidx * kQuantGroup + lane * 4);
        const float scale = scales[gidx];
        const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(q & 0xffffu), __NV_E4M3);
        const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(q >> 16), __NV_E4M3);
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
        const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
        __nv_bfloat162 o0 = __floats2bfloat162_rn(__fmul_rn(f01.x, scale), __fmul_rn(f01.y, scale));
        __nv_bfloat162 o1 = __floats2bfloat162_rn(__fmul_rn(f23.x, scale), __fmul_rn(f23.y, scale));
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&o0);
        packed.y = *reinterpret_cast<uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(dst + gidx * kQuantGroup + lane * 4) = packed;
      }
    }
    ptx::fence_proxy_async_smem();   // generic-proxy writes to out[] before the bulk store reads them
    __syncthreads();
    if (tid == 0) {
      if (elems > 0) {
        if (PACK) {
          ptx::bulk_s2g(reinterpret_cast<void*>(s_dst[st]), sm.out[ob], (uint32_t)elems);
          ptx::bulk_s2g(reinterpret_cast<void*>(s_dst2[st]), sm.out_scales[ob], (uint32_t)groups * 4);
        } else {
          ptx::bulk_s2g(reinterpret_cast<void*>(s_dst[st]), sm.out[ob], (uint32_t)elems * 2);
        }
      }
      ptx::bulk_commit();
    }
  }
  if (tid == 0) {
    ptx::bulk_wait<0>();
    if (s_abort) err |= KV_ERR_WAIT_EXPIRED;
    if (err && p.status)
      for (int b = 0; b < kStatusWords; ++b)
        if (err & (1 << b)) reinterpret_cast<volatile int32_t*>(p.status)[b] = 1;
  }
}

}  // namespace

cudaError_t launch_kv_quant_fp8(const KvCopyParams& p, int num_ctas, cudaStream_t stream) {
  if (p.num_pairs <= 0 || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return cudaSuccess;
  const int64_t chunk_elems = p.chunk_bytes / 2;
  if ((p.chunk_bytes & 1) || chunk_elems % 512 != 0 || !kv_copy_tma_eligible(p)) return cudaErrorInvalidValue;
  const int tiles_per_chunk = (int)((chunk_elems + kTileElems - 1) / kTileElems);
  const int64_t total = (int64_t)p.num_pairs * p.num_layers * p.kv_dim * tiles_per_chunk;
  int ctas = num_ctas > 0 ? num_ctas : 32;
  if ((int64_t)ctas > total) ctas = (int)total;
  const int smem = (int)sizeof(Smem) + 128;
  cudaError_t e;
  if (p.h2d) {
    e = cudaFuncSetAttribute(kv_quant_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kv_quant_fp8_kernel<false><<<ctas, kThreads, smem, stream>>>(p, tiles_per_chunk);
  } else {
    e = cudaFuncSetAttribute(kv_quant_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kv_quant_fp8_kernel<true><<<ctas, kThreads, smem, stream>>>(p, tiles_per_chunk);
  }
  return cudaGetLastError();
}

}  // namespace fkv
