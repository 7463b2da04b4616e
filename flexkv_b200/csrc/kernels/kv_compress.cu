#include "kv_compress.h"

#include "kv_signal.cuh"
#include "ptx_sm100.cuh"

namespace fkv {
namespace {

// A CTA runs kGroups independent tile pipelines of kThreads threads each (own stage ring, own scratch, own
// named barrier): one pipeline keeps a single warp per scheduler and waits out every shared-memory round
// trip; two per SM overlap each other's latencies, so half as many SMs carry the same link rate.
constexpr int kThreads = 128;
constexpr int kGroups = 2;
constexpr int kWarps = kThreads / 32;
constexpr int kEpoch = 1024;                                  // tile sizes fetched per batch (decompress)
constexpr uint64_t kWaitBudgetNs = 2000000000ull;
constexpr int kTblBatch = 32;                                 // size-table entries written per bulk store (128 bytes)
constexpr uint32_t kFull = 0xffffffffu;

template <int IN_STAGES>
struct __align__(16) Smem {
  uint8_t in[IN_STAGES][kCompressTileSlot];
  uint8_t out[2][kCompressTileSlot];
};

// barrier among the kThreads threads of one pipeline (hardware barrier 1 + group; 0 is __syncthreads')
__device__ __forceinline__ void group_sync(int grp) {
  asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(kThreads) : "memory");
}

// Per-tile scratch of the coder (static shared memory).
struct Scratch {
  uint32_t hist[kWarps][256];   // per-warp exponent histograms
  uint32_t cnt[256];            // their sum
  uint32_t code[256];           // exponent -> code bits (low 24) | code length (high 8)
  uint8_t nz[256];              // exponents that occur, compacted
  uint8_t rank[256];            // exponent -> frequency rank (kCodeRanks and above: no code of its own)
  uint32_t seg[8];              // occurrences per 32-exponent segment
  uint32_t warp_tot[kWarps];
  uint32_t cost[2];             // sampled code bits under mode 1 and mode 2
};

// code of exponent e with frequency rank r under `mode` (see kv_compress.h): bits (low 24, LSB first) | length << 24
__device__ __forceinline__ uint32_t code_of(int mode, int r, int e) {
  if (mode == 1) {
    if (r < kCodeShortRanks) return (uint32_t)r | (2u << 24);
    if (r < kCodeRanks) {
      const int n = r - kCodeShortRanks;                   // n ones between the "11" marker and the closing zero
      return 3u | (((1u << n) - 1u) << 2) | ((uint32_t)(n + 3) << 24);
    }
    return 3u | (((1u << kCodeEscapeOnes) - 1u) << 2) | ((uint32_t)e << (2 + kCodeEscapeOnes)) |
           ((uint32_t)(2 + kCodeEscapeOnes + 8) << 24);
  }
  if (r < kCodeRanks) {
    const int q = r >> 2;                                  // q ones, a zero, two bits
    return ((1u << q) - 1u) | ((uint32_t)(r & 3) << (q + 1)) | ((uint32_t)(q + 3) << 24);
  }
  return ((1u << kCodeFlatEscapeOnes) - 1u) | ((uint32_t)e << kCodeFlatEscapeOnes) |
         ((uint32_t)(kCodeFlatEscapeOnes + 8) << 24);
}
__device__ __forceinline__ uint32_t code_len(int mode, int r) { return code_of(mode, r, 0) >> 24; }

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, Scratch& sc, uint32_t& total, int grp) {
  const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) & (kWarps - 1);
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t u = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += u;
  }
  if (lane == 31) sc.warp_tot[warp] = incl;
  group_sync(grp);
  uint32_t base = 0;
  total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const uint32_t t = sc.warp_tot[w];
    if (w < warp) base += t;
    total += t;
  }
  return base + incl - v;
}

// Packs `elems` bf16 values at `in` into `out`; every thread returns the packed size (a multiple of 16).
__device__ uint32_t compress_tile(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int elems, Scratch& sc,
                                  int grp) {
  const int tid = threadIdx.x & (kThreads - 1), lane = tid & 31, warp = tid >> 5;
  const int n_chunks = elems / kCodeChunkVals;
  const uint32_t* in32 = reinterpret_cast<const uint32_t*>(in);
  const int off_sm = kCodeHeaderBytes + n_chunks, off_exp = off_sm + elems;
  constexpr int W = kCodeChunkVals / 2;     // words per chunk
  for (int i = tid; i < kWarps * 256; i += kThreads) (&sc.hist[0][0])[i] = 0;
  if (tid < kCodeRanks) out[16 + tid] = 0;
  if (tid < 2) sc.cost[tid] = 0;
  // this thread's chunk stays in registers for the three passes over it
  uint32_t x[W];
  const bool active = tid < n_chunks;
  if (active) {
#pragma unroll
    for (int k = 0; k < W; ++k) x[k] = in32[k * n_chunks + tid];
  } else {
#pragma unroll
    for (int k = 0; k < W; ++k) x[k] = 0;
  }
  group_sync(grp);
  // 1: exponent histogram over a sample (the first kCodeSampleWords words of every chunk: ranks only steer
  //    the code lengths, any table decodes) and the sign|mantissa plane
  if (active) {
    uint16_t* sm16 = reinterpret_cast<uint16_t*>(out + off_sm);
#pragma unroll
    for (int k = 0; k < W; ++k) {
      if (k % kCodeSampleStride == 0) {
        atomicAdd(&sc.hist[warp][(x[k] >> 7) & 0xffu], 1u);
        atomicAdd(&sc.hist[warp][(x[k] >> 23) & 0xffu], 1u);
      }
      sm16[k * n_chunks + tid] = (uint16_t)(((x[k] >> 8) & 0x80u) | (x[k] & 0x7fu) |
                                            ((((x[k] >> 24) & 0x80u) | ((x[k] >> 16) & 0x7fu)) << 8));
    }
  }
  group_sync(grp);
  // 2: counts, the exponents that occur, their frequency ranks -> code table and symbol table
  uint32_t c0 = 0, c1 = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) { c0 += sc.hist[w][tid]; c1 += sc.hist[w][tid + 128]; }
  sc.cnt[tid] = c0;
  sc.cnt[tid + 128] = c1;
  sc.rank[tid] = 255;
  sc.rank[tid + 128] = 255;
  const uint32_t b0 = __ballot_sync(kFull, c0 > 0), b1 = __ballot_sync(kFull, c1 > 0);
  if (lane == 0) { sc.seg[warp] = __popc(b0); sc.seg[4 + warp] = __popc(b1); }
  group_sync(grp);
  uint32_t base0 = 0, base1 = 0, n_nz = 0;
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const uint32_t v = sc.seg[s];
    if (s < warp) base0 += v;
    if (s < 4 + warp) base1 += v;
    n_nz += v;
  }
  const uint32_t lt = (1u << lane) - 1u;
  if (c0 > 0) sc.nz[base0 + __popc(b0 & lt)] = (uint8_t)tid;
  if (c1 > 0) sc.nz[base1 + __popc(b1 & lt)] = (uint8_t)(tid + 128);
  group_sync(grp);
  if (n_nz <= 32) {
    // the usual case: one warp ranks all occurring exponents through shuffles
    if (warp == 0) {
      const int b = lane < (int)n_nz ? sc.nz[lane] : 256;
      const uint32_t c = lane < (int)n_nz ? sc.cnt[b] : 0u;
      int r = 0;
      for (int j = 0; j < (int)n_nz; ++j) {
        const uint32_t co = __shfl_sync(kFull, c, j);
        const int bo = __shfl_sync(kFull, b, j);
        r += (co > c || (co == c && bo < b)) ? 1 : 0;
      }
      if (lane < (int)n_nz) {
        sc.rank[b] = (uint8_t)(r < kCodeRanks ? r : kCodeRanks);
        if (r < kCodeRanks) out[16 + r] = (uint8_t)b;
      }
      // what the sample would cost under either code
      uint32_t a1 = c * code_len(1, r < kCodeRanks ? r : kCodeRanks), a2 = c * code_len(2, r < kCodeRanks ? r : kCodeRanks);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        a1 += __shfl_xor_sync(kFull, a1, o);
        a2 += __shfl_xor_sync(kFull, a2, o);
      }
      if (lane == 0) { sc.cost[0] = a1; sc.cost[1] = a2; }
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t c = h ? c1 : c0;
      const int b = tid + 128 * h;
      if (c == 0) continue;
      int r = 0;
      for (uint32_t i = 0; i < n_nz; ++i) {
        const int bo = sc.nz[i];
        const uint32_t co = sc.cnt[bo];
        r += (co > c || (co == c && bo < b)) ? 1 : 0;
      }
      sc.rank[b] = (uint8_t)(r < kCodeRanks ? r : kCodeRanks);
      if (r < kCodeRanks) out[16 + r] = (uint8_t)b;
      atomicAdd(&sc.cost[0], c * code_len(1, r < kCodeRanks ? r : kCodeRanks));
      atomicAdd(&sc.cost[1], c * code_len(2, r < kCodeRanks ? r : kCodeRanks));
    }
  }
  group_sync(grp);
  // the code shape that is shorter for the sample; every exponent's code under it
  const int mode = sc.cost[1] < sc.cost[0] ? 2 : 1;
  {
    const int r0 = sc.rank[tid], r1 = sc.rank[tid + 128];
    sc.code[tid] = code_of(mode, r0 < kCodeRanks ? r0 : kCodeRanks, tid);
    sc.code[tid + 128] = code_of(mode, r1 < kCodeRanks ? r1 : kCodeRanks, tid + 128);
  }
  group_sync(grp);
  // 3: coded size of every chunk, their offsets, and whether coding pays at all
  uint32_t bits = 0;
  if (active) {
#pragma unroll
    for (int k = 0; k < W; ++k)
      bits += (sc.code[(x[k] >> 7) & 0xffu] >> 24) + (sc.code[(x[k] >> 23) & 0xffu] >> 24);
    out[kCodeHeaderBytes + tid] = (uint8_t)((bits + 7) >> 3);
  }
  const uint32_t nbytes = (bits + 7) >> 3;
  uint32_t total_exp;
  const uint32_t myoff = block_exclusive_scan(nbytes, sc, total_exp, grp);
  const uint32_t coded_total = ((uint32_t)off_exp + total_exp + 15u) & ~15u;
  const uint32_t raw_total = 16u + (uint32_t)elems * 2u;
  const bool coded = coded_total < raw_total;
  if (coded) {
    // 4a: the prefix codes of this thread's 64 exponents, bytes appended at the chunk's offset
    if (active) {
      uint8_t* dst = out + off_exp + myoff;
      uint64_t acc = 0;
      int nb = 0;
#pragma unroll
      for (int k = 0; k < W; ++k) {
        const uint32_t ca = sc.code[(x[k] >> 7) & 0xffu], cb = sc.code[(x[k] >> 23) & 0xffu];
        acc |= (uint64_t)(ca & 0xffffffu) << nb;
        nb += (int)(ca >> 24);
        if (nb >= 32) {                              // at most 31 + 23 bits are pending here (mode 2: 31 + 12)
          dst[0] = (uint8_t)acc; dst[1] = (uint8_t)(acc >> 8); dst[2] = (uint8_t)(acc >> 16); dst[3] = (uint8_t)(acc >> 24);
          dst += 4; acc >>= 32; nb -= 32;
        }
        acc |= (uint64_t)(cb & 0xffffffu) << nb;
        nb += (int)(cb >> 24);
        if (nb >= 32) {
          dst[0] = (uint8_t)acc; dst[1] = (uint8_t)(acc >> 8); dst[2] = (uint8_t)(acc >> 16); dst[3] = (uint8_t)(acc >> 24);
          dst += 4; acc >>= 32; nb -= 32;
        }
      }
      while (nb > 0) { *dst++ = (uint8_t)acc; acc >>= 8; nb -= 8; }
    }
    if (tid == 0) {
      for (uint32_t i = (uint32_t)off_exp + total_exp; i < coded_total; ++i) out[i] = 0;
      out[0] = (uint8_t)mode;
      out[1] = (uint8_t)(n_nz < (uint32_t)kCodeRanks ? n_nz : (uint32_t)kCodeRanks);
      *reinterpret_cast<uint16_t*>(out + 2) = (uint16_t)n_chunks;
      *reinterpret_cast<uint32_t*>(out + 4) = coded_total;
      *reinterpret_cast<uint32_t*>(out + 8) = (uint32_t)elems;
      *reinterpret_cast<uint32_t*>(out + 12) = 0;
    }
    return coded_total;
  }
  // 4b: exponents too spread out for the code to pay: the tile travels raw behind its header
  const uint4* src = reinterpret_cast<const uint4*>(in);
  uint4* dstv = reinterpret_cast<uint4*>(out + 16);
  for (int i = tid; i < elems / 8; i += kThreads) dstv[i] = src[i];
  if (tid == 0) {
    out[0] = 0;
    out[1] = 0;
    *reinterpret_cast<uint16_t*>(out + 2) = 0;
    *reinterpret_cast<uint32_t*>(out + 4) = raw_total;
    *reinterpret_cast<uint32_t*>(out + 8) = (uint32_t)elems;
    *reinterpret_cast<uint32_t*>(out + 12) = 0;
  }
  return raw_total;
}

// Unpacks a tile of `size` bytes at `in` into `elems` bf16 values at `out`. False (for every thread) when the
// header or the chunk table does not describe a tile of this shape and size; nothing past the slot is read.
__device__ bool decompress_tile(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int elems, uint32_t size,
                                Scratch& sc, int grp) {
  const int tid = threadIdx.x & (kThreads - 1);
  const int mode = in[0];
  const uint32_t total = *reinterpret_cast<const uint32_t*>(in + 4);
  const uint32_t elems_h = *reinterpret_cast<const uint32_t*>(in + 8);
  if (total != size || elems_h != (uint32_t)elems || mode > 2) return false;
  if (mode == 0) {
    if (size != 16u + (uint32_t)elems * 2u) return false;
    const uint4* src = reinterpret_cast<const uint4*>(in + 16);
    uint4* dst = reinterpret_cast<uint4*>(out);
    for (int i = tid; i < elems / 8; i += kThreads) dst[i] = src[i];
    return true;
  }
  const int n_chunks = elems / kCodeChunkVals;
  if (*reinterpret_cast<const uint16_t*>(in + 2) != n_chunks) return false;
  const int off_sm = kCodeHeaderBytes + n_chunks, off_exp = off_sm + elems;
  const uint32_t nbytes = tid < n_chunks ? in[kCodeHeaderBytes + tid] : 0u;
  uint32_t total_exp;
  const uint32_t myoff = block_exclusive_scan(nbytes, sc, total_exp, grp);
  if ((uint32_t)off_exp + total_exp > size) return false;       // same value in every thread
  if (tid < n_chunks) {
    const uint32_t* in32 = reinterpret_cast<const uint32_t*>(in);
    const uint16_t* sm16 = reinterpret_cast<const uint16_t*>(in + off_sm);
    const uint8_t* syms = in + 16;
    uint32_t* out32 = reinterpret_cast<uint32_t*>(out);
    const uint32_t B = (uint32_t)off_exp + myoff;
    uint32_t wi = B >> 2;
    const int sh = (int)(B & 3u) * 8;
    uint64_t buf = ((uint64_t)in32[wi] | ((uint64_t)in32[wi + 1] << 32)) >> sh;   // reads stay inside the stage ring
    int avail = 64 - sh;
    wi += 2;
    auto refill = [&](int len) {
      buf >>= len;
      avail -= len;
      if (avail < 32) { buf |= (uint64_t)in32[wi++] << avail; avail += 32; }
    };
    auto next_steep = [&]() -> uint32_t {                        // mode 1
      const uint32_t v = (uint32_t)buf;
      const uint32_t c = v & 3u, t = v >> 2;
      const int n = __ffs((int)~t) - 1;                        // ones that follow the "11" marker
      const bool esc = n >= kCodeEscapeOnes;
      const int len = c != 3u ? 2 : (esc ? 2 + kCodeEscapeOnes + 8 : n + 3);
      const uint32_t e = c != 3u ? syms[c] : (esc ? ((t >> kCodeEscapeOnes) & 0xffu) : syms[kCodeShortRanks + n]);
      refill(len);
      return e;
    };
    auto next_flat = [&]() -> uint32_t {                         // mode 2
      const uint32_t v = (uint32_t)buf;
      const int q = __ffs((int)(~v | (1u << kCodeFlatEscapeOnes))) - 1;   // leading ones of the code, at most 4
      const bool esc = q >= kCodeFlatEscapeOnes;
      const int len = esc ? kCodeFlatEscapeOnes + 8 : q + 3;
      const uint32_t e = esc ? ((v >> kCodeFlatEscapeOnes) & 0xffu) : syms[(q << 2) | ((v >> (q + 1)) & 3u)];
      refill(len);
      return e;
    };
    auto emit = [&](int k, uint32_t ea, uint32_t eb) {
      const int w = k * n_chunks + tid;
      const uint32_t s = sm16[w];
      const uint32_t lo = ((s & 0x80u) << 8) | (ea << 7) | (s & 0x7fu);
      const uint32_t hi = ((s & 0x8000u)) | (eb << 7) | ((s >> 8) & 0x7fu);
      out32[w] = lo | (hi << 16);
    };
    if (mode == 1) {
#pragma unroll 2
      for (int k = 0; k < kCodeChunkVals / 2; ++k) {
        const uint32_t ea = next_steep(), eb = next_steep();
        emit(k, ea, eb);
      }
    } else {
#pragma unroll 2
      for (int k = 0; k < kCodeChunkVals / 2; ++k) {
        const uint32_t ea = next_flat(), eb = next_flat();
        emit(k, ea, eb);
      }
    }
  }
  return true;
}

// static shared state of one pipeline
template <bool COMPRESS, int IN_STAGES>
struct __align__(128) GroupState {
  uint32_t tbl[3][kTblBatch];
  uint64_t full[IN_STAGES];
  uint64_t dst[IN_STAGES];
  uint64_t table_idx[IN_STAGES];
  int32_t elems[IN_STAGES];
  uint32_t in_bytes[IN_STAGES];
  uint32_t sizes[COMPRESS ? 1 : kEpoch];
  Scratch sc;
  int abort;
};

template <bool COMPRESS, int kInStages>
__global__ void __launch_bounds__(kThreads * kGroups, 1)
kv_compress_kernel(const __grid_constant__ KvCopyParams p, uint32_t* __restrict__ size_table, int layers_total,
                   int tiles_per_chunk) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ GroupState<COMPRESS, kInStages> gstate[kGroups];
  const int grp = threadIdx.x / kThreads;
  const int tid = threadIdx.x % kThreads;
  Smem<kInStages>& sm = reinterpret_cast<Smem<kInStages>*>(smem_raw)[grp];
  GroupState<COMPRESS, kInStages>& gs = gstate[grp];
  uint64_t* full = gs.full;
  uint64_t* s_dst = gs.dst;
  uint64_t* s_table_idx = gs.table_idx;
  uint32_t(*s_tbl)[kTblBatch] = gs.tbl;
  int32_t* s_elems = gs.elems;
  uint32_t* s_in_bytes = gs.in_bytes;
  uint32_t* s_sizes = gs.sizes;
  Scratch& sc = gs.sc;
  int& s_abort = gs.abort;
  // every pipeline is a CTA of its own as far as the work split and the completion count go
  const int64_t vcta = (int64_t)blockIdx.x * kGroups + grp, vgrid = (int64_t)gridDim.x * kGroups;

  if (tid == 0) {
    for (int s = 0; s < kInStages; ++s) ptx::mbar_init(&full[s], 1);
    s_abort = 0;
    ptx::fence_mbar_init();
  }
  group_sync(grp);

  const int64_t chunk_elems = p.chunk_bytes / 2;
  const bool by_layer = !COMPRESS && p.layer_major;
  // tiles of one major unit: a pair (all its layers), or, walking layer by layer, a layer (all its pairs)
  const int32_t span = (by_layer ? p.num_pairs : p.num_layers) * p.kv_dim * tiles_per_chunk;
  const int64_t total = (int64_t)span * (by_layer ? p.num_layers : p.num_pairs);
  // Pair-major: every CTA owns one contiguous run of tiles, so consecutive tiles share their block ids
  // (fetched once per pair, possibly over PCIe) and their size-table neighbourhood. Layer by layer the CTAs
  // interleave instead, so that all of them finish a layer at about the same time.
  // (whole blocks per pipeline when there are enough of them: runs that start inside a block showed up as a
  // 10-15 % dip in link rate at pipeline counts that do not divide the block count)
  const int64_t per_cta = !by_layer && p.num_pairs >= 4 * vgrid ? (p.num_pairs + vgrid - 1) / vgrid * span
                                                                 : (total + vgrid - 1) / vgrid;
  const int64_t first = by_layer ? vcta : vcta * per_cta;
  const int64_t step = by_layer ? vgrid : 1;
  const int64_t n_mine = first >= total ? 0
                         : by_layer   ? (total - first + step - 1) / step
                                      : (total - first < per_cta ? total - first : per_cta);
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
  int32_t signalled = 0;   // thread 0, layer by layer: layers [0, signalled) already reported by this CTA

  auto layer_rel_of = [&](int64_t it) -> int32_t { return (int32_t)((first + it * step) / span); };

  // decodes tile `it` of this CTA; returns false for a pair whose ids are out of range
  auto locate = [&](int64_t it, uint64_t& g, uint64_t& c, uint64_t& tidx, int32_t& elems, bool cached) -> bool {
    const int64_t t = first + it * step;
    const int32_t major = (int32_t)(t / span), r = (int32_t)(t % span);
    const int s_ = r % tiles_per_chunk, q = r / tiles_per_chunk;
    const int kv = q % p.kv_dim;
    const int32_t pair = by_layer ? q / p.kv_dim : major;
    const int layer = p.layer_start + (by_layer ? major : q / p.kv_dim);
    int64_t gblk, cblk;
    if (cached && !by_layer) pair_ids(pair, gblk, cblk);
    else { gblk = __ldg(p.gpu_blocks + pair); cblk = __ldg(p.cpu_blocks + pair); }
    bool ok = true;
    if (p.gpu_num_blocks > 0 && (gblk < 0 || gblk >= p.gpu_num_blocks)) { err |= KV_ERR_GPU_BLOCK_RANGE; ok = false; }
    if (p.cpu_num_blocks > 0 && (cblk < 0 || cblk >= p.cpu_num_blocks)) { err |= KV_ERR_CPU_BLOCK_RANGE; ok = false; }
    const int64_t e0 = (int64_t)s_ * kCompressTileElems;
    const int64_t left = chunk_elems - e0;
    elems = (int32_t)(left < kCompressTileElems ? left : kCompressTileElems);
    g = kv_gpu_tensor(p, layer * p.idx_layer_mul + kv * p.idx_kv_mul) + layer * p.g_layer_stride + kv * p.g_kv_stride +
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
      s_in_bytes[st] = (uint32_t)elems * 2;
      ptx::mbar_expect_tx(&full[st], (uint32_t)elems * 2);
      ptx::bulk_g2s(sm.in[st], reinterpret_cast<const void*>(g), (uint32_t)elems * 2, &full[st]);
    } else {
      s_dst[st] = g;
      const uint32_t sz = s_sizes[it % kEpoch];
      const uint32_t cap = 16u + 2u * (uint32_t)elems;
      if (sz < 32 || sz > cap || (sz & 15u)) {   // a slot that was never written or a corrupt table entry
        err |= KV_ERR_PAYLOAD_OVERFLOW;
        s_elems[st] = 0;
        ptx::mbar_arrive(&full[st]);
        return;
      }
      s_in_bytes[st] = sz;
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

  if (!COMPRESS) { fetch_sizes(0); group_sync(grp); }
  if (tid == 0)
    for (int64_t it = 0; it < n_mine && it < kInStages - 1; ++it) issue_load(it);

  for (int64_t it = 0; it < n_mine; ++it) {
    const int st = (int)(it % kInStages), ob = (int)(it & 1);
    if (!COMPRESS) {
      // the prefetch below reaches kInStages-1 tiles ahead: refill the size ring before it crosses into a new epoch
      const int64_t ahead = it + kInStages - 1;
      if (ahead % kEpoch == 0 && ahead > 0 && ahead < n_mine) { group_sync(grp); fetch_sizes(ahead); group_sync(grp); }
    }
    if (tid == 0) {
      if (by_layer && p.done_counter) {
        const int32_t lr = layer_rel_of(it);
        if (lr > signalled) {
          // first tile of a later layer: everything this CTA owned in the earlier layers is committed;
          // wait for those stores to be performed and report the layers
          ptx::bulk_wait<0>();
          signal_layers(p, signalled, lr, (unsigned)vgrid);
          signalled = lr;
        }
      }
      if (it + kInStages - 1 < n_mine) issue_load(it + kInStages - 1);
      if (it >= 2) ptx::bulk_wait_read<1>();
    }
    group_sync(grp);
    const int ok = ptx::mbar_wait_bounded(&full[st], (phases >> st) & 1u, kWaitBudgetNs) ? 1 : 0;
    phases ^= 1u << st;
    if (!ok) s_abort = 1;                 // any thread whose wait ran out; the pipeline leaves together
    group_sync(grp);
    if (*reinterpret_cast<volatile int*>(&s_abort)) break;
    const int elems = s_elems[st];
    uint32_t out_bytes = 0;
    if (elems > 0) {
      if (COMPRESS) {
        out_bytes = compress_tile(sm.in[st], sm.out[ob], elems, sc, grp);
      } else {
        if (decompress_tile(sm.in[st], sm.out[ob], elems, s_in_bytes[st], sc, grp)) out_bytes = (uint32_t)elems * 2;
        else err |= KV_ERR_PAYLOAD_OVERFLOW;   // same verdict in every thread; thread 0 reports it
      }
    }
    ptx::fence_proxy_async_smem();
    group_sync(grp);
    if (tid == 0) {
      if (out_bytes > 0) {
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
    // the status words are written before any flag of a layer this CTA did not finish is released
    if (err && p.status) report_status(p.status, err);
    if (by_layer) signal_layers(p, signalled, p.num_layers, (unsigned)vgrid);
    else signal_done(p, (unsigned)vgrid);
  }
}

}  // namespace

cudaError_t launch_kv_compress_bf16(const KvCopyParams& p, uint32_t* size_table, int layers_total, int num_ctas,
                                    cudaStream_t stream) {
  if (p.num_pairs <= 0 || p.num_layers <= 0 || p.kv_dim <= 0 || p.chunk_bytes <= 0) return cudaSuccess;
  const int64_t chunk_elems = p.chunk_bytes / 2;
  if ((p.chunk_bytes & 1) || chunk_elems % 1024 != 0 || size_table == nullptr || !kv_copy_tma_eligible(p))
    return cudaErrorInvalidValue;
  if (p.layer_major && !p.h2d) return cudaErrorInvalidValue;   // per-layer signalling exists for restores only
  const int tiles_per_chunk = (int)compress_tiles_per_chunk(chunk_elems);
  const int64_t total = (int64_t)p.num_pairs * p.num_layers * p.kv_dim * tiles_per_chunk;
  // `num_ctas` counts 128-thread tile pipelines; two of them share a CTA (and an SM)
  int64_t pipes = num_ctas > 0 ? num_ctas : 32;
  if (pipes > total) pipes = total;
  const int ctas = (int)((pipes + kGroups - 1) / kGroups);
  cudaError_t e;
  if (p.h2d) {
    // host reads need several tiles in flight per pipeline to cover the PCIe round trip
    constexpr int kIn = 4;
    const int smem = (int)sizeof(Smem<kIn>) * kGroups + 128;
    e = cudaFuncSetAttribute(kv_compress_kernel<false, kIn>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kv_compress_kernel<false, kIn><<<ctas, kThreads * kGroups, smem, stream>>>(p, size_table, layers_total,
                                                                               tiles_per_chunk);
  } else {
    constexpr int kIn = 3;
    const int smem = (int)sizeof(Smem<kIn>) * kGroups + 128;
    e = cudaFuncSetAttribute(kv_compress_kernel<true, kIn>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kv_compress_kernel<true, kIn><<<ctas, kThreads * kGroups, smem, stream>>>(p, size_table, layers_total,
                                                                              tiles_per_chunk);
  }
  return cudaGetLastError();
}

}  // namespace fkv
