#include "kv_hash.h"

namespace fkv {
namespace {

constexpr uint64_t P1 = 0x9E3779B185EBCA87ULL;
constexpr uint64_t P2 = 0xC2B2AE3D27D4EB4FULL;
constexpr uint64_t P3 = 0x165667B19E3779F9ULL;
constexpr uint64_t P4 = 0x85EBCA77C2B2AE63ULL;
constexpr uint64_t P5 = 0x27D4EB2F165667C5ULL;

__device__ __forceinline__ uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
__device__ __forceinline__ uint64_t xround(uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; }
__device__ __forceinline__ uint64_t xmerge(uint64_t h, uint64_t v) { return (h ^ xround(0, v)) * P1 + P4; }
__device__ __forceinline__ uint64_t avalanche(uint64_t h) {
  h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
  return h;
}

// The input is a stream of 64-bit words w[0], w[1], ... (namespace prefix, then tokens). XXH64 consumes
// it in stripes of four words; word k of a stripe feeds accumulator k. Lane `q` of a quad owns
// accumulator q and therefore reads words q, q+4, q+8, ... — fully parallel until a digest is due.
// A digest after `n` words: the n/4 complete stripes are in the accumulators, the last n%4 words are
// the "tail" and are folded in sequentially (done by every lane redundantly, it is at most 3 words).
__global__ void __launch_bounds__(128)
kv_block_hashes_kernel(const int64_t* __restrict__ tokens, const int64_t* __restrict__ offsets, int64_t num_seqs,
                       int tpb, const int64_t* __restrict__ ns, int64_t ns_len, uint64_t* __restrict__ out,
                       const int64_t* __restrict__ out_offsets) {
  const int64_t quad = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 2;
  const int q = threadIdx.x & 3;
  const unsigned qmask = 0xFu << ((threadIdx.x & 31) & ~3);
  if (quad >= num_seqs) return;
  const int64_t t0 = offsets[quad];
  const int64_t ntok = offsets[quad + 1] - t0;
  const int64_t nblk = ntok / tpb;
  uint64_t* o = out + out_offsets[quad];
  auto word = [&](int64_t i) -> uint64_t {      // i-th word of the stream
    return (uint64_t)(i < ns_len ? ns[i] : tokens[t0 + (i - ns_len)]);
  };
  uint64_t acc = q == 0 ? P1 + P2 : (q == 1 ? P2 : (q == 2 ? 0 : 0 - P1));
  int64_t done = 0;                             // complete stripes consumed so far
  for (int64_t b = 0; b < nblk; ++b) {
    const int64_t n = ns_len + (b + 1) * (int64_t)tpb;    // words covered by this digest
    const int64_t stripes = n >> 2;
    for (int64_t s = done; s < stripes; ++s) acc = xround(acc, word(4 * s + q));
    done = stripes;
    uint64_t h;
    if (n >= 4) {
      const uint64_t v0 = __shfl_sync(qmask, acc, 0, 4), v1 = __shfl_sync(qmask, acc, 1, 4);
      const uint64_t v2 = __shfl_sync(qmask, acc, 2, 4), v3 = __shfl_sync(qmask, acc, 3, 4);
      h = rotl(v0, 1) + rotl(v1, 7) + rotl(v2, 12) + rotl(v3, 18);
      h = xmerge(h, v0); h = xmerge(h, v1); h = xmerge(h, v2); h = xmerge(h, v3);
    } else {
      h = P5;                                    // seed 0
    }
    h += (uint64_t)n * 8;
    for (int64_t i = 4 * stripes; i < n; ++i) {  // at most three trailing words
      h ^= xround(0, word(i));
      h = rotl(h, 27) * P1 + P4;
    }
    h = avalanche(h);
    if (q == 0) o[b] = h;
  }
}

}  // namespace

cudaError_t launch_kv_block_hashes(const int64_t* tokens, const int64_t* offsets, int64_t num_seqs, int tokens_per_block,
                                   const int64_t* ns_prefix, int64_t ns_len, uint64_t* out, const int64_t* out_offsets,
                                   cudaStream_t stream) {
  if (num_seqs <= 0) return cudaSuccess;
  if (tokens_per_block <= 0 || ns_len < 0) return cudaErrorInvalidValue;
  const int threads = 128;                       // 32 sequences per CTA
  const int64_t blocks = (num_seqs * 4 + threads - 1) / threads;
  kv_block_hashes_kernel<<<(unsigned)blocks, threads, 0, stream>>>(tokens, offsets, num_seqs, tokens_per_block, ns_prefix,
                                                                   ns_len, out, out_offsets);
  return cudaGetLastError();
}

}  // namespace fkv
