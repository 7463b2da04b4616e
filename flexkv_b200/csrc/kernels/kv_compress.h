// Lossless exponent-packing codec for bf16 KV, fused into the paged copy.
//
// bf16 = sign(1) | exponent(8) | mantissa(7). Inside a group of 128 neighbouring
// values the exponents span only a few binades, so each group stores its largest
// exponent once and every value's distance to it in w bits (w = 0..8 chosen per
// group), next to the untouched sign+mantissa byte. Any bit pattern round-trips
// exactly (zeros, denormals, NaN, Inf included: they only widen w).
//
// GPU->host ("compress"): tile staged from HBM by TMA, packed in shared memory,
// only the packed bytes are bulk-stored to the host slot and the tile's size goes
// to a uint32 size table in mapped host memory. Host->GPU is the mirror: sizes are
// read first, exactly that many bytes cross PCIe. On N(0,1) data the link carries
// about 0.76 of the raw bytes. The reference reaches the same goal with nvCOMP's
// ANS coder and a staging kernel (csrc/compression/ans/nvcomp_ans.cu:321-519,
// csrc/compression/common/staging_transfer.cuh:16-101); the host slot geometry
// idea is kept: a fixed-size slot per tile, payload in its first `size` bytes.
//
// Tile = 8192 values (16 KiB raw) = 64 groups. Packed tile:
//   [64 x (e_base u8, w u8)] [group 0: 128 sign|mantissa bytes, w*16 bytes of bit planes] [group 1] ...
// Bit plane (b, j) of a group is the 32-bit ballot, over the 32 lanes, of bit b of
// the exponent distance of element 4*lane + j.
// Host chunk slot = tiles_per_chunk * kCompressTileSlot bytes; chunk elements % 1024 == 0.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "kv_copy.h"

namespace fkv {

constexpr int kCompressTileElems = 8192;
constexpr int kCompressTileSlot = 2 * kCompressTileElems + 128;   // worst case: every group needs w = 8

inline int64_t compress_tiles_per_chunk(int64_t chunk_elems) {
  return (chunk_elems + kCompressTileElems - 1) / kCompressTileElems;
}
inline int64_t compress_chunk_slot_bytes(int64_t chunk_elems) {
  return compress_tiles_per_chunk(chunk_elems) * kCompressTileSlot;
}

// p.chunk_bytes = raw bf16 chunk bytes (GPU side); host strides are slot strides.
// size_table: mapped-host uint32 array indexed
//   ((cpu_block * layers_total + layer) * kv_dim + kv) * tiles_per_chunk + tile
cudaError_t launch_kv_compress_bf16(const KvCopyParams& p, uint32_t* size_table, int layers_total, int num_ctas,
                                    cudaStream_t stream);

}  // namespace fkv
