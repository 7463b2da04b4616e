// Lossless exponent coder for bf16 KV, fused into the paged copy.
//
// bf16 = sign(1) | exponent(8) | mantissa(7). Sign and mantissa of KV values are close to
// incompressible and travel as one byte per value; the exponents of a tile take only a handful of
// values with a steep frequency profile, so they are entropy coded with a prefix code over their
// frequency RANK in the tile. Any bit pattern round-trips exactly (zeros, denormals, NaN, Inf: a rare
// exponent costs an escape, and a tile whose exponents do not compress travels raw behind its header).
//
// GPU->host ("compress"): tile staged from HBM by TMA, packed in shared memory, only the packed bytes
// are bulk-stored to the host slot and the tile's size goes to a uint32 size table in mapped host
// memory. Host->GPU is the mirror: sizes are read first, exactly that many bytes cross PCIe. On N(0,1)
// data the link carries 0.675 of the raw bytes (the exponent's entropy bounds it at about 0.66). The
// reference reaches the same goal with nvCOMP's ANS coder and a staging kernel
// (csrc/compression/ans/nvcomp_ans.cu:321-519, csrc/compression/common/staging_transfer.cuh:16-101);
// the host slot geometry idea is kept: a fixed-size slot per tile, payload in its first `size` bytes.
//
// Tile = up to 8192 values (16 KiB raw), a multiple of 1024. Chunk t of the tile = the 64 values of the
// 32-bit words t, t + C, t + 2C, ... (C = number of chunks = elems / 64): one thread codes one chunk and
// neighbouring threads touch neighbouring words. Packed tile, every size a multiple of 16 bytes:
//   [0]  u8 mode (0 raw, 1 steep code, 2 flat code)  [1] u8 symbols in use  [2] u16 C  [4] u32 packed size
//   [8]  u32 elems  [12] 0
//   [16] 16 x u8: the exponent of rank 0..15 (most frequent first, ties by smaller exponent; frequencies are
//        counted over a sample, words 0, 8, 16 and 24 of every chunk, i.e. 8 values per chunk spread over the
//        whole tile: the table only steers code lengths)
//   [32] C x u8: coded bytes of each chunk
//   [32 + C] elems x u8: sign<<7 | mantissa of every value, in value order
//   then the chunks' codes back to back, each chunk padded to a byte, the tile padded to 16 bytes.
// Code of an exponent, bits written LSB first.
//   mode 1 (steep profiles, e.g. one scale per tile): rank 0..2 -> that rank in 2 bits; rank r = 3..15 -> "11",
//     r-3 one bits, a zero bit; any other exponent -> "11", 13 one bits, the 8 exponent bits (23 bits).
//   mode 2 (flat profiles, e.g. channels or tokens with different scales in one tile): rank r = 0..15 ->
//     r/4 one bits, a zero bit, r%4 in 2 bits (3..6 bits); any other exponent -> 4 one bits, the 8 exponent
//     bits (12 bits).
// The packer takes the mode whose code is shorter for the sampled frequencies (mode 1 on a tie).
// Raw tile: the 16-byte header with mode 0, then the values.
// Host chunk slot: kCompressTileSlot bytes per full tile, 2 * elems + 128 for a shorter last tile; tile s of a
// chunk starts s * kCompressTileSlot bytes into the chunk's slot; chunk elements % 1024 == 0.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "kv_copy.h"

namespace fkv {

constexpr int kCompressTileElems = 8192;
constexpr int kCompressTileSlot = 2 * kCompressTileElems + 128;   // a raw tile (16 + 16384 bytes) fits
constexpr int kCodeChunkVals = 64;      // values coded by one thread
constexpr int kCodeHeaderBytes = 32;    // header and symbol table
constexpr int kCodeRanks = 16;          // exponents with a code of their own
constexpr int kCodeShortRanks = 3;      // of which this many take 2 bits
constexpr int kCodeEscapeOnes = kCodeRanks - kCodeShortRanks;   // one bits that announce a literal exponent
constexpr int kCodeSampleWords = 4;     // the frequency ranks come from 4 words (8 values) of every chunk,
constexpr int kCodeSampleStride = kCodeChunkVals / 2 / kCodeSampleWords;   // every 8th word of the chunk
constexpr int kCodeFlatEscapeOnes = 4;  // mode 2: one bits that announce a literal exponent

inline int64_t compress_tiles_per_chunk(int64_t chunk_elems) {
  return (chunk_elems + kCompressTileElems - 1) / kCompressTileElems;
}
inline int64_t compress_chunk_slot_bytes(int64_t chunk_elems) {
  // full tiles take a full slot; the last, shorter tile takes what its own raw form needs (plus the same slack)
  const int64_t full = chunk_elems / kCompressTileElems, rest = chunk_elems % kCompressTileElems;
  return full * kCompressTileSlot + (rest ? 2 * rest + 128 : 0);
}

// p.chunk_bytes = raw bf16 chunk bytes (GPU side); host strides are slot strides.
// Restores (p.h2d) honour p.layer_major with p.done_counter / dev_flags / host_flags exactly as the plain
// copy kernel does: tiles are walked layer by layer and each layer's flag is published when it has landed.
// size_table: mapped-host uint32 array indexed
//   ((cpu_block * layers_total + layer) * kv_dim + kv) * tiles_per_chunk + tile
cudaError_t launch_kv_compress_bf16(const KvCopyParams& p, uint32_t* size_table, int layers_total, int num_ctas,
                                    cudaStream_t stream);

}  // namespace fkv
