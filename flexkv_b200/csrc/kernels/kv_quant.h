// Block-scaled FP8 offload fused into the paged KV copy.
//
// GPU->host ("pack"): a bf16 tile is staged from HBM by the TMA unit, every
// group of 128 consecutive values gets one fp32 scale (amax / 448) and is
// converted to e4m3, and the packed tile plus its scales are bulk-stored to the
// host block: 1.94x fewer bytes cross PCIe. Host->GPU ("unpack") is the mirror.
// There is no counterpart in the reference (it never interprets KV bytes).
//
// Host chunk format (one (layer, kv, block) chunk of E bf16 values):
//     [ E bytes e4m3 payload ][ E/128 fp32 scales ]          E % 512 == 0
// so the host chunk stride is E + E/32 bytes. The arithmetic is exact and
// reproducible: scale = fdiv_rn(amax, 448), q = cvt_rn_satfinite(fdiv_rn(x, scale)),
// x' = bf16_rn(float(q) * scale); an all-zero group stores scale 1.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "kv_copy.h"

namespace fkv {

constexpr int kQuantGroup = 128;

inline int64_t fp8_packed_chunk_bytes(int64_t chunk_elems) { return chunk_elems + (chunk_elems / kQuantGroup) * 4; }

// `p.chunk_bytes` is the bf16 chunk size on the GPU side; the host strides must be
// those of the packed format. p.h2d selects unpack (1) or pack (0).
cudaError_t launch_kv_quant_fp8(const KvCopyParams& p, int num_ctas, cudaStream_t stream);

}  // namespace fkv
