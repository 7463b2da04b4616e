// Copy-engine path for GPU<->host block moves.
//
// The DMA engines move long contiguous spans a few percent faster than SM-issued
// traffic on PCIe (no SM time at all), but cost one driver call per span. An op is
// therefore analysed into maximal runs of consecutive (gpu, cpu) block-id pairs and
// routed: whole-run single copies when the block is laid out identically on both
// sides, one pitched 2-D copy per (run, layer, kv) when only the chunk is contiguous,
// and the persistent TMA kernel when the runs are too short to amortise the calls.
// Same role as the reference's adaptive copy-engine dispatcher (csrc/ce_transfer.cu:37-104,
// path list csrc/ce_transfer.h:42-49); staging buffers and CPU gather/scatter pools of
// that design are not needed because scattered ops go to the kernel instead.
#pragma once
#include <cstdint>
#include <vector>

#include <cuda_runtime.h>

#include "kernels/kv_copy.h"

namespace fkv {

struct CeRun {
  int64_t gpu_block, cpu_block, len;
};

struct CeAnalysis {
  std::vector<CeRun> runs;
  int64_t num_blocks = 0;
  int64_t longest = 0;
  int status = 0;  // KvCopyStatus range bits for ids that were dropped
};

enum class CePath : int {
  KERNEL = 0,        // leave the op to the copy kernel
  CONTIG_BLOCKS = 1, // one cudaMemcpyAsync per run (identical block geometry on both sides)
  SEGMENT_2D = 2,    // one cudaMemcpy2DAsync per (run, layer, kv)
};

struct CePolicy {
  int64_t max_copies = 4096;         // driver calls per op above which the kernel wins
  // measured on B200 (2 MiB blocks, 32 KiB chunks): 16 MiB per driver copy gives 54.6 GB/s against the
  // kernel's 52.0; 2 MiB per copy gives 50.5, below the kernel
  int64_t min_bytes_per_copy = 8 << 20;
};

// `gpu_blocks`/`cpu_blocks` must be host-readable. Out-of-range ids are skipped and
// recorded in `status`.
CeAnalysis ce_analyze(const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n, int64_t gpu_num_blocks,
                      int64_t cpu_num_blocks);
CePath ce_choose(const CeAnalysis& a, const KvCopyParams& p, const CePolicy& pol);
int64_t ce_num_copies(const CeAnalysis& a, const KvCopyParams& p, CePath path);
// Issues the copies on `stream`; returns the first CUDA error.
cudaError_t ce_copy(const KvCopyParams& p, const CeAnalysis& a, CePath path, cudaStream_t stream);

}  // namespace fkv
