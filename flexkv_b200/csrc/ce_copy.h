// Copy-engine path for GPU<->host block moves.
//
// The DMA engines move long contiguous spans a few percent faster than SM-issued
// traffic on PCIe (no SM time at all), but cost one driver call per span. An op is
// therefore analysed into maximal runs of consecutive (gpu, cpu) block-id pairs and
// routed: whole-run single copies when the block is laid out identically on both
// sides, one pitched 2-D copy per (run, layer, kv) when only the chunk is contiguous,
// and the persistent TMA kernel when the runs are too short to amortise the calls.
// Same role as the reference's adaptive copy-engine dispatcher (csrc/ce_transfer.cu:37-104,
// path list csrc/ce_transfer.h:42-49). A fourth route covers the common case of scattered GPU pages whose
// host blocks were allocated in a row (a fresh pool, or blocks recycled sequence by sequence): the copy
// kernel gathers the pages into a double-buffered device staging area in host block format, at HBM speed, and
// the DMA engine moves each staged piece to the contiguous host span with one large copy (and the reverse for
// restores), the reference's GATHER_DIRECT idea (csrc/ce_transfer.cu:643-812). Host blocks that are scattered
// too stay on the kernel: per-block driver copies of 2 MiB reach 50.6 / 49.5 GB/s on B200 with any number of
// streams, below the kernel's 52.8 / 51.5, and a host-side scatter would spend CPU cores and memory bandwidth.
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
  GATHER_STAGED = 3, // kernel gather into device staging + one large copy per piece of a host run
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

// ---- staged route -------------------------------------------------------------------------------------------
struct CeHostRun {
  int64_t first;      // index of the run's first pair in the op's id arrays
  int64_t cpu_block;  // its first host block
  int64_t len;
};

// Device staging of one GPU (owned by the caller's per-rank state; allocated on first use, freed by ce_staging_free).
struct CeStaging {
  uint8_t* buf[2] = {nullptr, nullptr};
  int64_t* iota = nullptr;            // device array 0, 1, 2, ...: the staged block ids
  cudaEvent_t kernel_done[2] = {nullptr, nullptr}, copy_done[2] = {nullptr, nullptr};
  cudaStream_t copy_stream = nullptr;
  int64_t blocks = 0, block_bytes = 0;
  bool used[2] = {false, false};
};
void ce_staging_free(CeStaging& st);

// Maximal runs of consecutive host block ids over consecutive pairs. Returns false (and leaves `runs` unspecified)
// unless every pair lies in a run of at least `min_run` blocks, all ids are in range, the op covers whole host
// blocks (layer_start == 0, every layer) and consecutive host blocks abut in memory in [layer][kv][chunk] order.
bool ce_host_runs(const KvCopyParams& p, const int64_t* gpu_blocks, const int64_t* cpu_blocks, int64_t n,
                  int total_layers, int64_t min_run, std::vector<CeHostRun>& runs);
// Moves the op through the staging area: pieces of at most `staging_blocks` blocks, gather/scatter kernel on
// `stream`, large copies on the staging's own stream, two buffers in flight. When it returns, everything has
// been queued and `stream` waits for the last copy.
cudaError_t ce_copy_staged(const KvCopyParams& p, const std::vector<CeHostRun>& runs, CeStaging& st,
                           int64_t staging_blocks, const KvCopyLaunch& cfg, cudaStream_t stream);

}  // namespace fkv
