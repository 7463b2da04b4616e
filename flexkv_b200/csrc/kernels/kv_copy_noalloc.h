// fkv_layerwise_copy_noalloc: a layer-by-layer signalled restore for callers that
// must not allocate.
//
// This entry point has no counterpart in the reference. It exists for hosts of
// this library that cannot call cudaMalloc at the moment they need a restore:
// an inference engine that has already handed every free byte of HBM to its own
// KV pool (a late allocation fails or fragments it), a plugin that runs under a
// fixed device-memory budget it does not own, or a latency-critical thread for
// which the implicit device-wide synchronisation of cudaMalloc/cudaFree is not
// acceptable. The ordinary path (LayerwiseGroup) allocates its per-layer
// completion counters with cudaMalloc when the group is built; this one keeps
// them in a fixed array inside the library image instead.
//
// What it does: the same single-launch, layer-major host -> GPU copy as the
// ordinary path, publishing `epoch` to dev_flags[layer] / host_flags[layer] as
// each layer lands. The caller passes every input and output (tensor table,
// host pool, block ids, flag arrays, status words); only the scratch counters
// are internal.
//
// Limits and rules:
//  * num_layers <= FKV_NOALLOC_MAX_LAYERS (1024); more is rejected with an error
//    and nothing is launched. The array costs 4 KiB of device memory on every GPU
//    that loads the library, for the life of the process.
//  * The first call on a device resolves the array's device address (once per
//    device, with that device current). Make that first call outside of any
//    stream capture.
//  * All calls on one GPU share the one array. Calls whose kernels may overlap on
//    the GPU race on it: serialise them (one stream, or an event between them).
//    The counters are cleared on the stream at the start of every call, so a call
//    that was cut short cannot poison the next one.
//  * The tensor table must cover every (layer, kv plane) the call addresses:
//    (num_layers-1)*idx_layer_mul + (kv_dim-1)*idx_kv_mul < num_gpu_ptrs, no addressed
//    entry null. A short or holed table is rejected (-1) before anything is queued.
//  * Arguments are checked before the first CUDA call: a rejected call has put
//    nothing on the stream and has not touched the shared array.
//  * num_pairs == 0 copies nothing and publishes `epoch` to every layer's flags in
//    stream order (two tiny launches), so waiters of an empty restore are released.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FKV_NOALLOC_MAX_LAYERS 1024
#define FKV_NOALLOC_MAX_PTRS 256

typedef struct FkvNoAllocArgs {
  // GPU side: table of tensor base addresses and byte strides (see kv_copy.h for the addressing rule)
  const uint64_t* gpu_ptrs;       // host array of num_gpu_ptrs device addresses
  int32_t num_gpu_ptrs;
  int32_t idx_layer_mul, idx_kv_mul;
  int64_t g_layer_stride, g_kv_stride, g_block_stride;
  // host pool (mapped pinned memory)
  uint64_t cpu_base;
  int64_t c_layer_stride, c_kv_stride, c_block_stride, c_off;
  // work: block-id arrays readable by the GPU (device memory or mapped pinned host memory)
  const int64_t* gpu_blocks;
  const int64_t* cpu_blocks;
  int32_t num_pairs;
  int32_t num_layers, kv_dim;
  int64_t chunk_bytes;
  int64_t gpu_num_blocks, cpu_num_blocks;
  // outputs
  uint32_t* dev_flags;            // device uint32[num_layers] or null
  uint32_t* host_flags;           // mapped host uint32[num_layers] or null
  int32_t* status;                // int32[8], one word per error bit, or null
  uint32_t epoch;
  // launch shape
  int32_t num_ctas, tile_bytes;
} FkvNoAllocArgs;

// Returns 0 on success. On failure returns a non-zero code (a cudaError_t value, or
// -1 for rejected arguments) and writes a message into errbuf when it is non-null.
// `stream` is a cudaStream_t.
int fkv_layerwise_copy_noalloc(const FkvNoAllocArgs* args, void* stream, char* errbuf, int errbuf_len);

#ifdef __cplusplus
}
#endif
