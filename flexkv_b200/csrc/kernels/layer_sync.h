// Device-side consumer of the layerwise ready flags, and a stand-in for a
// model layer: waits (bounded) until the restore of its layer has published
// `epoch`, then occupies the SMs for a fixed time.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace fkv {

// status word (device or mapped): set to 1 if the wait gave up after budget_ns.
cudaError_t launch_layer_stub(const uint32_t* flag, uint32_t epoch, uint64_t busy_ns, uint64_t budget_ns,
                              int32_t* status, uint64_t* t_start_ns, int num_ctas, cudaStream_t stream);

// Consumer-side check used by tests: bounded wait on `flag`, then a 64-bit sum of `num_bytes` at `data`
// is added to *out_sum (zero it first). All probe CTAs must be resident at once (they spin).
cudaError_t launch_layer_probe(const uint32_t* flag, uint32_t epoch, const void* data, int64_t num_bytes,
                               uint64_t budget_ns, int32_t* status, uint64_t* out_sum, int num_ctas,
                               cudaStream_t stream);

cudaError_t launch_set_flags(uint32_t* flags, int n, uint32_t value, cudaStream_t stream);

}  // namespace fkv
