#include "layer_sync.h"
#include "ptx_sm100.cuh"

namespace fkv {
namespace {

__global__ void layer_stub_kernel(const uint32_t* flag, uint32_t epoch, uint64_t busy_ns, uint64_t budget_ns,
                                  int32_t* status, uint64_t* t_start_ns) {
  __shared__ int go;
  if (threadIdx.x == 0) {
    go = 1;
    if (flag != nullptr) {
      const uint64_t t0 = ptx::globaltimer_ns();
      // flags carry a monotonically increasing epoch; signed difference tolerates wrap-around
      while ((int32_t)(ptx::ld_acquire_gpu(flag) - epoch) < 0) {
        if (ptx::globaltimer_ns() - t0 > budget_ns) {
          go = 0;
          if (status) *reinterpret_cast<volatile int32_t*>(status) = 1;
          break;
        }
        __nanosleep(200);
      }
    }
    if (blockIdx.x == 0 && t_start_ns) *t_start_ns = ptx::globaltimer_ns();
  }
  __syncthreads();
  if (!go) return;
  const uint64_t t1 = ptx::globaltimer_ns();
  while (ptx::globaltimer_ns() - t1 < busy_ns) __nanosleep(100);
}

// Waits (bounded) for a layer's flag and at once sums the layer's bytes as 64-bit words: if a flag were
// published before the data it guards is visible, the sum would be taken over stale bytes.
__global__ void layer_probe_kernel(const uint32_t* flag, uint32_t epoch, const uint64_t* data, int64_t num_words,
                                   uint64_t budget_ns, int32_t* status, unsigned long long* out_sum) {
  __shared__ int go;
  if (threadIdx.x == 0) {
    go = 1;
    const uint64_t t0 = ptx::globaltimer_ns();
    while ((int32_t)(ptx::ld_acquire_gpu(flag) - epoch) < 0) {
      if (ptx::globaltimer_ns() - t0 > budget_ns) {
        go = 0;
        if (status) *reinterpret_cast<volatile int32_t*>(status) = 1;
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (!go) return;
  unsigned long long acc = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < num_words; i += (int64_t)gridDim.x * blockDim.x)
    acc += __ldcg(data + i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(out_sum, acc);
}

__global__ void set_flags_kernel(uint32_t* flags, int n, uint32_t value) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ptx::st_release_gpu(flags + i, value);
}

}  // namespace

cudaError_t launch_layer_stub(const uint32_t* flag, uint32_t epoch, uint64_t busy_ns, uint64_t budget_ns,
                              int32_t* status, uint64_t* t_start_ns, int num_ctas, cudaStream_t stream) {
  layer_stub_kernel<<<num_ctas > 0 ? num_ctas : 1, 128, 0, stream>>>(flag, epoch, busy_ns, budget_ns, status,
                                                                      t_start_ns);
  return cudaGetLastError();
}

cudaError_t launch_layer_probe(const uint32_t* flag, uint32_t epoch, const void* data, int64_t num_bytes,
                               uint64_t budget_ns, int32_t* status, uint64_t* out_sum, int num_ctas,
                               cudaStream_t stream) {
  if (flag == nullptr || data == nullptr || out_sum == nullptr || (num_bytes & 7)) return cudaErrorInvalidValue;
  layer_probe_kernel<<<num_ctas > 0 ? num_ctas : 4, 256, 0, stream>>>(
      flag, epoch, static_cast<const uint64_t*>(data), num_bytes / 8, budget_ns, status,
      reinterpret_cast<unsigned long long*>(out_sum));
  return cudaGetLastError();
}

cudaError_t launch_set_flags(uint32_t* flags, int n, uint32_t value, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  set_flags_kernel<<<(n + 127) / 128, 128, 0, stream>>>(flags, n, value);
  return cudaGetLastError();
}

}  // namespace fkv
