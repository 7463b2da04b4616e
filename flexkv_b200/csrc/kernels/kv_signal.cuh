// Device-side helpers shared by the movers: error reporting into the status words and the
// last-CTA-out publication of completion flags (whole launch, or layer by layer).
#pragma once
#include "kv_copy.h"
#include "ptx_sm100.cuh"

namespace fkv {

// Error reporting without atomics: `status` is an array of kStatusWords words,
// one per KvCopyStatus bit, and a CTA that saw error bit b stores 1 to word b.
// Plain idempotent stores cannot lose a bit when several CTAs report at once,
// and they work on mapped host memory whether or not the platform offers PCIe
// atomics. The host ORs the words back into a bit mask.
__device__ __forceinline__ void report_status(int32_t* status, int err) {
#pragma unroll
  for (int b = 0; b < kStatusWords; ++b)
    if (err & (1 << b)) reinterpret_cast<volatile int32_t*>(status)[b] = 1;
}

// Last-CTA-out publication of the completion flags (see KvCopyParams). Called by
// one thread per CTA after all of the CTA's stores are complete.
// `arrivals` = how many callers the launch has (its CTAs, or its pipelines when a CTA runs several).
__device__ __forceinline__ void signal_done(const KvCopyParams& p, unsigned arrivals = 0) {
  if (p.done_counter == nullptr) return;
  if (arrivals == 0) arrivals = gridDim.x;
  ptx::fence_proxy_async_all();  // order the bulk (async proxy) stores before the generic-proxy flag traffic
  __threadfence();
  const unsigned prev = atomicAdd(p.done_counter, 1u);
  if (prev == arrivals - 1) {
    *reinterpret_cast<volatile uint32_t*>(p.done_counter) = 0;
    __threadfence();
    for (int l = p.layer_start; l < p.layer_start + p.num_layers; ++l) {
      if (p.dev_flags) ptx::st_release_gpu(p.dev_flags + l, p.epoch);
      if (p.host_flags) ptx::st_release_sys(p.host_flags + l, p.epoch);
    }
  }
}

// Per-layer publication for layer-major launches: this CTA has finished (and
// drained) everything it owns in layers [from, to); the last CTA to say so for
// a layer resets that layer's counter and publishes the flags.
__device__ __forceinline__ void signal_layers(const KvCopyParams& p, int from, int to, unsigned arrivals = 0) {
  if (p.done_counter == nullptr || from >= to) return;
  if (arrivals == 0) arrivals = gridDim.x;
  // The caller has waited for its bulk stores of these layers (wait_group 0: the writes are performed).
  // No async-proxy fence here: it would also wait for the loads in flight and drain the pipeline at every
  // layer boundary; the release below orders the completed stores before the counter and flag updates.
  __threadfence();
  for (int l = from; l < to; ++l) {
    const unsigned prev = atomicAdd(p.done_counter + l, 1u);
    if (prev == arrivals - 1) {
      reinterpret_cast<volatile uint32_t*>(p.done_counter)[l] = 0;
      __threadfence();
      if (p.dev_flags) ptx::st_release_gpu(p.dev_flags + p.layer_start + l, p.epoch);
      if (p.host_flags) ptx::st_release_sys(p.host_flags + p.layer_start + l, p.epoch);
    }
  }
}

}  // namespace fkv
