// Direct launch entry points for the CUDA kernels (used by flexkv_b200.ops and
// by tests that compare a kernel with a PyTorch reference on one stream).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include "kernels/kv_copy.h"
#include "kernels/kv_fanout.h"
#include "kernels/kv_quant.h"
#include "kernels/kv_compress.h"
#include "kernels/kv_hash.h"
#include "ce_copy.h"
#include "ptr_table.h"
#include "ipc.h"
#include "vmm_handle.h"

namespace py = pybind11;
using namespace fkv;

static void throw_on(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

// `on_host`: the call executes on the CPU (host_kv_copy, planning, checks), so a table beyond the inline
// limit stays in host memory; otherwise it is uploaded to the current device, where the launch goes.
KvCopyParams kv_params_from_dict(const py::dict& d, bool on_host = false) {
  KvCopyParams p;
  std::memset(&p, 0, sizeof(p));
  auto ptrs = d["gpu_ptrs"].cast<std::vector<uint64_t>>();
  int device = -1;
  auto table_device = [&]() {
    if (on_host) return -1;
    if (device < 0 && cudaGetDevice(&device) != cudaSuccess) {
      (void)cudaGetLastError();
      throw std::runtime_error("no CUDA device for a tensor table of more than " + std::to_string(kMaxGpuPtrs) +
                               " entries");
    }
    return device;
  };
  kv_set_gpu_table(p, ptrs, (int)ptrs.size() > kMaxGpuPtrs ? table_device() : -1);
  auto geti = [&](const char* k, int64_t dflt) { return d.contains(k) ? d[k].cast<int64_t>() : dflt; };
  p.idx_layer_mul = (int32_t)geti("idx_layer_mul", 1);
  p.idx_kv_mul = (int32_t)geti("idx_kv_mul", 0);
  p.g_layer_stride = geti("g_layer_stride", 0);
  p.g_kv_stride = geti("g_kv_stride", 0);
  p.g_block_stride = geti("g_block_stride", 0);
  p.g_off = geti("g_off", 0);
  p.cpu_base = d.contains("cpu_base") ? d["cpu_base"].cast<uint64_t>() : 0;
  if (d.contains("c_ptrs")) {
    auto cp = d["c_ptrs"].cast<std::vector<uint64_t>>();
    kv_set_c_table(p, cp, (int)cp.size() > kMaxGpuPtrs ? table_device() : -1);
    p.c_use_table = 1;
    p.c_idx_layer_mul = (int32_t)geti("c_idx_layer_mul", 1);
    p.c_idx_kv_mul = (int32_t)geti("c_idx_kv_mul", 0);
  }
  p.c_layer_stride = geti("c_layer_stride", 0);
  p.c_kv_stride = geti("c_kv_stride", 0);
  p.c_block_stride = geti("c_block_stride", 0);
  p.c_off = geti("c_off", 0);
  p.gpu_blocks = (const int64_t*)(uintptr_t)d["gpu_blocks_ptr"].cast<uint64_t>();
  p.cpu_blocks = (const int64_t*)(uintptr_t)d["cpu_blocks_ptr"].cast<uint64_t>();
  p.num_pairs = (int32_t)geti("num_pairs", 0);
  p.layer_start = (int32_t)geti("layer_start", 0);
  p.num_layers = (int32_t)geti("num_layers", 0);
  p.kv_dim = (int32_t)geti("kv_dim", 1);
  p.chunk_bytes = geti("chunk_bytes", 0);
  p.gpu_num_blocks = geti("gpu_num_blocks", 0);
  p.cpu_num_blocks = geti("cpu_num_blocks", 0);
  p.status = (int32_t*)(uintptr_t)(uint64_t)geti("status_ptr", 0);
  p.h2d = (int32_t)geti("h2d", 0);
  p.done_counter = (uint32_t*)(uintptr_t)(uint64_t)geti("done_counter_ptr", 0);
  p.dev_flags = (uint32_t*)(uintptr_t)(uint64_t)geti("dev_flags_ptr", 0);
  p.host_flags = (uint32_t*)(uintptr_t)(uint64_t)geti("host_flags_ptr", 0);
  p.epoch = (uint32_t)geti("epoch", 0);
  p.layer_major = (int32_t)geti("layer_major", 0);
  return p;
}

void init_kernel_bindings(py::module_& m) {
  m.def("kv_copy", [](py::dict params, int num_ctas, int tile_bytes, int engine, uint64_t stream) {
    KvCopyParams p = kv_params_from_dict(params);
    KvCopyLaunch cfg{num_ctas, tile_bytes, engine};
    throw_on(launch_kv_copy(p, cfg, (cudaStream_t)(uintptr_t)stream), "kv_copy launch");
  }, py::arg("params"), py::arg("num_ctas") = 16, py::arg("tile_bytes") = 16384, py::arg("engine") = 0,
     py::arg("stream") = 0);

  m.def("kv_copy_refshape", [](py::dict params, int num_ctas, uint64_t stream) {
    KvCopyParams p = kv_params_from_dict(params);
    throw_on(launch_kv_copy_refshape(p, num_ctas, (cudaStream_t)(uintptr_t)stream), "kv_copy_refshape launch");
  }, py::arg("params"), py::arg("num_ctas") = 4, py::arg("stream") = 0);

  m.def("kv_fanout", [](py::dict params, int64_t mc_delta, uint64_t mc_flag_ptr, int num_ctas, int tile_bytes,
                        uint64_t stream) {
    KvFanoutParams fp;
    // "mc_ptrs" (optional): multicast address of every tensor in gpu_ptrs
    std::vector<uint64_t> mc;
    if (params.contains("mc_ptrs")) mc = params["mc_ptrs"].cast<std::vector<uint64_t>>();
    fp.base = kv_params_from_dict(params);
    fp.base.h2d = 1;
    if (!mc.empty()) {
      if ((int)mc.size() != fp.base.num_gpu_ptrs) throw std::invalid_argument("mc_ptrs must match gpu_ptrs");
      int dev = -1;
      if ((int)mc.size() > kMaxGpuPtrs) throw_on(cudaGetDevice(&dev), "cudaGetDevice");
      kv_set_c_table(fp.base, mc, dev);
    }
    fp.mc_delta = mc_delta;
    fp.mc_flag = (uint32_t*)(uintptr_t)mc_flag_ptr;
    throw_on(launch_kv_fanout(fp, num_ctas, tile_bytes, (cudaStream_t)(uintptr_t)stream), "kv_fanout launch");
  }, py::arg("params"), py::arg("mc_delta"), py::arg("mc_flag_ptr") = (uint64_t)0, py::arg("num_ctas") = 8,
     py::arg("tile_bytes") = 16384, py::arg("stream") = (uint64_t)0);

  m.def("kv_quant_fp8", [](py::dict params, int num_ctas, uint64_t stream) {
    KvCopyParams p = kv_params_from_dict(params);
    throw_on(launch_kv_quant_fp8(p, num_ctas, (cudaStream_t)(uintptr_t)stream), "kv_quant_fp8 launch");
  }, py::arg("params"), py::arg("num_ctas") = 32, py::arg("stream") = (uint64_t)0);
  m.def("fp8_packed_chunk_bytes", &fp8_packed_chunk_bytes);

  m.def("kv_compress_bf16", [](py::dict params, uint64_t size_table_ptr, int layers_total, int num_ctas,
                               uint64_t stream) {
    KvCopyParams p = kv_params_from_dict(params);
    throw_on(launch_kv_compress_bf16(p, (uint32_t*)(uintptr_t)size_table_ptr, layers_total, num_ctas,
                                     (cudaStream_t)(uintptr_t)stream), "kv_compress_bf16 launch");
  }, py::arg("params"), py::arg("size_table_ptr"), py::arg("layers_total"), py::arg("num_ctas") = 32,
     py::arg("stream") = (uint64_t)0);
  m.def("compress_chunk_slot_bytes", &compress_chunk_slot_bytes);
  m.def("compress_tiles_per_chunk", &compress_tiles_per_chunk);
  m.attr("COMPRESS_TILE_SLOT") = kCompressTileSlot;
  m.attr("COMPRESS_TILE_ELEMS") = kCompressTileElems;

  m.def("ipc_export", [](uint64_t ptr) {
    IpcExport e = ipc_export(ptr);
    return py::make_tuple(py::bytes(e.handle), e.offset, e.alloc_bytes);
  });
  m.def("ipc_import", &ipc_import);
  m.def("ipc_close", &ipc_close);

  // Memory from the virtual-memory API (cuMemCreate): shareable handles instead of legacy IPC
  m.def("vmm_is_vmm_pointer", &vmm_is_vmm_pointer);
  m.def("vmm_export", [](uint64_t ptr, bool prefer_fabric) {
    VmmExport e = vmm_export(ptr, prefer_fabric);
    py::dict d;
    d["kind"] = e.kind == VmmHandleKind::FABRIC ? "fabric" : "posix_fd";
    d["fd"] = e.fd;
    d["fabric"] = py::bytes(e.fabric);
    d["base"] = e.base;
    d["size"] = e.size;
    d["offset"] = e.offset;
    return d;
  }, py::arg("device_ptr"), py::arg("prefer_fabric") = true);
  m.def("vmm_import_fd", [](int fd, uint64_t size, int device) {
    VmmMapping mp = vmm_import_fd(fd, size, device);
    return py::make_tuple(mp.va, mp.size);
  });
  m.def("vmm_import_fabric", [](const std::string& fabric, uint64_t size, int device) {
    VmmMapping mp = vmm_import_fabric(fabric, size, device);
    return py::make_tuple(mp.va, mp.size);
  });
  m.def("vmm_unmap", &vmm_unmap);
  m.def("vmm_alloc", [](uint64_t bytes, int device, bool fabric) {
    VmmMapping mp = vmm_alloc(bytes, device, fabric);
    return py::make_tuple(mp.va, mp.size);
  }, py::arg("bytes"), py::arg("device"), py::arg("fabric") = false);
  m.def("vmm_free", &vmm_free);

  // Batched block keys on the GPU; every pointer is a device (or mapped host) address.
  m.def("kv_block_hashes", [](uint64_t tokens, uint64_t offsets, int64_t num_seqs, int tokens_per_block, uint64_t ns,
                              int64_t ns_len, uint64_t out, uint64_t out_offsets, uint64_t stream) {
    throw_on(launch_kv_block_hashes((const int64_t*)(uintptr_t)tokens, (const int64_t*)(uintptr_t)offsets, num_seqs,
                                    tokens_per_block, (const int64_t*)(uintptr_t)ns, ns_len,
                                    (uint64_t*)(uintptr_t)out, (const int64_t*)(uintptr_t)out_offsets,
                                    (cudaStream_t)(uintptr_t)stream),
             "kv_block_hashes launch");
  }, py::arg("tokens"), py::arg("offsets"), py::arg("num_seqs"), py::arg("tokens_per_block"), py::arg("ns_prefix") = 0,
     py::arg("ns_len") = 0, py::arg("out") = 0, py::arg("out_offsets") = 0, py::arg("stream") = 0);

  m.def("host_kv_copy", [](py::dict params, int threads) {
    KvCopyParams p = kv_params_from_dict(params, true);
    py::gil_scoped_release rel;
    return host_kv_copy(p, threads);
  }, py::arg("params"), py::arg("threads") = 4);

  // Copy-engine planning, exposed for inspection and CPU tests: returns the runs as an
  // [R, 3] array (gpu block, cpu block, length), the chosen path, the number of driver
  // copies that path would issue, and the range-error bits of dropped ids.
  m.def("ce_plan", [](py::dict params, int64_t max_copies, int64_t min_bytes_per_copy) {
    KvCopyParams p = kv_params_from_dict(params, true);
    CeAnalysis a = ce_analyze(p.gpu_blocks, p.cpu_blocks, p.num_pairs, p.gpu_num_blocks, p.cpu_num_blocks);
    CePolicy pol;
    pol.max_copies = max_copies;
    pol.min_bytes_per_copy = min_bytes_per_copy;
    CePath path = ce_choose(a, p, pol);
    py::array_t<int64_t> runs(std::vector<py::ssize_t>{(py::ssize_t)a.runs.size(), 3});
    auto r = runs.mutable_unchecked<2>();
    for (size_t i = 0; i < a.runs.size(); ++i) {
      r(i, 0) = a.runs[i].gpu_block;
      r(i, 1) = a.runs[i].cpu_block;
      r(i, 2) = a.runs[i].len;
    }
    static const char* names[] = {"kernel", "contig_blocks", "segment_2d"};
    return py::make_tuple(runs, std::string(names[(int)path]), ce_num_copies(a, p, path), a.status);
  }, py::arg("params"), py::arg("max_copies") = 4096, py::arg("min_bytes_per_copy") = 8 << 20);

  m.def("kv_copy_tma_eligible", [](py::dict params) { return kv_copy_tma_eligible(kv_params_from_dict(params, true)); });
  m.def("ptr_table_cache_size", &ptr_table_cache_size);
  m.attr("MAX_GPU_PTRS_EXT") = kMaxGpuPtrsExt;
}
