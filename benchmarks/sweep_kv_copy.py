"""Launch-shape sweep of the paged KV copy: engines x CTA counts x tile sizes, the
reference-shaped kernel and a contiguous cudaMemcpy, on 4 GiB ops with random ids."""
import sys, os, time, json
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np, torch
from flexkv_b200 import _native
from flexkv_b200.models import get_shape, alloc_paged_cache
from flexkv_b200.storage.gpu_layout import register_tensors
C = _native.C
dev = torch.device("cuda:0")
shape = get_shape("llama3-8b")
NB = 4096
kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=1)
reg = register_tensors(kv, layout)
bb = shape.block_bytes
numa = C.gpu_numa_node(0)
print("numa node of gpu0:", numa, flush=True)
t0=time.time()
region = C.host_region_alloc(NB*bb, numa_node=numa, cuda_register=True, touch_threads=16)
print("host alloc+pin %.1f GiB: %.2fs hugepage=%s" % (NB*bb/2**30, time.time()-t0, region.hugepage), flush=True)
chunk = reg.chunk_bytes
host = dict(base=region.ptr, layer_stride=2*chunk, kv_stride=chunk, block_stride=bb, num_blocks=NB)
opts = dict(num_layers=32, kv_dim=2, chunk_bytes=chunk, max_blocks_per_op=NB)
grp = C.TransferGroup([reg.as_native()], host, opts)
rng = np.random.default_rng(0)
n = 2048
res = []
def run(h2d, engine, ctas, tile, reps=3):
    grp.set_launch(h2d, ctas, tile, engine)
    best = 1e9
    for r in range(reps+1):
        g = rng.permutation(NB)[:n].astype(np.int64); c = rng.permutation(NB)[:n].astype(np.int64)
        o = grp.transfer(g, c, h2d, 0, 32)
        assert o.status == 0, o.status
        if r > 0: best = min(best, o.gpu_ms)
    return n*bb/best/1e6
for engine in (0, 1):
    for ctas in (2, 4, 8, 16, 32, 64, 148):
        for tile in (4096, 8192, 16384, 32768):
            if engine == 1 and tile != 16384: continue
            d2h = run(False, engine, ctas, tile); h2d = run(True, engine, ctas, tile)
            row = dict(engine="tma" if engine == 0 else "simt", ctas=ctas, tile=tile, d2h_gbs=round(d2h,2), h2d_gbs=round(h2d,2))
            res.append(row); print(row, flush=True)
# reference-shaped baseline
for ctas in (4, 16):
    best=[1e9,1e9]
    for r in range(3):
        g = rng.permutation(NB)[:n].astype(np.int64); c = rng.permutation(NB)[:n].astype(np.int64)
        o1 = grp.transfer_refshape(g, c, False, ctas); o2 = grp.transfer_refshape(g, c, True, ctas)
        if r>0: best=[min(best[0],o1.gpu_ms), min(best[1],o2.gpu_ms)]
    row = dict(engine="refshape", ctas=ctas, d2h_gbs=round(n*bb/best[0]/1e6,2), h2d_gbs=round(n*bb/best[1]/1e6,2)); res.append(row); print(row, flush=True)
# cudaMemcpy contiguous upper bound
pin = torch.empty(4*2**30, dtype=torch.uint8).pin_memory(); d = torch.empty(4*2**30, dtype=torch.uint8, device=dev)
for name, a, b in (("memcpy_h2d", d, pin), ("memcpy_d2h", pin, d)):
    best = 1e9
    for r in range(3):
        e0=torch.cuda.Event(enable_timing=True); e1=torch.cuda.Event(enable_timing=True)
        e0.record(); a.copy_(b, non_blocking=True); e1.record(); torch.cuda.synchronize()
        best=min(best,e0.elapsed_time(e1))
    row = {name+"_gbs": round(4*2**30/best/1e6,2)}; res.append(row); print(row, flush=True)
out = sys.argv[1] if len(sys.argv) > 1 else "sweep_kv_copy.json"
json.dump(res, open(out, "w"), indent=1)
