"""In-tree build of the native module ``flexkv_b200._C`` for sm_100a.

The module is a single shared object made of
  * host C++ (control plane: XXH64 hasher, radix index, eviction, block pool,
    io_uring SSD engine, transfer thread groups, layerwise notifier), and
  * CUDA translation units (``csrc/kernels/*.cu``) compiled only for
    ``compute_100a/sm_100a``.

None of the sources include torch headers: tensors cross the boundary as raw
addresses (``tensor.data_ptr()``) and numpy arrays, so a full rebuild takes
seconds and the object depends only on the CUDA runtime (linked statically).

Objects are cached by content hash under ``flexkv_b200/csrc/build/`` so that
repeated ``build()`` calls are no-ops.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Tuple

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = CSRC / "build"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
TARGET = PKG_DIR / f"_C{EXT_SUFFIX}"

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.environ.get("NVCC", str(Path(CUDA_HOME) / "bin" / "nvcc"))
CXX = os.environ.get("CXX", "g++")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _includes() -> List[str]:
    import pybind11

    return [
        f"-I{CSRC}",
        f"-I{pybind11.get_include()}",
        f"-I{sysconfig.get_paths()['include']}",
        f"-I{CUDA_HOME}/include",
    ]


def _cxx_flags() -> List[str]:
    return ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall",
            "-Wno-unused-function", "-pthread", "-march=x86-64-v3"]


def _nvcc_flags() -> List[str]:
    return ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler",
            "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
            "--expt-relaxed-constexpr"] + ARCH_FLAGS


def _sources() -> Tuple[List[Path], List[Path]]:
    cpp = sorted(CSRC.glob("*.cpp"))
    cu = sorted((CSRC / "kernels").glob("*.cu"))
    return cpp, cu


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
                    + list((CSRC / "kernels").glob("*.cuh")) + list((CSRC / "kernels").glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _obj_for(src: Path, flags: List[str], hdr: str) -> Path:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(" ".join(flags).encode())
    h.update(hdr.encode())
    return BUILD_DIR / f"{src.stem}.{h.hexdigest()[:16]}.o"


def _run(cmd: List[str], log: Path | None = None) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"native build failed: {' '.join(cmd[:3])} ... (exit {proc.returncode})")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every C++/CUDA source and link ``_C``. Returns the .so path."""
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    cpp, cu = _sources()
    hdr = _headers_digest()
    inc = _includes()
    jobs = []
    objs: List[Path] = []
    for s in cpp:
        flags = _cxx_flags() + inc
        o = _obj_for(s, flags, hdr)
        objs.append(o)
        if force or not o.exists():
            jobs.append(([CXX, "-c", str(s), "-o", str(o)] + flags, BUILD_DIR / f"{s.stem}.log"))
    for s in cu:
        flags = _nvcc_flags() + inc
        o = _obj_for(s, flags, hdr)
        objs.append(o)
        if force or not o.exists():
            jobs.append(([NVCC, "-c", str(s), "-o", str(o)] + flags, BUILD_DIR / f"{s.stem}.ptxas.log"))

    stamp = BUILD_DIR / "link.stamp"
    want = "\n".join(str(o.name) for o in objs)
    if not jobs and TARGET.exists() and stamp.exists() and stamp.read_text() == want and not force:
        return TARGET

    if jobs:
        if verbose:
            print(f"[flexkv_b200] compiling {len(jobs)} translation units", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _run(*j), jobs))

    # drop stale objects of the same stems
    keep = {o.name for o in objs}
    for old in BUILD_DIR.glob("*.o"):
        if old.name not in keep:
            try:
                old.unlink()
            except OSError:
                pass

    link = [CXX, "-shared", "-o", str(TARGET) + ".tmp"] + [str(o) for o in objs] + [
        f"-L{CUDA_HOME}/lib64", "-lcudart_static", "-ldl", "-lrt", "-pthread",
        "-Wl,--no-undefined", "-Wl,--exclude-libs,ALL",
    ]
    # libcuda is resolved at run time through the runtime; python symbols stay undefined
    link.remove("-Wl,--no-undefined")
    _run(link)
    os.replace(str(TARGET) + ".tmp", TARGET)
    stamp.write_text(want)
    return TARGET


def clean() -> None:
    if BUILD_DIR.exists():
        shutil.rmtree(BUILD_DIR)
    if TARGET.exists():
        TARGET.unlink()


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True)
    print(p)
