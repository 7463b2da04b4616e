#!/usr/bin/env python
"""Build the unmodified reference KV manager into ``baseline/_ref`` for ``bench.py --impl reference``.

The reference's sources are copied to a scratch directory and built with its own ``setup.py``
through pip. Nothing of the reference is edited; only what the offline image lacks is supplied:

* ``third_party/spdlog/include``  <- the spdlog headers that flashinfer vendors in site-packages
* ``build/include/xxhash.h``      <- the xxHash header that pyarrow vendors; ``build/lib/libxxhash.a``
                                    is that header compiled with ``XXH_IMPLEMENTATION``
* ``build/include/liburing.h`` + ``build/lib/liburing.a``  <- ``baseline/shims/liburing`` (raw syscalls)
* Python modules ``nvtx``, ``expiring_dict``, ``redis``    <- ``baseline/shims/py`` (put on the arm's
  ``sys.path`` at run time, not installed)

Static archives are used so the built extension carries no run-time dependency on the scratch tree.
Usage: ``python baseline/build_reference.py [--src /path/to/reference] [--cython]``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import site
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")


def find_in_site(rel: str) -> str:
    for base in site.getsitepackages():
        p = os.path.join(base, rel)
        if os.path.exists(p):
            return p
    raise SystemExit(f"{rel} not found in site-packages")


def run(cmd, **kw):
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True, **kw)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default="/root/reference")
    ap.add_argument("--scratch", default="/tmp/flexkv_ref_build")
    ap.add_argument("--cython", action="store_true",
                    help="release mode: cythonize the Python package as the reference's default build does "
                         "(slow); default is its FLEXKV_DEBUG=1 mode, which builds only the C++/CUDA extension")
    ap.add_argument("--arch", default="10.0")
    args = ap.parse_args()

    if os.path.isdir(args.scratch):
        shutil.rmtree(args.scratch)
    shutil.copytree(args.src, args.scratch, symlinks=True)
    inc = os.path.join(args.scratch, "build", "include")
    lib = os.path.join(args.scratch, "build", "lib")
    os.makedirs(inc, exist_ok=True)
    os.makedirs(lib, exist_ok=True)

    # spdlog: header-only, bundled fmt
    spd = find_in_site("flashinfer/data/spdlog/include")
    dst = os.path.join(args.scratch, "third_party", "spdlog", "include")
    shutil.copytree(spd, dst)

    # xxHash: vendored single header -> header + static archive
    xxh = find_in_site("pyarrow/include/arrow/vendored/xxhash/xxhash.h")
    shutil.copy(xxh, os.path.join(inc, "xxhash.h"))
    with open(os.path.join(lib, "xxhash_impl.c"), "w") as f:
        f.write('#define XXH_STATIC_LINKING_ONLY\n#define XXH_IMPLEMENTATION\n#include "xxhash.h"\n')
    run(["gcc", "-O3", "-fPIC", "-I", inc, "-c", os.path.join(lib, "xxhash_impl.c"), "-o",
         os.path.join(lib, "xxhash_impl.o")])
    run(["ar", "rcs", os.path.join(lib, "libxxhash.a"), os.path.join(lib, "xxhash_impl.o")])

    # liburing: shim over raw syscalls
    shutil.copy(os.path.join(SHIMS, "liburing", "liburing.h"), os.path.join(inc, "liburing.h"))
    run(["gcc", "-O2", "-fPIC", "-I", inc, "-c", os.path.join(SHIMS, "liburing", "liburing.c"), "-o",
         os.path.join(lib, "liburing.o")])
    run(["ar", "rcs", os.path.join(lib, "liburing.a"), os.path.join(lib, "liburing.o")])

    env = dict(os.environ)
    env.update({"FLEXKV_ENABLE_METRICS": "0", "TORCH_CUDA_ARCH_LIST": args.arch, "MAX_JOBS": str(os.cpu_count() or 4),
                "FLEXKV_DEBUG": "0" if args.cython else "1",
                "PYTHONPATH": os.path.join(SHIMS, "py") + os.pathsep + env.get("PYTHONPATH", "")})
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
         "--find-links", "/opt/wheelhouse", "--target", DEST, args.scratch], env=env)
    with open(os.path.join(DEST, "BUILD_INFO.txt"), "w") as f:
        f.write(f"source={args.src}\nmode={'cython' if args.cython else 'FLEXKV_DEBUG=1'}\narch={args.arch}\n"
                f"spdlog={spd}\nxxhash={xxh}\nliburing=baseline/shims/liburing\n")
    print("installed into", DEST)
    return 0


if __name__ == "__main__":
    sys.exit(main())
