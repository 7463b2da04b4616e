"""Builds the C++ control plane with AddressSanitizer + UBSan and with ThreadSanitizer and runs a
randomized stress of the index, pools, hashing, leases and the peer view (no GPU, no Python
inside the binary). Skipped when the toolchain lacks the sanitizer runtimes."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "flexkv_b200", "csrc")
SOURCES = [os.path.join(CSRC, f) for f in ("radix_index.cpp", "dist_index.cpp", "native_log.cpp", "hasher.cpp", "graph_scheduler.cpp")] + \
    [os.path.join(HERE, "native", "stress_index.cpp")]


def _build(tmp_path, flags, name):
    # the configured compiler may ship without sanitizer runtimes: try the system one as well
    candidates = []
    for c in (os.environ.get("CXX"), "g++", "/usr/bin/g++", "clang++"):
        w = shutil.which(c) if c else None
        if w and w not in candidates:
            candidates.append(w)
    if not candidates:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path / name)
    last = ""
    for cxx in candidates:
        cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-I{CSRC}", *flags, *SOURCES, "-pthread",
               "-o", exe]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode == 0:
            return exe
        last = p.stderr
        if not any(w in last for w in ("sanitize", "libasan", "libtsan", "lasan", "ltsan", "cannot find")):
            raise AssertionError(last[-3000:])
    pytest.skip("sanitizer runtime not available: " + last.strip().splitlines()[-1][:200])


def _run(exe, args, env_extra):
    env = dict(os.environ, **env_extra)
    p = subprocess.run([exe, *args], capture_output=True, text=True, timeout=200, env=env)
    if p.returncode != 0 and "FATAL: ThreadSanitizer: unexpected memory mapping" in p.stderr:
        pytest.skip("ThreadSanitizer cannot map its shadow memory in this container")
    assert p.returncode == 0, (p.stdout + p.stderr)[-4000:]
    assert "OK" in p.stdout


def test_address_and_undefined_behaviour_sanitizers(tmp_path):
    exe = _build(tmp_path, ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "stress_asan")
    _run(exe, [], {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"})


def test_thread_sanitizer(tmp_path):
    exe = _build(tmp_path, ["-fsanitize=thread"], "stress_tsan")
    _run(exe, ["threads"], {"TSAN_OPTIONS": "halt_on_error=1"})
