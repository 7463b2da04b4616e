"""flexkv_b200: a Blackwell-native multi-tier KV-cache manager.

GPU paged KV cache <-> pinned/hugepage host pool <-> SSD <-> peers, with a
radix-tree prefix index keyed by cumulative XXH64 block hashes. The public
surface mirrors FlexKV's: ``KVManager``, ``KVTPClient``, ``ModelConfig``,
``CacheConfig``, ``KVResponse``.
"""
from .common.config import CacheConfig, ModelConfig  # noqa: F401
from .common.request import KVResponse, KVResponseStatus  # noqa: F401
from .common.storage import KVCacheLayout, KVCacheLayoutType  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name == "KVManager":
        from .kvmanager import KVManager
        return KVManager
    if name == "KVTPClient":
        from .server.client import KVTPClient
        return KVTPClient
    if name == "KVDPClient":
        from .server.client import KVDPClient
        return KVDPClient
    if name == "KVServer":
        from .server.server import KVServer
        return KVServer
    if name == "__git_commit__":
        # the commit the package was built from, when it sits in a git checkout (the reference exposes the
        # same attribute on its native module, csrc/bindings.cpp:429)
        import os
        import subprocess
        try:
            out = subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5,
                                 cwd=os.path.dirname(os.path.abspath(__file__)))
            return out.stdout.strip() or "unknown"
        except (OSError, subprocess.SubprocessError):
            return "unknown"
    raise AttributeError(name)
