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
    raise AttributeError(name)
