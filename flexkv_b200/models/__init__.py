"""KV-cache shapes of the model families the benchmarks and tests use, and
builders for synthetic paged caches in each engine's layout."""
from .shapes import KVShape, SHAPES, get_shape, make_model_config  # noqa: F401
from .paged_cache import alloc_paged_cache  # noqa: F401
