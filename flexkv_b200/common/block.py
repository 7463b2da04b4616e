"""Token sequence -> block keys.

Only whole blocks are keyed; key *i* is the XXH64 digest (seed 0) of the
namespace prefix followed by tokens ``[0, (i+1) * tokens_per_block)``, so keys
are prefix-cumulative (flexkv/common/block.py:11-20,44-90; csrc/hash.cpp:47-66).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from .. import _native


def namespace_prefix(namespace: Optional[List[str]]) -> Optional[np.ndarray]:
    """One int64 per UTF-8 byte of ``"\\0".join(namespace)``."""
    if not namespace:
        return None
    raw = "\x00".join(str(s) for s in namespace).encode("utf-8")
    return np.frombuffer(raw, dtype=np.uint8).astype(np.int64)


def hash_blocks(token_ids: np.ndarray, tokens_per_block: int,
                namespace: Optional[List[str]] = None) -> np.ndarray:
    tok = np.ascontiguousarray(token_ids, dtype=np.int64)
    return _native.C.gen_hashes(tok, tokens_per_block, namespace_prefix(namespace))


def format_block_hash(value: Optional[int]) -> str:
    """Signed or unsigned 64-bit key as fixed-width hex, ``-`` for none (log lines; flexkv/common/block.py:37-41)."""
    if value is None:
        return "-"
    return f"0x{int(value) & ((1 << 64) - 1):016x}"


@dataclass
class SequenceMeta:
    token_ids: np.ndarray
    tokens_per_block: int
    namespace: Optional[List[str]] = None
    block_hashes: np.ndarray = field(default=None, repr=False)  # type: ignore[assignment]

    def __post_init__(self) -> None:
        self.token_ids = np.ascontiguousarray(self.token_ids, dtype=np.int64)
        if self.block_hashes is None:
            self.block_hashes = hash_blocks(self.token_ids, self.tokens_per_block, self.namespace)

    @property
    def num_blocks(self) -> int:
        return len(self.token_ids) // self.tokens_per_block

    @property
    def length(self) -> int:
        return len(self.token_ids)

    def has_hashes(self) -> bool:
        return self.block_hashes is not None

    def get_hash(self, block_id: int) -> Optional[int]:
        if block_id >= self.num_blocks:
            return None
        return int(self.block_hashes[block_id])

    def gen_hashes(self) -> None:
        """Keys are computed at construction; kept for callers written against the reference."""

    @property
    def namespace_id(self) -> Optional[int]:
        """XXH64 of the namespace prefix alone (None without a namespace): one id per tenant / LoRA / salt
        combination, equal for equal namespaces (flexkv/common/block.py:80-90)."""
        pre = namespace_prefix(self.namespace)
        if pre is None:
            return None
        return int(_native.C.xxh64(pre, 0))
