"""Block keys: XXH64 vectors, streaming/cumulative property, namespaces
(reference behaviour pinned by tests/test_namespace_isolation.py)."""
import os

import numpy as np
import pytest

from flexkv_b200.common.block import SequenceMeta, hash_blocks, namespace_prefix

# published XXH64 test vectors (seed 0)
VECTORS = {b"": 0xEF46DB3751D8E999, b"a": 0xD24EC4F1A98C6E5B, b"abc": 0x44BC2CF5AD770999}


def test_known_vectors(native):
    for data, want in VECTORS.items():
        assert native.xxh64(data) == want


def test_matches_xxhash_package_on_all_tail_lengths(native):
    xxhash = pytest.importorskip("xxhash")
    rng = np.random.default_rng(0)
    for n in list(range(0, 70)) + [127, 128, 129, 1000, 4097]:
        data = rng.integers(0, 256, size=n, dtype=np.uint8).tobytes()
        for seed in (0, 1, 2**63 + 5):
            assert native.xxh64(data, seed) == xxhash.xxh64(data, seed=seed).intdigest()


def test_block_hashes_are_cumulative_streaming_digests(native):
    xxhash = pytest.importorskip("xxhash")
    tok = np.random.default_rng(1).integers(0, 128256, size=16 * 9 + 5, dtype=np.int64)
    h = hash_blocks(tok, 16)
    assert h.dtype == np.uint64 and len(h) == 9          # the partial trailing block has no key
    st = xxhash.xxh64(seed=0)
    for i in range(9):
        st.update(tok[i * 16:(i + 1) * 16].tobytes())
        assert int(h[i]) == st.intdigest()
    # a shared prefix gives shared keys, a change at block 4 changes every later key
    tok2 = tok.copy()
    tok2[4 * 16 + 3] += 1
    h2 = hash_blocks(tok2, 16)
    assert np.array_equal(h[:4], h2[:4]) and not np.any(h[4:] == h2[4:])


def test_namespace_isolation(native):
    tok = np.arange(64, dtype=np.int64)
    base = hash_blocks(tok, 16)
    a = hash_blocks(tok, 16, ["lora-a"])
    b = hash_blocks(tok, 16, ["lora-b"])
    a2 = hash_blocks(tok, 16, ["lora-a"])
    multi = hash_blocks(tok, 16, ["lora-a", "salt"])
    assert np.array_equal(a, a2)
    assert not np.any(a == b) and not np.any(a == base) and not np.any(a == multi)
    # the prefix is one int64 per UTF-8 byte of the NUL-joined parts, fed before the tokens
    pre = namespace_prefix(["lora-a", "salt"])
    assert pre.dtype == np.int64 and bytes(pre.astype(np.uint8)) == b"lora-a\x00salt"
    xxhash = pytest.importorskip("xxhash")
    st = xxhash.xxh64(seed=0)
    st.update(pre.tobytes())
    st.update(tok[:16].tobytes())
    assert int(multi[0]) == st.intdigest()


def test_batch_hashing_matches_single(native):
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, 1000, size=n, dtype=np.int64) for n in (0, 5, 16, 100, 1000)]
    out = native.gen_hashes_batch(seqs, 16, None, 3)
    for s, o in zip(seqs, out):
        assert np.array_equal(o, native.gen_hashes(s, 16))


def test_sequence_meta():
    s = SequenceMeta(np.arange(40), 16)
    assert s.num_blocks == 2 and len(s.block_hashes) == 2 and s.token_ids.dtype == np.int64


def test_namespace_identity_and_key_formatting(native):
    """Reference scenarios of tests/test_namespace_isolation.py at the level of SequenceMeta: an empty namespace is
    no namespace, equal namespaces share an id, prefix-cumulative keys hold inside a namespace, and every element of
    a multi-part namespace matters."""
    from flexkv_b200.common.block import format_block_hash
    assert format_block_hash(None) == "-"
    assert format_block_hash(1) == "0x0000000000000001" and format_block_hash(-1) == "0xffffffffffffffff"
    tok = np.arange(1, 9, dtype=np.int64)
    none, empty = SequenceMeta(tok, 4, None), SequenceMeta(tok, 4, [])
    named, again = SequenceMeta(tok, 4, ["ns"]), SequenceMeta(tok, 4, ["ns"])
    assert np.array_equal(none.block_hashes, empty.block_hashes) and none.namespace_id is None and empty.namespace_id is None
    assert named.namespace_id is not None and named.namespace_id == again.namespace_id
    assert named.namespace_id != SequenceMeta(tok, 4, ["other"]).namespace_id
    assert not np.any(named.block_hashes == none.block_hashes)
    # a longer sequence of the same namespace extends the shorter one's keys
    longer = SequenceMeta(np.arange(1, 17, dtype=np.int64), 4, ["ns"])
    assert np.array_equal(longer.block_hashes[:2], named.block_hashes)
    assert named.get_hash(1) == int(named.block_hashes[1]) and named.get_hash(2) is None
    # multi-part namespaces: LoRA id, cache salt, user hierarchy
    full = SequenceMeta(tok, 4, ["lora-1", "salt-a", "org", "user"])
    for other in (["lora-2", "salt-a", "org", "user"], ["lora-1", "salt-b", "org", "user"],
                  ["lora-1", "salt-a", "org", "user2"], ["lora-1", "salt-a", "org"]):
        assert not np.any(full.block_hashes == SequenceMeta(tok, 4, other).block_hashes)
    named.gen_hashes()          # accepted, keys exist already
    assert named.has_hashes()
