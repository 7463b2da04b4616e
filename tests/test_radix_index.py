"""Prefix index semantics, run against both back-ends (native C++ and the
pure-Python specification) and differentially against each other. Mirrors what
the reference pins in tests/test_cache_engine.py (ready prefix :275, stale
insert :324,:371, eviction policies :631-1189)."""
import numpy as np
import pytest

from flexkv_b200 import _native
from flexkv_b200.cache.radixtree import RadixTreeIndex


def make(kind, **kw):
    if kind == "native":
        return _native.C.RadixIndex(kw.pop("tokens_per_block", 16), kw.pop("max_num_blocks", 0),
                                    kw.pop("eviction_policy", "lru"), kw.pop("hit_reward_seconds", 0.0),
                                    kw.pop("slru_threshold", 2))
    return RadixTreeIndex(kw.pop("tokens_per_block", 16), kw.pop("max_num_blocks", 0),
                          kw.pop("eviction_policy", "lru"), kw.pop("hit_reward_seconds", 0.0),
                          kw.pop("slru_threshold", 2))


def H(*xs):
    return np.asarray(xs, dtype=np.uint64)


def B(*xs):
    return np.asarray(xs, dtype=np.int64)


KINDS = ["native", "python"]


@pytest.mark.parametrize("kind", KINDS)
def test_insert_match_split(kind):
    t = make(kind)
    assert t.is_empty()
    m = t.match_prefix(H(1, 2, 3, 4))
    assert m.num_matched_blocks == 0 and t.is_root(m.last_node)
    n1 = t.insert(B(10, 11, 12, 13), H(1, 2, 3, 4), -1, True, m)
    assert t.total_cached_blocks() == 4 and t.num_nodes() == 2
    m = t.match_prefix(H(1, 2, 9, 9))
    assert m.num_matched_blocks == 2 and m.last_node_matched_length == 2
    assert list(m.physical_blocks) == [10, 11]
    n2 = t.insert(B(20, 21), H(1, 2, 9, 9), -1, True, m)        # splits n1 after two blocks
    assert t.num_nodes() == 4 and t.total_cached_blocks() == 6
    assert t.node_size(n1) == 2 and t.node_size(n2) == 2        # the old handle now names the suffix
    m = t.match_prefix(H(1, 2, 3, 4, 5))
    assert m.num_matched_blocks == 4 and list(m.physical_blocks) == [10, 11, 12, 13]
    m = t.match_prefix(H(1, 2, 9, 9))
    assert m.num_matched_blocks == 4 and list(m.physical_blocks) == [10, 11, 20, 21]
    assert t.insert(B(), H(1, 2), -1, True, None) is None       # nothing new


@pytest.mark.parametrize("kind", KINDS)
def test_ready_match_is_a_contiguous_prefix(kind):
    t = make(kind)
    a = t.insert(B(1, 2), H(1, 2), -1, True, None)
    b = t.insert(B(3, 4), H(1, 2, 3, 4), -1, False, None)      # unready middle
    c = t.insert(B(5, 6), H(1, 2, 3, 4, 5, 6), -1, True, None)  # ready tail behind it
    m = t.match_prefix(H(1, 2, 3, 4, 5, 6))
    assert m.num_matched_blocks == 6 and m.num_ready_matched_blocks == 2
    assert m.last_ready_node == a
    t.set_ready(b, True, 2)
    m = t.match_prefix(H(1, 2, 3, 4, 5, 6))
    assert m.num_ready_matched_blocks == 6 and m.last_ready_node == c


@pytest.mark.parametrize("kind", KINDS)
def test_stale_insert_is_rejected_without_mutation(kind):
    t = make(kind)
    t.insert(B(1, 2, 3, 4), H(1, 2, 3, 4), -1, True, None)
    m_old = t.match_prefix(H(1, 2, 3, 4, 5, 6), -1, False)         # full match of the 4-block node
    # someone else extends the same path first
    t.insert(B(5, 6), H(1, 2, 3, 4, 5, 6), -1, True, None)
    before = (t.total_cached_blocks(), t.num_nodes())
    with pytest.raises(RuntimeError, match="stale"):
        t.insert(B(7, 8), H(1, 2, 3, 4, 5, 6), -1, True, m_old)   # target child exists now
    assert (t.total_cached_blocks(), t.num_nodes()) == before
    # concurrent split: the matched node shrank under the old result
    m_old = t.match_prefix(H(1, 2, 3, 4, 50), -1, False)
    t.insert(B(30), H(1, 2, 30), -1, True, None)                   # splits [1,2,3,4] into [1,2] + [3,4]
    with pytest.raises(RuntimeError, match="stale"):
        t.insert(B(51), H(1, 2, 3, 4, 50), -1, True, m_old)
    # evicted node: handle no longer resolves
    t2 = make(kind)
    t2.insert(B(1), H(1), -1, True, None)
    m = t2.match_prefix(H(1, 2), -1, False)
    t2.evict(1)
    with pytest.raises(RuntimeError):
        t2.insert(B(2), H(1, 2), -1, True, m)
    # wrong block count
    t3 = make(kind)
    with pytest.raises((ValueError, RuntimeError)):
        t3.insert(B(1, 2, 3), H(1, 2), -1, True, None)


@pytest.mark.parametrize("kind", KINDS)
def test_locks_and_unready_nodes_are_not_evicted(kind):
    t = make(kind)
    a = t.insert(B(1, 2), H(1, 2), -1, True, None)
    b = t.insert(B(3), H(1, 2, 3), -1, True, None)
    c = t.insert(B(4), H(7), -1, False, None)
    t.lock(b)
    blocks, hashes = t.evict(10)
    assert len(blocks) == 0                                     # b locked, a not a leaf, c unready
    t.unlock(b)
    with pytest.raises(RuntimeError):
        t.unlock(b)
    blocks, hashes = t.evict(10)
    assert sorted(blocks) == [1, 2, 3] and sorted(hashes) == [1, 2, 3]   # leaf first, then its parent
    assert not t.alive(a) and not t.alive(b) and t.alive(c)
    assert list(t.remove_unready_leaf(c)) == [4] and t.is_empty()


@pytest.mark.parametrize("kind", KINDS)
def test_partial_shrink_takes_the_tail(kind):
    t = make(kind)
    n = t.insert(B(1, 2, 3, 4, 5), H(1, 2, 3, 4, 5), -1, True, None)
    blocks, hashes = t.evict(2)
    assert list(blocks) == [4, 5] and list(hashes) == [4, 5]
    assert t.alive(n) and t.node_size(n) == 3 and t.total_cached_blocks() == 3
    assert t.match_prefix(H(1, 2, 3, 4, 5)).num_matched_blocks == 3


def _three(kind, policy, **kw):
    t = make(kind, eviction_policy=policy, **kw)
    t.set_clock_override(100)
    t.insert(B(1), H(1), -1, True, None)
    t.set_clock_override(200)
    t.insert(B(2), H(2), -1, True, None)
    t.set_clock_override(300)
    t.insert(B(3), H(3), -1, True, None)
    return t


@pytest.mark.parametrize("kind", KINDS)
def test_eviction_orders(kind):
    order = lambda t: [int(t.evict(1)[0][0]) for _ in range(3)]  # noqa: E731
    assert order(_three(kind, "lru")) == [1, 2, 3]
    assert order(_three(kind, "fifo")) == [1, 2, 3]
    assert order(_three(kind, "mru")) == [3, 2, 1]
    assert order(_three(kind, "filo")) == [3, 2, 1]
    # LRU follows access time, FIFO ignores it
    for policy, want in (("lru", [2, 3, 1]), ("fifo", [1, 2, 3]), ("mru", [1, 3, 2])):
        t = _three(kind, policy)
        t.set_clock_override(400)
        t.match_prefix(H(1))
        assert order(t) == want, policy
    # LFU: hit count first, then last access
    t = _three(kind, "lfu")
    t.set_clock_override(400)
    t.match_prefix(H(1)); t.match_prefix(H(1)); t.match_prefix(H(3))
    assert order(t) == [2, 3, 1]
    # SLRU: probationary (fewer than `threshold` hits) leaves before protected
    t = _three(kind, "slru", slru_threshold=2)
    t.set_clock_override(400)
    t.match_prefix(H(1)); t.match_prefix(H(1))       # 1 becomes protected
    t.set_clock_override(500)
    t.match_prefix(H(2))                              # one hit: still probationary, but recent
    assert order(t) == [3, 2, 1]


@pytest.mark.parametrize("kind", KINDS)
def test_hit_reward_extends_grace(kind):
    t = _three(kind, "lru", hit_reward_seconds=1000.0)
    t.set_clock_override(150)
    t.match_prefix(H(1))                              # grace(1) = max(100,150) + 1000 s
    assert [int(t.evict(1)[0][0]) for _ in range(3)] == [2, 3, 1]


@pytest.mark.parametrize("kind", KINDS)
def test_set_ready_walks_up_and_reset(kind):
    t = make(kind)
    a = t.insert(B(1, 2), H(1, 2), -1, False, None)
    b = t.insert(B(3), H(1, 2, 3), -1, False, None)
    t.set_ready(b, True, 3)
    assert t.node_ready(a) and t.node_ready(b) and t.total_ready_blocks() == 3
    assert t.num_evictable_blocks() == 3
    t.lock(b)
    assert t.num_evictable_blocks() == 0
    assert sorted(t.reset()) == [1, 2, 3]
    assert t.is_empty() and t.total_cached_blocks() == 0 and not t.alive(a)


def test_differential_native_vs_python_spec():
    rng = np.random.default_rng(7)
    nat, py = make("native", eviction_policy="lru"), make("python", eviction_policy="lru")
    clock = 1000
    next_block = 0
    seqs = []
    for step in range(400):
        clock += 10
        nat.set_clock_override(clock); py.set_clock_override(clock)
        r = rng.random()
        if r < 0.55 or not seqs:
            # new sequence sharing a random prefix of an old one
            if seqs and rng.random() < 0.7:
                base = seqs[rng.integers(len(seqs))]
                keep = int(rng.integers(0, len(base) + 1))
                h = np.concatenate([base[:keep], rng.integers(1, 2**62, size=int(rng.integers(1, 6)), dtype=np.uint64)])
            else:
                h = rng.integers(1, 2**62, size=int(rng.integers(1, 8)), dtype=np.uint64)
            seqs.append(h)
            mn, mp = nat.match_prefix(h), py.match_prefix(h)
            assert mn.num_matched_blocks == mp.num_matched_blocks
            assert mn.num_ready_matched_blocks == mp.num_ready_matched_blocks
            assert list(mn.physical_blocks) == list(mp.physical_blocks)
            k = len(h) - mn.num_matched_blocks
            ids = np.arange(next_block, next_block + k, dtype=np.int64)
            next_block += k
            ready = bool(rng.random() < 0.8)
            a, b = nat.insert(ids, h, -1, ready, mn), py.insert(ids, h, -1, ready, mp)
            assert (a is None) == (b is None)
        elif r < 0.8:
            h = seqs[rng.integers(len(seqs))]
            n = int(rng.integers(0, len(h) + 1))
            mn, mp = nat.match_prefix(h, n), py.match_prefix(h, n)
            assert (mn.num_matched_blocks, mn.num_ready_matched_blocks, mn.last_node_matched_length) == \
                (mp.num_matched_blocks, mp.num_ready_matched_blocks, mp.last_node_matched_length)
        else:
            n = int(rng.integers(1, 6))
            (bn, hn), (bp, hp) = nat.evict(n), py.evict(n)
            assert list(bn) == list(bp) and list(hn) == list(hp)
        assert nat.total_cached_blocks() == py.total_cached_blocks()
        assert nat.num_nodes() == py.num_nodes() and nat.num_leaves() == py.num_leaves()
        assert nat.num_evictable_blocks() == py.num_evictable_blocks()


@pytest.mark.parametrize("kind", KINDS)
def test_long_sequences(kind):
    t = make(kind)
    for n in (1, 10, 100, 1000, 10000):
        h = np.arange(1, n + 1, dtype=np.uint64) * np.uint64(2654435761) + np.uint64(n)
        t.insert(np.arange(n, dtype=np.int64), h, -1, True, None)
        m = t.match_prefix(h)
        assert m.num_matched_blocks == n and m.num_ready_matched_blocks == n
        assert m.physical_blocks[-1] == n - 1
