"""Window snapshots mounted on radix nodes (invariants pinned by the reference's
tests/test_swa_node_mount.py: one snapshot per node at its trailing block, snapshots are
a subset of full KV, snapshot-only eviction prefers interior nodes, full locks >= window
locks, match returns the deepest fully matched ready node with a live snapshot)."""
import numpy as np
import pytest

from flexkv_b200 import _native

C = _native.C


def _h(*v):
    return np.array(v, dtype=np.uint64)


def _p(*v):
    return np.array(v, dtype=np.int64)


def _idx():
    return C.RadixIndex(2, 64, "lru", 0.0)


def test_match_returns_deepest_snapshot():
    idx = _idx()
    n1 = idx.insert(_p(0, 1, 2, 3), _h(1, 2, 3, 4), 4, True, None)
    idx.set_swa(n1, 100)
    assert idx.has_swa(n1) and idx.swa_slot(n1) == 100 and idx.total_swa_slots() == 1
    m = idx.match_prefix(_h(1, 2, 3, 4))
    assert m.num_matched_blocks == 4 and m.last_swa_node == n1 and m.swa_hit_blocks == 4 and m.swa_slot == 100
    # a partial match of the node must not expose its trailing-block snapshot
    m = idx.match_prefix(_h(1, 2, 3))
    assert m.num_matched_blocks == 3 and m.last_swa_node is None and m.swa_hit_blocks == 0


def test_split_keeps_snapshot_on_the_suffix_half():
    idx = _idx()
    n1 = idx.insert(_p(0, 1, 2, 3), _h(1, 2, 3, 4), 4, True, None)
    idx.set_swa(n1, 200)
    h2 = _h(1, 2, 55, 66)
    m = idx.match_prefix(h2)
    assert m.num_matched_blocks == 2
    idx.insert(_p(8, 9), h2, 4, True, m)
    assert idx.has_swa(n1) and idx.swa_slot(n1) == 200 and idx.node_size(n1) == 2
    parent = idx.node_parent(n1)
    assert not idx.is_root(parent) and not idx.has_swa(parent)
    assert idx.drain_freed_swa_slots().tolist() == []
    m = idx.match_prefix(_h(1, 2, 3, 4))
    assert m.last_swa_node == n1 and m.swa_hit_blocks == 4
    # the prefix half can get its own snapshot; the deeper one still wins on a full match
    idx.set_swa(parent, 201)
    assert idx.match_prefix(_h(1, 2, 3, 4)).swa_slot == 200
    assert idx.match_prefix(_h(1, 2, 77)).swa_slot == 201


def test_full_eviction_frees_the_snapshot_slot():
    idx = _idx()
    na = idx.insert(_p(0, 1), _h(1, 2), 2, True, None)
    idx.set_swa(na, 300)
    blocks, _ = idx.evict(2)
    assert len(blocks) == 2
    assert idx.drain_freed_swa_slots().tolist() == [300] and idx.total_swa_slots() == 0
    # partial shrink drops the trailing block, so the snapshot goes too
    nb = idx.insert(_p(4, 5, 6), _h(11, 12, 13), 3, True, None)
    idx.set_swa(nb, 301)
    blocks, _ = idx.evict(1)
    assert blocks.tolist() == [6] and idx.drain_freed_swa_slots().tolist() == [301] and not idx.has_swa(nb)


def test_snapshot_eviction_prefers_interior_and_deletes_unlocked_leaves():
    idx = _idx()
    leaf = idx.insert(_p(0, 1, 2, 3), _h(1, 2, 3, 4), 4, True, None)
    h2 = _h(1, 2, 99, 98)
    idx.insert(_p(8, 9), h2, 4, True, idx.match_prefix(h2))
    inner = idx.node_parent(leaf)
    idx.set_swa(inner, 401)          # older
    idx.set_swa(leaf, 400)           # newer
    blocks, hashes, freed = idx.evict_swa(1)
    assert freed == 1 and blocks.size == 0
    assert idx.drain_freed_swa_slots().tolist() == [401]
    assert not idx.has_swa(inner) and idx.node_size(inner) == 2 and idx.has_swa(leaf)
    # an unlocked leaf that loses its snapshot is deleted whole
    blocks, hashes, freed = idx.evict_swa(1)
    assert freed == 1 and sorted(blocks.tolist()) == [2, 3] and hashes.tolist() == [3, 4]
    assert idx.drain_freed_swa_slots().tolist() == [400] and not idx.alive(leaf)


def test_locks():
    idx = _idx()
    n = idx.insert(_p(0, 1), _h(1, 2), 2, True, None)
    with pytest.raises(RuntimeError):
        idx.lock_swa(n)                       # nothing to lock yet
    idx.set_swa(n, 600)
    idx.lock_swa(n)
    assert idx.swa_lock_cnt(n) == 1 and idx.node_lock_cnt(n) == 1     # full locks >= window locks
    assert idx.evict_swa(1)[2] == 0                                   # window-locked: untouched
    idx.unlock_swa(n)
    idx.lock(n)                               # full lock only: the node stays, the snapshot goes
    blocks, _, freed = idx.evict_swa(1)
    assert freed == 1 and blocks.size == 0 and idx.alive(n) and not idx.has_swa(n)
    idx.unlock(n)
    # replacing a snapshot returns the old slot; reset forgets everything
    idx.set_swa(n, 601)
    idx.set_swa(n, 602)
    assert idx.drain_freed_swa_slots().tolist() == [600, 601]
    idx.reset()
    assert idx.total_swa_slots() == 0 and idx.drain_freed_swa_slots().tolist() == []


def test_python_specification_and_native_index_agree_on_random_snapshot_workloads():
    """Same random script of inserts, snapshot mounts, matches, full and snapshot-only evictions and locks
    on the native index and on the Python specification; every observable must agree."""
    from flexkv_b200.cache.radixtree import RadixTreeIndex
    for seed in range(6):
        rng = np.random.default_rng(seed)
        nat, py = C.RadixIndex(2, 0, "lru", 0.0), RadixTreeIndex(2, 0, "lru", 0.0)
        nat.set_clock_override(1000)
        py._clock_override = 1000
        seqs, handles, next_block, next_slot, clock = [], [], 0, 0, 1000
        for step in range(300):
            clock += 1
            nat.set_clock_override(clock)
            py._clock_override = clock
            op = int(rng.integers(0, 10))
            if op < 4 or not seqs:
                if seqs and rng.random() < 0.5:
                    base = seqs[int(rng.integers(len(seqs)))]
                    k = int(rng.integers(1, len(base) + 1))
                    h = np.concatenate([base[:k], rng.integers(1, 2**62, size=int(rng.integers(1, 5)), dtype=np.uint64)])
                else:
                    h = rng.integers(1, 2**62, size=int(rng.integers(1, 6)), dtype=np.uint64)
                mn, mp = nat.match_prefix(h), py.match_prefix(h)
                assert mn.num_matched_blocks == mp.num_matched_blocks
                need = len(h) - mn.num_matched_blocks
                if need:
                    phys = np.arange(next_block, next_block + need, dtype=np.int64)
                    next_block += need
                    hn, hp = nat.insert(phys, h, len(h), True, mn), py.insert(phys, h, len(h), True, mp)
                    handles.append((hn, hp))
                    seqs.append(h)
            elif op < 6 and handles:
                hn, hp = handles[int(rng.integers(len(handles)))]
                if nat.alive(hn):
                    assert py.alive(hp)
                    nat.set_swa(hn, next_slot); py.set_swa(hp, next_slot)
                    next_slot += 1
            elif op < 8:
                h = seqs[int(rng.integers(len(seqs)))]
                k = int(rng.integers(1, len(h) + 1))
                mn, mp = nat.match_prefix(h[:k]), py.match_prefix(h[:k])
                assert (mn.num_matched_blocks, mn.swa_hit_blocks, mn.swa_slot) == \
                    (mp.num_matched_blocks, mp.swa_hit_blocks, mp.swa_slot), (seed, step)
            elif op == 8:
                n = int(rng.integers(1, 4))
                bn, hn_, fn = nat.evict_swa(n)
                bp, hp_, fp = py.evict_swa(n)
                assert fn == fp and sorted(bn.tolist()) == sorted(bp.tolist()), (seed, step)
            else:
                n = int(rng.integers(1, 6))
                bn, _ = nat.evict(n)
                bp, _ = py.evict(n)
                assert sorted(bn.tolist()) == sorted(bp.tolist()), (seed, step)
            assert sorted(nat.drain_freed_swa_slots().tolist()) == sorted(py.drain_freed_swa_slots().tolist()), (seed, step)
            assert nat.total_swa_slots() == py.total_swa_slots()
            assert nat.total_cached_blocks() == py._total_blocks


INDEXES = [("native", lambda: C.RadixIndex(2, 64, "lru", 0.0))]


def _py_index():
    from flexkv_b200.cache.radixtree import RadixTreeIndex
    return RadixTreeIndex(2, 64, "lru", 0.0)


INDEXES.append(("python", _py_index))


def _clock(idx, t):
    if hasattr(idx, "set_clock_override"):
        idx.set_clock_override(t)
    else:
        idx._clock_override = t


@pytest.mark.parametrize("name,make", INDEXES)
def test_a_real_match_refreshes_the_snapshot_and_a_probe_does_not(name, make):
    """Snapshot-only eviction takes the least recently used snapshot; a match that updates cache information
    counts as a use, a probe (update_cache_info=False) does not (reference: tests/test_swa_node_mount.py
    reuse-promotes / probe-does-not-promote, both index back ends)."""
    for update, survivor in ((True, "a"), (False, "b")):
        idx = make()
        _clock(idx, 100)
        a = idx.insert(_p(0, 1), _h(1, 2), 2, True, None)
        idx.set_swa(a, 10)
        b = idx.insert(_p(2, 3), _h(5, 6), 2, True, None)
        idx.set_swa(b, 11)
        _clock(idx, 200)
        m = idx.match_prefix(_h(1, 2), 2, update)
        assert m.swa_slot == 10
        assert idx.evict_swa(1)[2] == 1
        alive = {"a": idx.alive(a) and idx.has_swa(a), "b": idx.alive(b) and idx.has_swa(b)}
        assert alive == {"a": survivor == "a", "b": survivor == "b"}, (name, update)


@pytest.mark.parametrize("name,make", INDEXES)
def test_window_locked_nodes_and_the_root_survive_full_eviction(name, make):
    idx = make()
    assert len(idx.evict(1)[0]) == 0                       # an empty index has nothing to give
    n = idx.insert(_p(0, 1), _h(1, 2), 2, True, None)
    idx.set_swa(n, 5)
    idx.lock_swa(n)
    assert len(idx.evict(2)[0]) == 0 and idx.alive(n) and idx.has_swa(n)
    idx.unlock_swa(n)
    assert sorted(idx.evict(2)[0].tolist()) == [0, 1] and idx.drain_freed_swa_slots().tolist() == [5]


def _fork(idx, snapshot):
    """root -> A(1,2) -> {a(3,4) [snapshot 901], b(55,66)}"""
    a = idx.insert(_p(0, 1, 2, 3), _h(1, 2, 3, 4), 4, True, None)
    if snapshot:
        idx.set_swa(a, 901)
    h2 = _h(1, 2, 55, 66)
    b = idx.insert(_p(8, 9), h2, 4, True, idx.match_prefix(h2))
    return idx.node_parent(a), a, b


@pytest.mark.parametrize("name,make", INDEXES)
def test_full_eviction_takes_ancestors_left_as_leaves_without_a_snapshot(name, make):
    """With window snapshots in use, a leaf without one serves no window-aware request: once both children are
    gone the parent goes too, beyond the number of blocks asked for; a locked parent stays; an index that never
    saw a snapshot keeps the plain rule (reference: tests/test_swa_node_mount.py:836-893)."""
    idx = make()
    A, a, b = _fork(idx, snapshot=True)
    blocks, hashes = idx.evict(4)
    assert sorted(blocks.tolist()) == [0, 1, 2, 3, 8, 9] and len(hashes) == 6
    assert not idx.alive(A) and idx.total_swa_slots() == 0 and idx.drain_freed_swa_slots().tolist() == [901]
    assert idx.match_prefix(_h(1, 2)).num_matched_blocks == 0

    idx = make()
    A, a, b = _fork(idx, snapshot=True)
    idx.lock(A)                                            # the parent's blocks are still referenced
    blocks, _ = idx.evict(4)
    assert sorted(blocks.tolist()) == [2, 3, 8, 9] and idx.alive(A) and idx.node_size(A) == 2
    idx.unlock(A)

    idx = make()                                           # never armed: exactly what was asked for
    A, a, b = _fork(idx, snapshot=False)
    blocks, _ = idx.evict(4)
    assert sorted(blocks.tolist()) == [2, 3, 8, 9] and idx.alive(A)
    assert idx.match_prefix(_h(1, 2)).num_matched_blocks == 2


@pytest.mark.parametrize("name,make", INDEXES)
def test_snapshot_eviction_of_a_leaf_takes_its_bare_ancestors_along(name, make):
    idx = make()
    A = idx.insert(_p(0, 1), _h(1, 2), 2, True, None)
    leaf = idx.insert(_p(2, 3), _h(1, 2, 3, 4), 4, True, idx.match_prefix(_h(1, 2, 3, 4)))
    idx.set_swa(leaf, 7)
    blocks, hashes, freed = idx.evict_swa(1)
    assert freed == 1 and sorted(blocks.tolist()) == [0, 1, 2, 3] and sorted(hashes.tolist()) == [1, 2, 3, 4]
    assert not idx.alive(A) and not idx.alive(leaf) and idx.drain_freed_swa_slots().tolist() == [7]
