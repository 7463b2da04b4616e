"""Lease-aware local index, published block records and the read-only view of peers
(reference: csrc/dist/local_radix_tree.cpp:193-245,351-454,
csrc/dist/distributed_radix_tree.cpp:119-204,272-416)."""
import threading
import time

import numpy as np

from flexkv_b200 import _native

C = _native.C


def _h(*v):
    return np.array(v, dtype=np.uint64)


def _local(nid, ch, **kw):
    kw.setdefault("start_thread", False)
    kw.setdefault("lease_ttl_ms", 1000)
    kw.setdefault("renew_margin_ms", 400)
    return C.LocalRadixTree(nid, 4, 64, "lru", 0.0, ch, **kw)


def test_publish_renew_and_remote_match():
    ch = C.InProcMetaChannel()
    a = _local(1, ch)
    hashes = _h(11, 12, 13, 14)
    a.set_clock_override_ms(10_000)
    a.insert(np.array([7, 8, 9, 10], dtype=np.int64), hashes, 4, True, None)
    a.refresh_once(10_000)
    rows = sorted(ch.load(1), key=lambda r: r[3])
    assert [(r[0], r[1], r[2], r[3], r[4], r[5]) for r in rows] == [
        (0, 7, 1, 11, 11_000, 0), (11, 8, 1, 12, 11_000, 0), (12, 9, 1, 13, 11_000, 0), (13, 10, 1, 14, 11_000, 0)]

    view = C.DistributedRadixTree(2, ch, start_thread=False, safety_ttl_ms=100)
    view.refresh_once()
    n, pbs, nids = view.match_prefix(_h(11, 12, 13, 99), now_ms=10_100)
    assert n == 3 and pbs.tolist() == [7, 8, 9] and nids.tolist() == [1, 1, 1]
    # a wrong parent chain does not match even when the hash is known
    n, _, _ = view.match_prefix(_h(12, 13), now_ms=10_100)
    assert n == 0
    # too close to lease expiry: readers stay away
    n, _, _ = view.match_prefix(hashes, now_ms=10_950)
    assert n == 0
    # the owner renews once less than the margin is left
    a.refresh_once(10_500)
    assert a.stats()["renewed"] == 0
    a.refresh_once(10_700)
    assert a.stats()["renewed"] == 4
    view.refresh_once()
    n, _, _ = view.match_prefix(hashes, now_ms=10_950)
    assert n == 4
    # the owner's own view never contains its own blocks
    own = C.DistributedRadixTree(1, ch, start_thread=False)
    own.refresh_once()
    assert own.num_remote_blocks() == 0


def test_unready_blocks_are_not_published_until_set_ready():
    ch = C.InProcMetaChannel()
    a = _local(1, ch)
    node = a.insert(np.array([1, 2], dtype=np.int64), _h(21, 22), 2, False, None)
    a.refresh_once(1000)
    assert ch.load(1) == []
    a.set_ready(node, True, 2)
    a.refresh_once(1000)
    assert len(ch.load(1)) == 2


def test_leased_blocks_survive_eviction_until_the_lease_runs_out():
    ch = C.InProcMetaChannel()
    a = _local(1, ch)
    a.set_clock_override_ms(0)
    a.insert(np.array([1, 2, 3], dtype=np.int64), _h(31, 32, 33), 3, True, None)
    a.insert(np.array([4, 5], dtype=np.int64), _h(41, 42), 2, True, None)        # never published below
    a.refresh_once(0)                                                             # publishes both, lease to t=1000
    a.insert(np.array([6], dtype=np.int64), _h(51), 1, True, None)                # unpublished: evictable at once
    blocks, hashes = a.evict(4)
    assert sorted(blocks.tolist()) == [6]                                         # only the unleased block left
    assert a.stats()["marked_about_to_evict"] >= 3
    a.refresh_once(100)                                                           # announces, does not renew those
    states = {r[3]: r[5] for r in ch.load(1)}
    assert any(s == 1 for s in states.values())
    view = C.DistributedRadixTree(2, ch, start_thread=False)
    view.refresh_once()
    marked = [h for h, s in states.items() if s == 1]
    assert view.match_prefix(_h(*sorted(marked)), now_ms=100)[0] == 0             # peers stop using them
    a.set_clock_override_ms(1001)                                                 # lease over
    blocks, hashes = a.evict(3)
    assert len(blocks) == 3
    a.refresh_once(1001)
    left = {r[3] for r in ch.load(1)}
    assert not (set(hashes.tolist()) & left)                                      # withdrawn from the channel
    assert a.stats()["withdrawn"] == 3


def test_nearest_owner_wins_and_reset_withdraws():
    ch = C.InProcMetaChannel()
    trees = {nid: _local(nid, ch) for nid in (1, 2, 5)}
    for nid, t in trees.items():
        t.insert(np.array([100 + nid], dtype=np.int64), _h(61), 1, True, None)
        t.refresh_once(0)
    view = C.DistributedRadixTree(4, ch, start_thread=False)
    view.refresh_once()
    n, pbs, nids = view.match_prefix(_h(61), now_ms=10)
    assert n == 1 and nids.tolist() == [5] and pbs.tolist() == [105]
    trees[5].reset()
    view.refresh_once()
    assert view.match_prefix(_h(61), now_ms=10)[2].tolist() == [2]
    assert ch.list_nodes() == [1, 2]


class _PyChannel:
    """Channel written in Python; the native refresh threads call into it."""

    def __init__(self):
        self.d, self.lock, self.calls = {}, threading.Lock(), 0

    def publish(self, nid, rows):
        with self.lock:
            self.calls += 1
            self.d.setdefault(nid, {}).update({r[3]: tuple(r) for r in rows})

    def remove(self, nid, hashes):
        with self.lock:
            for h in hashes:
                self.d.get(nid, {}).pop(h, None)

    def list_nodes(self):
        with self.lock:
            return sorted(self.d)

    def load(self, nid):
        with self.lock:
            return list(self.d.get(nid, {}).values())

    def clear_node(self, nid):
        with self.lock:
            self.d.pop(nid, None)


def test_python_channel_with_background_threads():
    ch = _PyChannel()
    a = C.LocalRadixTree(1, 4, 64, "lru", 0.0, ch, lease_ttl_ms=2000, renew_margin_ms=1900, refresh_interval_ms=10)
    view = C.DistributedRadixTree(2, ch, refresh_interval_ms=10)
    a.insert(np.array([3, 4], dtype=np.int64), _h(71, 72), 2, True, None)
    deadline = time.time() + 5
    n = 0
    while time.time() < deadline and n < 2:
        time.sleep(0.02)
        n = view.match_prefix(_h(71, 72))[0]
    assert n == 2
    assert view.generation > 0 and ch.calls >= 1
    time.sleep(0.25)
    assert a.stats()["renewed"] >= 2          # margin of 1.9 s on a 2 s lease: renewed on the next passes
    a.shutdown()
    view.shutdown()
    del a, view
