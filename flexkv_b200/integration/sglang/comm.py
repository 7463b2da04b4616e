"""Rank coordination for the SGLang connector and the engine-side layer hook.

``FlexKVComm``: only the sync leader of a replica owns a KVManager; it scatters
per-request manifests (matched lengths, task ids, slot mappings) to the other
TP / CP / PP ranks, and block counts are agreed with an all-reduce(MIN), over a
CPU (gloo) process group (flexkv/integration/sglang/comm.py:81-560).

``FlexKVLayerDoneCounter``: ``num_counters`` sets of per-layer eventfds (triple
buffering, so a new restore can be prepared while the previous one is being
consumed). The model's layer hook calls ``wait_until(layer)``, which blocks on
that layer's eventfd of the consumer set once per restore in flight
(flexkv/integration/sglang/comm.py:611-983).
"""
from __future__ import annotations

import os
import select
import threading
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist


class FlexKVComm:
    def __init__(self, world_group=None, tp_size: int = 1, cp_size: int = 1, pp_size: int = 1,
                 rank: Optional[int] = None) -> None:
        self.group = world_group
        self.enabled = dist.is_available() and dist.is_initialized()
        self.rank = rank if rank is not None else (dist.get_rank(self.group) if self.enabled else 0)
        self.world = dist.get_world_size(self.group) if self.enabled else 1
        self.tp_size, self.cp_size, self.pp_size = tp_size, cp_size, pp_size
        self.leader = 0
        if self.enabled and dist.get_backend(self.group) != "gloo":
            # manifests are CPU objects: coordination needs a CPU-capable group
            self.group = dist.new_group(backend="gloo")

    @property
    def is_leader(self) -> bool:
        return self.rank == self.leader

    def scatter(self, data: Optional[List[Any]] = None) -> Any:
        """Leader passes one payload per rank; every rank returns its own."""
        if not self.enabled or self.world == 1:
            return data[0] if data is not None else None
        out: List[Any] = [None]
        dist.scatter_object_list(out, data if self.is_leader else None, src=self.leader, group=self.group)
        return out[0]

    def broadcast(self, data: Any = None) -> Any:
        if not self.enabled or self.world == 1:
            return data
        box = [data if self.is_leader else None]
        dist.broadcast_object_list(box, src=self.leader, group=self.group)
        return box[0]

    def scatter_pp(self, data: Any = None) -> Any:
        """Pipeline-only fan-out: the leader of stage 0 hands ``data`` to the leader of every other
        stage; ranks that lead no stage return None (flexkv/integration/sglang/comm.py:342-352).
        Ranks are laid out stage-major: stage s owns ranks [s * world / pp, (s + 1) * world / pp)."""
        if not self.enabled or self.pp_size <= 1 or self.world == 1:
            return data
        per_stage = self.world // self.pp_size
        leaders = [s * per_stage for s in range(self.pp_size)]
        if self.rank not in leaders:
            return None
        if self.rank == leaders[0]:
            for r in leaders[1:]:
                dist.send_object_list([data], dst=r, group=self.group)
            return data
        box: List[Any] = [None]
        dist.recv_object_list(box, src=leaders[0], group=self.group)
        return box[0]

    def all_reduce_min(self, value: int) -> int:
        if not self.enabled or self.world == 1:
            return int(value)
        t = torch.tensor([int(value)], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return int(t.item())

    def barrier(self) -> None:
        if self.enabled and self.world > 1:
            dist.barrier(group=self.group)


def layerwise_wait_timeout_s() -> float:
    """How long a layer hook waits for its restore before it gives up (FLEXKV_LAYERWISE_WAIT_TIMEOUT_S, 240 s;
    a value that does not parse keeps the default: flexkv/integration/sglang/comm.py:775-781)."""
    raw = os.environ.get("FLEXKV_LAYERWISE_WAIT_TIMEOUT_S", "240")
    try:
        v = float(raw)
        return v if v > 0 else 240.0
    except ValueError:
        return 240.0


class FlexKVLayerLoadingEvent:
    """One set of per-layer eventfds plus the number of restores that will signal it."""

    def __init__(self, num_layers: int) -> None:
        self.num_layers = num_layers
        self.fds = [os.eventfd(0, os.EFD_NONBLOCK | os.EFD_SEMAPHORE) for _ in range(num_layers)]
        self._pending = 0
        self._lock = threading.Lock()

    def _drain(self) -> None:
        for fd in self.fds:
            while True:
                try:
                    os.read(fd, 8)
                except BlockingIOError:
                    break

    finished = True          # nothing registered, nothing being waited for: the set may be handed out again
    wait_started = False     # a forward pass began consuming this set

    def reset_for_new_transfer(self) -> None:
        with self._lock:
            self._drain()
            self._pending = 0
            self.finished, self.wait_started = False, False

    def mark_reusable(self) -> None:
        """Returns the set to the ring. The caller has made sure that no restore can still signal it (every
        launched layerwise task was waited for) - flexkv/integration/sglang/comm.py:672-682."""
        with self._lock:
            self._drain()
            self._pending = 0
            self.finished, self.wait_started = True, False

    def add_transfer(self) -> None:
        with self._lock:
            self._pending += 1

    def remove_transfer(self) -> None:
        with self._lock:
            self._pending = max(0, self._pending - 1)

    def pending_transfers(self) -> int:
        return self._pending

    def wait(self, layer: int, timeout: float = 240.0) -> None:
        """Blocks until every restore registered on this set has signalled `layer`."""
        need = self._pending
        self.wait_started = True
        fd = self.fds[layer]
        deadline = time.monotonic() + timeout
        got = 0
        while got < need:
            left = deadline - time.monotonic()
            if left <= 0:
                raise TimeoutError(f"layer {layer}: {got} of {need} restores signalled within {timeout} s")
            r, _, _ = select.select([fd], [], [], min(left, 1.0))
            if r:
                try:
                    os.read(fd, 8)      # semaphore mode: one unit per read
                    got += 1
                except BlockingIOError:
                    pass

    def close(self) -> None:
        for fd in self.fds:
            try:
                os.close(fd)
            except OSError:
                pass
        self.fds = []


class FlexKVLayerDoneCounter:
    def __init__(self, num_layers: int, num_counters: int = 3, world_rank: int = -1) -> None:
        self.num_layers, self.num_counters, self.world_rank = num_layers, num_counters, world_rank
        self.events = [FlexKVLayerLoadingEvent(num_layers) for _ in range(num_counters)]
        self._producer = -1
        self._consumer = -1
        self._task_to_counter: Dict[int, int] = {}

    def fds_per_counter(self) -> List[List[int]]:
        return [list(e.fds) for e in self.events]

    def update_producer(self) -> int:
        """Chooses the next set for a new restore and clears it."""
        self._producer = (self._producer + 1) % self.num_counters
        self.events[self._producer].reset_for_new_transfer()
        return self._producer

    def register_task(self, task_id: int, producer_id: int) -> None:
        self._task_to_counter[task_id] = producer_id
        self.events[producer_id].add_transfer()

    def expected_transfer_count(self, counter_id: int) -> int:
        """Checks, without changing anything, that a restore may still be added to set ``counter_id`` and returns
        how many are registered on it. Followers call it with the leader's choice, so that a rank whose batch
        boundary differs from the leader's fails loudly instead of waiting on the wrong set
        (flexkv/integration/sglang/comm.py:798-844)."""
        if not 0 <= counter_id < self.num_counters:
            raise ValueError(f"invalid counter id {counter_id}, must be in [0, {self.num_counters})")
        ev = self.events[counter_id]
        if ev.wait_started:
            raise RuntimeError(f"counter {counter_id} is already being consumed by a forward pass")
        if self._consumer == counter_id and ev.finished:
            raise RuntimeError(f"counter {counter_id} is marked finished but still selected for consumption")
        return ev.pending_transfers()

    def register_task_with_explicit_counter_id(self, task_id: int, counter_id: int) -> None:
        """Follower side of a batched restore: the leader chose the set."""
        self.expected_transfer_count(counter_id)
        if task_id in self._task_to_counter:
            raise RuntimeError(f"task {task_id} is already registered")
        ev = self.events[counter_id]
        if ev.finished:
            ev.reset_for_new_transfer()
        self._producer = counter_id
        self.register_task(task_id, counter_id)

    def abort_unregistered_selection(self, producer_id: int) -> None:
        """Gives back a set the leader selected with ``update_producer`` when nothing was registered on it after
        all (the plan turned out empty)."""
        if not 0 <= producer_id < self.num_counters:
            raise ValueError(f"invalid producer id {producer_id}, must be in [0, {self.num_counters})")
        ev = self.events[producer_id]
        if self._consumer == producer_id or ev.wait_started:
            raise RuntimeError(f"counter {producer_id} is already being consumed")
        if ev.pending_transfers() != 0:
            raise RuntimeError(f"counter {producer_id} already has registered transfers")
        ev.mark_reusable()
        if self._producer == producer_id:
            self._producer = (producer_id - 1) % self.num_counters

    def rollback_prepared_transfer(self, task_id: int) -> None:
        c = self._task_to_counter.pop(task_id, None)
        if c is not None:
            self.events[c].remove_transfer()

    def set_consumer(self, task_id: int) -> None:
        """The forward pass that is about to run consumes the set this task signals."""
        self._consumer = self._task_to_counter.pop(task_id, self._consumer)

    def wait_until(self, layer: int, timeout: Optional[float] = None) -> None:
        if self._consumer < 0:
            return
        if timeout is None:
            timeout = layerwise_wait_timeout_s()
        self.events[self._consumer].wait(layer, timeout)
        if layer == self.num_layers - 1:
            self.events[self._consumer].mark_reusable()
            self._consumer = -1

    def reset(self) -> None:
        for e in self.events:
            e.mark_reusable()
        self._producer = self._consumer = -1
        self._task_to_counter.clear()

    def close(self) -> None:
        for e in self.events:
            e.close()
