"""Transfer IR: ops, the per-task op graph and batch merging.

A ``get``/``put`` plan is a small DAG of block moves between tiers. Op kinds
and their names follow the reference (flexkv/common/transfer.py:91-118); the
graph object here is a plain dependency counter with late binding of GPU block
ids (the engine hands over its slot mapping only at launch,
flexkv/common/transfer.py:369-404) and a merge step that folds the graphs of
many tasks into one op per tier hop (flexkv/common/transfer.py:761-1042).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum, IntEnum
from typing import Dict, Iterable, List, NamedTuple, Optional, Sequence, Set, Tuple

import numpy as np


class DeviceType(IntEnum):
    CPU = 0
    GPU = 1
    SSD = 2
    REMOTE = 3
    PEERCPU = 4
    PEERSSD = 5
    PEERGPU = 6      # another rank's HBM, reached over NVLink


class TransferType(Enum):
    H2D = "H2D"
    D2H = "D2H"
    DISK2H = "DISK2H"
    H2DISK = "H2DISK"
    DISK2D = "DISK2D"
    D2DISK = "D2DISK"
    REMOTE2H = "REMOTE2H"
    H2REMOTE = "H2REMOTE"
    PEERH2H = "PEERH2H"
    H2PEERH = "H2PEERH"
    PEERSSD2H = "PEERSSD2H"
    H2PEERSSD = "H2PEERSSD"
    PEERD2D = "PEERD2D"       # NVLink pull from a peer GPU's block table
    VIRTUAL = "Virtual"       # no data; joins its predecessors
    LAYERWISE = "LAYERWISE"   # fused DISK2H + per-layer H2D with notifications


class WorkerKey(NamedTuple):
    dp_client_id: int = 0
    pp_rank: int = 0


class TransferOpStatus(Enum):
    PENDING = 0
    RUNNING = 1
    COMPLETED = 2
    FAILED = 3


_op_ids = itertools.count()
_graph_ids = itertools.count()
_EMPTY = np.zeros(0, dtype=np.int64)


def _ids(a: Optional[Sequence[int]]) -> np.ndarray:
    if a is None:
        return _EMPTY
    return np.ascontiguousarray(a, dtype=np.int64)


@dataclass
class TransferOp:
    graph_id: int
    transfer_type: TransferType
    src_block_ids: np.ndarray
    dst_block_ids: np.ndarray
    dp_client_id: int = 0
    # Late GPU binding: the side named by `gpu_side` ("src" or "dst") is filled by
    # TransferOpGraph.set_gpu_blocks from the head (or, for DISK2D / D2DISK, the
    # tail) of the block ids the engine passes at launch
    gpu_side: Optional[str] = None
    gpu_bind: str = "head"
    gpu_offset: int = 0           # head binding starts this many blocks into the launch-time list
    is_swa: bool = False
    allow_partial: bool = False   # a per-block failure does not fail the op: the planner adopts the good prefix
    remote_node_ids: Optional[np.ndarray] = None      # owner node / rank per block (peer ops)
    block_hashes: Optional[np.ndarray] = None         # key-addressed remote stores
    layer_start: int = 0
    num_layers: int = -1                              # -1 = all
    op_id: int = field(default_factory=lambda: next(_op_ids))
    predecessors: Set[int] = field(default_factory=set)
    successors: Set[int] = field(default_factory=set)
    status: TransferOpStatus = TransferOpStatus.PENDING
    pending_count: int = 0                            # PP siblings still running
    block_results: Optional[Tuple[bool, ...]] = None  # per-block success of partial-capable backends
    merged_from: List[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        self.src_block_ids = _ids(self.src_block_ids)
        self.dst_block_ids = _ids(self.dst_block_ids)
        if self.transfer_type not in (TransferType.VIRTUAL, TransferType.LAYERWISE) and self.gpu_side is None \
                and self.src_block_ids.size != self.dst_block_ids.size:
            raise ValueError(f"{self.transfer_type.value}: src has {self.src_block_ids.size} blocks, "
                             f"dst has {self.dst_block_ids.size}")

    @property
    def valid_block_num(self) -> int:
        if self.gpu_side == "src":
            return int(self.dst_block_ids.size)
        return int(self.src_block_ids.size)


@dataclass
class LayerwiseTransferOp(TransferOp):
    """SSD->host for all layers, then host->GPU layer by layer with one
    notification per layer (flexkv/common/transfer.py:185-249)."""
    src_block_ids_h2d: np.ndarray = field(default_factory=lambda: _EMPTY)
    dst_block_ids_h2d: np.ndarray = field(default_factory=lambda: _EMPTY)
    src_block_ids_disk2h: np.ndarray = field(default_factory=lambda: _EMPTY)
    dst_block_ids_disk2h: np.ndarray = field(default_factory=lambda: _EMPTY)
    counter_id: int = 0

    def __post_init__(self) -> None:
        self.transfer_type = TransferType.LAYERWISE
        super().__post_init__()
        for n in ("src_block_ids_h2d", "dst_block_ids_h2d", "src_block_ids_disk2h", "dst_block_ids_disk2h"):
            setattr(self, n, _ids(getattr(self, n)))
        if self.src_block_ids_h2d.size != self.dst_block_ids_h2d.size:
            raise ValueError("layerwise h2d id arrays differ in size")
        if self.src_block_ids_disk2h.size != self.dst_block_ids_disk2h.size:
            raise ValueError("layerwise disk2h id arrays differ in size")


@dataclass
class CompletedOp:
    graph_id: int
    op_id: int
    success: bool = True
    failed_graph: bool = False                       # the whole graph was abandoned
    block_results: Optional[Tuple[bool, ...]] = None
    gpu_ms: float = 0.0
    num_bytes: int = 0

    def is_graph_completed(self) -> bool:
        return self.op_id == -1

    @staticmethod
    def graph_done(graph_id: int, success: bool = True) -> "CompletedOp":
        return CompletedOp(graph_id=graph_id, op_id=-1, success=success, failed_graph=not success)


class TransferOpGraph:
    def __init__(self) -> None:
        self.graph_id: int = next(_graph_ids)
        self._ops: Dict[int, TransferOp] = {}
        self._ready: Set[int] = set()
        self._unfinished: int = 0
        self._gpu_bound = True
        self.failed = False

    # ---- construction ---------------------------------------------------------
    @classmethod
    def create_empty_graph(cls) -> "TransferOpGraph":
        return cls()

    def add_transfer_op(self, op: TransferOp) -> int:
        op.graph_id = self.graph_id
        self._ops[op.op_id] = op
        self._ready.add(op.op_id)
        self._unfinished += 1
        if op.gpu_side is not None and not op.is_swa:   # window side ops are bound (or dropped) at launch
            self._gpu_bound = False
        return op.op_id

    def add_virtual_op(self, predecessors: Iterable[int]) -> int:
        op = TransferOp(self.graph_id, TransferType.VIRTUAL, _EMPTY, _EMPTY)
        self.add_transfer_op(op)
        for p in predecessors:
            self.add_dependency(op.op_id, p)
        return op.op_id

    def add_dependency(self, successor_op_id: int, predecessor_op_id: int) -> None:
        s, p = self._ops[successor_op_id], self._ops[predecessor_op_id]
        if p.status == TransferOpStatus.COMPLETED:
            return
        s.predecessors.add(predecessor_op_id)
        p.successors.add(successor_op_id)
        self._ready.discard(successor_op_id)

    # ---- late binding ---------------------------------------------------------
    def set_gpu_blocks(self, gpu_block_ids: np.ndarray) -> None:
        gpu_block_ids = _ids(gpu_block_ids)
        for op in self._ops.values():
            if op.gpu_side is None or op.is_swa:
                continue
            if isinstance(op, LayerwiseTransferOp):
                n = int(op.src_block_ids_h2d.size)
            else:
                n = int(op.dst_block_ids.size if op.gpu_side == "src" else op.src_block_ids.size)
            if n + (op.gpu_offset if op.gpu_bind == "head" else 0) > gpu_block_ids.size:
                raise ValueError(f"slot mapping covers {gpu_block_ids.size} blocks, op needs "
                                 f"{n} at offset {op.gpu_offset}")
            ids = gpu_block_ids[op.gpu_offset:op.gpu_offset + n] if op.gpu_bind == "head" \
                else gpu_block_ids[gpu_block_ids.size - n:]
            if op.gpu_side == "src":
                op.src_block_ids = ids
            else:
                op.dst_block_ids = ids
            if isinstance(op, LayerwiseTransferOp):
                op.dst_block_ids_h2d = ids
            op._late_side = op.gpu_side
        self._gpu_bound = True

    @property
    def gpu_bound(self) -> bool:
        return self._gpu_bound

    def set_swa_pages(self, page_ids: Optional[np.ndarray]) -> None:
        """Binds the GPU side of sliding-window side ops to the caller's window pages. With
        ``None`` the side ops are turned into no-ops (the caller moves no window state)."""
        for op in self._ops.values():
            if not op.is_swa:
                continue
            if page_ids is None and (op.gpu_side is not None or
                                     op.transfer_type in (TransferType.H2DISK, TransferType.DISK2H, TransferType.H2REMOTE,
                                                          TransferType.REMOTE2H)):
                # the whole window chain goes, tier-to-tier hops included: their source never arrives
                op.transfer_type = TransferType.VIRTUAL
                op.src_block_ids = op.dst_block_ids = _EMPTY
                op.gpu_side = None
                continue
            if op.gpu_side is None:
                continue
            n = int(op.dst_block_ids.size if op.gpu_side == "src" else op.src_block_ids.size)
            ids = _ids(page_ids)
            if ids.size < n:
                raise ValueError(f"window side op needs {n} page(s), {ids.size} given")
            if op.gpu_side == "src":
                op.src_block_ids = ids[:n]
            else:
                op.dst_block_ids = ids[:n]
            op.gpu_side = None

    # ---- execution ------------------------------------------------------------
    set_swa_gpu_blocks = set_swa_pages      # the reference's name for the same binding step

    _GPU_SIDE_OF = {"D2H": "src", "H2D": "dst", "DISK2D": "dst", "D2DISK": "src", "PEERD2D": "dst"}

    def clear_gpu_blocks(self, force: bool = False) -> None:
        """Forgets the bound GPU side of every late-bound op so that another pipeline stage (whose
        engine uses its own block ids) can bind the same plan again (flexkv/kvtask.py:438-444).
        ``force`` also unbinds ops whose GPU pages were known when the plan was made (a put, a one-call get):
        which side is the GPU's follows from the op's type, its place in the page list from its binding rule."""
        for op in self._ops.values():
            side = getattr(op, "_late_side", None)
            if side is None and force and not op.is_swa:
                side = self._GPU_SIDE_OF.get(op.transfer_type.value)
                if side is None and isinstance(op, LayerwiseTransferOp):
                    side = "dst"
            if side is None or op.is_swa:
                continue
            if side == "src":
                op.src_block_ids = _EMPTY
            else:
                op.dst_block_ids = _EMPTY
            op.gpu_side = side
            self._gpu_bound = False

    def is_graph_failed(self) -> bool:
        return bool(self.failed)

    def visualize(self) -> str:
        """Text dump of the DAG: one line per op with type, block counts, state and predecessors."""
        lines = [f"graph {self.graph_id}: {len(self._ops)} ops, {self._unfinished} unfinished"
                 f"{', FAILED' if self.failed else ''}"]
        for oid in sorted(self._ops):
            op = self._ops[oid]
            dep = ",".join(str(p) for p in sorted(op.predecessors)) or "-"
            lines.append(f"  op {oid:>5} {op.transfer_type.value:<10} src={op.src_block_ids.size:<6} "
                         f"dst={op.dst_block_ids.size:<6} {op.status.name:<9} after [{dep}]"
                         f"{' swa' if op.is_swa else ''}{' late:' + op.gpu_side if op.gpu_side else ''}")
        return "\n".join(lines)

    def take_ready_ops(self) -> List[TransferOp]:
        """Ops whose predecessors are all done and that were not handed out yet."""
        out = []
        for oid in sorted(self._ready):
            op = self._ops[oid]
            if op.status == TransferOpStatus.PENDING:
                op.status = TransferOpStatus.RUNNING
                out.append(op)
        self._ready.clear()
        return out

    def requeue(self, op_id: int) -> None:
        """Hands an op that was taken but not started back to the ready set."""
        op = self._ops[op_id]
        if op.status == TransferOpStatus.RUNNING:
            op.status = TransferOpStatus.PENDING
            self._ready.add(op_id)

    def mark_completed(self, op_id: int, success: bool = True) -> List[int]:
        """Returns ids of ops that became ready."""
        op = self._ops[op_id]
        if op.status in (TransferOpStatus.COMPLETED, TransferOpStatus.FAILED):
            return []
        op.status = TransferOpStatus.COMPLETED if success else TransferOpStatus.FAILED
        self._unfinished -= 1
        newly = []
        if not success:
            self.failed = True
            return newly
        for s in op.successors:
            so = self._ops[s]
            so.predecessors.discard(op_id)
            if not so.predecessors and so.status == TransferOpStatus.PENDING:
                self._ready.add(s)
                newly.append(s)
        return newly

    def all_transfer_ops_completed(self) -> bool:
        return self._unfinished == 0

    def running_ops(self) -> List[int]:
        return [o.op_id for o in self._ops.values() if o.status == TransferOpStatus.RUNNING]

    def pending_ops(self) -> List[int]:
        return [o.op_id for o in self._ops.values() if o.status == TransferOpStatus.PENDING]

    @property
    def num_ops(self) -> int:
        return len(self._ops)

    def ops(self) -> List[TransferOp]:
        return list(self._ops.values())

    def get_op(self, op_id: int) -> TransferOp:
        return self._ops[op_id]

    def has_op(self, op_id: int) -> bool:
        return op_id in self._ops

    def __repr__(self) -> str:
        body = ", ".join(f"{o.op_id}:{o.transfer_type.value}[{o.valid_block_num}]<-{sorted(o.predecessors)}"
                         for o in self._ops.values())
        return f"TransferOpGraph(id={self.graph_id}, {body})"


def _cat(arrs: List[np.ndarray]) -> np.ndarray:
    arrs = [a for a in arrs if a is not None and a.size]
    return np.concatenate(arrs) if arrs else _EMPTY


_MERGE_ORDER_GET = [TransferType.DISK2H, TransferType.REMOTE2H, TransferType.PEERH2H, TransferType.PEERSSD2H,
                    TransferType.PEERD2D, TransferType.DISK2D, TransferType.H2D]
_MERGE_ORDER_PUT = [TransferType.D2H, TransferType.H2DISK, TransferType.H2REMOTE, TransferType.D2DISK]
_STAGE_IN = (TransferType.DISK2H, TransferType.REMOTE2H, TransferType.PEERH2H, TransferType.PEERSSD2H)


def merge_to_batch_graph(graphs: List[TransferOpGraph], layerwise: bool = False, counter_id: int = 0
                         ) -> Tuple[TransferOpGraph, Dict[int, int]]:
    """Folds the (GPU-bound) graphs of several tasks into one graph with one op
    per transfer type. Returns the merged graph and ``old_op_id -> new_op_id``.

    GET side: every host-staging op (DISK2H, REMOTE2H, peer reads) precedes the
    single H2D; PUT side: the single D2H precedes H2DISK / H2REMOTE. With
    ``layerwise`` the DISK2H and H2D ops are folded into one LAYERWISE op.
    """
    merged = TransferOpGraph()
    remap: Dict[int, int] = {}
    by_type: Dict[TransferType, List[TransferOp]] = {}
    swa_ops: List[TransferOp] = []
    for g in graphs:
        if not g.gpu_bound:
            raise ValueError("merge_to_batch_graph needs GPU block ids bound on every graph")
        for op in g.ops():
            if op.transfer_type == TransferType.VIRTUAL:
                continue
            if op.is_swa:
                swa_ops.append(op)
                continue
            by_type.setdefault(op.transfer_type, []).append(op)

    new_ops: Dict[TransferType, TransferOp] = {}

    def fold(tt: TransferType) -> Optional[TransferOp]:
        ops = by_type.get(tt)
        if not ops:
            return None
        first = ops[0]
        nodes = _cat([o.remote_node_ids for o in ops if o.remote_node_ids is not None])
        hashes = _cat([o.block_hashes for o in ops if o.block_hashes is not None])
        new = TransferOp(merged.graph_id, tt, _cat([o.src_block_ids for o in ops]),
                         _cat([o.dst_block_ids for o in ops]), dp_client_id=first.dp_client_id,
                         remote_node_ids=nodes if nodes.size else None,
                         block_hashes=hashes if hashes.size else None)
        new.merged_from = [o.op_id for o in ops]
        for o in ops:
            remap[o.op_id] = new.op_id
        merged.add_transfer_op(new)
        new_ops[tt] = new
        return new

    if layerwise and TransferType.H2D in by_type:
        h2d = by_type.pop(TransferType.H2D)
        d2h = by_type.pop(TransferType.DISK2H, [])
        lw = LayerwiseTransferOp(merged.graph_id, TransferType.LAYERWISE, _EMPTY, _EMPTY,
                                 dp_client_id=h2d[0].dp_client_id,
                                 src_block_ids_h2d=_cat([o.src_block_ids for o in h2d]),
                                 dst_block_ids_h2d=_cat([o.dst_block_ids for o in h2d]),
                                 src_block_ids_disk2h=_cat([o.src_block_ids for o in d2h]),
                                 dst_block_ids_disk2h=_cat([o.dst_block_ids for o in d2h]),
                                 counter_id=counter_id)
        lw.merged_from = [o.op_id for o in h2d + d2h]
        for o in h2d + d2h:
            remap[o.op_id] = lw.op_id
        merged.add_transfer_op(lw)
        new_ops[TransferType.LAYERWISE] = lw

    for tt in _MERGE_ORDER_GET + _MERGE_ORDER_PUT:
        fold(tt)
    for tt in list(by_type):
        if tt not in new_ops and tt != TransferType.LAYERWISE:
            fold(tt)

    consumer = new_ops.get(TransferType.H2D) or new_ops.get(TransferType.LAYERWISE)
    if consumer is not None:
        for tt in _STAGE_IN:
            if tt in new_ops:
                merged.add_dependency(consumer.op_id, new_ops[tt].op_id)
    if TransferType.D2H in new_ops:
        for tt in (TransferType.H2DISK, TransferType.H2REMOTE, TransferType.H2PEERH, TransferType.H2PEERSSD):
            if tt in new_ops:
                merged.add_dependency(new_ops[tt].op_id, new_ops[TransferType.D2H].op_id)
    # SWA side ops keep their own identity (different pool, different worker)
    for op in swa_ops:
        clone = TransferOp(merged.graph_id, op.transfer_type, op.src_block_ids, op.dst_block_ids,
                           dp_client_id=op.dp_client_id, is_swa=True)
        clone.merged_from = [op.op_id]
        remap[op.op_id] = clone.op_id
        merged.add_transfer_op(clone)
    # a window chain (tier hop, then the GPU copy) keeps its order inside the merged graph
    for op in swa_ops:
        for pred in op.predecessors:
            if pred in remap and remap[pred] != remap[op.op_id]:
                merged.add_dependency(remap[op.op_id], remap[pred])
    return merged, remap
