"""Transfer IR: dependency tracking, late GPU binding, batch merge
(reference: tests/test_batch_kvtask.py, tests/test_transfer_scheduler_incremental.py)."""
import numpy as np
import pytest

from flexkv_b200.common.transfer import (LayerwiseTransferOp, TransferOp, TransferOpGraph, TransferType,
                                         merge_to_batch_graph)

A = lambda *x: np.asarray(x, dtype=np.int64)  # noqa: E731


def test_ready_set_follows_dependencies():
    g = TransferOpGraph()
    a = g.add_transfer_op(TransferOp(g.graph_id, TransferType.DISK2H, A(1, 2), A(3, 4)))
    b = g.add_transfer_op(TransferOp(g.graph_id, TransferType.H2D, A(3, 4), A(5, 6)))
    g.add_dependency(b, a)
    v = g.add_virtual_op([a, b])
    assert [o.op_id for o in g.take_ready_ops()] == [a]
    assert g.take_ready_ops() == []                    # handed out once
    assert g.mark_completed(a) == [b]
    assert [o.op_id for o in g.take_ready_ops()] == [b]
    assert g.mark_completed(b) == [v]
    assert not g.all_transfer_ops_completed()
    g.take_ready_ops()
    g.mark_completed(v)
    assert g.all_transfer_ops_completed()


def test_failure_blocks_successors():
    g = TransferOpGraph()
    a = g.add_transfer_op(TransferOp(g.graph_id, TransferType.D2H, A(1), A(2)))
    b = g.add_transfer_op(TransferOp(g.graph_id, TransferType.H2DISK, A(2), A(3)))
    g.add_dependency(b, a)
    g.take_ready_ops()
    assert g.mark_completed(a, success=False) == [] and g.failed
    assert g.take_ready_ops() == [] and g.pending_ops() == [b]


def test_size_mismatch_rejected_and_late_binding():
    with pytest.raises(ValueError):
        TransferOp(0, TransferType.H2D, A(1, 2), A(3))
    g = TransferOpGraph()
    h2d = TransferOp(g.graph_id, TransferType.H2D, A(1, 2, 3), A(), gpu_side="dst")
    d2d = TransferOp(g.graph_id, TransferType.DISK2D, A(7, 8), A(), gpu_side="dst", gpu_bind="tail")
    g.add_transfer_op(h2d); g.add_transfer_op(d2d)
    assert not g.gpu_bound
    with pytest.raises(ValueError):
        g.set_gpu_blocks(A(1, 2))
    g.set_gpu_blocks(A(10, 11, 12, 13, 14))
    assert list(h2d.dst_block_ids) == [10, 11, 12] and list(d2d.dst_block_ids) == [13, 14] and g.gpu_bound


def _get_graph(cpu, gpu, ssd=None, stage=None):
    g = TransferOpGraph()
    h = TransferOp(g.graph_id, TransferType.H2D, A(*cpu, *(stage or [])), A(*gpu))
    g.add_transfer_op(h)
    if ssd:
        d = TransferOp(g.graph_id, TransferType.DISK2H, A(*ssd), A(*stage))
        g.add_transfer_op(d)
        g.add_dependency(h.op_id, d.op_id)
    return g


def test_merge_get_graphs():
    g1 = _get_graph([1, 2], [10, 11, 12], ssd=[50], stage=[3])
    g2 = _get_graph([4], [20])
    merged, remap = merge_to_batch_graph([g1, g2])
    kinds = {o.transfer_type: o for o in merged.ops()}
    assert set(kinds) == {TransferType.H2D, TransferType.DISK2H}
    assert list(kinds[TransferType.H2D].src_block_ids) == [1, 2, 3, 4]
    assert list(kinds[TransferType.H2D].dst_block_ids) == [10, 11, 12, 20]
    assert kinds[TransferType.H2D].predecessors == {kinds[TransferType.DISK2H].op_id}
    assert set(remap) == {o.op_id for g in (g1, g2) for o in g.ops()}
    assert sorted(kinds[TransferType.H2D].merged_from) == sorted(o.op_id for g in (g1, g2) for o in g.ops()
                                                                if o.transfer_type == TransferType.H2D)


def test_merge_put_graphs_and_layerwise_fold():
    gs = []
    for gpu, cpu, ssd in (([1, 2], [5, 6], [9, 8]), ([3], [7], [4])):
        g = TransferOpGraph()
        a = g.add_transfer_op(TransferOp(g.graph_id, TransferType.D2H, A(*gpu), A(*cpu)))
        b = g.add_transfer_op(TransferOp(g.graph_id, TransferType.H2DISK, A(*cpu), A(*ssd)))
        g.add_dependency(b, a)
        gs.append(g)
    merged, _ = merge_to_batch_graph(gs)
    kinds = {o.transfer_type: o for o in merged.ops()}
    assert list(kinds[TransferType.D2H].dst_block_ids) == [5, 6, 7]
    assert list(kinds[TransferType.H2DISK].dst_block_ids) == [9, 8, 4]
    assert kinds[TransferType.H2DISK].predecessors == {kinds[TransferType.D2H].op_id}
    lw, remap = merge_to_batch_graph([_get_graph([1, 2], [10, 11, 12], ssd=[50], stage=[3]), _get_graph([4], [20])],
                                     layerwise=True, counter_id=2)
    assert lw.num_ops == 1
    op = lw.ops()[0]
    assert isinstance(op, LayerwiseTransferOp) and op.counter_id == 2
    assert list(op.src_block_ids_h2d) == [1, 2, 3, 4] and list(op.dst_block_ids_h2d) == [10, 11, 12, 20]
    assert list(op.src_block_ids_disk2h) == [50] and list(op.dst_block_ids_disk2h) == [3]
    assert set(remap.values()) == {op.op_id}


def test_merge_requires_bound_graphs():
    g = TransferOpGraph()
    g.add_transfer_op(TransferOp(g.graph_id, TransferType.H2D, A(1), A(), gpu_side="dst"))
    with pytest.raises(ValueError):
        merge_to_batch_graph([g])


def test_even_tile_bytes_cuts_chunks_without_a_ragged_tile():
    from flexkv_b200.transfer.workers import even_tile_bytes
    assert even_tile_bytes(73728) == 24576          # 64 tokens x 576 x bf16 (MLA)
    assert even_tile_bytes(32768) == 16384
    assert even_tile_bytes(65536) == 16384
    assert even_tile_bytes(2048) == 2048
    assert even_tile_bytes(4680) == 16384           # no 16-byte-aligned even cut: the default tile
    for c in (73728, 32768, 147456, 9216):
        t = even_tile_bytes(c)
        assert c % t == 0 and t % 16 == 0 and t <= 24576
