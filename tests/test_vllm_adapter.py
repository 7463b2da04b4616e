"""vLLM connector contract with stand-in engine objects and the CPU data plane:
lookup -> bind -> launch -> finished, offload on finish, zero-hit cancel,
preemption, failed-get block reporting, config mapping (reference:
tests/test_vllm_abort_offload_directive.py and the adapter contract)."""
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.integration.config import FlexKVConfig
from flexkv_b200.integration.dynamo.collector import KVEventCollector
from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVSchedulerConnector, infer_vllm_gpu_layout
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def make():
    shape = KVShape("v", 2, 2, 16, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=80)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    return FlexKVSchedulerConnector(cfg, kv_manager=mgr), kv, mgr


def req(rid, tokens, **kw):
    return NS(request_id=rid, all_token_ids=list(tokens), lora_request=None, cache_salt=None, **kw)


def drain(conn, want_send=(), want_recv=()):
    import time
    s, r = set(), set()
    t0 = time.time()
    while (not set(want_send) <= s or not set(want_recv) <= r) and time.time() - t0 < 10:
        a, b = conn.query_finished_task()
        s |= a; r |= b
        time.sleep(0.005)
    return s, r


def test_offload_then_restore_cycle():
    conn, kv, mgr = make()
    try:
        events = KVEventCollector()
        events.attach(mgr.kv_task_engine.cache_engine)
        tok = np.arange(100, 100 + 6 * T + 2)
        r1 = req("a", tok)
        assert conn.get_num_new_matched_tokens(r1, 0) == (0, False)          # cold
        keep, _ = conn.request_finished(r1, [10, 11, 12, 13, 14, 15, 16])
        assert keep                                                           # blocks stay until the put lands
        conn.launch_tasks()
        s, _ = drain(conn, want_send={"a"})
        assert s == {"a"}
        stored = [e for e in events.take_events() if e.kind == "stored"]
        assert sum(len(e.block_hashes) for e in stored) == 6                  # ((26-1)//4)*4 = 24 tokens = 6 blocks
        # a second request with the same prompt: 2 blocks already computed on the GPU, 4 to restore
        r2 = req("b", tok)
        n, is_async = conn.get_num_new_matched_tokens(r2, 2 * T)
        assert (n, is_async) == (4 * T, True)
        saved = [t.clone() for t in kv]
        conn.update_state_after_alloc(r2, NS(get_block_ids=lambda: ([40, 41, 42, 43, 44, 45, 46],)), n)
        conn.launch_tasks()
        _, r = drain(conn, want_recv={"b"})
        assert r == {"b"} and conn.get_and_clear_failed_block_ids() == set()
        for l in range(2):
            assert torch.equal(kv[l][:, [42, 43, 44, 45]], saved[l][:, [12, 13, 14, 15]])
        # finishing it again offloads nothing new and frees the blocks immediately
        assert conn.request_finished(r2, [40, 41, 42, 43, 44, 45, 46]) == (False, None)
        assert conn.stats.num_get_requests == 2 and conn.stats.num_flexkv_matched_tokens == 4 * T
    finally:
        conn.shutdown()


def test_preemption_cancels_unlaunched_and_failed_get_reports_blocks():
    conn, kv, mgr = make()
    try:
        tok = np.arange(6 * T + 1)
        conn.request_finished(req("seed", tok), list(range(6)))
        conn.launch_tasks()
        drain(conn, want_send={"seed"})
        r = req("p", tok)
        n, _ = conn.get_num_new_matched_tokens(r, 0)
        assert n == 6 * T
        conn.handle_preemptions(["p"])
        conn.flush_cancels()
        cpu = mgr.kv_task_engine.cache_engine.cpu_cache_engine
        from flexkv_b200.common.block import SequenceMeta
        assert cpu.index.node_lock_cnt(cpu.match(SequenceMeta(tok[:24], T)).last_node) == 0   # lock released
        # a get whose transfer fails: its GPU blocks are reported for recomputation
        from flexkv_b200.common.transfer import TransferType, WorkerKey
        mgr.transfer_manager.engine.worker_for(WorkerKey(0, 0), TransferType.H2D).fail_next = 1
        r = req("f", tok)
        n, _ = conn.get_num_new_matched_tokens(r, 0)
        conn.update_state_after_alloc(r, [[20, 21, 22, 23, 24, 25]], n)
        conn.launch_tasks()
        _, done = drain(conn, want_recv={"f"})
        assert done == {"f"} and conn.get_and_clear_failed_block_ids() == {20, 21, 22, 23, 24, 25}
    finally:
        conn.shutdown()


def test_layout_inference_and_config_mapping():
    a = [torch.empty(2, 10, 16, 4, 64) for _ in range(3)]
    b = [torch.empty(10, 2, 16, 4, 64) for _ in range(3)]
    c = [torch.empty(10, 16, 576) for _ in range(3)]
    assert infer_vllm_gpu_layout(a, 16, 4, 64, False).type.value == "LAYERFIRST"
    assert infer_vllm_gpu_layout(b, 16, 4, 64, False).type.value == "LAYERBLOCK"
    packed = [torch.zeros(8, 4, 16, 72, dtype=torch.uint8) for _ in range(3)]      # no K/V axis: one region per block
    lay = infer_vllm_gpu_layout(packed, 16, 4, 72, False)
    assert (lay.kv_dim, lay.num_block, lay.tokens_per_block, lay.get_chunk_size()) == (1, 8, 16, 4 * 16 * 72)
    lay = infer_vllm_gpu_layout(c, 16, 1, 576, True)
    assert lay.is_mla and lay.kv_dim == 1 and lay.num_block == 10
    hf = NS(num_hidden_layers=32, num_key_value_heads=8, num_attention_heads=32, hidden_size=4096, head_dim=128)
    vcfg = NS(model_config=NS(hf_text_config=hf, hf_config=hf, dtype=torch.bfloat16, use_mla=False),
              parallel_config=NS(tensor_parallel_size=2, pipeline_parallel_size=1, data_parallel_size=1),
              cache_config=NS(block_size=16, cache_dtype="auto"))
    cfg = FlexKVConfig()
    cfg.user_config.cpu_cache_gb = 4
    cfg.post_init_from_vllm_config(vcfg)
    m = cfg.model_config
    assert (m.num_layers, m.num_kv_heads, m.head_size, m.tp_size) == (32, 8, 128, 2)
    assert cfg.cache_config.num_cpu_blocks == 4 * 2**30 // (2 * 2**20)
    with pytest.raises(AttributeError):
        m.num_layers = 3                                     # frozen after post-init
    cfg2 = FlexKVConfig(kv_cache_dtype="nvfp4")
    cfg2.post_init_from_vllm_config(vcfg)
    assert cfg2.model_config.dtype == torch.uint8 and cfg2.model_config.head_size == 64 + 8   # nibbles + scales


def test_blocking_waits_events_and_stats():
    conn, kv, mgr = make()
    try:
        conn.enable_kv_events()
        tok = np.arange(900, 900 + 4 * T + 1)
        keep, _ = conn.request_finished(req("p", tok), [1, 2, 3, 4, 5])
        assert keep
        rsp = conn.wait_for_all_put_tasks()
        assert len(rsp) == 1 and rsp[0].status.value == "success" and not conn.launched_put
        n, _ = conn.get_num_new_matched_tokens(req("g", tok), 0)
        assert n == 4 * T
        conn.update_state_after_alloc(req("g", tok), [20, 21, 22, 23, 24], n)
        rsp = conn.wait_for_all_get_tasks()
        assert len(rsp) == 1 and rsp[0].status.value == "success"
        ev = conn.collector.take_events()
        assert sum(len(e.block_hashes) for e in ev if e.kind == "stored") == 4
        assert conn.stats.num_put_requests == 1 and conn.stats.num_get_requests == 1
    finally:
        conn.shutdown()


def test_worker_registers_indexer_caches_as_a_second_group_and_the_manager_adopts_it():
    """Only the worker sees the indexer key caches (layer names with ``.k_cache``): the group list travels with
    its registration and a manager configured without groups moves both groups from then on."""
    from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVWorkerConnector
    from flexkv_b200.server.utils import unique_ipc_endpoint
    shape = KVShape("v", 2, 2, 16, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    cfg.gpu_register_port = unique_ipc_endpoint("vidx")
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True, gpu_register_port=cfg.gpu_register_port)
    mgr.start()
    kv, _ = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=81)
    g = torch.Generator().manual_seed(4)
    idx = [torch.randint(0, 256, (64, T, 12), dtype=torch.uint8, generator=g) for _ in range(2)]
    caches = {"model.layers.0.self_attn.attn": kv[0], "model.layers.0.self_attn.indexer.k_cache": idx[0],
              "model.layers.1.self_attn.attn": kv[1], "model.layers.1.self_attn.indexer.k_cache": idx[1]}
    worker = FlexKVWorkerConnector(cfg, dp_client_id=0, tp_rank=0, device_id=0)
    worker.client.register_to_server = (lambda f: lambda *a, **k: f(*a, mode="same_process", **k))(
        worker.client.register_to_server)
    try:
        worker.register_to_server(caches)
        mgr.wait_ready(30)
        groups = mgr.transfer_manager.model_config.layer_groups
        assert [(x.num_layers, x.num_kv_heads, x.head_size, x.kv_dim) for x in groups] == [(2, 2, 16, 2), (2, 1, 12, 1)]
        host = mgr.transfer_manager.storage.host
        assert host.block_bytes == 2 * 2 * T * 2 * 16 * 2 + 2 * T * 12
        tok = np.arange(5 * T, dtype=np.int64) + 40
        sl = lambda b: np.repeat(np.asarray(b), T) * T + np.tile(np.arange(T), len(b))   # noqa: E731
        src, dst = [3, 9, 1, 30, 12], [40, 41, 42, 43, 44]
        tid = mgr.put_async(tok, sl(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want_kv, want_idx = [t[:, src].clone() for t in kv], [t[src].clone() for t in idx]
        for t in kv:
            t[:, dst] = 0
        for t in idx:
            t[dst] = 0
        tid = mgr.get_async(tok, sl(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], want_kv[l]) and torch.equal(idx[l][dst], want_idx[l])
        # sleep mode: the engine drops both groups' tensors and comes back with new ones
        assert worker.before_device_sleep() == 0
        kv2 = [torch.zeros_like(t) for t in kv]
        idx2 = [torch.zeros_like(t) for t in idx]
        worker.after_device_wake({"model.layers.0.self_attn.attn": kv2[0],
                                  "model.layers.0.self_attn.indexer.k_cache": idx2[0],
                                  "model.layers.1.self_attn.attn": kv2[1],
                                  "model.layers.1.self_attn.indexer.k_cache": idx2[1]})
        tid = mgr.get_async(tok, sl(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv2[l][:, dst], want_kv[l]) and torch.equal(idx2[l][dst], want_idx[l])
    finally:
        mgr.shutdown()


def test_aborted_requests_offload_only_on_request():
    """An abort leaves nothing behind unless the caller set ``offload_kv_on_finish``; stop and length finishes
    offload as before (reference: tests/test_vllm_abort_offload_directive.py)."""
    conn, kv, mgr = make()
    try:
        blocks = [10, 11, 12, 13, 14]
        tok = np.arange(700, 700 + 4 * T + 1)
        aborted = req("x", tok, get_finished_reason=lambda: NS(name="ABORT"))
        assert conn.request_finished(aborted, blocks) == (False, None)
        assert conn.stats.num_put_requests == 0
        for reason in ("STOP", "LENGTH"):
            r = req("ok-" + reason, tok + (1 if reason == "LENGTH" else 0), get_finished_reason=lambda n=reason: NS(name=n))
            keep, _ = conn.request_finished(r, blocks)
            assert keep
        moved = req("y", tok + 7, get_finished_reason=lambda: NS(name="ABORT"), offload_kv_on_finish=True)
        keep, _ = conn.request_finished(moved, blocks)
        assert keep
        conn.launch_tasks()
        s, _ = drain(conn, want_send={"ok-STOP", "ok-LENGTH", "y"})
        assert s == {"ok-STOP", "ok-LENGTH", "y"}
    finally:
        conn.shutdown()


def test_impl_reports_finished_transfers_through_the_engines_connector_output():
    """The step loop as vLLM drives it: ``build_connector_meta`` launches, ``update_connector_output`` writes the
    finished request ids into the engine's own output record (merged with what is already there), and a scheduler
    output without ``preempted_req_ids`` gets the preempted set from the difference of consecutive steps."""
    import time
    from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl
    conn, kv, mgr = make()
    impl = FlexKVConnectorV1Impl.__new__(FlexKVConnectorV1Impl)
    impl.is_scheduler, impl.scheduler, impl.worker = True, conn, None
    impl._finished_sending, impl._finished_recving, impl._previous_scheduled = set(), set(), set()
    try:
        tok = np.arange(500, 500 + 5 * T + 1)
        keep, _ = impl.request_finished(req("a", tok), [1, 2, 3, 4, 5, 6])
        assert keep
        step = NS(scheduled_new_reqs=[NS(req_id="x")], scheduled_cached_reqs=NS(req_ids=["y"]), finished_req_ids=set())
        meta = impl.build_connector_meta(step)                      # launches the put
        out = NS(finished_sending={"earlier"}, finished_recving=None)
        t0 = time.time()
        while "a" not in (out.finished_sending or ()) and time.time() - t0 < 10:
            impl.update_connector_output(out)
            time.sleep(0.005)
        assert out.finished_sending == {"earlier", "a"} and not out.finished_recving
        assert hasattr(meta, "finished_sending")
        # next step: "x" is gone without having finished -> treated as preempted; "y" finished
        seen = []
        conn.handle_preemptions = lambda ids: seen.append(set(ids))
        impl.build_connector_meta(NS(scheduled_new_reqs=[], scheduled_cached_reqs=None, finished_req_ids={"y"}))
        assert seen == [{"x"}]
        impl.update_connector_output(None)                          # tolerated
    finally:
        conn.shutdown()


def test_operator_switches_skip_put_flag_and_synchronous_gets(monkeypatch, tmp_path):
    """FLEXKV_MAYBE_SKIP_PUT: offloads stop while a flag file exists, without a restart. FLEXKV_SYNC_GET: the
    step that launches a restore returns only after it has landed and reports it in the same step
    (reference: flexkv/integration/vllm/vllm_v1_adapter.py:264,534,1199)."""
    from flexkv_b200.integration.vllm import vllm_v1_adapter as A
    from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl
    flag = tmp_path / "skip_put"
    monkeypatch.setattr(A, "SKIP_PUT_FLAG", str(flag))
    monkeypatch.setenv("FLEXKV_MAYBE_SKIP_PUT", "1")
    monkeypatch.setenv("FLEXKV_SYNC_GET", "1")
    monkeypatch.setenv("FLEXKV_NUM_LOG_INTERVAL_REQUESTS", "7")
    conn, kv, mgr = make()
    assert conn.maybe_skip_put and conn.sync_get and conn.stats.log_interval == 7
    impl = FlexKVConnectorV1Impl.__new__(FlexKVConnectorV1Impl)
    impl.is_scheduler, impl.scheduler, impl.worker = True, conn, None
    impl._finished_sending, impl._finished_recving, impl._previous_scheduled = set(), set(), set()
    try:
        tok = np.arange(900, 900 + 4 * T + 1)
        flag.write_text("")
        assert conn.request_finished(req("a", tok), [1, 2, 3, 4, 5]) == (False, None)     # writing is paused
        assert conn.stats.num_put_requests == 0
        flag.unlink()
        keep, _ = conn.request_finished(req("a", tok), [1, 2, 3, 4, 5])
        assert keep
        conn.launch_tasks()
        assert drain(conn, want_send={"a"})[0] == {"a"}
        # synchronous get: finished within the step that launched it
        r2 = req("b", tok)
        n, _ = conn.get_num_new_matched_tokens(r2, 0)
        assert n == 4 * T
        conn.update_state_after_alloc(r2, NS(get_block_ids=lambda: ([20, 21, 22, 23, 24],)), n)
        meta = impl.build_connector_meta(NS(preempted_req_ids=set()))
        assert "b" in meta.finished_recving and not conn.launched_get
        for l in range(2):
            assert torch.equal(kv[l][:, [20, 21, 22, 23]], kv[l][:, [1, 2, 3, 4]])
    finally:
        conn.shutdown()


def test_layers_of_different_head_geometry_become_one_group_per_shape():
    """A hybrid model whose sliding-window layers and full-attention layers have different head counts and head
    sizes (the reference's Gemma-4 case, docs/gemma4_support.md: 16 x 256 beside 4 x 512, triton layout
    ``[blocks, 2, tokens, heads, dim]``, some layers sharing one tensor): the worker probes the shapes, registers
    one layer group per shape, the manager adopts the groups, and a put / get moves every layer."""
    from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVWorkerConnector
    from flexkv_b200.server.utils import unique_ipc_endpoint
    shape = KVShape("g", 5, 4, 8, tokens_per_block=T)                 # what the engine config alone would say
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    cfg.gpu_register_port = unique_ipc_endpoint("vgem")
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True, gpu_register_port=cfg.gpu_register_port)
    mgr.start()
    g = torch.Generator().manual_seed(12)
    NB = 48
    swa = [torch.randn(NB, 2, T, 4, 8, generator=g).to(torch.bfloat16) for _ in range(3)]      # sliding-window layers
    full = [torch.randn(NB, 2, T, 1, 16, generator=g).to(torch.bfloat16) for _ in range(2)]    # full-attention layers
    caches = {"model.layers.0.attn": swa[0], "model.layers.1.attn": swa[1], "model.layers.2.attn": full[0],
              "model.layers.3.attn": swa[2], "model.layers.4.attn": full[1],
              "model.layers.5.attn": full[1]}                          # shares layer 4's tensor
    worker = FlexKVWorkerConnector(cfg, dp_client_id=0, tp_rank=0, device_id=0)
    worker.client.register_to_server = (lambda f: lambda *a, **k: f(*a, mode="same_process", **k))(
        worker.client.register_to_server)
    try:
        worker.register_to_server(caches)
        mgr.wait_ready(30)
        groups = mgr.transfer_manager.model_config.layer_groups
        assert [(x.num_layers, x.num_kv_heads, x.head_size, x.kv_dim) for x in groups] == [(3, 4, 8, 2), (2, 1, 16, 2)]
        assert [list(x.layer_ids) for x in groups] == [[0, 1, 3], [2, 4]]
        host = mgr.transfer_manager.storage.host
        assert host.block_bytes == (3 * 2 * T * 4 * 8 + 2 * 2 * T * 1 * 16) * 2
        tok = np.arange(4 * T, dtype=np.int64) + 77
        sl = lambda b: np.repeat(np.asarray(b), T) * T + np.tile(np.arange(T), len(b))   # noqa: E731
        src, dst = [3, 9, 1, 30], [40, 41, 42, 43]
        tid = mgr.put_async(tok, sl(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want = [t[src].clone() for t in swa + full]
        for t in swa + full:
            t[dst] = 0
        tid = mgr.get_async(tok, sl(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for t, w in zip(swa + full, want):
            assert torch.equal(t[dst], w)
        # wake with new tensors of the same shapes
        assert worker.before_device_sleep() == 0
        swa2, full2 = [torch.zeros_like(t) for t in swa], [torch.zeros_like(t) for t in full]
        worker.after_device_wake({"model.layers.0.attn": swa2[0], "model.layers.1.attn": swa2[1],
                                  "model.layers.2.attn": full2[0], "model.layers.3.attn": swa2[2],
                                  "model.layers.4.attn": full2[1], "model.layers.5.attn": full2[1]})
        tid = mgr.get_async(tok, sl(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for t, w in zip(swa2 + full2, want):
            assert torch.equal(t[dst], w)
    finally:
        mgr.shutdown()
