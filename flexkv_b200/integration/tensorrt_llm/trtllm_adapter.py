"""TensorRT-LLM KV-cache connector pair. TRT-LLM registers ONE tensor per worker,
``[num_blocks, num_layers, kv, tokens_per_block * heads * head_dim]``-shaped; the
scheduler side follows the same lookup / bind / offload / step-loop contract as
the vLLM adapter (flexkv/integration/tensorrt_llm/trtllm_adapter.py:29-650)."""
from __future__ import annotations

from typing import Any, Dict, Optional, Sequence, Set, Tuple

import torch

from ...common.storage import KVCacheLayout, KVCacheLayoutType
from ..config import FlexKVConfig
from ..vllm.vllm_v1_adapter import FlexKVSchedulerConnector as _SchedulerCore
from .meta import FlexKVConnectorMetadata, FlexKVTask
from .utils import RequestWrapper, extract_namespace, physical_device_id


def trtllm_gpu_layout(kv_cache_tensor: torch.Tensor, num_layers: int, kv_dim: int, tokens_per_block: int,
                      heads_per_rank: int, head_size: int) -> KVCacheLayout:
    nb = kv_cache_tensor.shape[0]
    per_block = kv_cache_tensor.numel() // nb
    want = num_layers * kv_dim * tokens_per_block * heads_per_rank * head_size
    if per_block != want:
        raise ValueError(f"TRT-LLM pool has {per_block} elements per block, the model needs {want}")
    return KVCacheLayout(KVCacheLayoutType.BLOCKFIRST, num_layers, nb, tokens_per_block, heads_per_rank, head_size,
                         kv_dim_override=kv_dim)


class FlexKVSchedulerConnector:
    def __init__(self, config: Any = None, flexkv_config: Optional[FlexKVConfig] = None, kv_manager: Any = None) -> None:
        if flexkv_config is None:
            flexkv_config = FlexKVConfig.from_env()
            flexkv_config.post_init_from_trt_config(config, getattr(config, "mapping", None))
        self.core = _SchedulerCore(flexkv_config, kv_manager=kv_manager)
        self.tasks: Dict[str, FlexKVTask] = {}        # per-request records with match / execute timers

    def is_ready(self) -> bool:
        return self.core.is_ready()

    @staticmethod
    def _extract_namespace(request: Any):
        return extract_namespace(request)

    def get_num_new_matched_tokens(self, request: Any, num_computed_tokens: int) -> Tuple[int, bool]:
        """Tokens beyond ``num_computed_tokens`` that the host / SSD / remote tiers can restore, and whether the
        restore is asynchronous. The match is isolated by the request's namespace (LoRA task, cache salt,
        user hierarchy)."""
        import time
        w = RequestWrapper(request)
        t0 = time.perf_counter()
        n, is_async = self.core.get_num_new_matched_tokens(w, num_computed_tokens)
        if n > 0:
            core_task = self.core.req_to_get.get(str(w.req_id))
            self.tasks[str(w.req_id)] = FlexKVTask(getattr(core_task, "task_id", -1), w, "get",
                                                   num_computed_tokens=num_computed_tokens,
                                                   num_new_matched_tokens=n, match_start_time=t0,
                                                   match_end_time=time.perf_counter())
        return n, is_async

    def update_state_after_alloc(self, request: Any, block_ids: Sequence[int]) -> None:
        v = RequestWrapper(request)
        task = self.core.req_to_get.get(str(v.req_id))
        self.core.update_state_after_alloc(v, list(block_ids), task.num_tokens if task else 0)
        rec = self.tasks.get(str(v.req_id))
        if rec is not None:
            rec.launched()

    def request_finished(self, request: Any, cache_block_ids: Sequence[int]) -> bool:
        """True while a transfer still needs the request's blocks. A request that did not finish normally
        (cancelled, errored) leaves nothing behind (flexkv/integration/tensorrt_llm/trtllm_adapter.py:291-297)."""
        def flag(name: str) -> bool:
            v = getattr(request, name, True)
            return bool(v() if callable(v) else v)
        if not (flag("is_finished") and flag("is_finished_normal")):
            return False
        return self.core.request_finished(RequestWrapper(request), cache_block_ids)[0]

    def build_connector_meta(self, scheduler_output: Any = None) -> FlexKVConnectorMetadata:
        self.core.flush_cancels()
        self.core.launch_tasks()
        s, r = self.core.query_finished_task()
        for rid in r:
            rec = self.tasks.pop(str(rid), None)
            if rec is not None:
                rec.finished()
        return FlexKVConnectorMetadata(finished_sending=sorted(s), finished_recving=sorted(r))

    # the step-loop pieces, for engines that drive them separately
    def launch_tasks(self) -> None:
        self.core.launch_tasks()

    def cancel_tasks(self) -> None:
        self.core.flush_cancels()

    def query_finished_task(self) -> Tuple[Set[str], Set[str]]:
        return self.core.query_finished_task()

    def wait_for_all_get_tasks(self):
        return self.core.wait_for_all_get_tasks()

    def wait_for_all_put_tasks(self):
        return self.core.wait_for_all_put_tasks()

    def shutdown(self) -> None:
        self.core.shutdown()


class FlexKVWorkerConnector:
    """Worker side: registers the rank's single pool tensor with the data plane. On the first local rank of a
    node other than the master's it also starts that node's transfer manager in a process of its own
    (TensorRT-LLM owns MPI in the worker processes; the data plane must not live inside them:
    flexkv/integration/tensorrt_llm/trtllm_adapter.py:507-597)."""

    def __init__(self, config: Any = None, flexkv_config: Optional[FlexKVConfig] = None, tp_rank: int = 0,
                 dp_client_id: int = 0, pp_rank: int = 0, node_rank: int = 0, local_rank: Optional[int] = None,
                 remote_endpoints: Optional[Tuple[str, str, str]] = None) -> None:
        import os
        from ...server.client import KVTPClient
        if flexkv_config is None:
            flexkv_config = FlexKVConfig.from_env()
            flexkv_config.post_init_from_trt_config(config, getattr(config, "mapping", None))
        self.cfg = flexkv_config
        self.remote_process = None
        m = flexkv_config.model_config
        local_rank = tp_rank if local_rank is None else local_rank
        if getattr(m, "nnodes", 1) > 1 and node_rank > 0 and local_rank == 0:
            from ...transfer_manager import TransferManagerOnRemote
            host = getattr(m, "master_host", "127.0.0.1")
            ports = getattr(m, "master_ports", ("5556", "5557", "5558"))
            eps = remote_endpoints or (f"tcp://*:{ports[0]}", f"tcp://{host}:{ports[1]}", f"tcp://*:{ports[2]}")
            self.remote_process = TransferManagerOnRemote.create_process(
                m, flexkv_config.cache_config, *eps, gpu_register_port=flexkv_config.gpu_register_port)
        dev = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device_id = physical_device_id(dev, os.environ.get("CUDA_VISIBLE_DEVICES"))
        self.client = KVTPClient(flexkv_config.gpu_register_port, dp_client_id, self.device_id, tp_rank=tp_rank,
                                 pp_rank=pp_rank)
        self._metadata = FlexKVConnectorMetadata()

    def register_kv_caches(self, kv_cache_tensor: torch.Tensor) -> None:
        """``kv_cache_tensor``: [blocks, layers, kv (1 for MLA), tokens_per_block * heads * head_dim]."""
        m, c = self.cfg.model_config, self.cfg.cache_config
        if m.use_mla or m.kv_dim == 1:
            if kv_cache_tensor.dim() != 4 or kv_cache_tensor.shape[2] != 1:
                raise ValueError(f"an MLA pool is [blocks, layers, 1, page], got {tuple(kv_cache_tensor.shape)}")
        heads = 1 if m.use_mla else m.num_kv_heads // max(1, m.tp_size)
        layout = trtllm_gpu_layout(kv_cache_tensor, m.num_layers_per_pp_stage, m.kv_dim, c.tokens_per_block, heads,
                                   m.head_size)
        self.client.register_to_server([kv_cache_tensor], layout)

    def bind_connector_meta(self, metadata: FlexKVConnectorMetadata) -> None:
        self._metadata = metadata

    # data moves outside the forward pass
    def start_load_kv(self, stream: Any = None) -> None: ...
    def wait_for_layer_load(self, layer_idx: int, stream: Any = None) -> None: ...
    def save_kv_layer(self, layer_idx: int, stream: Any = None) -> None: ...
    def wait_for_save(self, stream: Any = None) -> None: ...

    def get_finished(self, finished_gen_req_ids: Sequence[Any] = (), started_loading_req_ids: Sequence[Any] = ()):
        """Requests whose offload / restore the scheduler side saw end this step (from the bound metadata)."""
        return list(self._metadata.finished_sending), list(self._metadata.finished_recving)

    def shutdown(self) -> None:
        self.client.shutdown()
        p, self.remote_process = self.remote_process, None
        if p is not None:
            p.terminate()
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=5)
