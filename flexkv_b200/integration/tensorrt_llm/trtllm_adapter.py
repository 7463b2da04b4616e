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


def trtllm_gpu_layout(kv_cache_tensor: torch.Tensor, num_layers: int, kv_dim: int, tokens_per_block: int,
                      heads_per_rank: int, head_size: int) -> KVCacheLayout:
    nb = kv_cache_tensor.shape[0]
    per_block = kv_cache_tensor.numel() // nb
    want = num_layers * kv_dim * tokens_per_block * heads_per_rank * head_size
    if per_block != want:
        raise ValueError(f"TRT-LLM pool has {per_block} elements per block, the model needs {want}")
    return KVCacheLayout(KVCacheLayoutType.BLOCKFIRST, num_layers, nb, tokens_per_block, heads_per_rank, head_size,
                         kv_dim_override=kv_dim)


class _LlmRequestView:
    """Adapts a TRT-LLM LlmRequest to the attribute names the scheduler core reads."""

    def __init__(self, req: Any) -> None:
        self._r = req
        self.request_id = getattr(req, "request_id", None) or getattr(req, "py_request_id", None)
        toks = req.get_tokens(0) if hasattr(req, "get_tokens") else getattr(req, "tokens", [])
        self.all_token_ids = list(toks)
        self.lora_request = None
        lora = getattr(req, "lora_task_id", None)
        self.cache_salt = str(lora) if lora is not None else getattr(req, "cache_salt", None)


class FlexKVSchedulerConnector:
    def __init__(self, config: Any = None, flexkv_config: Optional[FlexKVConfig] = None, kv_manager: Any = None) -> None:
        if flexkv_config is None:
            flexkv_config = FlexKVConfig.from_env()
            flexkv_config.post_init_from_trt_config(config, getattr(config, "mapping", None))
        self.core = _SchedulerCore(flexkv_config, kv_manager=kv_manager)

    def is_ready(self) -> bool:
        return self.core.is_ready()

    def get_num_new_matched_tokens(self, request: Any, num_computed_tokens: int) -> Tuple[int, bool]:
        return self.core.get_num_new_matched_tokens(_LlmRequestView(request), num_computed_tokens)

    def update_state_after_alloc(self, request: Any, block_ids: Sequence[int]) -> None:
        v = _LlmRequestView(request)
        task = self.core.req_to_get.get(str(v.request_id))
        self.core.update_state_after_alloc(v, list(block_ids), task.num_tokens if task else 0)

    def request_finished(self, request: Any, cache_block_ids: Sequence[int]) -> bool:
        """True while a transfer still needs the request's blocks. A request that did not finish normally
        (cancelled, errored) leaves nothing behind (flexkv/integration/tensorrt_llm/trtllm_adapter.py:291-297)."""
        def flag(name: str) -> bool:
            v = getattr(request, name, True)
            return bool(v() if callable(v) else v)
        if not (flag("is_finished") and flag("is_finished_normal")):
            return False
        return self.core.request_finished(_LlmRequestView(request), cache_block_ids)[0]

    def build_connector_meta(self, scheduler_output: Any = None) -> Dict[str, Set[str]]:
        self.core.flush_cancels()
        self.core.launch_tasks()
        s, r = self.core.query_finished_task()
        return {"finished_sending": s, "finished_recving": r}

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
    def __init__(self, config: Any = None, flexkv_config: Optional[FlexKVConfig] = None, tp_rank: int = 0,
                 dp_client_id: int = 0) -> None:
        from ...server.client import KVTPClient
        if flexkv_config is None:
            flexkv_config = FlexKVConfig.from_env()
            flexkv_config.post_init_from_trt_config(config, getattr(config, "mapping", None))
        self.cfg = flexkv_config
        dev = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.client = KVTPClient(flexkv_config.gpu_register_port, dp_client_id, dev, tp_rank=tp_rank)

    def register_kv_caches(self, kv_cache_tensor: torch.Tensor) -> None:
        m, c = self.cfg.model_config, self.cfg.cache_config
        heads = 1 if m.use_mla else m.num_kv_heads // max(1, m.tp_size)
        layout = trtllm_gpu_layout(kv_cache_tensor, m.num_layers_per_pp_stage, m.kv_dim, c.tokens_per_block, heads,
                                   m.head_size)
        self.client.register_to_server([kv_cache_tensor], layout)

    # data moves outside the forward pass
    def start_load_kv(self, stream: Any = None) -> None: ...
    def wait_for_layer_load(self, layer_idx: int, stream: Any = None) -> None: ...
    def save_kv_layer(self, layer_idx: int, stream: Any = None) -> None: ...
    def wait_for_save(self, stream: Any = None) -> None: ...

    def get_finished(self, finished_gen_req_ids: Sequence[Any] = (), started_loading_req_ids: Sequence[Any] = ()):
        return list(finished_gen_req_ids), list(started_loading_req_ids)

    def shutdown(self) -> None:
        self.client.shutdown()
