"""Public facade. Same methods and semantics as the reference's ``KVManager``
(flexkv/kvmanager.py:34-394): tasks are ints, results are ``KVResponse``.

In-process mode owns a ``KVTaskEngine`` whose data plane runs on threads of
this process. With ``dp_size > 1``, several engine instances or
``FLEXKV_SERVER_CLIENT_MODE=1`` the manager becomes a client of one
``KVServer`` that owns the shared index (flexkv/kvmanager.py:69-131).
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from .common.debug import flexkv_logger
from .common.request import KVResponse
from .common.storage import KVCacheLayout


def _np(x, dtype=None):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().numpy()
    x = np.asarray(x)
    return x.astype(dtype, copy=False) if dtype is not None else x


class KVManager:
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, dp_client_id: int = 0,
                 server_recv_port: Optional[str] = None, gpu_register_port: Optional[str] = None,
                 require_gpu: Optional[bool] = None, in_process: Optional[bool] = None,
                 remote_transfer_endpoints: Optional[Sequence[tuple]] = None,
                 transfer_manager_mode: Optional[str] = None) -> None:
        env = GLOBAL_CONFIG_FROM_ENV
        self.model_config = model_config
        self.cache_config = cache_config
        self.dp_client_id = dp_client_id
        self.server_recv_port = server_recv_port or env.server_recv_port
        self.gpu_register_port = gpu_register_port
        safe = {k: ("***" if "password" in k else v) for k, v in vars(cache_config).items() if not k.startswith("_")}
        flexkv_logger.debug("KVManager config: %s | %s", model_config, safe)
        for name, why in cache_config.settings_without_effect():
            flexkv_logger.warning("configuration: %s has no effect here: %s", name, why)
        # `in_process=True` keeps everything in this process even with several DP ranks (one process
        # that sees every GPU, e.g. tests and single-process benchmarks)
        self.server_client_mode = bool(env.server_client_mode or model_config.dp_size > 1
                                       or model_config.instance_num > 1) if in_process is None else not in_process
        self.server_handle = None
        self.dp_client = None
        self.kv_task_engine = None
        self.transfer_manager = None
        self._metrics = None
        self._shut = False
        import atexit
        import weakref
        ref = weakref.ref(self)
        atexit.register(lambda: ref() is not None and ref().shutdown())
        if self.server_client_mode:
            from .server.client import KVDPClient
            from .server.server import KVServer
            # dp client 0 of instance 0 hosts the server unless one is launched externally
            if dp_client_id == 0 and env.instance_id == 0 and env.server_launch_mode != "external":
                self.server_handle = KVServer.create_server(model_config, cache_config, self.server_recv_port,
                                                            gpu_register_port=gpu_register_port,
                                                            mode=env.server_launch_mode if env.server_launch_mode
                                                            in ("thread", "process") else "thread",
                                                            require_gpu=require_gpu)
            self.dp_client = KVDPClient(self.server_recv_port, model_config, dp_client_id)
        else:
            from .kvtask import KVTaskEngine
            from .transfer_manager import TransferManager
            if require_gpu is None:
                require_gpu = torch.cuda.is_available()
            if env.crash_diagnostics:
                from .common.debug import install_crash_diagnostics
                install_crash_diagnostics()
            tm_mode = transfer_manager_mode or env.transfer_manager_mode
            if transfer_manager_mode is None and getattr(model_config, "use_trtllm_subprocess", False) \
                    and "FLEXKV_TRANSFER_MANAGER_MODE" not in os.environ:
                # TensorRT-LLM owns MPI in the serving processes: the data plane goes to a child process started
                # from a fresh interpreter (the reference runs it as a remote-mode subprocess on
                # FLEXKV_TRT_SUBPROCESS_HOST/PORTS for the same reason: flexkv/kvtask.py:172-199)
                tm_mode = "process"
            if tm_mode == "process":
                # the data plane in a child process (pipe EOF in both directions, SIGTERM-safe unpinning)
                from .transfer_process import TransferManagerProcessHandle
                self.transfer_manager = TransferManagerProcessHandle(model_config, cache_config, gpu_register_port,
                                                                     require_gpu=require_gpu)
            else:
                self.transfer_manager = TransferManager(model_config, cache_config, gpu_register_port,
                                                        require_gpu=require_gpu)
            handles = [self.transfer_manager]
            # other nodes of a TP/PP group: one handle per (command, result, query) endpoint triple; a graph
            # is finished when every node reported it
            # a fourth element True: that node numbers its GPU pages itself and sends them per task
            # (KVTPClient.set_slot_mapping on its ranks); graphs go there with their GPU side unbound
            for cmd, res, qry, *more in (remote_transfer_endpoints or []):
                from .transfer_manager import TransferManagerMultiNodeHandle
                handles.append(TransferManagerMultiNodeHandle(cmd, res, qry, rebind_gpu_blocks=bool(more and more[0])))
            self.kv_task_engine = KVTaskEngine(model_config, cache_config, transfer_handles=handles)
            if env.enable_metrics:
                from .metrics.collector import get_collector
                self._metrics = get_collector(start_server=True)
                self.kv_task_engine.set_metrics_collector(self._metrics)
                self.transfer_manager.set_metrics_collector(self._metrics)

    # ---- in-process registration (engine worker and manager share the process) --------------
    def register_gpu_tensors(self, tensors: Sequence[torch.Tensor], gpu_layout: KVCacheLayout, tp_rank: int = 0,
                             pp_rank: int = 0, dp_client_id: Optional[int] = None, group_id: int = -1,
                             multicast=None) -> None:
        """``group_id`` names the layer group of a multi-group cache (``ModelConfig.layer_groups``): call once
        per group with that group's tensors and layout.

        ``multicast``: the ``parallel.nvls.SymmetricKVPool`` (or ``SymmetricKVBuffer``) the tensors were carved
        from, when the ranks of a shared-KV (MLA) tensor-parallel group allocated their caches as symmetric
        memory. This ONE registration, made by the rank that lives in the manager's process, then stands for the
        whole group: a restore reads each host block once and `multimem.st` writes it into every rank's cache
        (``NvlsFanoutWorker``); an offload reads this rank's copy."""
        if self.server_client_mode:
            raise RuntimeError("in server-client mode GPU tensors are registered through KVTPClient")
        if hasattr(self.transfer_manager, "register_gpu_tensors"):      # data plane in a child process
            self.transfer_manager.register_gpu_tensors(tensors, gpu_layout, tp_rank=tp_rank, pp_rank=pp_rank,
                                                       dp_client_id=self.dp_client_id if dp_client_id is None
                                                       else dp_client_id, group_id=group_id)
            return
        from .storage.gpu_layout import register_tensors
        reg = register_tensors(tensors, gpu_layout, tp_rank=tp_rank, pp_rank=pp_rank,
                               dp_client_id=self.dp_client_id if dp_client_id is None else dp_client_id,
                               group_id=group_id)
        if multicast is not None:
            if hasattr(multicast, "mc_of"):
                reg.mc_ptrs = [int(multicast.mc_of(int(p))) for p in reg.ptrs]
            else:
                reg.mc_ptrs = [int(p) + int(multicast.mc_delta) for p in reg.ptrs]
            reg.mc_flag_ptr = int(multicast.flag_mc_ptr)
            reg.keepalive = (reg.keepalive, multicast)
        self.transfer_manager.register_gpu(reg)

    def register_swa_tensors(self, tensors: Sequence[torch.Tensor], tp_rank: int = 0, pp_rank: int = 0,
                             dp_client_id: Optional[int] = None, group_id: int = 0) -> None:
        """Sliding-window pages of one rank: one tensor per window layer, shaped
        [num_pages, ...] with a contiguous page; call before ``start()``. ``group_id`` g >= 1 registers
        the g-th sidecar group of ``SWAPoolConfig.sidecar_groups`` (state saved with the same slot).
        Engine ranks in other processes use ``KVTPClient.register_swa_to_server``."""
        if self.server_client_mode:
            raise RuntimeError("in server-client mode the engine ranks register their window pages themselves")
        from .storage.gpu_layout import swa_registration
        reg = swa_registration([int(t.data_ptr()) for t in tensors], [tuple(t.shape) for t in tensors],
                               [tuple(t.stride()) for t in tensors], tensors[0].dtype,
                               (tensors[0].device.index or 0) if tensors[0].is_cuda else -1)
        reg.dp_client_id = self.dp_client_id if dp_client_id is None else dp_client_id
        reg.pp_rank, reg.tp_rank, reg.group_id, reg.keepalive = pp_rank, tp_rank, int(group_id), list(tensors)
        self.transfer_manager.register_swa(reg)

    # ---- sleep / wake of the engine's GPU memory ---------------------------------------
    def suspend_gpu_mappings(self, dp_client_id: Optional[int] = None, timeout: float = 60.0) -> bool:
        """Returns once no transfer touches this client's GPU tensors; later GPU ops wait for
        ``resume_gpu_mappings``. The host cache stays intact."""
        if self.server_client_mode:
            raise RuntimeError("in server-client mode use KVTPClient.suspend_gpu_mappings")
        dp = self.dp_client_id if dp_client_id is None else dp_client_id
        pd = self.kv_task_engine.cache_engine.peer_directory
        if pd is not None:
            pd.clear_rank(dp)           # nobody may plan a pull out of memory that is about to go away
        return self.transfer_manager.suspend_gpu_mappings(dp, timeout)

    def resume_gpu_mappings(self, tensors: Optional[Sequence[torch.Tensor]] = None,
                            gpu_layout: Optional[KVCacheLayout] = None, tp_rank: int = 0, pp_rank: int = 0,
                            dp_client_id: Optional[int] = None) -> None:
        """Pass the re-created tensors when the engine re-allocated its cache on wake."""
        if self.server_client_mode:
            raise RuntimeError("in server-client mode use KVTPClient.resume_gpu_mappings")
        dp = self.dp_client_id if dp_client_id is None else dp_client_id
        regs = []
        if tensors is not None:
            from .storage.gpu_layout import register_tensors
            regs.append(register_tensors(tensors, gpu_layout, tp_rank=tp_rank, pp_rank=pp_rank, dp_client_id=dp))
        self.transfer_manager.resume_gpu_mappings(dp, regs)

    # ---- lifecycle ------------------------------------------------------------
    def start(self) -> None:
        if self.server_client_mode:
            self.dp_client.start_server_and_register()
        else:
            self.kv_task_engine.start()

    def is_ready(self) -> bool:
        if self.server_client_mode:
            return self.dp_client.is_ready()
        return self.kv_task_engine.is_ready()

    def wait_ready(self, timeout: float = 600.0) -> None:
        t0 = time.monotonic()
        while not self.is_ready():
            if time.monotonic() - t0 > timeout:
                raise TimeoutError("KVManager did not become ready")
            time.sleep(0.01)

    def shutdown(self) -> None:
        """Stops the data plane, unpins host memory and leaves the registry; safe to call twice.
        Also runs at interpreter exit for managers that were never shut down."""
        if self._shut:
            return
        self._shut = True
        # a constructor that raised half way leaves some of these unset
        if self.server_client_mode:
            if self.dp_client is not None:
                self.dp_client.shutdown()
            if self.server_handle is not None:
                self.server_handle.shutdown()
                self.server_handle = None
        elif self.kv_task_engine is not None:
            self.kv_task_engine.shutdown()
        elif self.transfer_manager is not None:
            self.transfer_manager.shutdown()

    # ---- requests -------------------------------------------------------------
    def get_async(self, token_ids, slot_mapping, token_mask=None, namespace: Optional[List[str]] = None) -> int:
        token_ids, slot_mapping, token_mask = _np(token_ids, np.int64), _np(slot_mapping, np.int64), _np(token_mask)
        if self.server_client_mode:
            return self.dp_client.get_async(token_ids, slot_mapping, token_mask, namespace=namespace)
        return self.kv_task_engine.get_async(token_ids, slot_mapping, token_mask, self.dp_client_id, namespace)[0]

    def get_match(self, token_ids, token_mask=None, cpu_only: bool = False, namespace: Optional[List[str]] = None,
                  swa_aware: bool = False) -> Tuple[int, np.ndarray]:
        token_ids, token_mask = _np(token_ids, np.int64), _np(token_mask)
        if self.server_client_mode:
            return self.dp_client.get_match(token_ids, token_mask, cpu_only=cpu_only, namespace=namespace,
                                            swa_aware=swa_aware)
        return self.kv_task_engine.get_match(token_ids, token_mask, self.dp_client_id, cpu_only, namespace, swa_aware)

    def put_async(self, token_ids, slot_mapping, token_mask=None, namespace: Optional[List[str]] = None) -> int:
        token_ids, slot_mapping, token_mask = _np(token_ids, np.int64), _np(slot_mapping, np.int64), _np(token_mask)
        if self.server_client_mode:
            return self.dp_client.put_async(token_ids, slot_mapping, token_mask, namespace=namespace)
        return self.kv_task_engine.put_async(token_ids, slot_mapping, token_mask, self.dp_client_id, namespace)[0]

    def put_match(self, token_ids, token_mask=None, namespace: Optional[List[str]] = None) -> Tuple[int, np.ndarray]:
        token_ids, token_mask = _np(token_ids, np.int64), _np(token_mask)
        if self.server_client_mode:
            return self.dp_client.put_match(token_ids, token_mask, namespace=namespace)
        return self.kv_task_engine.put_match(token_ids, token_mask, self.dp_client_id, namespace)

    def prefetch_async(self, token_ids, namespace: Optional[List[str]] = None, swa_aware: bool = False) -> int:
        token_ids = _np(token_ids, np.int64)
        if self.server_client_mode:
            return self.dp_client.prefetch_async(token_ids, namespace=namespace, swa_aware=swa_aware)
        return self.kv_task_engine.prefetch_async(token_ids, self.dp_client_id, namespace, swa_aware)

    def launch(self, task_ids: Union[int, List[int]], slot_mappings, swa_slot_mappings=None, as_batch: bool = False,
               layerwise_transfer: bool = False, counter_id: int = 0) -> List[int]:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        if not isinstance(slot_mappings, (list, tuple)):
            slot_mappings = [slot_mappings]
        slot_mappings = [_np(s, np.int64) for s in slot_mappings]
        if self.server_client_mode:
            return self.dp_client.launch_tasks(task_ids, slot_mappings, swa_slot_mappings=swa_slot_mappings,
                                               as_batch=as_batch, layerwise_transfer=layerwise_transfer,
                                               counter_id=counter_id)
        return self.kv_task_engine.launch_tasks(task_ids, slot_mappings, swa_slot_mappings=swa_slot_mappings,
                                                as_batch=as_batch, layerwise_transfer=layerwise_transfer,
                                                counter_id=counter_id)

    def cancel(self, task_ids: Union[int, List[int]]) -> None:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        if self.server_client_mode:
            self.dp_client.cancel_tasks(task_ids)
        else:
            self.kv_task_engine.cancel_tasks(task_ids)

    def wait(self, task_ids: Union[int, List[int]], timeout: float = 20.0, completely: bool = False
             ) -> Dict[int, KVResponse]:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        if self.server_client_mode:
            return self.dp_client.wait(task_ids, timeout, completely)
        return self.kv_task_engine.wait(task_ids, timeout, completely)

    def try_wait(self, task_ids: Union[int, List[int]]) -> Dict[int, KVResponse]:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        if self.server_client_mode:
            return self.dp_client.try_wait(task_ids)
        return self.kv_task_engine.try_wait(task_ids)

    # ---- cross-rank GPU prefix reuse (NVLink) ------------------------------------------
    def publish_gpu_blocks(self, token_ids, slot_mapping, namespace: Optional[List[str]] = None,
                           dp_client_id: Optional[int] = None) -> int:
        """Tells the other ranks that these GPU blocks of this rank hold the prefix's
        KV, so their gets can pull it over NVLink. Returns the number of blocks published."""
        token_ids, slot_mapping = _np(token_ids, np.int64), _np(slot_mapping, np.int64)
        dp = self.dp_client_id if dp_client_id is None else dp_client_id
        if self.server_client_mode:
            return self.dp_client.publish_gpu_blocks(token_ids, slot_mapping, namespace=namespace)
        return self.kv_task_engine.publish_gpu_blocks(token_ids, slot_mapping, dp, namespace)

    def withdraw_gpu_blocks(self, gpu_block_ids, dp_client_id: Optional[int] = None) -> List[int]:
        """Call before the engine reuses the blocks; returns blocks a peer is still reading."""
        dp = self.dp_client_id if dp_client_id is None else dp_client_id
        if self.server_client_mode:
            return self.dp_client.withdraw_gpu_blocks(_np(gpu_block_ids, np.int64))
        return self.kv_task_engine.withdraw_gpu_blocks(_np(gpu_block_ids, np.int64), dp)

    def checkpoint_ssd_index(self) -> bool:
        """Writes the SSD tier's size table and index beside its files now (they are written at shutdown
        anyway when ``ssd_persist`` is on): a crash after this call restarts from this state instead of cold.
        Blocks still being written are left out, blocks stored later are simply not in the image, and the
        image is removed again as soon as the tier evicts a block (it would be rewritten). Returns False when
        the tier does not persist or lives in another process."""
        from .cache import persist
        if self.server_client_mode or not persist.persist_enabled(self.cache_config):
            return False
        tm, gce = self.transfer_manager, self.kv_task_engine.cache_engine
        if tm.storage is None or gce.ssd_cache_engine is None:
            return False
        with gce._cache_tree_lock:     # noqa: SLF001 - the index must not move between the two files
            # the index may only name blocks whose bytes are on the disk: with buffered descriptors (no O_DIRECT)
            # they may still sit in the page cache, and the blocks carry no checksum
            tm.storage.sync_ssd_files()
            persist.save_size_table(self.cache_config, tm.storage.ssd_size_table)
            return gce.checkpoint_ssd_index()

    def _clear_cpu_cache(self) -> None:
        if self.server_client_mode:
            flexkv_logger.error("clearing the host cache is not supported in server-client mode")
            return
        self.kv_task_engine._clear_cpu_cache()  # noqa: SLF001

    def reset(self) -> None:
        """Drops every tier's index and frees its pool (call after a weight update)."""
        if self.server_client_mode:
            self.dp_client.reset()
        else:
            self.kv_task_engine.reset_cache()
