"""Engine-facing configuration: builds ModelConfig / CacheConfig from an engine's
own config objects (flexkv/integration/config.py:180-281 vLLM, :385 SGLang, :644
TRT-LLM). Engine objects are read by attribute name only, so the functions work
with the real classes and with stand-ins in tests."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..common.config import (GLOBAL_CONFIG_FROM_ENV, NVFP4_NAMES, CacheConfig, ModelConfig, UserConfig, load_user_config_from_env,
                             nvfp4_head_bytes, parse_dtype, update_default_config_from_user_config)


def _attr(obj: Any, *names: str, default: Any = None) -> Any:
    for n in names:
        cur = obj
        ok = True
        for part in n.split("."):
            if cur is None or not hasattr(cur, part):
                ok = False
                break
            cur = getattr(cur, part)
        if ok and cur is not None:
            return cur() if callable(cur) and not isinstance(cur, type) else cur
    return default


@dataclass
class FlexKVConfig:
    model_config: ModelConfig = field(default_factory=ModelConfig)
    cache_config: CacheConfig = field(default_factory=CacheConfig)
    user_config: UserConfig = field(default_factory=UserConfig)
    server_recv_port: str = "ipc:///tmp/flexkv_server"
    gpu_register_port: str = "ipc:///tmp/flexkv_gpu_register"
    kv_cache_dtype: Optional[str] = None

    @classmethod
    def from_env(cls) -> "FlexKVConfig":
        import os
        cfg = cls(user_config=load_user_config_from_env())
        cfg.server_recv_port = os.getenv("FLEXKV_SERVER_RECV_PORT", cfg.server_recv_port)
        cfg.gpu_register_port = os.getenv("FLEXKV_GPU_REGISTER_PORT", cfg.server_recv_port + "_gpu_register")
        cfg.kv_cache_dtype = cfg.user_config.kv_cache_dtype
        return cfg

    # ---- shared -------------------------------------------------------------------
    def _apply_kv_dtype(self, engine_dtype: Any, head_size: int) -> None:
        """A packed NVFP4 cache is uint8 on the wire: the per-head width becomes
        head/2 nibble bytes + head/16 scale bytes and is never interpreted."""
        name = str(self.kv_cache_dtype or engine_dtype or "").lower().replace("torch.", "")
        m = self.model_config
        if name in NVFP4_NAMES:
            m.dtype = torch.uint8
            m.head_size = nvfp4_head_bytes(head_size)
        elif name and name != "auto":
            m.dtype = parse_dtype(name)
            m.head_size = head_size
        else:
            m.head_size = head_size

    def _finish(self, tokens_per_block: int) -> None:
        import os
        self.cache_config.tokens_per_block = tokens_per_block
        # where the transfer managers of a group that spans nodes reach the master's
        # (FLEXKV_MASTER_HOST / FLEXKV_MASTER_PORTS = command, result, query ports: flexkv/integration/config.py:250-253)
        if os.getenv("FLEXKV_MASTER_HOST"):
            self.model_config.master_host = os.environ["FLEXKV_MASTER_HOST"]
        if os.getenv("FLEXKV_MASTER_PORTS"):
            ports = tuple(p.strip() for p in os.environ["FLEXKV_MASTER_PORTS"].split(",") if p.strip())
            if len(ports) != 3:
                raise ValueError("FLEXKV_MASTER_PORTS needs three comma-separated ports")
            self.model_config.master_ports = ports
        self.model_config.instance_num = int(GLOBAL_CONFIG_FROM_ENV.instance_num)
        update_default_config_from_user_config(self.model_config, self.cache_config, self.user_config)
        self.model_config.freeze()

    # ---- vLLM ----------------------------------------------------------------------
    def post_init_from_vllm_config(self, vllm_config: Any) -> None:
        mc, pc, cc = _attr(vllm_config, "model_config"), _attr(vllm_config, "parallel_config"), \
            _attr(vllm_config, "cache_config")
        m = self.model_config
        m.num_layers = int(_attr(mc, "hf_text_config.num_hidden_layers", "hf_config.num_hidden_layers"))
        m.tp_size = int(_attr(pc, "tensor_parallel_size", default=1))
        m.pp_size = int(_attr(pc, "pipeline_parallel_size", default=1))
        m.dp_size = int(_attr(pc, "data_parallel_size", default=1))
        m.use_mla = bool(_attr(mc, "use_mla", default=False))
        if m.use_mla:
            hf = _attr(mc, "hf_text_config", "hf_config")
            m.num_kv_heads, m.kv_dim = 1, 1
            head = int(_attr(hf, "kv_lora_rank", default=512)) + int(_attr(hf, "qk_rope_head_dim", default=64))
        else:
            total_heads = _attr(mc, "hf_text_config.num_key_value_heads", "hf_config.num_key_value_heads",
                                "hf_text_config.num_attention_heads")
            m.num_kv_heads = max(int(total_heads), m.tp_size)
            head = int(_attr(mc, "hf_text_config.head_dim", "hf_config.head_dim", default=0)) or \
                int(_attr(mc, "hf_text_config.hidden_size")) // int(_attr(mc, "hf_text_config.num_attention_heads"))
        m.dtype = parse_dtype(_attr(mc, "dtype", default=torch.bfloat16))
        self._apply_kv_dtype(_attr(cc, "cache_dtype", default="auto"), head)
        self._finish(int(_attr(cc, "block_size", default=16)))

    # ---- SGLang --------------------------------------------------------------------
    def post_init_from_sglang_config(self, server_args: Any, model_config: Any, page_size: int, tp_size: int = 1,
                                     pp_size: int = 1, dp_size: int = 1, cp_size: int = 1) -> None:
        m = self.model_config
        m.num_layers = int(_attr(model_config, "num_hidden_layers", "hf_config.num_hidden_layers"))
        m.tp_size, m.pp_size, m.dp_size, m.cp_size = tp_size, pp_size, dp_size, cp_size
        m.attn_cp_size = cp_size
        m.use_mla = bool(_attr(model_config, "is_mla", "use_mla", default=False)) or \
            "mla" in str(_attr(model_config, "attention_arch", default="")).lower()
        if m.use_mla:
            m.num_kv_heads, m.kv_dim = 1, 1
            head = int(_attr(model_config, "kv_lora_rank", default=512)) + \
                int(_attr(model_config, "qk_rope_head_dim", default=64))
        else:
            m.num_kv_heads = max(int(_attr(model_config, "num_key_value_heads", "get_total_num_kv_heads")), tp_size)
            head = int(_attr(model_config, "head_dim"))
        m.dtype = parse_dtype(_attr(model_config, "dtype", default=torch.bfloat16))
        self._apply_kv_dtype(_attr(server_args, "kv_cache_dtype", default="auto"), head)
        if m.use_mla and _attr(model_config, "index_head_dim", default=None) is not None and \
                m.dtype == torch.float8_e4m3fn:
            # sparse-attention fp8 latent cache: fp8 latent + one fp32 scale per 128 values + bf16 rope part,
            # all counted in bytes of the 1-byte element (flexkv/integration/config.py:506-518)
            rank = int(_attr(model_config, "kv_lora_rank", default=512))
            rope = int(_attr(model_config, "qk_rope_head_dim", default=64))
            if rank % 128:
                raise ValueError(f"kv_lora_rank {rank} must be a multiple of 128 for the fp8 latent cache layout")
            m.head_size = rank + rank // 128 * 4 + rope * torch.bfloat16.itemsize
        self._finish(int(page_size))

    # ---- TensorRT-LLM --------------------------------------------------------------
    def post_init_from_trt_config(self, llm_args: Any, mapping: Any = None) -> None:
        m = self.model_config
        cfg = _attr(llm_args, "model_config", "pretrained_config", default=llm_args)
        m.num_layers = int(_attr(cfg, "num_hidden_layers"))
        m.tp_size = int(_attr(mapping, "tp_size", default=_attr(llm_args, "tensor_parallel_size", default=1)))
        m.pp_size = int(_attr(mapping, "pp_size", default=_attr(llm_args, "pipeline_parallel_size", default=1)))
        m.num_kv_heads = max(int(_attr(cfg, "num_key_value_heads", "num_attention_heads")), m.tp_size)
        head = int(_attr(cfg, "head_dim", default=0)) or int(_attr(cfg, "hidden_size")) // int(
            _attr(cfg, "num_attention_heads"))
        m.dtype = parse_dtype(_attr(cfg, "torch_dtype", "dtype", default=torch.bfloat16))
        m.use_trtllm_subprocess = True
        self._apply_kv_dtype(_attr(llm_args, "kv_cache_config.dtype", default="auto"), head)
        self._finish(int(_attr(llm_args, "kv_cache_config.tokens_per_block", default=32)))
