"""Named KV shapes (layers, KV heads, head size, dtype, block size)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..common.config import ModelConfig, nvfp4_head_bytes


@dataclass(frozen=True)
class KVShape:
    name: str
    num_layers: int
    num_kv_heads: int
    head_size: int
    dtype: torch.dtype = torch.bfloat16
    use_mla: bool = False
    tokens_per_block: int = 16
    engine_layout: str = "vllm"      # vllm | sglang | trtllm

    @property
    def kv_dim(self) -> int:
        return 1 if self.use_mla else 2

    @property
    def bytes_per_token(self) -> int:
        return self.num_layers * self.kv_dim * self.num_kv_heads * self.head_size * self.dtype.itemsize

    @property
    def block_bytes(self) -> int:
        return self.bytes_per_token * self.tokens_per_block


SHAPES: Dict[str, KVShape] = {
    # 32 layers x 8 KV heads x 128, bf16, 16-token blocks: 2 MiB of K+V per block
    "llama3-8b": KVShape("llama3-8b", 32, 8, 128),
    # TP=8 SGLang deployment: 80 layers, 8 KV heads (one per rank)
    "llama3-70b": KVShape("llama3-70b", 80, 8, 128, engine_layout="sglang"),
    # MLA latent cache: 512 kv_lora + 64 rope = 576 per token, 64-token blocks
    "deepseek-v3": KVShape("deepseek-v3", 61, 1, 576, use_mla=True, tokens_per_block=64),
    # packed NVFP4 cache moved as bytes: head width = D/2 nibble bytes + D/16 scale bytes
    "qwen3-32b-nvfp4": KVShape("qwen3-32b-nvfp4", 64, 8, nvfp4_head_bytes(128), dtype=torch.uint8),
    "qwen3-32b": KVShape("qwen3-32b", 64, 8, 128),
    "tiny": KVShape("tiny", 2, 2, 16, tokens_per_block=4),
    "tiny-mla": KVShape("tiny-mla", 3, 1, 64, use_mla=True, tokens_per_block=4),
}


def get_shape(name: str) -> KVShape:
    if name not in SHAPES:
        raise KeyError(f"unknown KV shape {name}; known: {sorted(SHAPES)}")
    return SHAPES[name]


def make_model_config(shape: KVShape, tp_size: int = 1, dp_size: int = 1, pp_size: int = 1, nnodes: int = 1
                      ) -> ModelConfig:
    return ModelConfig(num_layers=shape.num_layers, num_kv_heads=shape.num_kv_heads, head_size=shape.head_size,
                       kv_dim=shape.kv_dim, use_mla=shape.use_mla, dtype=shape.dtype, tp_size=tp_size,
                       dp_size=dp_size, pp_size=pp_size, nnodes=nnodes)
