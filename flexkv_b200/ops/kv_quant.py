"""Block-scaled FP8 (e4m3, one fp32 scale per 128 values) offload fused with the
paged KV copy, and its PyTorch fp32 reference.

Host chunk format for a chunk of ``E`` bf16 values: ``E`` payload bytes followed
by ``E/128`` fp32 scales (``E % 512 == 0``).
"""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch

from .. import _native
from ..storage.gpu_layout import GpuRegistration
from .kv_copy import HostSide, make_params

GROUP = 128


def packed_chunk_bytes(chunk_elems: int) -> int:
    return chunk_elems + (chunk_elems // GROUP) * 4


def kv_quant_fp8(reg: GpuRegistration, host: HostSide, gpu_blocks, cpu_blocks, h2d: bool, layer_start: int = 0,
                 num_layers: int = -1, num_ctas: int = 32, status: Optional[torch.Tensor] = None,
                 stream: Optional[torch.cuda.Stream] = None) -> List[Any]:
    """pack (GPU bf16 -> host fp8, ``h2d=False``) or unpack (``h2d=True``) on the current stream.
    ``host`` strides are those of the packed format."""
    if reg.dtype != torch.bfloat16:
        raise TypeError("fp8 offload packs bf16 caches")
    keep: List[Any] = []
    p = make_params(reg, host, gpu_blocks, cpu_blocks, h2d, layer_start, num_layers,
                    status_ptr=status.data_ptr() if status is not None else 0, keep=keep)
    s = stream if stream is not None else torch.cuda.current_stream()
    _native.C.kv_quant_fp8(p, num_ctas, s.cuda_stream)
    return keep


def reference_pack(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 reference of the pack: ``x`` bf16 ``[..., E]`` -> (uint8 payload ``[..., E]``, fp32 scales ``[..., E/128]``)."""
    # computed on the CPU with tensor / tensor divisions: IEEE round-to-nearest fp32 division, which is what
    # the kernel's fdiv_rn does (a GPU division by a Python scalar may be turned into a reciprocal multiply)
    dev = x.device
    xf = x.detach().cpu().float().reshape(*x.shape[:-1], -1, GROUP)
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / torch.full_like(amax, 448.0), torch.ones_like(amax))
    q = (xf / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(*x.shape).to(dev), scale.squeeze(-1).to(dev)


def reference_unpack(payload: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    dev = payload.device
    q = payload.detach().cpu().view(torch.float8_e4m3fn).float().reshape(*payload.shape[:-1], -1, GROUP)
    return (q * scales.detach().cpu().unsqueeze(-1)).to(torch.bfloat16).reshape(*payload.shape).to(dev)
