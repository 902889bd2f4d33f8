"""Packed-sequence (varlen) causal attention on CUDA.

Training and prefill attention go through :func:`varlen_attention_cuda`. The hand-written sm_100a kernel is
used when the library exports it; until then the call is served by the flash-attn library kernel, which is
the same kernel the reference calls (cosmos_rl/policy/model/gpt/__init__.py:264-273) and therefore the
baseline, not the product.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import native


def _have_native_flash() -> bool:
    return hasattr(native.lib(), "b200_flash_fwd")


def varlen_attention_cuda(q, k, v, cu_seqlens, max_seqlen: int, scale: Optional[float] = None):
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    from flash_attn import flash_attn_varlen_func
    cu = cu_seqlens.to(torch.int32)
    return flash_attn_varlen_func(q, k, v, cu, cu, max_seqlen, max_seqlen, dropout_p=0.0, softmax_scale=scale,
                                  causal=True)
