"""Packed-sequence (varlen) causal attention on CUDA.

Forward runs the hand-written tcgen05 kernel (``csrc/flash_fwd.cu``: head_dim 128, GQA, packed sequences, queries
aligned to the end of the keys). It returns the output and the log-sum-exp the backward pass and the
context-parallel merge need. Head dims other than 128 (tiny test models) are served by the flash-attn library
kernel, which is what the reference calls (cosmos_rl/policy/kernel/modeling_utils.py:65-173).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import native


def native_flash_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and q.stride(-1) == 1
            and k.stride(-1) == 1 and v.stride(-1) == 1 and q.stride(1) == 128 and k.stride(1) == 128
            and v.stride(1) == 128 and q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0 and v.stride(0) % 8 == 0
            and q.shape[1] % k.shape[1] == 0)


def flash_fwd(q, k, v, cu_q, cu_k, max_q: int, scale: float, causal: bool = True
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [Tq, hq, 128], k / v [Tk, hkv, 128] (token-strided views are fine). Returns (out [Tq, hq, 128] bf16,
    lse [hq, Tq] fp32)."""
    Tq, hq, d = q.shape
    Tk, hkv = k.shape[0], k.shape[1]
    out = torch.empty(Tq, hq, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(hq, Tq, dtype=torch.float32, device=q.device)
    st = native.status_word(q.device)
    native.check(native.lib().b200_flash_fwd(
        native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(out), native.ptr(lse), native.ptr(cu_q),
        native.ptr(cu_k), cu_q.numel() - 1, Tq, Tk, hq, hkv, d, q.stride(0), k.stride(0), v.stride(0), out.stride(0),
        int(max_q), 1 if causal else 0, float(scale), native.ptr(st), native.stream()), "flash_fwd")
    return out, lse


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, scale, causal=True):
        out, lse = flash_fwd(q, k, v, cu_q, cu_k, max_q, scale, causal)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.max_q, ctx.max_k, ctx.scale, ctx.causal = max_q, max_k, scale, causal
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        return flash_bwd(dout.contiguous(), q, k, v, out, lse, cu_q, ctx.max_q, ctx.scale, cu_k=cu_k,
                         max_k=ctx.max_k, causal=ctx.causal) + (None, None, None, None, None, None)


def flash_attention(q, k, v, cu_q, cu_k, max_q: int, scale: Optional[float] = None, max_k: Optional[int] = None,
                    causal: bool = True):
    """Differentiable attention over packed sequences. Causal: the queries of a sequence are aligned to the end of
    its keys. Non-causal (``causal=False``): every query sees every key of its sequence (bidirectional self-attention
    of diffusion transformers, cross-attention onto a text sequence of another length)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    i32 = lambda t: t if t.dtype == torch.int32 else t.to(torch.int32)
    if max_k is None:
        max_k = int((cu_k[1:] - cu_k[:-1]).max().item()) if cu_k is not cu_q else max_q
    return _FlashAttn.apply(q, k, v, i32(cu_q), i32(cu_k), int(max_q), int(max_k), scale, bool(causal))


def flash_bwd(dout, q, k, v, out, lse, cu, max_seqlen: int, scale: float, cu_k=None, max_k=None,
              causal: bool = True):
    """Gradients of packed causal attention from the saved output and log-sum-exp (tcgen05 kernel)."""
    Tq, hq, d = q.shape
    Tk, hkv = k.shape[0], k.shape[1]
    cu_k = cu if cu_k is None else cu_k
    dq_acc = torch.zeros(Tq, hq, d, dtype=torch.float32, device=q.device)
    dk = torch.empty(Tk, hkv, d, dtype=k.dtype, device=q.device)
    dv = torch.empty(Tk, hkv, d, dtype=v.dtype, device=q.device)
    delta = torch.empty(hq, Tq, dtype=torch.float32, device=q.device)
    st = native.status_word(q.device)
    native.check(native.lib().b200_flash_bwd(
        native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(out), native.ptr(dout), native.ptr(lse),
        native.ptr(dq_acc), native.ptr(dk), native.ptr(dv), native.ptr(delta), native.ptr(cu), native.ptr(cu_k),
        cu.numel() - 1, Tq, Tk, hq, hkv, d, q.stride(0), k.stride(0), v.stride(0), out.stride(0), dout.stride(0),
        dk.stride(0), dv.stride(0), int(max_k if max_k is not None else max_seqlen), 1 if causal else 0, float(scale),
        native.ptr(st), native.stream()), "flash_bwd")
    return dq_acc.to(q.dtype), dk, dv


def flash_bwd_library(dout, q, k, v, out, lse, cu, max_seqlen: int, scale: float):
    """The flash-attn library's backward on the same saved tensors (comparison baseline in the kernel cases)."""
    from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _flash_attn_varlen_backward(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, max_seqlen, max_seqlen, 0.0, scale,
                                True, -1, -1, 0.0, None, False, None)
    return dq, dk, dv


def full_attention_cuda(q, k, v, cu_q, cu_k, max_q: int, max_k: int, scale: Optional[float] = None):
    """Non-causal packed attention (own kernel for head_dim 128, the flash-attn library otherwise)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    i32 = lambda t: t if t.dtype == torch.int32 else t.to(torch.int32)
    if native_flash_supported(q, k, v):
        return _FlashAttn.apply(q, k, v, i32(cu_q), i32(cu_k), int(max_q), int(max_k), scale, False)
    from flash_attn import flash_attn_varlen_func
    return flash_attn_varlen_func(q, k, v, i32(cu_q), i32(cu_k), max_q, max_k, dropout_p=0.0, softmax_scale=scale,
                                  causal=False)


def varlen_attention_cuda(q, k, v, cu_seqlens, max_seqlen: int, scale: Optional[float] = None):
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    cu = cu_seqlens if cu_seqlens.dtype == torch.int32 else cu_seqlens.to(torch.int32)
    if native_flash_supported(q, k, v):
        return _FlashAttn.apply(q, k, v, cu, cu, int(max_seqlen), int(max_seqlen), scale)
    from flash_attn import flash_attn_varlen_func
    return flash_attn_varlen_func(q, k, v, cu, cu, max_seqlen, max_seqlen, dropout_p=0.0, softmax_scale=scale,
                                  causal=True)
