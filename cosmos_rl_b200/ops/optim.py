"""Fused optimizer kernels on flat buffers: AdamW with fp32 master weights / bf16 shadow copy, gradient
sum-of-squares and the clip coefficient (kept on the device, so no host sync sits between the gradient
reduction and the update). Reference behaviour: torch.optim.AdamW(fused=True) in
cosmos_rl/policy/trainer/optm/__init__.py:365-400 and gradient_norm_clipping in
cosmos_rl/utils/distributed.py:306-407.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional, Tuple

import torch

from . import native, reference


def grad_sumsq(grads: Iterable[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sum of squares of all gradient tensors, accumulated into a 1-element fp32 device tensor."""
    grads = [g for g in grads if g is not None]
    dev = grads[0].device
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=dev)
    if dev.type != "cuda":
        for g in grads:
            out += g.float().pow(2).sum()
        return out
    L = native.lib()
    for g in grads:
        assert g.is_contiguous()
        native.check(L.b200_sumsq(native.ptr(g), 1 if g.dtype == torch.float32 else 0, g.numel(), native.ptr(out),
                                  native.stream()), "sumsq")
    return out


def clip_coef_from_sumsq(sumsq: torch.Tensor, max_norm: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (norm, coef) as 1-element device tensors; coef = min(1, max_norm / (norm + 1e-6))."""
    if sumsq.device.type != "cuda":
        norm = sumsq.sqrt()
        coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
        return norm, coef
    norm = torch.empty_like(sumsq)
    coef = torch.empty_like(sumsq)
    native.check(native.lib().b200_clip_coef(native.ptr(sumsq), float(max_norm), native.ptr(coef), native.ptr(norm),
                                             native.stream()), "clip_coef")
    return norm, coef


def grad_norm_and_clip(grads: Iterable[torch.Tensor], max_norm: float):
    return clip_coef_from_sumsq(grad_sumsq(grads), max_norm)


def adamw_flat(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
               shadow: Optional[torch.Tensor], *, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, grad_scale: Optional[torch.Tensor] = None) -> None:
    """One AdamW step on flat fp32 ``master/m/v`` with a bf16 or fp32 ``grad``; ``shadow`` (bf16 compute copy of
    the weights) is rewritten in the same pass. ``grad_scale`` is a 1-element device tensor (clip coefficient)."""
    n = master.numel()
    if master.device.type != "cuda":
        gs = float(grad_scale) if grad_scale is not None else 1.0
        reference.adamw_step(master, m, v, grad, lr, beta1, beta2, eps, weight_decay, step, gs)
        if shadow is not None:
            shadow.copy_(master.to(shadow.dtype))
        return
    bias1 = 1.0 - beta1 ** step
    bias2 = 1.0 - beta2 ** step
    native.check(native.lib().b200_adamw(native.ptr(master), native.ptr(m), native.ptr(v), native.ptr(grad),
                                         1 if grad.dtype == torch.float32 else 0, native.ptr(shadow), n, lr, beta1,
                                         beta2, eps, weight_decay, bias1, bias2, native.ptr(grad_scale),
                                         native.stream()), "adamw")
