"""Differentiable front-ends of the sm_100a kernels.

CUDA tensors always run the hand-written kernels from ``libb200rl.so`` (a missing library raises);
CPU tensors run the fp32 PyTorch statements in :mod:`cosmos_rl_b200.ops.reference`, which are also the
test oracles. Tensor layouts follow the packed ("varlen") convention used across the framework:
activations are ``[T, ...]`` with ``T`` the total number of tokens of the micro-batch.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import native, reference

_N_PARTIAL_NORM = 296  # CTAs (2 per SM) that accumulate RMSNorm weight-gradient partials


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# --------------------------------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual):
        shape = x.shape
        H = shape[-1]
        x2 = _c(x).view(-1, H)
        T = x2.shape[0]
        res2 = _c(residual).view(-1, H) if residual is not None else None
        y = torch.empty_like(x2)
        res_out = torch.empty_like(x2) if residual is not None else None
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        L = native.lib()
        native.check(L.b200_rmsnorm_fwd(native.ptr(x2), native.ptr(res2), native.ptr(weight), native.ptr(y),
                                        native.ptr(res_out), native.ptr(rstd), T, H, eps, native.stream()),
                     "rmsnorm_fwd")
        h = res_out if residual is not None else x2
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = residual is not None
        ctx.shape = shape
        if residual is not None:
            return y.view(shape), res_out.view(shape)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dres_out):
        h, weight, rstd = ctx.saved_tensors
        H = h.shape[-1]
        T = h.shape[0]
        dy2 = _c(dy).view(-1, H)
        dres2 = _c(dres_out).view(-1, H) if dres_out is not None else None
        dx = torch.empty_like(h)
        dw = torch.zeros(H, dtype=torch.float32, device=h.device)
        native.check(native.lib().b200_rmsnorm_bwd2(native.ptr(dy2), native.ptr(h), native.ptr(weight),
                                                    native.ptr(rstd), native.ptr(dres2), native.ptr(dx),
                                                    native.ptr(dw), T, H, native.stream()), "rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        return dxv, dw.to(weight.dtype), None, (dxv if ctx.has_res else None)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None):
    """Returns ``(y, new_residual)``; ``new_residual`` is ``x + residual`` (or ``None`` without residual)."""
    if x.is_cuda:
        if x.dtype != torch.bfloat16:
            raise TypeError("rms_norm on CUDA expects bf16 activations")
        return _RMSNorm.apply(x, weight, eps, residual)
    return reference.rms_norm(x, weight, eps, residual)


# --------------------------------------------------------------------------------------------------
# RoPE (in place on views of the fused qkv projection)
# --------------------------------------------------------------------------------------------------
def _rope_native(q, k, positions, theta, backward):
    T, hq, d = q.shape
    hkv = k.shape[1] if k is not None else 0
    assert q.stride(-1) == 1 and q.stride(1) == d
    if k is not None:
        assert k.stride(-1) == 1 and k.stride(1) == d
    L = native.lib()
    native.check(L.b200_rope_inplace(native.ptr(q), native.ptr(k), native.ptr(positions), T, hq, hkv, d, q.stride(0),
                                     k.stride(0) if k is not None else 0, float(theta), 1 if backward else 0,
                                     native.stream()), "rope")


class _RoPE(torch.autograd.Function):
    """Out-of-place on separate q / k tensors (the fused-qkv form below rotates in place)."""

    @staticmethod
    def forward(ctx, q, k, positions, theta):
        q, k = q.clone(memory_format=torch.contiguous_format), k.clone(memory_format=torch.contiguous_format)
        _rope_native(q, k, positions, theta, False)
        ctx.save_for_backward(positions)
        ctx.theta = theta
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        (positions,) = ctx.saved_tensors
        dq, dk = dq.clone(memory_format=torch.contiguous_format), dk.clone(memory_format=torch.contiguous_format)
        _rope_native(dq, dk, positions, ctx.theta, True)
        return dq, dk, None, None


def apply_rope(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, theta: float):
    """Rotary embedding of ``q [T, hq, d]`` and ``k [T, hkv, d]`` (int64 positions on CUDA). With autograd the
    result is a new pair of tensors; without, the rotation is done in place."""
    if q.is_cuda:
        positions = positions.to(torch.int64)
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad):
            return _RoPE.apply(q, k, positions, theta)
        _rope_native(q, k, positions, theta, False)
        return q, k
    return reference.apply_rope(q, k, positions, theta)


class _RoPEQKV(torch.autograd.Function):
    """In-place rotation of the q and k column blocks of a fused ``[T, (hq + 2 hkv) d]`` projection."""

    @staticmethod
    def forward(ctx, qkv, positions, hq, hkv, d, theta):
        T = qkv.shape[0]
        q = qkv[:, : hq * d].unflatten(-1, (hq, d))
        k = qkv[:, hq * d: (hq + hkv) * d].unflatten(-1, (hkv, d))
        _rope_native(q, k, positions, theta, False)
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(positions)
        ctx.cfg = (hq, hkv, d, theta)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        (positions,) = ctx.saved_tensors
        hq, hkv, d, theta = ctx.cfg
        dqkv = dqkv.clone(memory_format=torch.contiguous_format)
        q = dqkv[:, : hq * d].unflatten(-1, (hq, d))
        k = dqkv[:, hq * d: (hq + hkv) * d].unflatten(-1, (hkv, d))
        _rope_native(q, k, positions, theta, True)
        return dqkv, None, None, None, None, None


def rope_qkv_(qkv: torch.Tensor, positions: torch.Tensor, hq: int, hkv: int, d: int, theta: float) -> torch.Tensor:
    """Rotary embedding applied to the q and k blocks of a fused qkv projection ``[T, (hq + 2 hkv) d]``.
    In place on CUDA (returns the same tensor); a new tensor on CPU."""
    if qkv.is_cuda:
        positions = positions.to(torch.int64)
        if torch.is_grad_enabled() and qkv.requires_grad:
            return _RoPEQKV.apply(qkv, positions, hq, hkv, d, theta)
        q = qkv[:, : hq * d].unflatten(-1, (hq, d))
        k = qkv[:, hq * d: (hq + hkv) * d].unflatten(-1, (hkv, d))
        _rope_native(q, k, positions, theta, False)
        return qkv
    T = qkv.shape[0]
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k = reference.apply_rope(q.reshape(T, hq, d), k.reshape(T, hkv, d), positions, theta)
    return torch.cat([q.reshape(T, -1), k.reshape(T, -1), v], dim=-1)


# --------------------------------------------------------------------------------------------------
# SwiGLU
# --------------------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        I2 = gate_up.shape[-1]
        gu = _c(gate_up).view(-1, I2)
        out = torch.empty(gu.shape[0], I2 // 2, dtype=gu.dtype, device=gu.device)
        native.check(native.lib().b200_swiglu_fwd(native.ptr(gu), native.ptr(out), gu.shape[0], I2 // 2,
                                                  native.stream()), "swiglu_fwd")
        ctx.save_for_backward(gu)
        ctx.shape = gate_up.shape
        return out.view(*gate_up.shape[:-1], I2 // 2)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        d2 = _c(dout).view(-1, gu.shape[1] // 2)
        dgu = torch.empty_like(gu)
        native.check(native.lib().b200_swiglu_bwd(native.ptr(d2), native.ptr(gu), native.ptr(dgu), gu.shape[0],
                                                  gu.shape[1] // 2, native.stream()), "swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    if gate_up.is_cuda:
        return _SwiGLU.apply(gate_up)
    return reference.swiglu(gate_up)


# --------------------------------------------------------------------------------------------------
# dense GEMM (tcgen05)
# --------------------------------------------------------------------------------------------------
def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
            accumulate: bool = False) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T`` on the tcgen05 kernel (bf16 in, bf16 or fp32 out)."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and a.dim() == 2 and b.dim() == 2
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    st = native.status_word(a.device)
    dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
    native.check(native.lib().b200_gemm_bf16_nt(native.ptr(a), native.ptr(b), native.ptr(out), M, N, K, a.stride(0),
                                                b.stride(0), out.stride(0), 1 if out.dtype == torch.float32 else 0,
                                                1 if accumulate else 0, native.ptr(st), native.num_sms(dev),
                                                native.stream()), "gemm_bf16_nt")
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, accumulate: bool = False,
         bias: Optional[torch.Tensor] = None, swiglu: bool = False, path: int = 0) -> torch.Tensor:
    """General tcgen05 GEMM ``C[M, N] (+)= A . B^T (+ bias)`` on row-major bf16 tensors.

    ``a_mn``: ``a`` is stored ``[K, M]`` instead of ``[M, K]``; ``b_mn``: ``b`` is stored ``[K, N]`` instead of
    ``[N, K]``. ``bias [N]`` (bf16 or fp32) is added in the epilogue. ``swiglu``: ``b`` is a fused gate/up weight
    ``[2 I, K]`` and the result is ``silu(A Bg^T) * (A Bu^T)`` of shape ``[M, I]``. ``path``: 0 lets the library choose
    between the CTA-pair kernel (256-row tiles over two SMs) and the single-CTA kernel, 1 / 2 force one of them."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and a.dim() == 2 and b.dim() == 2
    K, M = (a.shape[0], a.shape[1]) if a_mn else (a.shape[1], a.shape[0])
    Kb, N = (b.shape[0], b.shape[1]) if b_mn else (b.shape[1], b.shape[0])
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N // 2 if swiglu else N, dtype=out_dtype, device=a.device)
    if bias is not None:
        assert bias.is_contiguous() and bias.numel() == N and bias.dtype in (torch.bfloat16, torch.float32)
    st = native.status_word(a.device)
    dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
    native.check(native.lib().b200_gemm_bf16_ex(native.ptr(a), native.ptr(b), native.ptr(out), M, N, K, a.stride(0),
                                                b.stride(0), out.stride(0), int(a_mn), int(b_mn),
                                                1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                                                native.ptr(bias), 1 if bias is not None and bias.dtype == torch.bfloat16 else 0,
                                                1 if swiglu else 0, N // 2 if swiglu else 0, path,
                                                native.ptr(st), native.num_sms(dev), native.stream()), "gemm_bf16")
    return out


def _tc_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The tensor-core GEMMs move rows with TMA: feature dimensions must give 16-byte rows."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2
            and weight.stride(-1) == 1 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
            and weight.stride(0) % 8 == 0)


class _LinearTC(torch.autograd.Function):
    """``y = x W^T (+ b)`` with forward, dgrad and wgrad on the tcgen05 GEMM. The bias is added in the forward
    epilogue; when ``W.grad`` already exists the weight gradient is accumulated into it by the GEMM epilogue itself
    (no separate add pass)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = _c(x).view(-1, x.shape[-1])
        # the result is allocated in its final shape: callers rotate / scale it in place, which autograd forbids on
        # a view returned by a custom function
        y = torch.empty(*x.shape[:-1], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        y2 = y.view(-1, weight.shape[0])
        gemm(x2, weight, out=y2, bias=bias if (bias is not None and x2.shape[0] > 128) else None)
        if bias is not None and x2.shape[0] <= 128:
            y2 += bias
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = _c(dy).view(-1, weight.shape[0])
        dx = gemm(dy2, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            if weight.grad is not None and weight.grad.dtype in (torch.bfloat16, torch.float32) \
                    and weight.grad.stride(-1) == 1:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=weight.grad, accumulate=True)
                dw = None  # accumulated in place
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        db = dy2.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return (dx.view(ctx.shape) if dx is not None else None), dw, db


def linear_tc(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Linear layer on this library's GEMM (CUDA bf16); CPU tensors use ``torch.nn.functional.linear``."""
    if _tc_ok(x, weight):
        if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad or
                                        (bias is not None and bias.requires_grad)):
            return _LinearTC.apply(x, weight, bias)
        x2 = _c(x).view(-1, x.shape[-1])
        return linear_infer(x2, weight, bias).view(*x.shape[:-1], weight.shape[0])
    return torch.nn.functional.linear(x, weight, bias)


def _dims_ok(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(-1) == 1 and t.stride(0) % 8 == 0
               and t.shape[1] % 8 == 0 for t in ts)


def mm_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T`` (a forward projection) without autograd: this library's GEMM for bf16 CUDA tensors."""
    return gemm(x, w) if _dims_ok(x, w) else x @ w.t()


def mm_nn(gy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``gy [M, N] @ w [N, K]`` (the input gradient of a projection): ``w`` is read as stored, no transposed copy."""
    return gemm(gy, w, b_mn=True) if _dims_ok(gy, w) else gy @ w


def mm_tn(gy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
          accumulate: bool = False) -> torch.Tensor:
    """``gy [T, N]^T @ x [T, K]`` (the weight gradient of a projection), contracting over the token axis of both."""
    if _dims_ok(gy, x) and (out is None or (out.is_cuda and out.stride(-1) == 1)):
        return gemm(gy, x, a_mn=True, b_mn=True, out=out, out_dtype=out_dtype, accumulate=accumulate)
    r = gy.t() @ x
    if out is None:
        return r.to(out_dtype)
    return out.add_(r) if accumulate else out.copy_(r)


def linear_infer(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inference linear on ``x2 [M, K]``: the CTA-pair kernel for wide batches, the weight-streaming split-K kernel
    for decode-sized ones (``M <= 256``), where reading ``weight`` once is the whole cost."""
    M = x2.shape[0]
    if M <= _SKINNY_MAX_M:
        return gemm_skinny(x2, weight, bias=bias, out=out)
    return gemm(x2, weight, bias=bias, out=out)


# --------------------------------------------------------------------------------------------------
# decode-sized projections: weight-streaming split-K GEMM + fused reductions
# --------------------------------------------------------------------------------------------------
_SKINNY_MAX_M = 256
_SKINNY_WS_FLOATS = 148 * 2 * 128 * 128      # splits * tiles <= SMs, a tile is 128 x 128 fp32: this bound always holds
_skinny_ws: dict = {}


def _skinny_workspace(device: torch.device) -> torch.Tensor:
    """fp32 split-K workspace, one per (device, stream) so that concurrent streams never share partial sums. It is
    created by the first decode-sized projection on that stream (do that once outside CUDA-graph capture)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), native.stream())
    w = _skinny_ws.get(key)
    if w is None:
        w = _skinny_ws[key] = torch.empty(_SKINNY_WS_FLOATS, dtype=torch.float32, device=device)
    return w


def _skinny_launch(x2, weight, N, swiglu, out, use_ws, bias=None):
    M, K = x2.shape
    assert x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M <= _SKINNY_MAX_M
    assert x2.stride(-1) == 1 and weight.stride(-1) == 1
    dev = x2.device.index if x2.device.index is not None else torch.cuda.current_device()
    sms = native.num_sms(dev)
    L = native.lib()
    splits = 1 if swiglu else L.b200_gemm_skinny_splits(M, N, K, 0, sms)
    ws = _skinny_workspace(x2.device) if (use_ws or splits > 1) else None
    if ws is not None:
        assert splits * M * N <= ws.numel()
    st = native.status_word(x2.device)
    native.check(L.b200_gemm_skinny(native.ptr(x2), native.ptr(weight), native.ptr(out) if ws is None else None,
                                    native.ptr(ws), M, N, K, x2.stride(0), weight.stride(0),
                                    out.stride(0) if out is not None else 0, native.ptr(bias),
                                    1 if bias is not None and bias.dtype == torch.bfloat16 else 0,
                                    1 if swiglu else 0, N if swiglu else 0, splits, native.ptr(st), sms,
                                    native.stream()), "gemm_skinny")
    return ws, splits


def gemm_skinny(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x2 [M <= 256, K] @ weight [N, K]^T (+ bias)`` in bf16 on the weight-streaming kernel."""
    M, N = x2.shape[0], weight.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x2.device)
    ws, splits = _skinny_launch(x2, weight, N, False, out, False, bias)
    if ws is not None:
        native.check(native.lib().b200_splitk_reduce(native.ptr(ws), splits, M, N, native.ptr(bias),
                                                     1 if bias is not None and bias.dtype == torch.bfloat16 else 0,
                                                     native.ptr(out), out.stride(0), native.stream()), "splitk_reduce")
    return out


def skinny_gate_up_swiglu(x2: torch.Tensor, gate_up_weight: torch.Tensor) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` for a fused ``[2 I, K]`` weight: the product is formed in the GEMM epilogue."""
    M, I = x2.shape[0], gate_up_weight.shape[0] // 2
    out = torch.empty(M, I, dtype=torch.bfloat16, device=x2.device)
    _skinny_launch(x2, gate_up_weight, I, True, out, False)
    return out


def skinny_linear_residual_rmsnorm(x2: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor],
                                   norm_weight: torch.Tensor, eps: float):
    """``res' = x2 @ weight^T + residual``; returns ``(rmsnorm(res') * norm_weight, res')``: the split-K reduction of
    the projection, the residual add and the normalisation are one kernel."""
    M, H = x2.shape[0], weight.shape[0]
    ws, splits = _skinny_launch(x2, weight, H, False, None, True)
    y = torch.empty(M, H, dtype=torch.bfloat16, device=x2.device)
    res_out = torch.empty_like(y)
    assert norm_weight.dtype == torch.bfloat16 and (residual is None or residual.is_contiguous())
    native.check(native.lib().b200_splitk_reduce_residual_rmsnorm(native.ptr(ws), splits, M, H, native.ptr(residual),
                                                                  native.ptr(norm_weight), float(eps),
                                                                  native.ptr(res_out), native.ptr(y), native.stream()),
                 "splitk_reduce_residual_rmsnorm")
    return y, res_out


def skinny_qkv_rope_append(x2: torch.Tensor, qkv_weight: torch.Tensor, bias: Optional[torch.Tensor],
                           positions: torch.Tensor, slot_mapping: torch.Tensor, theta: float, hq: int, hkv: int, d: int,
                           cache: torch.Tensor, v_transposed: bool) -> torch.Tensor:
    """Fused qkv projection of a decode step: returns rotated ``q [M, hq, d]``; the rotated K rows and the V rows are
    written into the paged ``cache [pages, 2, hkv, page, d]`` at ``slot_mapping`` by the reduction kernel."""
    M, N = x2.shape[0], qkv_weight.shape[0]
    assert N == (hq + 2 * hkv) * d and positions.dtype == torch.int64 and slot_mapping.dtype == torch.int32
    ws, splits = _skinny_launch(x2, qkv_weight, N, False, None, True)
    q = torch.empty(M, hq, d, dtype=torch.bfloat16, device=x2.device)
    native.check(native.lib().b200_splitk_reduce_qkv_rope_append(
        native.ptr(ws), splits, M, hq, hkv, d, native.ptr(bias),
        1 if bias is not None and bias.dtype == torch.bfloat16 else 0, native.ptr(positions), native.ptr(slot_mapping),
        float(theta), native.ptr(q), native.ptr(cache), cache.shape[3], 1 if v_transposed else 0, native.stream()),
        "splitk_reduce_qkv_rope_append")
    return q


# --------------------------------------------------------------------------------------------------
# fused lm_head + log-prob + entropy
# --------------------------------------------------------------------------------------------------
def _pick_nsplit(T: int, V: int, sms: int) -> int:
    num_m = (T + 127) // 128
    num_n = (V + 255) // 256
    best, best_score = 1, -1.0
    for ns in range(1, min(num_n, 64) + 1):
        units = num_m * ns
        waves = math.ceil(units / sms)
        eff = units / (waves * sms)
        # prefer full waves, then fewer splits (less scratch, fewer partial merges)
        score = eff - 0.002 * ns
        if score > best_score:
            best, best_score = ns, score
    return best


_DLOGITS_CHUNK = int(os.environ.get("B200RL_DLOGITS_CHUNK", "16384"))


class _FusedLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature, want_entropy):
        T, H = hidden.shape
        V = weight.shape[0]
        hidden = _c(hidden)
        dev = hidden.device.index if hidden.device.index is not None else torch.cuda.current_device()
        sms = native.num_sms(dev)
        nsplit = _pick_nsplit(T, V, sms)
        partial = torch.empty(T, nsplit, 4, dtype=torch.float32, device=hidden.device)
        lp = torch.empty(T, dtype=torch.float32, device=hidden.device)
        lse = torch.empty_like(lp)
        ent = torch.empty_like(lp)
        st = native.status_word(hidden.device)
        L = native.lib()
        native.check(L.b200_lmhead_logprob_partial(native.ptr(hidden), native.ptr(weight), native.ptr(labels),
                                                   native.ptr(partial), T, V, H, hidden.stride(0), weight.stride(0),
                                                   1.0 / temperature, nsplit, native.ptr(st), sms, native.stream()),
                     "lmhead_logprob_partial")
        native.check(L.b200_logprob_combine(native.ptr(partial), native.ptr(labels), native.ptr(lp), native.ptr(lse),
                                            native.ptr(ent), T, nsplit, native.stream()), "logprob_combine")
        ctx.save_for_backward(hidden, weight, labels, lse, ent)
        ctx.temperature = temperature
        ctx.want_entropy = want_entropy
        ctx.sms = sms
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, labels, lse, ent = ctx.saved_tensors
        T, H = hidden.shape
        V = weight.shape[0]
        g_lp = _c(g_lp.float())
        use_ent = ctx.want_entropy and g_ent is not None
        g_ent_t = _c(g_ent.float()) if use_ent else None
        st = native.status_word(hidden.device)
        L = native.lib()
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dh = torch.zeros(T, H, dtype=torch.float32, device=hidden.device) if need_dh else None
        dw = torch.empty_like(weight) if need_dw else None
        chunk = min(_DLOGITS_CHUNK, V)
        buf = torch.empty(T, chunk, dtype=torch.bfloat16, device=hidden.device)
        for v0 in range(0, V, chunk):
            vc = min(chunk, V - v0)
            dl = buf[:, :vc]
            native.check(L.b200_lmhead_dlogits(native.ptr(hidden), native.ptr(weight), native.ptr(labels),
                                               native.ptr(lse), native.ptr(g_lp), native.ptr(g_ent_t),
                                               native.ptr(ent) if use_ent else None, native.ptr(buf), T, V, H,
                                               hidden.stride(0), weight.stride(0), v0, vc, buf.stride(0),
                                               1.0 / ctx.temperature, native.ptr(st), ctx.sms, native.stream()),
                         "lmhead_dlogits")
            # both products on this library's GEMM: dh accumulates in fp32 through the epilogue's reduce-add,
            # dW of this vocabulary slice contracts dlogits^T and hidden over the token axis as stored
            if need_dh:
                if _dims_ok(dl, weight):
                    gemm(dl, weight[v0:v0 + vc], b_mn=True, out=dh, accumulate=True)
                else:
                    dh.add_(torch.mm(dl, weight[v0:v0 + vc]))
            if need_dw:
                mm_tn(dl, hidden, out=dw[v0:v0 + vc])
        return (dh.to(hidden.dtype) if need_dh else None), dw, None, None, None


def fused_logprob(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                  want_entropy: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Log-prob of ``labels [T]`` and entropy under ``softmax(hidden @ weight.T / temperature)`` without
    materialising the logits. ``hidden [T, H]`` bf16, ``weight [V, H]`` bf16. Returns fp32 ``(logprob, entropy)``."""
    if hidden.is_cuda:
        labels = labels.to(torch.int64)
        return _FusedLogprob.apply(hidden, weight, labels, float(temperature), want_entropy)
    return reference.logprob_entropy(hidden, weight, labels, temperature)


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
def varlen_attention(q, k, v, cu_seqlens, max_seqlen: int, scale: Optional[float] = None):
    """Causal GQA attention over packed sequences."""
    if q.is_cuda:
        from . import attention
        return attention.varlen_attention_cuda(q, k, v, cu_seqlens, max_seqlen, scale)
    return reference.varlen_attention(q, k, v, cu_seqlens, scale)


def full_attention(q, k, v, cu_q, cu_k, max_q: int, max_k: int, scale: Optional[float] = None):
    """Bidirectional attention over packed sequences: ``q [Tq, hq, d]``, ``k/v [Tk, hkv, d]``; sequence i owns queries
    ``cu_q[i]:cu_q[i+1]`` and keys ``cu_k[i]:cu_k[i+1]`` (self-attention when ``cu_q is cu_k``, else cross-attention)."""
    if q.is_cuda:
        from . import attention
        return attention.full_attention_cuda(q, k, v, cu_q, cu_k, max_q, max_k, scale)
    return reference.varlen_attention(q, k, v, cu_q, scale, causal=False, cu_k=cu_k)


def tc_decode_supported(d: int, page_size: int, hq: int, hkv: int) -> bool:
    """The tcgen05 decode kernel needs head_dim 128, 128-token pages and a GQA group of at most 8."""
    return d == 128 and page_size == 128 and hq % hkv == 0 and hq // hkv <= 8


def kv_append(k, v, cache, slot_mapping, v_transposed: bool = False):
    """Write new K/V rows into the paged cache ``[pages, 2, hkv, page_size, d]``. With ``v_transposed`` the V
    slabs are stored as ``[d, page_size]`` (the layout the tensor-core decode kernel consumes)."""
    if k.is_cuda:
        T, hkv, d = k.shape
        assert k.stride(-1) == 1 and k.stride(1) == d and v.stride(-1) == 1 and v.stride(1) == d
        fn = native.lib().b200_kv_append_vt if v_transposed else native.lib().b200_kv_append
        native.check(fn(native.ptr(k), native.ptr(v), native.ptr(cache), native.ptr(slot_mapping), T, hkv, d,
                        k.stride(0), v.stride(0), cache.shape[3], native.stream()), "kv_append")
    else:
        reference.kv_append(k, v, cache, slot_mapping, v_transposed)


def paged_decode(q, cache, block_table, seq_lens, scale: Optional[float] = None, nsplit: Optional[int] = None,
                 scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 v_transposed: bool = False, prefix_pages: Optional[torch.Tensor] = None, group: int = 0,
                 max_shared: int = 0):
    """Decode attention of ``q [B, hq, d]`` against the paged cache ``[pages, 2, hkv, page_size, d]``.
    ``v_transposed`` selects the tcgen05 kernel (V slabs stored ``[d, page_size]``).

    Shared-prefix mode (tcgen05 kernel only): sequences ``[g * group, (g + 1) * group)`` form a group whose first
    ``prefix_pages[b]`` pages (int32 [B], at most ``max_shared``) are the same physical pages; they are read once
    per group instead of once per sequence. The result is the same attention over all ``seq_lens[b]`` tokens."""
    if not q.is_cuda:
        return reference.paged_decode(q, cache, block_table, seq_lens, scale, v_transposed)
    B, hq, d = q.shape
    hkv, page_size = cache.shape[2], cache.shape[3]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    dev = q.device.index if q.device.index is not None else torch.cuda.current_device()
    sms = native.num_sms(dev)
    if nsplit is None:
        if v_transposed:
            # persistent kernel: at least ~2 work items per SM, splits only when B * hkv under-fills the machine
            nsplit = max(1, min(8, (2 * sms) // max(1, B * hkv)))
        else:
            nsplit = max(1, min(16, (2 * sms) // max(1, B * hkv)))
    if out is None:
        out = torch.empty_like(q)
    if nsplit > 1 and scratch is None:
        scratch = torch.empty(B * hq * nsplit * (d + 2), dtype=torch.float32, device=q.device)
    qc = _c(q)
    if v_transposed and prefix_pages is not None and group > 1 and max_shared > 0 and group * (hq // hkv) <= 128:
        need = B * hq * (max_shared + nsplit) * (d + 2)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        st = native.status_word(q.device)
        native.check(native.lib().b200_paged_decode_prefix_tc(
            native.ptr(qc), native.ptr(cache), cache.shape[0], native.ptr(block_table), native.ptr(seq_lens),
            native.ptr(out), native.ptr(scratch), B, hq, hkv, d, page_size, block_table.shape[1], nsplit, scale,
            native.ptr(prefix_pages), group, max_shared, native.ptr(st), sms, native.stream()), "paged_decode_prefix_tc")
        return out
    if v_transposed:
        st = native.status_word(q.device)
        native.check(native.lib().b200_paged_decode_tc(
            native.ptr(qc), native.ptr(cache), cache.shape[0], native.ptr(block_table), native.ptr(seq_lens),
            native.ptr(out), native.ptr(scratch), B, hq, hkv, d, page_size, block_table.shape[1], nsplit, scale,
            native.ptr(st), sms, native.stream()), "paged_decode_tc")
        return out
    native.check(native.lib().b200_paged_decode(native.ptr(qc), native.ptr(cache), native.ptr(block_table),
                                                native.ptr(seq_lens), native.ptr(out), native.ptr(scratch), B, hq,
                                                hkv, d, page_size, block_table.shape[1], nsplit, scale,
                                                native.stream()), "paged_decode")
    return out


# --------------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperature=None, top_p=None, top_k=None, seed: int = 0, offset: int = 0,
           generator: Optional[torch.Generator] = None, offset_dev: Optional[torch.Tensor] = None,
           out_tokens: Optional[torch.Tensor] = None, out_logprobs: Optional[torch.Tensor] = None):
    """Returns ``(tokens [B] int64, logprobs [B] fp32)``; per-row ``temperature/top_p`` fp32 and ``top_k`` int32."""
    if not logits.is_cuda:
        return reference.sample(logits, temperature, top_p, top_k, generator)
    B, V = logits.shape
    assert logits.stride(-1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    toks = out_tokens if out_tokens is not None else torch.empty(B, dtype=torch.int64, device=logits.device)
    lps = out_logprobs if out_logprobs is not None else torch.empty(B, dtype=torch.float32, device=logits.device)
    native.check(native.lib().b200_sample(native.ptr(logits), 1 if logits.dtype == torch.bfloat16 else 0,
                                          logits.stride(0), B, V, native.ptr(temperature), native.ptr(top_p),
                                          native.ptr(top_k), seed & (2 ** 64 - 1), offset & (2 ** 64 - 1),
                                          native.ptr(offset_dev), native.ptr(toks), native.ptr(lps), native.stream()), "sample")
    return toks, lps


# --------------------------------------------------------------------------------------------------
# fp8 block quantisation
# --------------------------------------------------------------------------------------------------
def quant_fp8_block(w: torch.Tensor, block_rows: int = 128):
    """bf16 ``[R, C]`` -> (e4m3 ``[R, C]``, fp32 scales ``[ceil(R/block_rows), ceil(C/128)]``)."""
    if not w.is_cuda:
        return reference.quant_fp8_block(w, block_rows, 128)
    R, C = w.shape
    assert w.stride(-1) == 1 and w.dtype == torch.bfloat16
    q = torch.empty(R, C, dtype=torch.float8_e4m3fn, device=w.device)
    scales = torch.empty((R + block_rows - 1) // block_rows, (C + 127) // 128, dtype=torch.float32, device=w.device)
    native.check(native.lib().b200_quant_fp8_block(native.ptr(w), w.stride(0), native.ptr(q), q.stride(0),
                                                   native.ptr(scales), R, C, block_rows, native.stream()),
                 "quant_fp8_block")
    return q, scales


def gemm_fp8_block(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(aq * sa) @ (bq * sb)^T`` with aq [M, K] e4m3 + 1x128 scales [M, K/128] and bq [N, K] e4m3 + 128x128
    scales [N/128, K/128]; fp32 accumulation with per-k-block promotion, bf16 result."""
    if not aq.is_cuda:
        a = reference.dequant_fp8_block(aq, sa, 1, 128)
        b = reference.dequant_fp8_block(bq, sb, 128, 128)
        return (a @ b.t()).to(torch.bfloat16)
    M, K = aq.shape
    N = bq.shape[0]
    assert aq.stride(-1) == 1 and bq.stride(-1) == 1 and sa.stride(-1) == 1 and sb.stride(-1) == 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    st = native.status_word(aq.device)
    dev = aq.device.index if aq.device.index is not None else torch.cuda.current_device()
    native.check(native.lib().b200_gemm_fp8_block(native.ptr(aq), native.ptr(sa), native.ptr(bq), native.ptr(sb),
                                                  native.ptr(out), M, N, K, aq.stride(0), bq.stride(0), out.stride(0),
                                                  sa.stride(0), sb.stride(0), native.ptr(st), native.num_sms(dev),
                                                  native.stream()), "gemm_fp8_block")
    return out


def fp8_linear(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor) -> torch.Tensor:
    """Inference linear layer on block-scaled fp8 weights: the activation is quantised 1x128 on the fly."""
    xq, xs = quant_fp8_block(x.contiguous(), 1)
    return gemm_fp8_block(xq, xs, wq, ws)


class _Fp8TrainLinear(torch.autograd.Function):
    """``y = x @ w^T`` with all three GEMMs of the layer on the block-scaled fp8 kernel: activations and output
    gradients are quantised 1 x 128 along the contraction axis of the GEMM they enter, weights (and the second
    operand of the weight-gradient GEMM) 128 x 128. bf16 copies of x and w are what is saved, so memory matches bf16
    training (train.fp8: cosmos_rl/utils/fp8/fp8_util.py:139-153 does this through torchao row-wise scaling)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        xq, xs = quant_fp8_block(x.contiguous(), 1)
        wq, ws = quant_fp8_block(w.contiguous(), 128)
        return gemm_fp8_block(xq, xs, wq, ws).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gq, gs = quant_fp8_block(gy, 1)                           # along N
            wtq, wts = quant_fp8_block(w.t().contiguous(), 128)       # [K, N]
            gx = gemm_fp8_block(gq, gs, wtq, wts).to(x.dtype)
        if ctx.needs_input_grad[1]:
            if x.shape[0] % 16 == 0:
                gtq, gts = quant_fp8_block(gy.t().contiguous(), 1)    # [N, M], along the token axis
                xtq, xts = quant_fp8_block(x.t().contiguous(), 128)   # [K, M]
                gw = gemm_fp8_block(gtq, gts, xtq, xts).to(w.dtype)
            else:                                                     # ragged token count: 16-byte rows are needed
                gw = gy.t() @ x
        return gx, gw


def fp8_train_supported(w: torch.Tensor) -> bool:
    """Both dimensions of the weight are contraction axes of one of the three GEMMs: they must give 16-byte rows."""
    return w.dim() == 2 and w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0


def linear_maybe_fp8(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w^T + b``. A weight that carries block-scaled fp8 data (``w._fp8 = (e4m3 [N, K], scales)``, attached
    by the rollout's fp8 weight store) is used through the fp8 GEMM in inference; a weight marked ``_fp8_train`` (by
    the trainer, ``train.fp8.enable_fp8``) runs forward and both backward GEMMs in fp8; everything else runs this
    library's bf16 tcgen05 GEMM (forward, dgrad and wgrad; ``linear_tc``)."""
    if getattr(w, "_fp8_train", False) and x.dtype in (torch.bfloat16, torch.float32):
        y = _Fp8TrainLinear.apply(x.reshape(-1, x.shape[-1]), w).view(*x.shape[:-1], w.shape[0])
        return y if b is None else y + b
    f8 = getattr(w, "_fp8", None)
    if f8 is not None and x.is_cuda and not torch.is_grad_enabled() and x.dtype == torch.bfloat16:
        y = fp8_linear(x.reshape(-1, x.shape[-1]), f8[0], f8[1]).view(*x.shape[:-1], f8[0].shape[0])
        return y if b is None else y + b
    return linear_tc(x, w, b)


# --------------------------------------------------------------------------------------------------
# microscaling fp4 (weights of mxfp4-served experts: cosmos_rl/rollout/vllm_rollout/monkey_patch_for_mxfp4.py)
# --------------------------------------------------------------------------------------------------
def mxfp4_scale_bytes(R: int, C: int, swizzle: bool) -> int:
    return ((R + 127) // 128) * ((C // 32 + 3) // 4) * 512 if swizzle else R * (C // 32)


def quant_mxfp4(w: torch.Tensor, swizzle: bool = False):
    """bf16 ``[R, C]`` -> (packed E2M1 ``[R, C/2]`` uint8, E8M0 scale bytes). ``swizzle`` stores the scales in the
    128 x 4 tile interleaving of block-scaled tensor-core MMA; otherwise row-major ``[R, C/32]``."""
    if not w.is_cuda:
        return reference.quant_mxfp4(w, swizzle)
    R, C = w.shape
    assert w.dtype == torch.bfloat16 and w.stride(-1) == 1 and C % 32 == 0
    q = torch.empty(R, C // 2, dtype=torch.uint8, device=w.device)
    sf = torch.zeros(mxfp4_scale_bytes(R, C, swizzle), dtype=torch.uint8, device=w.device)
    native.check(native.lib().b200_quant_mxfp4(native.ptr(w), w.stride(0), native.ptr(q), native.ptr(sf), R, C,
                                               1 if swizzle else 0, native.stream()), "quant_mxfp4")
    return q, sf


def dequant_mxfp4(q: torch.Tensor, sf: torch.Tensor, swizzle: bool = False) -> torch.Tensor:
    if not q.is_cuda:
        return reference.dequant_mxfp4(q, sf, swizzle)
    R, C = q.shape[0], q.shape[1] * 2
    out = torch.empty(R, C, dtype=torch.bfloat16, device=q.device)
    native.check(native.lib().b200_dequant_mxfp4(native.ptr(q), native.ptr(sf), native.ptr(out), out.stride(0), R, C,
                                                 1 if swizzle else 0, native.stream()), "dequant_mxfp4")
    return out
