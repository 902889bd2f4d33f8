"""Mixture-of-experts layer ops: router, permutation, grouped expert GEMMs, weighted combine.

``moe_experts`` is the differentiable expert computation
``out[t] = sum_j prob[t, j] * down_e( silu(gate_e(x_t)) * up_e(x_t) )`` over the top-k experts ``e = idx[t, j]``.
On CUDA it runs the sm_100a kernels (``csrc/moe.cu``, ``csrc/grouped_gemm.cu``): tokens are sorted by expert
into a buffer whose expert blocks start on multiples of 128 rows, the three grouped GEMM forms (forward,
dgrad, wgrad) run on the tcgen05 pipeline, and no step needs a host synchronisation. On CPU the same math is
a per-expert loop in PyTorch (also the test oracle); semantics of cosmos_rl/policy/kernel/moe/moe.py:147-284.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as tF

from . import functional as F
from . import native

ALIGN = 128


# --------------------------------------------------------------------------------------------------
# reference statements (CPU path and oracle)
# --------------------------------------------------------------------------------------------------
def route_topk_reference(logits: torch.Tensor, k: int, renorm: bool = True):
    p = torch.softmax(logits.float(), dim=-1)
    topv, topi = torch.topk(p, k, dim=-1)
    if renorm:
        topv = topv / topv.sum(-1, keepdim=True)
    return topv, topi.to(torch.int32)


def moe_experts_reference(x, probs, idx, w_gate_up, w_down):
    """x [T, H], probs/idx [T, k], w_gate_up [E, 2I, H], w_down [E, H, I]."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w_gate_up.shape[0]
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = tF.linear(x[tok].float(), w_gate_up[e].float())
        g, u = h.chunk(2, dim=-1)
        y = tF.linear(tF.silu(g) * u, w_down[e].float())
        out.index_add_(0, tok, y * probs[tok, slot].float()[:, None])
    return out.to(x.dtype)


# --------------------------------------------------------------------------------------------------
# CUDA path
# --------------------------------------------------------------------------------------------------
def route_topk(logits: torch.Tensor, k: int, renorm: bool = True, counts: Optional[torch.Tensor] = None):
    """Softmax + top-k of router logits ``[T, E]``; returns (probs [T, k] fp32, idx [T, k] int32). On CUDA the
    per-expert histogram is accumulated into ``counts`` (int32 [E], pre-zeroed) in the same kernel."""
    if not logits.is_cuda:
        pv, pi = route_topk_reference(logits, k, renorm)
        if counts is not None:
            counts += torch.bincount(pi.flatten().long(), minlength=counts.numel()).to(counts.dtype)
        return pv, pi
    T, E = logits.shape
    lg = logits.float().contiguous()
    probs = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    native.check(native.lib().b200_moe_route_topk(native.ptr(lg), T, E, k, int(renorm), native.ptr(probs),
                                                  native.ptr(idx), native.ptr(counts), native.stream()), "moe_route")
    return probs, idx


class _Dispatch:
    """Device-side description of one permutation (no host reads)."""

    def __init__(self, idx: torch.Tensor, E: int, counts: Optional[torch.Tensor] = None):
        T, k = idx.shape
        dev = idx.device
        self.T, self.k, self.E = T, k, E
        self.max_rows = (T * k + E * (ALIGN - 1)) // ALIGN * ALIGN + ALIGN
        self.max_tiles = self.max_rows // ALIGN
        if counts is None:
            counts = torch.zeros(E, dtype=torch.int32, device=dev)
            counts.index_add_(0, idx.flatten().long(), torch.ones(T * k, dtype=torch.int32, device=dev))
        self.counts = counts
        self.offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        self.tile_expert = torch.zeros(self.max_tiles, dtype=torch.int32, device=dev)
        self.n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        self.cursor = torch.empty(E, dtype=torch.int32, device=dev)
        self.row_map = torch.empty(T, k, dtype=torch.int32, device=dev)
        native.check(native.lib().b200_moe_offsets(native.ptr(counts), E, native.ptr(self.offsets),
                                                   native.ptr(self.tile_expert), native.ptr(self.n_tiles),
                                                   native.ptr(self.cursor), self.max_tiles, native.stream()),
                     "moe_offsets")


def _grouped(x, w, disp: _Dispatch, mode: int, n_out: int) -> torch.Tensor:
    K = x.shape[1]
    y = torch.empty(disp.max_rows, n_out, dtype=torch.bfloat16, device=x.device)
    st = native.status_word(x.device)
    dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
    native.check(native.lib().b200_grouped_gemm(native.ptr(x), native.ptr(w), native.ptr(y), disp.max_rows, n_out, K,
                                                disp.E, x.stride(0), y.stride(0), native.ptr(disp.tile_expert),
                                                native.ptr(disp.n_tiles), mode, 0, native.ptr(st),
                                                native.num_sms(dev), native.stream()), "grouped_gemm")
    return y


def _grouped_wgrad(dy, x, disp: _Dispatch, out: torch.Tensor, accumulate: bool) -> None:
    st = native.status_word(x.device)
    dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
    native.check(native.lib().b200_grouped_wgrad(native.ptr(dy), native.ptr(x), native.ptr(out), disp.max_rows,
                                                 dy.shape[1], x.shape[1], disp.E, dy.stride(0), x.stride(0),
                                                 native.ptr(disp.offsets), 1 if out.dtype == torch.float32 else 0,
                                                 int(accumulate), native.ptr(st), native.num_sms(dev),
                                                 native.stream()), "grouped_wgrad")


class _MoEExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, idx, w_gate_up, w_down, counts):
        T, H = x.shape
        E, I2, _ = w_gate_up.shape
        I = I2 // 2
        k = idx.shape[1]
        L = native.lib()
        disp = _Dispatch(idx, E, counts)
        xp = torch.zeros(disp.max_rows, H, dtype=torch.bfloat16, device=x.device)
        native.check(L.b200_moe_permute(native.ptr(x.contiguous()), native.ptr(idx), native.ptr(disp.offsets),
                                        native.ptr(disp.cursor), native.ptr(disp.row_map), native.ptr(xp), T, k, H,
                                        native.stream()), "moe_permute")
        h1 = _grouped(xp, w_gate_up, disp, 0, I2)
        act = F.swiglu(h1)
        y = _grouped(act, w_down, disp, 0, H)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        probs = probs.float().contiguous()
        native.check(L.b200_moe_combine(native.ptr(y), native.ptr(probs), native.ptr(disp.row_map), native.ptr(out), T,
                                        k, H, native.stream()), "moe_combine")
        ctx.save_for_backward(xp, h1, y, probs, w_gate_up, w_down)
        ctx.disp = disp
        return out

    @staticmethod
    def backward(ctx, dout):
        xp, h1, y, probs, w_gate_up, w_down = ctx.saved_tensors
        disp = ctx.disp
        T, k, E = disp.T, disp.k, disp.E
        H = xp.shape[1]
        I2 = h1.shape[1]
        L = native.lib()
        dout = dout.contiguous()
        dprob = torch.empty(T, k, dtype=torch.float32, device=dout.device)
        native.check(L.b200_moe_combine_dprob(native.ptr(dout), native.ptr(y), native.ptr(disp.row_map),
                                              native.ptr(dprob), T, k, H, native.stream()), "moe_dprob")
        dy = torch.zeros(disp.max_rows, H, dtype=torch.bfloat16, device=dout.device)
        native.check(L.b200_moe_scatter_scaled(native.ptr(dout), native.ptr(probs), native.ptr(disp.row_map),
                                               native.ptr(dy), T, k, H, native.stream()), "moe_scatter")
        act = F.swiglu(h1)                                  # recomputed: cheaper than keeping [Mp, I] alive
        dact = _grouped(dy, w_down, disp, 1, I2 // 2)       # dY . W_down[e]   (W_down [E, H, I])
        dw_down = torch.empty_like(w_down)
        _grouped_wgrad(dy, act, disp, dw_down, False)
        dh1 = torch.empty_like(h1)
        native.check(L.b200_swiglu_bwd(native.ptr(dact), native.ptr(h1), native.ptr(dh1), h1.shape[0], I2 // 2,
                                       native.stream()), "swiglu_bwd")
        dxp = _grouped(dh1, w_gate_up, disp, 1, H)          # dH1 . W_gu[e]     (W_gu [E, 2I, H])
        dw_gu = torch.empty_like(w_gate_up)
        _grouped_wgrad(dh1, xp, disp, dw_gu, False)
        dx = torch.empty(T, H, dtype=torch.bfloat16, device=dout.device)
        native.check(L.b200_moe_combine(native.ptr(dxp), None, native.ptr(disp.row_map), native.ptr(dx), T, k, H,
                                        native.stream()), "moe_unpermute")
        return dx, dprob, None, dw_gu, dw_down, None


def moe_experts(x: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.is_cuda:
        return _MoEExperts.apply(x, probs, idx, w_gate_up, w_down, counts)
    return moe_experts_reference(x, probs, idx, w_gate_up, w_down)


# ---------------------------------------------------------------------------------------------- index utilities
def indices_to_multihot(idx: torch.Tensor, probs: torch.Tensor, n_experts: int):
    """Top-k ``idx [T, k]`` / ``probs [T, k]`` -> dense ``(mask [T, E] bool, weights [T, E])``; negative indices are
    padding (the layout dense dispatchers take; cosmos_rl/policy/kernel/megatron_moe/fused_indices_converter.py:24-178)."""
    T = idx.shape[0]
    valid = idx >= 0
    safe = idx.clamp_min(0).long()
    mask = torch.zeros(T, n_experts, dtype=torch.bool, device=idx.device)
    w = torch.zeros(T, n_experts, dtype=probs.dtype, device=idx.device)
    rows = torch.arange(T, device=idx.device)[:, None].expand_as(safe)
    mask[rows[valid], safe[valid]] = True
    w[rows[valid], safe[valid]] = probs[valid]
    return mask, w


def multihot_to_indices(mask: torch.Tensor, weights: torch.Tensor, k: int):
    """Inverse of ``indices_to_multihot``: ``(idx [T, k] int32, probs [T, k])`` in ascending expert order, padded
    with -1 / 0 for tokens routed to fewer than k experts."""
    T, E = mask.shape
    order = torch.where(mask, torch.arange(E, device=mask.device)[None, :], torch.full_like(mask, E, dtype=torch.long))
    pos = order.sort(dim=1).values[:, :k]
    valid = pos < E
    idx = torch.where(valid, pos, torch.full_like(pos, -1)).to(torch.int32)
    probs = torch.where(valid, weights.gather(1, pos.clamp_max(E - 1)), torch.zeros_like(weights[:, :k]))
    return idx, probs


def fill_indices(tokens_per_expert_group: torch.Tensor, experts_per_rank: int, ep_size: int,
                 max_len: Optional[int] = None) -> torch.Tensor:
    """Permutation that turns rows received in (source rank, local expert) order into (local expert, source rank)
    order, i.e. groups each local expert's tokens together for the grouped GEMM.
    ``tokens_per_expert_group[r * experts_per_rank + e]`` = rows rank r sent for local expert e. Returns the source
    row of every output row (-1 beyond the total when ``max_len`` pads); the reference builds it with a Triton kernel,
    cosmos_rl/policy/kernel/moe/indices.py:25-111."""
    counts = tokens_per_expert_group.view(ep_size, experts_per_rank).long()
    starts = (counts.flatten().cumsum(0) - counts.flatten()).view(ep_size, experts_per_rank)
    pieces = []
    for e in range(experts_per_rank):
        for r in range(ep_size):
            n = int(counts[r, e])
            if n:
                pieces.append(torch.arange(n, device=counts.device) + starts[r, e])
    out = torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.long, device=counts.device)
    if max_len is not None and max_len > out.numel():
        out = torch.cat([out, torch.full((max_len - out.numel(),), -1, dtype=torch.long, device=counts.device)])
    return out
