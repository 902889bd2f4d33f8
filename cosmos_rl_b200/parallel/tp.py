"""Tensor parallelism of the dense decoder: column-parallel qkv / gate_up, row-parallel o / down,
vocabulary-parallel embedding and lm_head (plan of cosmos_rl/policy/model/gpt/parallelize.py:233-340).

The collectives here are the NCCL (library) statements; the fused sm_100a GEMM + all-reduce / reduce-scatter
kernel (``tp_fused.FusedTP``) replaces them for row-parallel projections once ``attach_fused`` has been called.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _F():
    from ..ops import functional
    return functional


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _AllGatherLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world):
        ctx.group, ctx.world = group, world
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        r = dist.get_rank(ctx.group)
        return g.chunk(ctx.world, dim=-1)[r].contiguous(), None, None


def _gather_rows(x: torch.Tensor, group, world: int) -> torch.Tensor:
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def _reduce_scatter_rows(x: torch.Tensor, group, world: int, rank: int) -> torch.Tensor:
    """Sum over ranks, keep this rank's block of rows. NCCL has the collective; gloo takes all-reduce + slice."""
    x = x.contiguous()
    n = x.shape[0] // world
    if x.is_cuda:
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    dist.all_reduce(x, group=group)
    return x[rank * n:(rank + 1) * n].clone()


class _GatherRows(torch.autograd.Function):
    """Sequence shards -> full sequence. What follows is computed identically on every rank (or reduces its own
    gradient, as the vocabulary-parallel log-prob does), so the backward pass just takes this rank's rows."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _gather_rows(x, tp.group, tp.size)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        n = g.shape[0] // tp.size
        return g[tp.rank * n:(tp.rank + 1) * n].contiguous(), None


class _ScatterRowsSum(torch.autograd.Function):
    """Partial sums over the full sequence -> summed rows of this rank (embedding output); backward all-gathers."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _reduce_scatter_rows(x, tp.group, tp.size, tp.rank)

    @staticmethod
    def backward(ctx, g):
        return _gather_rows(g, ctx.tp.group, ctx.tp.size), None


class _GatherGemm(torch.autograd.Function):
    """Column-parallel projection on a sequence-sharded input: ``Y = gather(x) @ w^T`` with x [T/tp, K], w [N/tp, K].
    Forward and the input gradient (``dx = reduce_scatter(dY @ w)``) run the fused all-gather -> GEMM and
    GEMM -> reduce-scatter kernels when attached; the weight gradient re-gathers x (cheaper than keeping the gathered
    activations of every layer alive)."""

    @staticmethod
    def forward(ctx, x, w, tp):
        ctx.tp = tp
        ag = tp.fused_ag
        if ag is not None and x.is_cuda and x.dtype == torch.bfloat16 and ag.fits(x.shape[0] * tp.size, x.shape[1]):
            ctx.kept = False
            ctx.save_for_backward(x, w)
            return ag.gemm(x.contiguous(), w)
        xg = _gather_rows(x, tp.group, tp.size)
        # keeping the gathered rows for the weight gradient saves an all-gather in backward (communication then equals
        # the plain tensor-parallel plan); dropping them keeps only T / tp rows alive per projection
        ctx.kept = bool(tp.keep_gathered)
        ctx.save_for_backward(xg if ctx.kept else x, w)
        return _F().mm_nt(xg, w)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        gy = gy.contiguous()
        f = tp.fused
        if (f is not None and gy.is_cuda and gy.dtype == torch.bfloat16 and gy.shape[0] % (128 * tp.size) == 0
                and f.fits(gy.shape[0], w.shape[1], 1)):
            gx = f.gemm_reduce_scatter(gy, w.t().contiguous())
        else:
            gx = _reduce_scatter_rows(_F().mm_nn(gy, w), tp.group, tp.size, tp.rank)
        gw = _F().mm_tn(gy, x if ctx.kept else _gather_rows(x, tp.group, tp.size), out_dtype=w.dtype)
        return gx, gw, None


class _GemmScatter(torch.autograd.Function):
    """Row-parallel projection back to sequence shards: ``y = reduce_scatter(x @ w^T)`` with x [T, K/tp], w [N, K/tp];
    the input gradient is ``gather(dy) @ w`` (fused all-gather -> GEMM), the weight gradient ``gather(dy)^T x``."""

    @staticmethod
    def forward(ctx, x, w, tp):
        ctx.tp = tp
        ctx.save_for_backward(x, w)
        f = tp.fused
        if (f is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] % (128 * tp.size) == 0
                and f.fits(x.shape[0], w.shape[0], 1)):
            return f.gemm_reduce_scatter(x.contiguous(), w)
        return _reduce_scatter_rows(_F().mm_nt(x, w), tp.group, tp.size, tp.rank)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        gy = gy.contiguous()
        ag = tp.fused_ag
        gy_full = _gather_rows(gy, tp.group, tp.size)
        if ag is not None and gy.is_cuda and gy.dtype == torch.bfloat16 and ag.fits(gy.shape[0] * tp.size, gy.shape[1]):
            gx = ag.gemm(gy, w.t().contiguous())
        else:
            gx = _F().mm_nn(gy_full, w)
        return gx, _F().mm_tn(gy_full, x, out_dtype=w.dtype), None


class TensorParallel:
    def __init__(self, group: dist.ProcessGroup, size: int, rank: int, fused=None):
        self.group, self.size, self.rank = group, size, rank
        self.fused = fused
        self.fused_ag = None
        self.fused_min_rows = 4096
        # sequence parallelism: the residual stream, norms and dropout-free elementwise work hold T/tp rows per rank;
        # column-parallel projections gather the sequence, row-parallel ones scatter it again
        # (cosmos_rl/policy/model/gpt/parallelize.py:244-327)
        self.sequence_parallel = False
        self.keep_gathered = True          # sequence parallelism: keep gathered inputs for the weight gradients

    # ------------------------------------------------------------------ sequence-parallel building blocks
    def row_multiple(self, cuda: bool) -> int:
        """Token counts are padded to a multiple of this (the fused kernels work on 128-row blocks per rank)."""
        return self.size * (128 if cuda and (self.fused is not None or self.fused_ag is not None) else 1)

    def col_linear(self, x, w, b=None):
        """Column-parallel projection; ``x`` is a sequence shard in sequence-parallel mode, replicated otherwise."""
        if self.sequence_parallel:
            y = _GatherGemm.apply(x, w, self)
            return y if b is None else y + b
        if torch.is_grad_enabled():
            x = self.copy_to_region(x)
        from ..ops.functional import linear_maybe_fp8
        return linear_maybe_fp8(x, w, b)

    def gather_rows(self, x):
        return _GatherRows.apply(x, self)

    def scatter_rows_sum(self, x):
        return _ScatterRowsSum.apply(x, self)

    def shared_weight(self, w):
        """A replicated weight applied to this rank's sequence shard only: its gradient is summed over the ranks."""
        return self.copy_to_region(w) if (self.sequence_parallel and torch.is_grad_enabled()) else w

    def copy_to_region(self, x):
        return _CopyToTP.apply(x, self.group)

    def reduce_output(self, x):
        """Sum the partial outputs of a row-parallel projection."""
        return _AllReduce.apply(x, self.group)

    def row_linear(self, x, w):
        """Row-parallel projection + reduction. Inference on GPU with a peer-memory context attached runs the
        fused tcgen05 GEMM + all-reduce kernel; otherwise a GEMM followed by the library all-reduce."""
        if self.sequence_parallel:
            return _GemmScatter.apply(x, w, self)
        f = self.fused
        # below ~4k rows the projection is launch/latency bound and the library pair is faster (measured
        # crossover on 2 GPUs between 2048 and 8192 rows); prefill and training shapes take the fused kernel
        if (f is not None and x.is_cuda and not torch.is_grad_enabled() and x.dtype == torch.bfloat16
                and getattr(w, "_fp8", None) is None
                and x.dim() == 2 and x.shape[0] >= self.fused_min_rows and f.fits(x.shape[0], w.shape[0])):
            return f.gemm_all_reduce(x.contiguous(), w)
        from ..ops.functional import linear_maybe_fp8
        return _AllReduce.apply(linear_maybe_fp8(x, w), self.group)

    def attach_fused(self, device, max_rows: int, max_cols: int, all_gather_k: int = 0) -> None:
        """``all_gather_k`` > 0 also attaches the all-gather -> GEMM workspace (inner dimension up to that size),
        which the sequence-parallel training plan uses."""
        from .tp_fused import FusedAllGatherGemm, FusedTP
        self.fused = FusedTP(self.group, self.size, self.rank, device, max_rows, max_cols)
        if all_gather_k > 0:
            rows = (max_rows + 128 * self.size - 1) // (128 * self.size) * (128 * self.size)
            self.fused_ag = FusedAllGatherGemm(self.group, self.size, self.rank, device, rows, all_gather_k)

    def gather_vocab(self, logits_local):
        return _AllGatherLast.apply(logits_local, self.group, self.size)

    def vocab_parallel_embed(self, input_ids, weight_local):
        v_local = weight_local.shape[0]
        lo = self.rank * v_local
        mask = (input_ids >= lo) & (input_ids < lo + v_local)
        local = torch.where(mask, input_ids - lo, torch.zeros_like(input_ids))
        out = torch.nn.functional.embedding(local, weight_local) * mask.unsqueeze(-1).to(weight_local.dtype)
        if self.sequence_parallel:
            return self.scatter_rows_sum(out)
        return _AllReduce.apply(out, self.group)

    def vocab_parallel_logprob(self, hidden, weight_local, labels, temperature: float = 1.0):
        """Log-prob / entropy with the vocabulary sharded over TP ranks: each rank runs the fused kernel on
        its vocabulary slice and the (max, sum) statistics are combined across ranks."""
        from ..ops import functional as F
        v_local = weight_local.shape[0]
        lo = self.rank * v_local
        in_range = (labels >= lo) & (labels < lo + v_local)
        local_labels = torch.where(in_range, labels - lo, torch.full_like(labels, -100))
        hidden = self.copy_to_region(hidden)
        logits = F.linear_tc(hidden, weight_local).float() / temperature
        m_local = logits.max(dim=-1).values.detach()
        m = m_local.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
        ex = torch.exp(logits - m[:, None])
        s = _AllReduce.apply(ex.sum(-1), self.group)
        lse = m + torch.log(s)
        z = logits.gather(-1, local_labels.clamp_min(0)[:, None]).squeeze(-1) * in_range.float()
        z = _AllReduce.apply(z, self.group)
        pz = _AllReduce.apply((ex * logits).sum(-1), self.group) / s
        lp = torch.where(labels >= 0, z - lse, torch.zeros_like(z))
        return lp, lse - pz
