"""Tensor parallelism of the dense decoder: column-parallel qkv / gate_up, row-parallel o / down,
vocabulary-parallel embedding and lm_head (plan of cosmos_rl/policy/model/gpt/parallelize.py:233-340).

The collectives here are the NCCL (library) statements; the fused sm_100a GEMM + all-reduce / reduce-scatter
kernel (``tp_fused.FusedTP``) replaces them for row-parallel projections once ``attach_fused`` has been called.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


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


class TensorParallel:
    def __init__(self, group: dist.ProcessGroup, size: int, rank: int, fused=None):
        self.group, self.size, self.rank = group, size, rank
        self.fused = fused
        self.fused_min_rows = 4096

    def copy_to_region(self, x):
        return _CopyToTP.apply(x, self.group)

    def reduce_output(self, x):
        """Sum the partial outputs of a row-parallel projection."""
        return _AllReduce.apply(x, self.group)

    def row_linear(self, x, w):
        """Row-parallel projection + reduction. Inference on GPU with a peer-memory context attached runs the
        fused tcgen05 GEMM + all-reduce kernel; otherwise a GEMM followed by the library all-reduce."""
        f = self.fused
        # below ~4k rows the projection is launch/latency bound and the library pair is faster (measured
        # crossover on 2 GPUs between 2048 and 8192 rows); prefill and training shapes take the fused kernel
        if (f is not None and x.is_cuda and not torch.is_grad_enabled() and x.dtype == torch.bfloat16
                and getattr(w, "_fp8", None) is None
                and x.dim() == 2 and x.shape[0] >= self.fused_min_rows and f.fits(x.shape[0], w.shape[0])):
            return f.gemm_all_reduce(x.contiguous(), w)
        from ..ops.functional import linear_maybe_fp8
        return _AllReduce.apply(linear_maybe_fp8(x, w), self.group)

    def attach_fused(self, device, max_rows: int, max_cols: int) -> None:
        from .tp_fused import FusedTP
        self.fused = FusedTP(self.group, self.size, self.rank, device, max_rows, max_cols)

    def gather_vocab(self, logits_local):
        return _AllGatherLast.apply(logits_local, self.group, self.size)

    def vocab_parallel_embed(self, input_ids, weight_local):
        v_local = weight_local.shape[0]
        lo = self.rank * v_local
        mask = (input_ids >= lo) & (input_ids < lo + v_local)
        local = torch.where(mask, input_ids - lo, torch.zeros_like(input_ids))
        out = torch.nn.functional.embedding(local, weight_local) * mask.unsqueeze(-1).to(weight_local.dtype)
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
        logits = torch.nn.functional.linear(hidden, weight_local).float() / temperature
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
