"""Context parallelism for packed (varlen) causal attention.

Every sequence of the packed batch is split into ``cp`` equal contiguous chunks (sequences are padded to a
multiple of ``cp`` tokens by the caller); rank ``r`` of the CP group holds chunk ``r`` of every sequence, so all
token-wise layers (norms, projections, MLP, log-probs) run on ``T / cp`` tokens without communication. Attention
is the only layer that mixes positions. Two exchanges are provided:

* ``ulysses``: all-to-all that trades the sequence split for a head split (each rank attends the full sequences
  with ``heads / cp`` heads) and back; the reference's CP mode (cosmos_rl/utils/ulysses.py:30-545). Needs the
  number of KV heads to divide by ``cp``.
* ``kv-gather``: every rank gathers the K/V chunks of the ranks before it (K/V are small under GQA) and runs ONE
  attention call whose queries are aligned to the end of the keys of their sequence; the key prefix is exactly
  what a ring schedule would stream past this rank. Gradients of the gathered K/V flow back through a
  reduce-scatter. On GPUs the attention call is the tcgen05 kernel, which takes separate query/key offsets.

* ``ring``: K/V chunks travel around the ring one hop per step (point-to-point send / receive posted before the
  attention call on the chunk that is already here, so the transfer hides behind the math); every step yields a
  partial output and its log-sum-exp, merged on the fly. Only one foreign K/V chunk is resident at a time, so the
  key length per GPU stays ``T / cp`` however long the sequences are. The backward pass runs the ring again: each
  step's dK/dV chunk is computed from the global log-sum-exp and handed on to its owner.

* ``ring-zigzag``: the ring on a balanced layout. Every sequence is cut into ``2 cp`` chunks and rank ``r`` holds
  chunks ``r`` and ``2 cp - 1 - r``; with contiguous chunks the last rank does ``cp`` times the causal work of the first
  and everybody waits for it, here every hop is one attention call of the same size on every rank.

All are autograd functions over ``torch.distributed`` collectives, so they run on NCCL and (for tests) on gloo.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import reference


def split_for_cp(x: torch.Tensor, cu_seqlens: torch.Tensor, cp: int, rank: int, zigzag: bool = False) -> torch.Tensor:
    """Rows of the packed tensor ``x [T, ...]`` that belong to ``rank``: chunk ``rank`` of every sequence. With
    ``zigzag`` every sequence is cut into ``2 cp`` chunks and the rank holds chunks ``rank`` and ``2 cp - 1 - rank``
    (in that order), which gives every rank the same share of a causal attention's work."""
    cs = cu_seqlens.tolist()
    parts = []
    for s, e in zip(cs[:-1], cs[1:]):
        if zigzag:
            n = (e - s) // (2 * cp)
            assert n * 2 * cp == e - s, "sequence lengths must be multiples of twice the CP degree"
            parts.append(x[s + rank * n:s + (rank + 1) * n])
            parts.append(x[s + (2 * cp - 1 - rank) * n:s + (2 * cp - rank) * n])
            continue
        n = (e - s) // cp
        assert n * cp == e - s, "sequence lengths must be multiples of the CP degree"
        parts.append(x[s + rank * n:s + (rank + 1) * n])
    return torch.cat(parts) if parts else x[:0]


def local_cu_seqlens(cu_seqlens: torch.Tensor, cp: int) -> torch.Tensor:
    return (cu_seqlens // cp).to(cu_seqlens.dtype)


def _attention(q, k, v, cu_q, cu_k, max_q: int, scale: Optional[float]):
    """Attention with queries aligned to the end of the keys; differentiable."""
    if q.is_cuda:
        from ..ops import attention
        if attention.native_flash_supported(q, k, v):
            return attention.flash_attention(q, k, v, cu_q, cu_k, max_q, scale)
    return reference.varlen_attention(q, k, v, cu_q, scale, True, cu_k)


# ------------------------------------------------------------------------------------------------ all-to-all
class _SeqToHead(torch.autograd.Function):
    """[T_local, H, d] (all heads, my chunk of every sequence) -> [T, H / cp, d] (my heads, whole sequences)."""

    @staticmethod
    def forward(ctx, x, cu_local, group, cp):
        ctx.group, ctx.cp = group, cp
        ctx.save_for_backward(cu_local)
        return _a2a_seq_to_head(x, cu_local, group, cp)

    @staticmethod
    def backward(ctx, g):
        (cu_local,) = ctx.saved_tensors
        return _a2a_head_to_seq(g.contiguous(), cu_local, ctx.group, ctx.cp), None, None, None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu_local, group, cp):
        ctx.group, ctx.cp = group, cp
        ctx.save_for_backward(cu_local)
        return _a2a_head_to_seq(x, cu_local, group, cp)

    @staticmethod
    def backward(ctx, g):
        (cu_local,) = ctx.saved_tensors
        return _a2a_seq_to_head(g.contiguous(), cu_local, ctx.group, ctx.cp), None, None, None


def _interleave_index(cu_local: torch.Tensor, cp: int, device) -> torch.Tensor:
    """Permutation that turns rank-major order ([rank][sequence][chunk rows]) into sequence-major order."""
    cs = cu_local.tolist()
    t_local = cs[-1]
    idx = []
    for s, e in zip(cs[:-1], cs[1:]):
        for r in range(cp):
            idx.append(torch.arange(r * t_local + s, r * t_local + e))
    return torch.cat(idx).to(device) if idx else torch.zeros(0, dtype=torch.long, device=device)


def _a2a_seq_to_head(x, cu_local, group, cp):
    t, h, d = x.shape
    assert h % cp == 0, "heads must divide by the CP degree for the all-to-all exchange"
    send = x.view(t, cp, h // cp, d).transpose(0, 1).contiguous()          # [cp (dest rank), t, h/cp, d]
    recv = torch.empty_like(send)                                            # [cp (source rank), t, h/cp, d]
    dist.all_to_all_single(recv, send, group=group)
    return recv.view(cp * t, h // cp, d)[_interleave_index(cu_local, cp, x.device)]


def _a2a_head_to_seq(x, cu_local, group, cp):
    T, hl, d = x.shape
    t = T // cp
    inv = torch.empty(T, dtype=torch.long, device=x.device)
    inv[_interleave_index(cu_local, cp, x.device)] = torch.arange(T, device=x.device)
    send = x[inv].view(cp, t, hl, d).contiguous()                            # [cp (dest = owner of the rows), t, hl, d]
    recv = torch.empty_like(send)                                            # [cp (source = owner of the heads), ...]
    dist.all_to_all_single(recv, send, group=group)
    return recv.transpose(0, 1).reshape(t, cp * hl, d)


def ulysses_attention(q, k, v, cu_local, max_local: int, group, scale: Optional[float] = None):
    cp = dist.get_world_size(group)
    qf = _SeqToHead.apply(q.contiguous(), cu_local, group, cp)
    kf = _SeqToHead.apply(k.contiguous(), cu_local, group, cp)
    vf = _SeqToHead.apply(v.contiguous(), cu_local, group, cp)
    cu_full = cu_local * cp
    o = _attention(qf, kf, vf, cu_full, cu_full, max_local * cp, scale)
    return _HeadToSeq.apply(o.contiguous(), cu_local, group, cp)


# ------------------------------------------------------------------------------------------------ KV gather
class _GatherKV(torch.autograd.Function):
    """All-gather the K (or V) chunks of the group and lay the chunks of ranks ``0 .. rank`` of every sequence
    out contiguously. Backward: scatter the gradient back to chunk order and reduce-scatter it."""

    @staticmethod
    def forward(ctx, x, cu_local, group, cp, rank):
        parts = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(parts, x.contiguous(), group=group)
        full = torch.cat(parts)                                              # rank-major
        cs = cu_local.tolist()
        t_local = cs[-1]
        idx = []
        for s, e in zip(cs[:-1], cs[1:]):
            for r in range(rank + 1):
                idx.append(torch.arange(r * t_local + s, r * t_local + e))
        idx = torch.cat(idx).to(x.device) if idx else torch.zeros(0, dtype=torch.long, device=x.device)
        ctx.group, ctx.cp, ctx.shape = group, cp, full.shape
        ctx.save_for_backward(idx)
        return full[idx]

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        full = torch.zeros(ctx.shape, dtype=g.dtype, device=g.device)
        full[idx] = g
        chunks = [c.contiguous() for c in full.chunk(ctx.cp, dim=0)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=ctx.group)
        return out, None, None, None, None


def kv_gather_attention(q, k, v, cu_local, max_local: int, group, scale: Optional[float] = None):
    cp, rank = dist.get_world_size(group), dist.get_rank(group)
    kg = _GatherKV.apply(k, cu_local, group, cp, rank)
    vg = _GatherKV.apply(v, cu_local, group, cp, rank)
    cu_k = cu_local * (rank + 1)
    return _attention(q, kg, vg, cu_local, cu_k, max_local, scale)


# ------------------------------------------------------------------------------------------------ ring
def _fwd_with_lse(q, k, v, cu, max_len: int, scale: float, causal: bool, cu_k=None):
    """(out fp32-mergeable, lse [h, T] natural log) of one chunk pair; ``cu_k`` when the keys are segmented
    differently from the queries (half chunks of the zig-zag ring; non-causal only)."""
    if q.is_cuda:
        from ..ops import attention
        if attention.native_flash_supported(q, k, v):
            i32 = lambda t: t if t.dtype == torch.int32 else t.to(torch.int32)
            return attention.flash_fwd(q, k, v, i32(cu), i32(cu if cu_k is None else cu_k), max_len, scale, causal)
    return reference.varlen_attention(q, k, v, cu, scale, causal, cu_k, return_lse=True)


def _bwd_from_lse(dout, q, k, v, out, lse, cu, max_len: int, scale: float, causal: bool, cu_k=None, max_k=None):
    """Gradients of one chunk pair given the GLOBAL output and log-sum-exp of the queries (the probabilities of this
    chunk are exp(s - lse), the softmax correction term is rowsum(dout * out) over the whole row). ``cu_k`` /
    ``max_k`` when the keys are segmented differently from the queries (non-causal only)."""
    if q.is_cuda:
        from ..ops import attention
        if attention.native_flash_supported(q, k, v):
            i32 = lambda t: t if t.dtype == torch.int32 else t.to(torch.int32)
            return attention.flash_bwd(dout, q, k, v, out, lse, i32(cu), max_len, scale,
                                       cu_k=None if cu_k is None else i32(cu_k), max_k=max_k, causal=causal)
    hq, hkv = q.shape[1], k.shape[1]
    g = hq // hkv
    dq, dk, dv = torch.zeros_like(q, dtype=torch.float32), torch.zeros_like(k, dtype=torch.float32), \
        torch.zeros_like(v, dtype=torch.float32)
    cs = cu.tolist()
    ks = cs if cu_k is None else cu_k.tolist()
    for s, e, ks0, ke0 in zip(cs[:-1], cs[1:], ks[:-1], ks[1:]):
        if e <= s or ke0 <= ks0:
            continue
        qi = q[s:e].float().transpose(0, 1)                               # [hq, L, d]
        ki = k[ks0:ke0].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vi = v[ks0:ke0].float().transpose(0, 1).repeat_interleave(g, dim=0)
        do, o = dout[s:e].float().transpose(0, 1), out[s:e].float().transpose(0, 1)
        sc = (qi @ ki.transpose(-1, -2)) * scale
        if causal:
            L = e - s
            sc = sc.masked_fill(~torch.ones(L, L, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        p = torch.exp(sc - lse[:, s:e, None])
        delta = (do * o).sum(-1, keepdim=True)
        ds = p * (do @ vi.transpose(-1, -2) - delta)
        dq[s:e] = ((ds @ ki) * scale).transpose(0, 1)
        dk[ks0:ke0] = ((ds.transpose(-1, -2) @ qi) * scale).view(hkv, g, ke0 - ks0, -1).sum(1).transpose(0, 1)
        dv[ks0:ke0] = (p.transpose(-1, -2) @ do).view(hkv, g, ke0 - ks0, -1).sum(1).transpose(0, 1)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _ring_exchange(send: torch.Tensor, group, cp: int, rank: int):
    """Post send-to-next / receive-from-previous; returns (recv buffer, requests)."""
    recv = torch.empty_like(send)
    nxt, prv = dist.get_global_rank(group, (rank + 1) % cp), dist.get_global_rank(group, (rank - 1) % cp)
    ops = [dist.P2POp(dist.isend, send, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
    return recv, dist.batch_isend_irecv(ops)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_local, max_local, group, scale):
        cp, rank = dist.get_world_size(group), dist.get_rank(group)
        d = q.shape[-1]
        scale = scale if scale is not None else d ** -0.5
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        kv = torch.stack([k, v])                                           # one message per hop
        out = lse = None
        for step in range(cp):
            src = (rank - step) % cp                                       # owner of the chunk held now
            if step < cp - 1:
                nxt_kv, reqs = _ring_exchange(kv, group, cp, rank)         # in flight during the attention below
            if src <= rank:                                                # later chunks are entirely in the future
                o_j, lse_j = _fwd_with_lse(q, kv[0], kv[1], cu_local, max_local, scale, causal=(src == rank))
                o_j = o_j.float()
                if out is None:
                    out, lse = o_j, lse_j
                else:
                    new = torch.logaddexp(lse, lse_j)
                    wa, wb = torch.exp(lse - new), torch.exp(lse_j - new)  # [h, T]
                    out = out * wa.t()[..., None] + o_j * wb.t()[..., None]
                    lse = new
            if step < cp - 1:
                for r_ in reqs:
                    r_.wait()
                kv = nxt_kv
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse, cu_local)
        ctx.group, ctx.max_local, ctx.scale = group, max_local, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_local = ctx.saved_tensors
        group = ctx.group
        cp, rank = dist.get_world_size(group), dist.get_rank(group)
        dout = dout.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack([k, v])
        dkv = torch.zeros_like(kv, dtype=torch.float32)                    # gradient of the chunk held now
        for step in range(cp):
            src = (rank - step) % cp
            if step < cp - 1:
                nxt_kv, reqs = _ring_exchange(kv, group, cp, rank)
            if src <= rank:
                dq_j, dk_j, dv_j = _bwd_from_lse(dout, q, kv[0], kv[1], out, lse, cu_local, ctx.max_local, ctx.scale,
                                                 causal=(src == rank))
                dq += dq_j.float()
                dkv[0] += dk_j.float()
                dkv[1] += dv_j.float()
            # the gradient travels with its chunk: after cp hops in total it is back at the owner
            nxt_dkv, greqs = _ring_exchange(dkv, group, cp, rank)
            if step < cp - 1:
                for r_ in reqs:
                    r_.wait()
                kv = nxt_kv
            for r_ in greqs:
                r_.wait()
            dkv = nxt_dkv
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None


def ring_attention(q, k, v, cu_local, max_local: int, group, scale: Optional[float] = None):
    return _RingAttention.apply(q, k, v, cu_local, max_local, group, scale)


# ------------------------------------------------------------------------------------------------ zig-zag ring
def _half_rows(cu_local: torch.Tensor, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row indices of the first and of the second half of every local sequence."""
    cs = cu_local.tolist()
    lo, hi = [], []
    for s, e in zip(cs[:-1], cs[1:]):
        m = (s + e) // 2
        lo.append(torch.arange(s, m))
        hi.append(torch.arange(m, e))
    cat = lambda xs: (torch.cat(xs) if xs else torch.zeros(0, dtype=torch.int64)).to(device)
    return cat(lo), cat(hi)


def _merge(out, lse, o_j, lse_j, rows=None):
    """Fold a partial result (for all rows, or for ``rows`` only) into the running output and log-sum-exp, in place
    (called inside autograd functions, where nothing is recorded)."""
    if out is None:
        return o_j.float(), lse_j
    if rows is None:
        new = torch.logaddexp(lse, lse_j)
        out.mul_(torch.exp(lse - new).t()[..., None]).add_(o_j.float() * torch.exp(lse_j - new).t()[..., None])
        return out, new
    cur_l = lse[:, rows]
    new = torch.logaddexp(cur_l, lse_j)
    upd = out[rows] * torch.exp(cur_l - new).t()[..., None] + o_j.float() * torch.exp(lse_j - new).t()[..., None]
    out.index_copy_(0, rows, upd)
    lse.index_copy_(1, rows, new)
    return out, lse


class _ZigzagRingAttention(torch.autograd.Function):
    """Ring attention on the zig-zag layout (rank r holds chunks r and 2 cp - 1 - r of every sequence). Per hop the
    chunk pair needs exactly one call of half the size of a full chunk pair on every rank: the rank's own chunks ->
    causal over the local order; chunks of an earlier rank -> all local queries against the first half of the keys;
    chunks of a later rank -> the second half of the local queries against all keys. No rank waits for another."""

    @staticmethod
    def forward(ctx, q, k, v, cu_local, max_local, group, scale):
        cp, rank = dist.get_world_size(group), dist.get_rank(group)
        scale = scale if scale is not None else q.shape[-1] ** -0.5
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        lo, hi = _half_rows(cu_local, q.device)
        cu_half = (cu_local // 2).to(cu_local.dtype)
        kv = torch.stack([k, v])
        out = lse = None
        for step in range(cp):
            src = (rank - step) % cp
            if step < cp - 1:
                nxt_kv, reqs = _ring_exchange(kv, group, cp, rank)
            if src == rank:
                o_j, l_j = _fwd_with_lse(q, kv[0], kv[1], cu_local, max_local, scale, True)
                out, lse = _merge(out, lse, o_j, l_j)
            elif src < rank:
                o_j, l_j = _fwd_with_lse(q, kv[0][lo].contiguous(), kv[1][lo].contiguous(), cu_local, max_local, scale,
                                         False, cu_k=cu_half)
                out, lse = _merge(out, lse, o_j, l_j)
            else:
                o_j, l_j = _fwd_with_lse(q[hi].contiguous(), kv[0], kv[1], cu_half, max_local // 2, scale, False,
                                         cu_k=cu_local)
                out, lse = _merge(out, lse, o_j, l_j, rows=hi)
            if step < cp - 1:
                for r_ in reqs:
                    r_.wait()
                kv = nxt_kv
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse, cu_local)
        ctx.group, ctx.max_local, ctx.scale = group, max_local, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_local = ctx.saved_tensors
        group = ctx.group
        cp, rank = dist.get_world_size(group), dist.get_rank(group)
        ml, scale = ctx.max_local, ctx.scale
        dout = dout.contiguous()
        lo, hi = _half_rows(cu_local, q.device)
        cu_half = (cu_local // 2).to(cu_local.dtype)
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack([k, v])
        dkv = torch.zeros_like(kv, dtype=torch.float32)
        for step in range(cp):
            src = (rank - step) % cp
            if step < cp - 1:
                nxt_kv, reqs = _ring_exchange(kv, group, cp, rank)
            if src == rank:
                dq_j, dk_j, dv_j = _bwd_from_lse(dout, q, kv[0], kv[1], out, lse, cu_local, ml, scale, True)
                dq += dq_j.float()
                dkv[0] += dk_j.float()
                dkv[1] += dv_j.float()
            elif src < rank:
                dq_j, dk_j, dv_j = _bwd_from_lse(dout, q, kv[0][lo].contiguous(), kv[1][lo].contiguous(), out, lse,
                                                 cu_local, ml, scale, False, cu_k=cu_half, max_k=ml // 2)
                dq += dq_j.float()
                dkv[0].index_add_(0, lo, dk_j.float())
                dkv[1].index_add_(0, lo, dv_j.float())
            else:
                dq_j, dk_j, dv_j = _bwd_from_lse(dout[hi].contiguous(), q[hi].contiguous(), kv[0], kv[1],
                                                 out[hi].contiguous(), lse[:, hi].contiguous(), cu_half, ml // 2, scale,
                                                 False, cu_k=cu_local, max_k=ml)
                dq.index_add_(0, hi, dq_j.float())
                dkv[0] += dk_j.float()
                dkv[1] += dv_j.float()
            nxt_dkv, greqs = _ring_exchange(dkv, group, cp, rank)
            if step < cp - 1:
                for r_ in reqs:
                    r_.wait()
                kv = nxt_kv
            for r_ in greqs:
                r_.wait()
            dkv = nxt_dkv
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None


def zigzag_ring_attention(q, k, v, cu_local, max_local: int, group, scale: Optional[float] = None):
    return _ZigzagRingAttention.apply(q, k, v, cu_local, max_local, group, scale)


class ContextParallel:
    """Attached to a model as ``model.cp``; the attention layer calls ``attention`` instead of the local kernel."""

    def __init__(self, group, size: int, rank: int, mode: str = "kv-gather"):
        assert mode in ("kv-gather", "ulysses", "ring", "ring-zigzag")
        self.group, self.size, self.rank, self.mode = group, size, rank, mode
        self.zigzag = mode == "ring-zigzag"
        self.seq_multiple = size * (2 if self.zigzag else 1)       # sequences are padded to multiples of this

    def attention(self, q, k, v, cu_local, max_local: int, scale: Optional[float] = None):
        fn = {"ulysses": ulysses_attention, "ring": ring_attention,
              "ring-zigzag": zigzag_ring_attention}.get(self.mode, kv_gather_attention)
        return fn(q, k, v, cu_local, max_local, self.group, scale)

    def shard(self, x, cu_seqlens):
        return split_for_cp(x, cu_seqlens, self.size, self.rank, self.zigzag)
