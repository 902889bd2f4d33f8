"""Padded -> packed ("varlen") conversion and token-balanced mini-batching
(cosmos_rl/utils/sequence_packing.py:22-399, cosmos_rl/utils/balance_seqlen.py:24-260)."""
from __future__ import annotations

import heapq
from typing import Any, Dict, List, Sequence, Tuple

import torch


def pack_sequences(seqs: Sequence[Sequence[int]], masks: Sequence[Sequence[int]], device=None,
                   pad_multiple: int = 1) -> Dict[str, Any]:
    """Concatenate token sequences. Returns input_ids [T], position_ids [T], cu_seqlens [B+1] (int32),
    max_seqlen, label_ids [T] (next token, -100 where not scored), seq_ids [T]."""
    ids: List[int] = []
    pos: List[int] = []
    labels: List[int] = []
    seq_ids: List[int] = []
    cu = [0]
    max_len = 0
    for si, (s, m) in enumerate(zip(seqs, masks)):
        n = len(s)
        ids.extend(s)
        pos.extend(range(n))
        # label for position i is token i+1 when mask[i] is set
        labels.extend([(s[i + 1] if (i + 1 < n and m[i]) else -100) for i in range(n)])
        seq_ids.extend([si] * n)
        pad = (-n) % pad_multiple
        if pad:
            ids.extend([0] * pad)
            pos.extend(range(n, n + pad))
            labels.extend([-100] * pad)
            seq_ids.extend([si] * pad)
        cu.append(len(ids))
        max_len = max(max_len, n + pad)
    t = lambda x, dt: torch.tensor(x, dtype=dt, device=device)
    return {"input_ids": t(ids, torch.long), "position_ids": t(pos, torch.long),
            "cu_seqlens": t(cu, torch.int32), "max_seqlen": max_len, "label_ids": t(labels, torch.long),
            "seq_ids": t(seq_ids, torch.long)}


def shard_packed(b: Dict[str, Any], cp: int, rank: int, zigzag: bool = False) -> Dict[str, Any]:
    """This context-parallel rank's part of a packed batch (sequences padded to multiples of ``cp``, or of ``2 cp`` for
    the zig-zag layout): chunk ``rank`` of every sequence (zig-zag: chunks ``rank`` and ``2 cp - 1 - rank``) for the
    token-wise tensors, local ``cu_seqlens`` / ``max_seqlen``; position ids stay global."""
    from ..parallel.context_parallel import local_cu_seqlens, split_for_cp
    out = dict(b)
    for k in ("input_ids", "position_ids", "label_ids", "seq_ids"):
        out[k] = split_for_cp(b[k], b["cu_seqlens"], cp, rank, zigzag)
    out["cu_seqlens"] = local_cu_seqlens(b["cu_seqlens"], cp)
    out["max_seqlen"] = b["max_seqlen"] // cp
    out["cu_seqlens_full"] = b["cu_seqlens"]
    return out


def padded_to_packed(input_ids: torch.Tensor, masks: torch.Tensor, seq_lens: Sequence[int]) -> Dict[str, Any]:
    seqs = [input_ids[i, :n].tolist() for i, n in enumerate(seq_lens)]
    ms = [masks[i, :n].tolist() for i, n in enumerate(seq_lens)]
    return pack_sequences(seqs, ms, device=input_ids.device)


def karmarkar_karp(lengths: Sequence[int], k: int, equal_size: bool = False) -> List[List[int]]:
    """Partition item indices into ``k`` groups with near-equal total length (largest differencing method)."""
    if k <= 1:
        return [list(range(len(lengths)))]
    # state: (-(max-min), counter, [ (sum, [idx...]) * k ])
    heap = []
    cnt = 0
    for i, L in sorted(enumerate(lengths), key=lambda x: -x[1]):
        parts = [(0, [])] * (k - 1) + [(L, [i])]
        heapq.heappush(heap, (-L, cnt, parts))
        cnt += 1
    while len(heap) > 1:
        d1, _, p1 = heapq.heappop(heap)
        d2, _, p2 = heapq.heappop(heap)
        p1 = sorted(p1, key=lambda x: x[0])
        p2 = sorted(p2, key=lambda x: -x[0])
        merged = [(a[0] + b[0], a[1] + b[1]) for a, b in zip(p1, p2)]
        spread = max(m[0] for m in merged) - min(m[0] for m in merged)
        heapq.heappush(heap, (-spread, cnt, merged))
        cnt += 1
    return [sorted(p[1]) for p in heap[0][2]]


def token_budget_batches(lengths: Sequence[int], max_tokens: int) -> List[List[int]]:
    """Greedy first-fit-decreasing into mini-batches of at most ``max_tokens`` tokens (each holds >= 1 item)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[Tuple[int, List[int]]] = []
    for i in order:
        L = lengths[i]
        for b in range(len(bins)):
            if bins[b][0] + L <= max_tokens:
                bins[b] = (bins[b][0] + L, bins[b][1] + [i])
                break
        else:
            bins.append((L, [i]))
    return [sorted(b[1]) for b in bins]
