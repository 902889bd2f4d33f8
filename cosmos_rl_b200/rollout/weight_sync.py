"""Policy -> rollout weight synchronisation transports.

``PeerWeightSync`` is the product path: the rollout rank maps the policy ranks' flat parameter buffers
(CUDA IPC over NVLink) and ONE kernel pulls every rectangle of the resharding plan straight into the
engine's own layout, optionally quantising to 128x128 block-scaled fp8 on the way
(``csrc/reshard.cu``). ``CollectiveWeightSync`` moves the same rectangles with point-to-point
send/recv of ``torch.distributed`` (NCCL on GPUs, gloo on CPU): it is the statement of what the reference
does (cosmos_rl/policy/worker/rl_worker.py:419-571, cosmos_rl/rollout/worker/rollout_control.py:674-1413),
kept as the measured baseline, for CPU runs and for replicas on different nodes.
"""
from __future__ import annotations

import ctypes
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import native
from ..parallel.reshard import merge_descriptors

TILE = 128


class PeerWeightSync:
    def __init__(self, dst_flat: torch.Tensor, plan: List[List[int]], src_ptrs: Dict[int, int],
                 fp8_dst: Optional[torch.Tensor] = None, fp8_scales: Optional[torch.Tensor] = None):
        """``plan`` rows: [src_rank, src_off, src_ld, dst_off, dst_ld, rows, cols] (elements of bf16)."""
        self.device = dst_flat.device
        self.dst = dst_flat
        plan = merge_descriptors(plan)
        self.n = len(plan)
        self.bytes = sum(d[5] * d[6] for d in plan) * 2
        descs = (native.CopyDesc * self.n)()
        prefix = []
        tiles = 0
        esz = dst_flat.element_size()
        base = dst_flat.data_ptr()
        for i, (src_rank, so, sld, do, dld, rows, cols) in enumerate(plan):
            descs[i].src = src_ptrs[src_rank] + so * esz
            descs[i].dst = base + do * esz
            descs[i].dst_scale = None
            descs[i].src_ld, descs[i].dst_ld = sld, dld
            descs[i].rows, descs[i].cols = rows, cols
            descs[i].ld_scale, descs[i].quant = 0, 0
            prefix.append(tiles)
            tiles += ((rows + TILE - 1) // TILE) * ((cols + TILE - 1) // TILE)
        self.total_tiles = tiles
        raw = bytes(descs)
        self.descs_dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)
        self.prefix_dev = torch.tensor(prefix, dtype=torch.int32, device=self.device)

    def pull(self) -> None:
        """Enqueue the pull on the current stream. The caller guarantees (control-plane handshake) that the
        source buffers hold the version to fetch and are not rewritten before the kernel has finished."""
        st = native.status_word(self.device)
        native.check(native.lib().b200_reshard_pull(self.descs_dev.data_ptr(), self.prefix_dev.data_ptr(), self.n,
                                                    self.total_tiles, st.data_ptr(), native.stream()),
                     "reshard_pull")


class CollectiveWeightSync:
    """Rectangle-by-rectangle send/recv over a process group that spans the policy and rollout ranks."""

    def __init__(self, group: Optional[dist.ProcessGroup], rank_map_policy: Dict[int, int],
                 rank_map_rollout: Dict[int, int], transfer_dtype: Optional[torch.dtype] = None, batch: int = 64):
        self.group = group
        self.pmap, self.rmap = rank_map_policy, rank_map_rollout   # replica-local rank -> rank in `group`
        self.transfer_dtype = transfer_dtype
        self.batch = batch

    @staticmethod
    def _view(flat: torch.Tensor, off: int, ld: int, rows: int, cols: int) -> torch.Tensor:
        return torch.as_strided(flat, (rows, cols), (ld, 1), storage_offset=flat.storage_offset() + off)

    def send(self, flat: torch.Tensor, send_plan: List[List[Any]]) -> None:
        """``send_plan`` rows: [dst_rank, [src_rank, src_off, src_ld, dst_off, dst_ld, rows, cols]]."""
        ops, keep = [], []
        for dst_rank, d in send_plan:
            t = self._view(flat, d[1], d[2], d[5], d[6]).contiguous()
            if self.transfer_dtype is not None:
                t = t.to(self.transfer_dtype)
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self.rmap[dst_rank], group=self.group))
            if len(ops) >= self.batch:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
                ops, keep = [], []
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def recv(self, flat: torch.Tensor, recv_plan: List[List[int]]) -> None:
        ops, pending = [], []

        def flush():
            nonlocal ops, pending
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
                for buf, d in pending:
                    self._view(flat, d[3], d[4], d[5], d[6]).copy_(buf)
            ops, pending = [], []

        for d in recv_plan:
            dt = self.transfer_dtype or flat.dtype
            buf = torch.empty(d[5], d[6], dtype=dt, device=flat.device)
            pending.append((buf, d))
            ops.append(dist.P2POp(dist.irecv, buf, self.pmap[d[0]], group=self.group))
            if len(ops) >= self.batch:
                flush()
        flush()
