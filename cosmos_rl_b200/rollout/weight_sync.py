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
from ..parallel.reshard import interleave_sources, merge_descriptors

TILE = 128


class Fp8WeightStore:
    """Block-scaled fp8 copies of the rollout model's linear weights (the reference re-quantises after the
    sync, cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:989-999; here the sync kernel writes them directly).

    ``q`` mirrors the element offsets of the bf16 flat buffer (one byte per element); ``scales`` holds one fp32 per
    128 x 128 block of every quantised matrix, row-major ``[N / 128, K / 128]``. Quantised: 2-D parameters with
    both dimensions multiples of 128, except embeddings and the output head (kept in bf16, as fp8 serving stacks do).
    ``attach`` hangs ``_fp8`` views on the parameters; ``ops.functional.linear_maybe_fp8`` picks them up."""

    def __init__(self, flat, skip=("embed", "lm_head")):
        self.flat = flat
        dev = flat.device
        self.q = torch.zeros(flat.total, dtype=torch.uint8, device=dev)
        self.table = []           # (offset, N, K, scale_offset), sorted by offset
        n_scales = 0
        for s in flat.slots:
            if len(s.shape) == 2 and s.shape[0] % TILE == 0 and s.shape[1] % TILE == 0 \
                    and not any(k in s.name for k in skip):
                self.table.append((s.offset, s.shape[0], s.shape[1], n_scales, s.name))
                n_scales += (s.shape[0] // TILE) * (s.shape[1] // TILE)
        self.table.sort()
        self._offsets = [t[0] for t in self.table]
        self.scales = torch.zeros(max(n_scales, 1), dtype=torch.float32, device=dev)

    def lookup(self, dst_off: int):
        """The quantised matrix that contains flat offset ``dst_off`` (or None)."""
        import bisect
        i = bisect.bisect_right(self._offsets, dst_off) - 1
        if i < 0:
            return None
        off, N, K, so, _ = self.table[i]
        return (off, N, K, so) if dst_off < off + N * K else None

    def views(self, entry):
        off, N, K, so = entry[:4]
        q = self.q[off:off + N * K].view(torch.float8_e4m3fn).view(N, K)
        return q, self.scales[so:so + (N // TILE) * (K // TILE)].view(N // TILE, K // TILE)

    def attach(self, module) -> int:
        by_name = dict(module.named_parameters())
        for e in self.table:
            by_name[e[4]]._fp8 = self.views(e)
        return len(self.table)

    def quantize_local(self) -> None:
        """Quantise from the bf16 flat buffer (weights that arrived by another route: checkpoint, collectives)."""
        from ..ops import functional as F
        for e in self.table:
            off, N, K = e[0], e[1], e[2]
            q, sc = F.quant_fp8_block(self.flat.data[off:off + N * K].view(N, K), TILE)
            qv, sv = self.views(e)
            qv.copy_(q)
            sv.copy_(sc)


class PeerWeightSync:
    def __init__(self, dst_flat: torch.Tensor, plan: List[List[int]], src_ptrs: Dict[int, int],
                 fp8: Optional[Fp8WeightStore] = None, dst_rank: int = 0):
        """``plan`` rows: [src_rank, src_off, src_ld, dst_off, dst_ld, rows, cols] (elements of bf16). With an
        ``fp8`` store, rectangles that land block-aligned inside a quantised matrix are written as e4m3 + scales by
        the same kernel pass (their bf16 copy is not refreshed); the rest stays bf16."""
        self.device = dst_flat.device
        self.dst = dst_flat
        plan = merge_descriptors(plan) if fp8 is None else [list(d) for d in plan]
        plan = interleave_sources(plan, first=dst_rank)     # every source at once, pullers staggered
        self.n = len(plan)
        self.n_quant = 0
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
            ent = fp8.lookup(do) if fp8 is not None else None
            if ent is not None:
                off, N, K, sc_off = ent
                r0, c0 = divmod(do - off, K)
                aligned = (dld == K and r0 % TILE == 0 and c0 % TILE == 0 and r0 + rows <= N and c0 + cols <= K
                           and (rows % TILE == 0 or r0 + rows == N) and (cols % TILE == 0 or c0 + cols == K))
                if not aligned:
                    raise ValueError(f"weight-sync rectangle at flat offset {do} is not 128-aligned inside its "
                                     f"{N}x{K} matrix: cannot be quantised in flight")
                descs[i].dst = fp8.q.data_ptr() + do
                descs[i].dst_scale = fp8.scales.data_ptr() + 4 * (sc_off + (r0 // TILE) * (K // TILE) + c0 // TILE)
                descs[i].ld_scale, descs[i].quant = K // TILE, 1
                self.n_quant += 1
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
        """``send_plan`` rows: [dst_rank, [src_rank, src_off, src_ld, dst_off, dst_ld, rows, cols]], the rectangles of
        one destination in the order of that destination's plan.

        Every group of point-to-point operations is matched by a group of the same composition on the other side:
        a sender walks the destinations in rank order and sends each one's rectangles in chunks of ``batch``; a
        receiver walks the sources in rank order and posts the receives of each in the same chunks. Groups of unequal
        composition on the two sides (receives from several sources in one group against sends to one destination)
        stalled on four GPUs."""
        by_dst: Dict[int, List[Any]] = {}
        for dst_rank, d in send_plan:
            by_dst.setdefault(dst_rank, []).append(d)
        for dst_rank in sorted(by_dst):
            rects = by_dst[dst_rank]
            for i in range(0, len(rects), self.batch):
                ops, keep = [], []
                for d in rects[i:i + self.batch]:
                    t = self._view(flat, d[1], d[2], d[5], d[6]).contiguous()
                    if self.transfer_dtype is not None:
                        t = t.to(self.transfer_dtype)
                    keep.append(t)
                    ops.append(dist.P2POp(dist.isend, t, self.rmap[dst_rank], group=self.group))
                for w in dist.batch_isend_irecv(ops):
                    w.wait()

    def recv(self, flat: torch.Tensor, recv_plan: List[List[int]]) -> None:
        by_src: Dict[int, List[List[int]]] = {}
        for d in recv_plan:
            by_src.setdefault(d[0], []).append(d)
        dt = self.transfer_dtype or flat.dtype
        for src in sorted(by_src):
            rects = by_src[src]
            for i in range(0, len(rects), self.batch):
                chunk = rects[i:i + self.batch]
                bufs = [torch.empty(d[5], d[6], dtype=dt, device=flat.device) for d in chunk]
                ops = [dist.P2POp(dist.irecv, b, self.pmap[src], group=self.group) for b in bufs]
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
                for b, d in zip(bufs, chunk):
                    self._view(flat, d[3], d[4], d[5], d[6]).copy_(b)
