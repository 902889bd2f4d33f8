"""Peer-memory context of the fused row-parallel GEMM + tensor-parallel reduction kernel (``csrc/tp_gemm.cu``).

One workspace per TP rank holds two call-counter words, the per-tile arrival counters (two sets) and the
staging slots (two sets x tp source ranks). Workspaces are exchanged as CUDA IPC handles over the TP process
group; afterwards ``gemm_all_reduce`` / ``gemm_reduce_scatter`` are single kernel launches with no library
collective (the reference's path is nn.Linear + NCCL all-reduce / reduce-scatter,
cosmos_rl/policy/model/gpt/parallelize.py:233-340).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native
from .peer import PeerBuffer, PeerMapping

_HEADER = 256


class FusedAllGatherGemm:
    """Workspace of ``csrc/ag_gemm.cu``: per rank two call-counter words, per-row-block arrival counters (two sets)
    and the gathered-activation buffer (two sets of ``max_rows x max_k`` bf16)."""

    def __init__(self, group, size: int, rank: int, device: torch.device, max_rows: int, max_k: int,
                 wait_s: float = 10.0):
        assert 1 <= size <= 8 and max_rows % (128 * size) == 0
        self.group, self.size, self.rank, self.device = group, size, rank, device
        self.max_blocks = max_rows // 128
        self.set_elems = max_rows * max_k
        self.flag_bytes = ((2 * self.max_blocks * 4 + 255) // 256) * 256
        self.nbytes = _HEADER + self.flag_bytes + 2 * self.set_elems * 2
        self.wait_ns = int(wait_s * 1e9)
        self.buf = PeerBuffer(self.nbytes, device)
        torch.cuda.synchronize(device)
        handles: List[Optional[bytes]] = [None] * size
        dist.all_gather_object(handles, self.buf.export(), group=group)
        self.maps: List[Optional[PeerMapping]] = []
        bases = []
        for r, h in enumerate(handles):
            if r == rank:
                self.maps.append(None)
                bases.append(self.buf.ptr)
            else:
                m = PeerMapping(h, self.nbytes, device)
                self.maps.append(m)
                bases.append(m.ptr)
        arr = ctypes.c_void_p * 8
        self._flags = arr(*[b + _HEADER for b in bases] + [None] * (8 - size))
        self._gathered = arr(*[b + _HEADER + self.flag_bytes for b in bases] + [None] * (8 - size))
        self._ctrl = self.buf.ptr
        dist.barrier(group=group)

    def fits(self, rows_total: int, k: int) -> bool:
        return (rows_total % (128 * self.size) == 0 and rows_total // 128 <= self.max_blocks
                and rows_total * k <= self.set_elems and k % 8 == 0)

    def gemm(self, x_local: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``gather(x) @ w^T``: x_local [M / tp, K] are this rank's rows, w [N, K]; returns [M, N] bf16."""
        assert x_local.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        assert x_local.stride(-1) == 1 and w.stride(-1) == 1
        m_local, K = x_local.shape
        M, N = m_local * self.size, w.shape[0]
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device)
        st = native.status_word(x_local.device)
        dev = x_local.device.index if x_local.device.index is not None else torch.cuda.current_device()
        native.check(native.lib().b200_ag_gemm(
            native.ptr(x_local), native.ptr(w), native.ptr(out), M, N, K, x_local.stride(0), w.stride(0),
            out.stride(0), self._gathered, self._flags, self._ctrl, self.size, self.rank, self.set_elems,
            self.max_blocks, self.wait_ns, native.ptr(st), native.num_sms(dev), native.stream()), "ag_gemm")
        return out

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for m in self.maps:
            if m is not None:
                m.close()
        self.buf.free()


class FusedTP:
    def __init__(self, group, size: int, rank: int, device: torch.device, max_rows: int, max_cols: int,
                 wait_s: float = 10.0):
        assert 1 <= size <= 8
        self.group, self.size, self.rank, self.device = group, size, rank, device
        self.max_tiles = ((max_rows + 127) // 128) * ((max_cols + 127) // 128)
        self.slot_elems = ((max_rows + 127) // 128) * 128 * max_cols
        self.flag_bytes = ((2 * self.max_tiles * 4 + 255) // 256) * 256
        self.nbytes = _HEADER + self.flag_bytes + 2 * size * self.slot_elems * 2
        self.wait_ns = int(wait_s * 1e9)
        self.buf = PeerBuffer(self.nbytes, device)          # zero-filled
        torch.cuda.synchronize(device)
        handles: List[Optional[bytes]] = [None] * size
        dist.all_gather_object(handles, self.buf.export(), group=group)
        self.maps: List[Optional[PeerMapping]] = []
        bases = []
        for r, h in enumerate(handles):
            if r == rank:
                self.maps.append(None)
                bases.append(self.buf.ptr)
            else:
                m = PeerMapping(h, self.nbytes, device)
                self.maps.append(m)
                bases.append(m.ptr)
        arr = ctypes.c_void_p * 8
        self._flags = arr(*[b + _HEADER for b in bases] + [None] * (8 - size))
        self._stage = arr(*[b + _HEADER + self.flag_bytes for b in bases] + [None] * (8 - size))
        self._ctrl = self.buf.ptr
        dist.barrier(group=group)

    @classmethod
    def with_silent_peers(cls, size: int, device: torch.device, max_rows: int, max_cols: int,
                          wait_s: float = 0.002) -> "FusedTP":
        """Rank 0 of a ``size``-rank context whose other ranks are plain buffers on the SAME GPU that nothing ever
        writes: a launch stages its tiles, waits ``wait_s`` for arrivals that never come, records the peer-flag
        timeout in the status word, frees its tensor memory and returns. Used to exercise the bounded waits on one
        GPU (no collective, no second process)."""
        self = cls.__new__(cls)
        self.group, self.size, self.rank, self.device = None, size, 0, device
        self.max_tiles = ((max_rows + 127) // 128) * ((max_cols + 127) // 128)
        self.slot_elems = ((max_rows + 127) // 128) * 128 * max_cols
        self.flag_bytes = ((2 * self.max_tiles * 4 + 255) // 256) * 256
        self.nbytes = _HEADER + self.flag_bytes + 2 * size * self.slot_elems * 2
        self.wait_ns = int(wait_s * 1e9)
        self.buf = PeerBuffer(self.nbytes, device)
        self._silent = [PeerBuffer(self.nbytes, device) for _ in range(size - 1)]
        self.maps = [None] * size
        bases = [self.buf.ptr] + [b.ptr for b in self._silent]
        arr = ctypes.c_void_p * 8
        self._flags = arr(*[b + _HEADER for b in bases] + [None] * (8 - size))
        self._stage = arr(*[b + _HEADER + self.flag_bytes for b in bases] + [None] * (8 - size))
        self._ctrl = self.buf.ptr
        torch.cuda.synchronize(device)
        return self

    def free_silent(self) -> None:
        torch.cuda.synchronize(self.device)
        for b in getattr(self, "_silent", []):
            b.free()
        self.buf.free()

    def fits(self, rows: int, cols: int, mode: int = 0) -> bool:
        r = rows if mode == 0 else rows // self.size
        return (r * cols <= self.slot_elems and cols % 8 == 0
                and ((rows + 127) // 128) * ((cols + 127) // 128) <= self.max_tiles)

    def _launch(self, a, w, out, residual, mode):
        M, K = a.shape
        N = w.shape[0]
        st = native.status_word(a.device)
        dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
        native.check(native.lib().b200_tp_gemm(
            native.ptr(a), native.ptr(w), native.ptr(out), native.ptr(residual) if residual is not None else None,
            M, N, K, a.stride(0), w.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
            self._stage, self._flags, self._ctrl, self.size, self.rank, mode, self.slot_elems, self.max_tiles,
            self.wait_ns, native.ptr(st), native.num_sms(dev), native.stream()), "tp_gemm")
        return out

    def gemm_all_reduce(self, a: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``sum_r a_r @ w_r^T (+ residual)`` on every rank; a [M, K/tp], w [N, K/tp], bf16."""
        assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(-1) == 1 and w.stride(-1) == 1
        if out is None:
            out = torch.empty(a.shape[0], w.shape[0], dtype=torch.bfloat16, device=a.device)
        return self._launch(a, w, out, residual, 0)

    def gemm_reduce_scatter(self, a: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows ``[rank * M/tp, (rank+1) * M/tp)`` of the summed product (sequence-parallel layout)."""
        assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] % (128 * self.size) == 0
        if out is None:
            out = torch.empty(a.shape[0] // self.size, w.shape[0], dtype=torch.bfloat16, device=a.device)
        return self._launch(a, w, out, residual, 1)

    def reset(self) -> None:
        """Re-arm after an error status (all ranks, between steps)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.buf.tensor(torch.uint8)[:_HEADER + self.flag_bytes].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for m in self.maps:
            if m is not None:
                m.close()
        self.buf.free()
