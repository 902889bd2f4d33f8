"""Expert-parallel token exchange over NVLink peer memory (``csrc/a2av.cu``).

``PeerAllToAll.exchange`` has the semantics of ``dist.all_to_all_single`` with split sizes for 2-D row tensors:
rows sorted by destination rank go out, rows sorted by source rank come back. Every rank owns a receive ring of two
sets (a peer can be one exchange ahead, never two: finishing exchange k+1 needs this rank's rows of k+1, which are
pushed after this rank finished exchange k) and two arrival counters. The split-size matrix travels as a small
object collective (the library path needs the same host-side sizes); the payload never touches a library collective.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import native
from .peer import PeerBuffer, PeerMapping, flag_wait

_HEADER = 256


class PeerAllToAll:
    def __init__(self, group, size: int, rank: int, device: torch.device, max_rows: int, row_bytes: int,
                 wait_s: float = 10.0):
        assert 1 <= size <= 8 and row_bytes % 16 == 0
        self.group, self.size, self.rank, self.device = group, size, rank, device
        self.max_rows, self.row_bytes = max_rows, row_bytes
        self.set_bytes = max_rows * row_bytes
        self.nbytes = _HEADER + 2 * self.set_bytes
        self.wait_ns = int(wait_s * 1e9)
        self.buf = PeerBuffer(self.nbytes, device)            # zero-filled: both counters start at 0
        torch.cuda.synchronize(device)
        handles: List[Optional[bytes]] = [None] * size
        dist.all_gather_object(handles, self.buf.export(), group=group)
        self.maps, self.bases = [], []
        for r, h in enumerate(handles):
            if r == rank:
                self.maps.append(None)
                self.bases.append(self.buf.ptr)
            else:
                m = PeerMapping(h, self.nbytes, device)
                self.maps.append(m)
                self.bases.append(m.ptr)
        self.calls = 0
        self._local = self.buf.tensor(torch.uint8)
        self._flags = self._local[:8].view(torch.int32)       # two uint32 arrival counters
        L = native.lib()
        L.b200_a2av_push.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                     ctypes.c_void_p]
        L.b200_a2av_push.restype = ctypes.c_int
        dist.barrier(group=group)

    def exchange(self, x: torch.Tensor, send_counts: Sequence[int], count_matrix: Sequence[Sequence[int]]
                 ) -> torch.Tensor:
        """``x [sum(send_counts), H]`` sorted by destination; ``count_matrix[s][d]`` = rows rank s sends to rank d
        (identical on every rank). Returns the received rows ``[sum_s count_matrix[s][rank], H]`` sorted by source."""
        ep, me = self.size, self.rank
        assert x.dim() == 2 and x.stride(1) == 1 and x.shape[1] * x.element_size() == self.row_bytes
        recv_rows = sum(count_matrix[s][me] for s in range(ep))
        if recv_rows > self.max_rows:
            raise ValueError(f"all-to-all receives {recv_rows} rows, the ring holds {self.max_rows}")
        st = self.calls & 1
        self.calls += 1
        off = [0]
        for d in range(ep):
            off.append(off[-1] + int(send_counts[d]))
        send_off = (ctypes.c_int * (ep + 1))(*off)
        dst_ptrs = (ctypes.c_void_p * ep)(*[b + _HEADER + st * self.set_bytes for b in self.bases])
        flag_ptrs = (ctypes.c_void_p * ep)(*[b + 4 * st for b in self.bases])
        dst_row = (ctypes.c_longlong * ep)(*[sum(count_matrix[s][d] for s in range(me)) for d in range(ep)])
        native.check(native.lib().b200_a2av_push(native.ptr(x), x.stride(0) * x.element_size(), self.row_bytes, ep,
                                                 send_off, dst_ptrs, dst_row, self.row_bytes, flag_ptrs,
                                                 native.stream()), "a2av_push")
        flag = self._flags[st:st + 1]
        if recv_rows > 0:
            flag_wait(flag.data_ptr(), recv_rows, self.device, self.wait_ns / 1e9)
        out = self._local[_HEADER + st * self.set_bytes:_HEADER + st * self.set_bytes + recv_rows * self.row_bytes] \
            .view(x.dtype).view(recv_rows, x.shape[1]).clone()      # the ring is reused two exchanges later
        flag.zero_()                                                # re-arm (stream ordered, before my next push)
        return out

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for m in self.maps:
            if m is not None:
                m.close()
        self.buf.free()
