"""Expert-parallel MoE forward with the token dispatch fused into the first grouped expert GEMM (``csrc/ep_gemm.cu``).

Inference / rollout path (no autograd). Nothing on the host depends on the routing result: buffers have fixed
capacities, the split sizes stay on the device (one small ``all_gather_into_tensor`` of the per-expert counts), the
layout is computed by a device kernel, and arrival is signalled through counters in peer memory. The library path
(``MoEFeedForward._forward_ep``) needs a host read of the split sizes on every layer.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native
from .peer import PeerBuffer, PeerMapping, flag_wait

_HEADER = 256
ALIGN = 128


class FusedEPForward:
    def __init__(self, group, ep: int, rank: int, device: torch.device, n_experts: int, hidden: int,
                 max_tokens: int, top_k: int, wait_s: float = 10.0):
        assert 1 <= ep <= 8 and n_experts % ep == 0 and hidden % 8 == 0
        self.group, self.ep, self.rank, self.device = group, ep, rank, device
        self.E, self.El, self.H, self.k = n_experts, n_experts // ep, hidden, top_k
        self.max_send = max_tokens * top_k
        self.max_recv = ((ep * self.max_send + self.El * (ALIGN - 1)) // ALIGN + 1) * ALIGN
        self.max_tiles = self.max_recv // ALIGN
        self.flag_bytes = 256 + ((self.max_tiles * 4 + 255) // 256) * 256     # return counter, then block counters
        self.recv_bytes = self.max_recv * hidden * 2
        self.ret_bytes = ((self.max_send * hidden * 2 + 255) // 256) * 256
        self.set_bytes = self.flag_bytes + self.recv_bytes + self.ret_bytes
        self.nbytes = _HEADER + 2 * self.set_bytes
        self.wait_s = wait_s
        self.buf = PeerBuffer(self.nbytes, device)
        torch.cuda.synchronize(device)
        handles: List[Optional[bytes]] = [None] * ep
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
        self.local = self.buf.tensor(torch.uint8)
        i32 = dict(dtype=torch.int32, device=device)
        self.counts_all = torch.zeros(ep * self.E, **i32)
        self.send_off = torch.zeros(self.E + 1, **i32)
        self.dst_base = torch.zeros(self.E, **i32)
        self.ret_base = torch.zeros(ep * self.E, **i32)
        self.block_start = torch.zeros(self.El + 1, **i32)
        self.tile_expert = torch.zeros(self.max_tiles, **i32)
        self.block_target = torch.zeros(self.max_tiles, **i32)
        self.n_tiles = torch.zeros(1, **i32)
        self.calls = 0
        L = native.lib()
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        L.b200_ep_layout.argtypes = [vp, ci, ci, ci, ci] + [vp] * 7 + [vp]
        L.b200_ep_dispatch_gemm.argtypes = [vp, cl, vp, vp, cl, ci, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp,
                                            ctypes.c_ulonglong, vp, ci, vp]
        L.b200_ep_combine_push.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]
        for n in ("b200_ep_layout", "b200_ep_dispatch_gemm", "b200_ep_combine_push"):
            getattr(L, n).restype = ci
        dist.barrier(group=group)

    def _set_view(self, st: int):
        base = _HEADER + st * self.set_bytes
        flags = self.local[base:base + self.flag_bytes]
        ret = self.local[base + self.flag_bytes + self.recv_bytes:base + self.set_bytes]
        return flags, ret

    @torch.no_grad()
    def forward(self, x: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor) -> torch.Tensor:
        """x [T, H] bf16, probs / idx [T, k]; w_gate_up [El, 2I, H], w_down [El, H, I] (this rank's experts)."""
        T, H = x.shape
        k, ep, E = idx.shape[1], self.ep, self.E
        assert H == self.H and T * k <= self.max_send and x.dtype == torch.bfloat16
        L, dev = native.lib(), self.device
        st = self.calls & 1
        self.calls += 1
        flat_e = idx.flatten().long()
        order = torch.argsort(flat_e, stable=True)
        tok = order // k
        send_x = x[tok]                                                     # sorted by global expert
        mine = torch.bincount(flat_e, minlength=E).to(torch.int32)
        dist.all_gather_into_tensor(self.counts_all, mine, group=self.group)
        native.check(L.b200_ep_layout(native.ptr(self.counts_all), ep, E, self.rank, self.max_tiles,
                                      native.ptr(self.send_off), native.ptr(self.dst_base), native.ptr(self.ret_base),
                                      native.ptr(self.block_start), native.ptr(self.tile_expert),
                                      native.ptr(self.block_target), native.ptr(self.n_tiles), native.stream()),
                     "ep_layout")
        set_base = [b + _HEADER + st * self.set_bytes for b in self.bases]
        VP = ctypes.c_void_p * ep
        blk_flags = VP(*[b + 256 for b in set_base])                        # first 256 bytes: the return counter
        recv_ptrs = VP(*[b + self.flag_bytes for b in set_base])
        ret_ptrs = VP(*[b + self.flag_bytes + self.recv_bytes for b in set_base])
        ret_flags = VP(*set_base)
        I2 = w_gate_up.shape[1]
        y1 = torch.empty(self.max_recv, I2, dtype=torch.bfloat16, device=dev)
        status = native.status_word(dev)
        di = dev.index if dev.index is not None else torch.cuda.current_device()
        native.check(L.b200_ep_dispatch_gemm(
            native.ptr(send_x), send_x.stride(0), native.ptr(w_gate_up), native.ptr(y1), y1.stride(0), self.max_recv,
            I2, H, E, ep, self.rank, native.ptr(self.send_off), native.ptr(self.dst_base), recv_ptrs, blk_flags,
            native.ptr(self.tile_expert), native.ptr(self.block_target), native.ptr(self.n_tiles),
            int(self.wait_s * 1e9), native.ptr(status), native.num_sms(di), native.stream()), "ep_dispatch_gemm")
        act = F.swiglu(y1)
        y2 = torch.empty(self.max_recv, H, dtype=torch.bfloat16, device=dev)
        native.check(L.b200_grouped_gemm(native.ptr(act), native.ptr(w_down), native.ptr(y2), self.max_recv, H,
                                         act.shape[1], self.El, act.stride(0), y2.stride(0),
                                         native.ptr(self.tile_expert), native.ptr(self.n_tiles), 0, 0,
                                         native.ptr(status), native.num_sms(di), native.stream()), "grouped_gemm")
        native.check(L.b200_ep_combine_push(native.ptr(y2), H, E, ep, self.rank, native.ptr(self.counts_all),
                                            native.ptr(self.block_start), native.ptr(self.ret_base), ret_ptrs,
                                            ret_flags, native.stream()), "ep_combine_push")
        flags, ret = self._set_view(st)
        flag_wait(flags.data_ptr(), T * k, dev, self.wait_s)                # every copy of my tokens is back
        back = ret[:T * k * H * 2].view(torch.bfloat16).view(T * k, H)
        w = probs.flatten()[order].to(back.dtype)[:, None]
        out = torch.zeros(T, H, dtype=back.dtype, device=dev).index_add_(0, tok, back * w)   # as the library path
        flags.zero_()                                                       # re-arm this set (reused two calls later)
        return out

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for m in self.maps:
            if m is not None:
                m.close()
        self.buf.free()
