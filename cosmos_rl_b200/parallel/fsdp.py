"""Peer-memory data parallelism for the flat optimizer (``csrc/fsdp_fused.cu``).

``PeerCollective`` is handed to :class:`cosmos_rl_b200.policy.optim.FlatAdamW`; it replaces the NCCL
reduce-scatter / all-gather pair by two fused kernels that read peers' gradients and write peers' weights
through NVLink. The ranks exchange the IPC handles of their flat buffers once, at construction.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native
from .flat import FlatParams
from .peer import PeerMapping


class PeerCollective:
    def __init__(self, flat: FlatParams, group: dist.ProcessGroup, object_group: Optional[dist.ProcessGroup] = None):
        self.flat = flat
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = flat.device
        data_buf = getattr(flat.data, "_peer_buffer", None)
        grad_buf = getattr(flat.grad, "_peer_buffer", None)
        if data_buf is None or grad_buf is None:
            raise RuntimeError("PeerCollective needs FlatParams allocated with parallel.peer.peer_allocator")
        mine = {"data": data_buf.export(), "grad": grad_buf.export(), "nbytes": data_buf.nbytes}
        everyone: List[dict] = [None] * self.world
        dist.all_gather_object(everyone, mine, group=object_group or group)
        self.maps: List[PeerMapping] = []
        data_ptrs, grad_ptrs = [], []
        for r, h in enumerate(everyone):
            if r == self.rank:
                data_ptrs.append(flat.data.data_ptr())
                grad_ptrs.append(flat.grad.data_ptr())
            else:
                md = PeerMapping(h["data"], h["nbytes"], self.device)
                mg = PeerMapping(h["grad"], h["nbytes"], self.device)
                self.maps += [md, mg]
                data_ptrs.append(md.ptr)
                grad_ptrs.append(mg.ptr)
        VP = ctypes.c_void_p * self.world
        self.data_ptrs = VP(*data_ptrs)
        self.grad_ptrs = VP(*grad_ptrs)
        self._token = torch.zeros(1, device=self.device)
        L = native.lib()
        L.b200_reduce_scatter_sumsq.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p]
        L.b200_adamw_publish.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                                                                ctypes.c_longlong] + [ctypes.c_float] * 7 + \
                                        [ctypes.c_void_p, ctypes.c_void_p]
        L.b200_reduce_scatter_sumsq.restype = ctypes.c_int
        L.b200_adamw_publish.restype = ctypes.c_int

    def stream_barrier(self) -> None:
        """Stream-ordered barrier: when it completes on this rank's stream, every rank's earlier work on its
        stream has completed."""
        dist.all_reduce(self._token, group=self.group)

    def reduce_scatter_sumsq(self, lo: int, hi: int, out_shard: torch.Tensor, sumsq: torch.Tensor) -> None:
        self.stream_barrier()   # every rank's backward is complete
        native.check(native.lib().b200_reduce_scatter_sumsq(
            ctypes.cast(self.grad_ptrs, ctypes.c_void_p), self.world, lo, hi - lo, out_shard.data_ptr(),
            sumsq.data_ptr(), 1.0 / self.world, native.stream()), "reduce_scatter_sumsq")
        self.stream_barrier()   # every rank has read all gradients: they may be cleared

    def adamw_publish(self, master, m, v, grad_shard, lo: int, hi: int, *, lr, beta1, beta2, eps, weight_decay, step,
                      grad_scale: torch.Tensor) -> None:
        bias1 = 1.0 - beta1 ** step
        bias2 = 1.0 - beta2 ** step
        native.check(native.lib().b200_adamw_publish(
            master.data_ptr(), m.data_ptr(), v.data_ptr(), grad_shard.data_ptr(),
            ctypes.cast(self.data_ptrs, ctypes.c_void_p), self.world, lo, hi - lo, lr, beta1, beta2, eps,
            weight_decay, bias1, bias2, grad_scale.data_ptr(), native.stream()), "adamw_publish")
        self.stream_barrier()   # every shard has landed everywhere before the next forward

    def all_reduce_grads(self, average: bool = True) -> None:
        """In-place (averaging) all-reduce of the flat gradient buffer over peer memory: one launch per rank, each
        rank reduces and republishes its own 1/world range. Used for gradient averaging between policy replicas that
        share a box; ``torch.distributed`` all-reduce is the route between boxes."""
        n = self.flat.total
        per = (n // self.world) // 8 * 8
        lo = self.rank * per
        cnt = per if self.rank < self.world - 1 else n - lo
        self.stream_barrier()
        L = native.lib()
        L.b200_peer_all_reduce.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong,
                                           ctypes.c_float, ctypes.c_void_p]
        L.b200_peer_all_reduce.restype = ctypes.c_int
        native.check(L.b200_peer_all_reduce(ctypes.cast(self.grad_ptrs, ctypes.c_void_p), self.world, lo, cnt,
                                            1.0 / self.world if average else 1.0, native.stream()), "peer_all_reduce")
        self.stream_barrier()

    def close(self) -> None:
        for m in self.maps:
            m.close()
        self.maps = []
