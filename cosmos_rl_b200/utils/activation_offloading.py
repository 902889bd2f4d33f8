"""Activation offloading: tensors saved for backward are copied to pinned host memory on a side stream during
forward and brought back just before they are needed (cosmos_rl/utils/activation_offloading.py:32-432).
Small tensors and parameters stay on the device."""
from __future__ import annotations

import contextlib
from typing import Dict, Optional, Tuple

import torch


class OffloadActivations(torch.autograd.graph.saved_tensors_hooks):
    def __init__(self, min_bytes: int = 1 << 20, use_pinned: bool = True, params: Optional[set] = None):
        self.min_bytes = min_bytes
        self.use_pinned = use_pinned
        self.param_ptrs = params or set()
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.stash: Dict[int, Tuple[torch.Tensor, Optional[torch.cuda.Event], torch.device]] = {}
        self.next_id = 0
        self.bytes_offloaded = 0

        def pack(t: torch.Tensor):
            if (not t.is_cuda or t.numel() * t.element_size() < self.min_bytes
                    or t.untyped_storage().data_ptr() in self.param_ptrs or isinstance(t, torch.nn.Parameter)):
                return ("keep", t)
            tid = self.next_id
            self.next_id += 1
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.use_pinned)
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                host.copy_(t, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            t.record_stream(self.stream)
            self.stash[tid] = (host, ev, t.device)
            self.bytes_offloaded += t.numel() * t.element_size()
            return ("off", tid)

        def unpack(packed):
            kind, v = packed
            if kind == "keep":
                return v
            host, ev, dev = self.stash.pop(v)
            ev.synchronize()
            return host.to(dev, non_blocking=True)

        super().__init__(pack, unpack)


@contextlib.contextmanager
def maybe_offload(enabled: bool, model: Optional[torch.nn.Module] = None, min_bytes: int = 1 << 20):
    if not enabled or not torch.cuda.is_available():
        yield None
        return
    ptrs = {p.untyped_storage().data_ptr() for p in model.parameters()} if model is not None else set()
    ctx = OffloadActivations(min_bytes=min_bytes, params=ptrs)
    with ctx:
        yield ctx
