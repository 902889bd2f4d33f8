"""Activation offloading: tensors saved for backward are copied to pinned host memory on a side stream during
forward and brought back just before they are needed (cosmos_rl/utils/activation_offloading.py:32-432).
Small tensors and parameters stay on the device."""
from __future__ import annotations

import contextlib
from typing import Dict, Optional, Tuple

import torch


class OffloadActivations(torch.autograd.graph.saved_tensors_hooks):
    """Forward: every large saved tensor is copied to pinned host memory on a side stream (the device copy is freed
    when autograd drops it). Backward: tensors come back in (roughly) reverse order of saving, so when tensor ``i`` is
    asked for, the copies of ``i - 1 .. i - prefetch`` are already enqueued on the side stream; the consumer's stream
    waits on the copy's event, the host never blocks (the reference prefetches the same way,
    cosmos_rl/utils/activation_offloading.py:138-330)."""

    def __init__(self, min_bytes: int = 1 << 20, use_pinned: bool = True, params: Optional[set] = None,
                 prefetch: int = 2):
        self.min_bytes = min_bytes
        self.use_pinned = use_pinned
        self.param_ptrs = params or set()
        self.prefetch = max(0, int(prefetch))
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.stash: Dict[int, Tuple[torch.Tensor, torch.device]] = {}            # id -> (host copy, device)
        self.inflight: Dict[int, Tuple[torch.Tensor, torch.cuda.Event]] = {}     # id -> (device copy, ready event)
        self.next_id = 0
        self.bytes_offloaded = 0
        self.n_prefetched = 0        # fetches that were already enqueued when their tensor was asked for

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
            t.record_stream(self.stream)
            self.stash[tid] = (host, t.device)
            self.bytes_offloaded += t.numel() * t.element_size()
            return ("off", tid)

        def fetch(tid: int) -> None:
            """Enqueue the host-to-device copy of ``tid`` on the side stream (which also ran its device-to-host copy,
            so the two are ordered without any host wait)."""
            host, dev = self.stash.pop(tid)
            with torch.cuda.stream(self.stream):
                d = host.to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.inflight[tid] = (d, ev)

        def unpack(packed):
            kind, v = packed
            if kind == "keep":
                return v
            if v in self.inflight:
                self.n_prefetched += 1
            else:
                fetch(v)
            for k in range(v - 1, v - 1 - self.prefetch, -1):     # the tensors backward asks for next
                if k in self.stash:
                    fetch(k)
            d, ev = self.inflight.pop(v)
            cur = torch.cuda.current_stream()
            cur.wait_event(ev)
            d.record_stream(cur)
            return d

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
