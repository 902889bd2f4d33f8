"""Flat parameter / gradient storage.

Every parameter of a model is a view into ONE contiguous buffer per dtype role (bf16 compute weights,
gradients), with each tensor starting on a 256-byte boundary. One buffer means: one fused AdamW launch for
the whole model, one reduce-scatter / all-gather (or one fused peer-memory kernel) per step for data
parallelism, rectangle descriptors for weight sync that all point into the same allocation (which is what
gets IPC-mapped into the rollout processes), and no per-parameter launch overheads anywhere. This replaces
the per-parameter DTensor bookkeeping of FSDP2 in the reference (cosmos_rl/policy/model/gpt/parallelize.py:366-423).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

ALIGN_ELEMS = 128  # 256 bytes of bf16


@dataclass
class FlatSlot:
    name: str
    offset: int
    numel: int
    shape: Tuple[int, ...]


class FlatParams:
    """Rebinds ``module``'s parameters (and their ``.grad``) to views of flat buffers."""

    def __init__(self, module: nn.Module, dtype: torch.dtype, device: torch.device, shard_multiple: int = 1,
                 allocator: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None,
                 with_grad: bool = True, local_filter: Optional[Callable[[str], bool]] = None):
        """``local_filter(name)`` marks parameters that are NOT replicas across the data-parallel ranks (the experts
        an expert-parallel rank owns). They are laid out after everything else: ``[0, shared_total)`` is the region
        the sharded optimizer reduces and republishes, ``[shared_total, total)`` stays local to the rank."""
        self.module = module
        self.dtype = dtype
        self.device = device
        self.slots: List[FlatSlot] = []
        seen: Dict[int, int] = {}
        owners: List[List[Tuple[nn.Module, str]]] = []
        olds: List[nn.Parameter] = []
        names: List[str] = []
        for mod_name, mod in module.named_modules():
            for pname, p in list(mod._parameters.items()):
                if p is None:
                    continue
                if id(p) in seen:  # tied parameter: one slot, several owners
                    owners[seen[id(p)]].append((mod, pname))
                    continue
                full = f"{mod_name}.{pname}" if mod_name else pname
                seen[id(p)] = len(olds)
                owners.append([(mod, pname)])
                olds.append(p)
                names.append(full)
        unit = ALIGN_ELEMS * max(1, shard_multiple)
        is_local = [bool(local_filter and local_filter(n)) for n in names]
        offsets = [0] * len(names)
        off = 0
        for i, (n, p) in enumerate(zip(names, olds)):
            if not is_local[i]:
                offsets[i] = off
                off += (p.numel() + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        self.shared_total = (off + unit - 1) // unit * unit
        off = self.shared_total
        for i, (n, p) in enumerate(zip(names, olds)):
            if is_local[i]:
                offsets[i] = off
                off += (p.numel() + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        for n, p, o in zip(names, olds, offsets):
            self.slots.append(FlatSlot(n, o, p.numel(), tuple(p.shape)))
        self.total = (off + unit - 1) // unit * unit if any(is_local) else self.shared_total
        alloc = allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        self.data = alloc(self.total, dtype, device)
        self.grad = alloc(self.total, dtype, device) if with_grad else None
        params: List[Tuple[str, nn.Parameter]] = []
        with torch.no_grad():
            for name, old, slot, own in zip(names, olds, self.slots, owners):
                view = self.data[slot.offset: slot.offset + slot.numel].view(slot.shape)
                if old.device.type != "meta":
                    view.copy_(old.data.to(dtype))
                # a fresh Parameter object (a meta parameter cannot be re-pointed at real storage)
                new = nn.Parameter(view, requires_grad=old.requires_grad)
                for mod, pname in own:
                    mod._parameters[pname] = new
                if with_grad and new.requires_grad:
                    new.grad = self.grad[slot.offset: slot.offset + slot.numel].view(slot.shape)
                params.append((name, new))
        self.params = params
        self.by_name = {s.name: s for s in self.slots}

    def view(self, name: str, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        s = self.by_name[name]
        b = self.data if buf is None else buf
        return b[s.offset: s.offset + s.numel].view(s.shape)

    def zero_grad(self) -> None:
        if self.grad is not None:
            self.grad.zero_()
            # autograd may have replaced .grad objects (e.g. after set_to_none); rebind
            for (name, p), slot in zip(self.params, self.slots):
                if p.requires_grad and (p.grad is None or p.grad.data_ptr() !=
                                        self.grad.data_ptr() + slot.offset * self.grad.element_size()):
                    p.grad = self.grad[slot.offset: slot.offset + slot.numel].view(slot.shape)

    def shard_range(self, rank: int, world: int) -> Tuple[int, int]:
        """This rank's slice of the replicated region (the rank-local tail is never sharded)."""
        per = self.shared_total // world
        return rank * per, (rank + 1) * per

    def trainable_mask(self) -> Optional[torch.Tensor]:
        """1.0 for elements of trainable parameters (None if everything is trainable)."""
        if all(p.requires_grad for _, p in self.params):
            return None
        mask = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        for (name, p), slot in zip(self.params, self.slots):
            if p.requires_grad:
                mask[slot.offset: slot.offset + slot.numel] = 1.0
        return mask
