"""Parameter-sharded data parallelism: every rank keeps 1/world of every unit of the model.

A *unit* is what is gathered together: the embedding, each transformer block, the final norm with the output
head. Persistent memory per rank is one bf16 shard of the weights, one fp32 shard of the gradients and the sharded
optimizer state; two rotating buffers hold the gathered bf16 weights of the unit that computes and of the unit
that is being fetched, two more hold their gradients. Forward gathers unit ``u + 1`` on a side stream while unit
``u`` computes; backward gathers unit ``u - 1`` while unit ``u`` computes, and reduce-scatters the gradients of a
unit as soon as its backward is over. This is the memory plan of the reference's ``fully_shard`` per block with
``reshard_after_forward`` (cosmos_rl/policy/model/gpt/parallelize.py:366-423) on a flat layout: one all-gather
and one reduce-scatter per unit, no per-parameter bookkeeping.

Unit ``u`` always lives in buffer ``u % 2``, so the parameters of a block are fixed views; only the contents of
the buffers change. Writes into the buffers go through a tensor that does not share a version counter with the
parameter views, so autograd's saved-tensor check does not object to a unit being gathered again for backward.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .flat import ALIGN_ELEMS, FlatSlot


@dataclass
class Unit:
    index: int
    base: int = 0            # offset of the unit in the concatenated (gathered) layout
    size: int = 0            # padded to world * ALIGN_ELEMS
    shard: int = 0           # size / world
    shard_off: int = 0       # offset of this rank's piece in the shard buffers
    names: List[str] = field(default_factory=list)


def default_units(module: nn.Module) -> Callable[[str], int]:
    """Unit of a parameter name for models with a ``layers`` list: sub-modules registered before the blocks are
    unit 0, block ``i`` is unit ``1 + i``, everything else (sub-modules after the blocks, parameters held by the
    model itself such as a final norm weight) is the last unit."""
    n_layers = len(getattr(module, "layers", []))
    before = []
    for child, _ in module.named_children():
        if child == "layers":
            break
        before.append(child)

    def unit_of(name: str) -> int:
        head = name.split(".")[0]
        if head == "layers":
            return 1 + int(name.split(".")[1])
        return 0 if head in before else n_layers + 1
    return unit_of


class _Begin(torch.autograd.Function):
    """Identity in front of a unit; its backward runs when the unit's backward is over."""

    @staticmethod
    def forward(ctx, sharder, u, defer, *xs):
        ctx.sharder, ctx.u, ctx.defer = sharder, u, defer
        return xs if len(xs) > 1 else xs[0]

    @staticmethod
    def backward(ctx, *gs):
        if not ctx.defer:
            ctx.sharder._reduce(ctx.u)
        return (None, None, None) + gs


class _End(torch.autograd.Function):
    """Identity behind a unit; its backward runs right before the unit's backward starts."""

    @staticmethod
    def forward(ctx, sharder, u, *xs):
        ctx.sharder, ctx.u = sharder, u
        return xs if len(xs) > 1 else xs[0]

    @staticmethod
    def backward(ctx, *gs):
        s, u = ctx.sharder, ctx.u
        s.in_backward = True
        s._wait_grad_buffer(u)
        s.ensure(u)
        if u > 0:
            s.prefetch(u - 1)
        s.dirty.add(u)
        return (None, None) + gs


class _OptimizerView:
    """What the flat AdamW needs to see: this rank's shard as if it were a whole, unsharded buffer."""

    def __init__(self, sp: "ShardedFlatParams"):
        self.sp = sp
        self.data, self.grad = sp.data, sp.grad
        self.device, self.dtype = sp.device, sp.dtype
        self.total = self.shared_total = sp.n_shard
        self.params, self.slots = [], []
        for (name, p), slot in zip(sp.params, sp.slots):
            un = sp.units[sp.unit_of_param[name]]
            a, b = slot.offset - un.base, slot.offset - un.base + slot.numel       # range inside the unit
            lo, hi = sp.rank * un.shard, (sp.rank + 1) * un.shard
            a, b = max(a, lo), min(b, hi)
            if a < b:
                self.params.append((name, p))
                self.slots.append(FlatSlot(name, un.shard_off + a - lo, b - a, (b - a,)))

    def shard_range(self, rank: int, world: int) -> Tuple[int, int]:
        return 0, self.total

    def trainable_mask(self) -> Optional[torch.Tensor]:
        if all(p.requires_grad for _, p in self.sp.params):
            return None
        mask = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        for (name, p), slot in zip(self.params, self.slots):
            if p.requires_grad:
                mask[slot.offset: slot.offset + slot.numel] = 1.0
        return mask

    def zero_grad(self) -> None:
        self.sp.zero_grad()


class ShardedFlatParams:
    sharded = True

    def __init__(self, module: nn.Module, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup], unit_of: Optional[Callable[[str], int]] = None,
                 reduce_dtype: Optional[torch.dtype] = None):
        self.module, self.dtype, self.device, self.group = module, dtype, device, group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.reduce_dtype = reduce_dtype or dtype
        unit_of = unit_of or default_units(module)
        seen: Dict[int, int] = {}
        owners: List[List[Tuple[nn.Module, str]]] = []
        olds: List[nn.Parameter] = []
        names: List[str] = []
        for mod_name, mod in module.named_modules():
            for pname, p in list(mod._parameters.items()):
                if p is None:
                    continue
                if id(p) in seen:
                    owners[seen[id(p)]].append((mod, pname))
                    continue
                seen[id(p)] = len(olds)
                owners.append([(mod, pname)])
                olds.append(p)
                names.append(f"{mod_name}.{pname}" if mod_name else pname)
        ids = [unit_of(n) for n in names]
        self.units: List[Unit] = [Unit(i) for i in range(max(ids) + 1)]
        self.unit_of_param: Dict[str, int] = dict(zip(names, ids))
        in_unit = [0] * len(names)
        for i, (n, p, u) in enumerate(zip(names, olds, ids)):
            un = self.units[u]
            in_unit[i] = un.size
            un.size += (p.numel() + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
            un.names.append(n)
        pad = ALIGN_ELEMS * self.world
        base = soff = 0
        for un in self.units:
            un.size = (un.size + pad - 1) // pad * pad
            un.shard = un.size // self.world
            un.base, un.shard_off = base, soff
            base += un.size
            soff += un.shard
        self.total = self.shared_total = base
        self.n_shard = soff
        self.max_unit = max(un.size for un in self.units)
        self.data = torch.zeros(self.n_shard, dtype=dtype, device=device)            # this rank's weights
        self.grad = torch.zeros(self.n_shard, dtype=torch.float32, device=device)    # this rank's gradients
        # gathered units: ``_w`` is written by the collectives, ``_w_params`` aliases the same memory with a version
        # counter of its own and is what the parameters are views of
        self._w = [torch.zeros(self.max_unit, dtype=dtype, device=device) for _ in range(2)]
        self._w_params = [w.data for w in self._w]
        self._g = [torch.zeros(self.max_unit, dtype=dtype, device=device) for _ in range(2)]
        self._rs_out = torch.zeros(max(un.shard for un in self.units), dtype=self.reduce_dtype, device=device)
        self.slots: List[FlatSlot] = []
        self.params: List[Tuple[str, nn.Parameter]] = []
        self._local: List[Tuple[int, int]] = []      # (buffer, offset in buffer) per parameter
        for i, (n, old, u, own) in enumerate(zip(names, olds, ids, owners)):
            if old.device.type != "meta":
                raise ValueError("the sharded layout builds from a model on the meta device; load weights afterwards")
            un = self.units[u]
            self.slots.append(FlatSlot(n, un.base + in_unit[i], old.numel(), tuple(old.shape)))
            k, o = u % 2, in_unit[i]
            new = nn.Parameter(self._w_params[k][o:o + old.numel()].view(old.shape), requires_grad=old.requires_grad)
            for mod, pname in own:
                mod._parameters[pname] = new
            self.params.append((n, new))
            self._local.append((k, o))
        self.by_name = {s.name: s for s in self.slots}
        self._bind_grads()
        self.resident: List[Optional[int]] = [None, None]
        self._pending: List[Optional[Tuple[int, object]]] = [None, None]
        self._grad_free: List[Optional[object]] = [None, None]
        self.dirty: set = set()
        self.in_backward = False
        self.cuda = device.type == "cuda"
        self.comm = torch.cuda.Stream(device) if self.cuda else None
        self.n_gathers = self.n_reduces = 0
        self._full: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ bookkeeping
    def _bind_grads(self) -> None:
        for (name, p), slot, (k, o) in zip(self.params, self.slots, self._local):
            if p.requires_grad:
                p.grad = self._g[k][o:o + slot.numel].view(slot.shape)

    def optimizer_view(self) -> _OptimizerView:
        return _OptimizerView(self)

    def shard_range(self, rank: int, world: int) -> Tuple[int, int]:
        return 0, self.n_shard

    def trainable_mask(self) -> Optional[torch.Tensor]:
        return self.optimizer_view().trainable_mask()

    def zero_grad(self) -> None:
        self.grad.zero_()
        for g in self._g:
            g.zero_()
        for (name, p), slot, (k, o) in zip(self.params, self.slots, self._local):
            if p.requires_grad and (p.grad is None or p.grad.data_ptr() != self._g[k].data_ptr() + o * self._g[k].element_size()):
                p.grad = self._g[k][o:o + slot.numel].view(slot.shape)
        self.dirty.clear()
        self.in_backward = False

    def invalidate(self) -> None:
        """The shard changed (optimizer step, checkpoint load, weights swapped): gathered copies are stale."""
        self.sync()
        self.resident = [None, None]

    # ------------------------------------------------------------------ gather / reduce
    def _shard_of(self, un: Unit, buf: torch.Tensor) -> torch.Tensor:
        return buf[un.shard_off: un.shard_off + un.shard]

    def _launch_gather(self, u: int) -> None:
        un, k = self.units[u], u % 2
        src, dst = self._shard_of(un, self.data), self._w[k][:un.size]
        if un.size == 0:
            self._pending[k] = (u, None)
            return
        self.n_gathers += 1
        if self.world == 1:
            dst.copy_(src)
            self._pending[k] = (u, None)
            return
        if not self.cuda:
            dist.all_gather_into_tensor(dst, src, group=self.group)
            self._pending[k] = (u, None)
            return
        ev = torch.cuda.Event()
        ev.record()                                   # everything that still reads buffer k is queued before this
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(ev)
            work = dist.all_gather_into_tensor(dst, src, group=self.group, async_op=True)
        self._pending[k] = (u, work)

    def prefetch(self, u: int) -> None:
        k = u % 2
        if self.resident[k] == u or (self._pending[k] is not None and self._pending[k][0] == u):
            return
        self._finish_pending(k)
        self._launch_gather(u)

    def _finish_pending(self, k: int) -> None:
        if self._pending[k] is not None:
            u, work = self._pending[k]
            if work is not None:
                work.wait()                          # the current stream waits; the host does not
            self.resident[k] = u
            self._pending[k] = None

    def ensure(self, u: int) -> None:
        k = u % 2
        if self.resident[k] == u and self._pending[k] is None:
            return
        if self._pending[k] is None or self._pending[k][0] != u:
            self._finish_pending(k)
            self._launch_gather(u)
        self._finish_pending(k)

    def _wait_grad_buffer(self, u: int) -> None:
        ev = self._grad_free[u % 2]
        if ev is not None and self.cuda:
            torch.cuda.current_stream().wait_event(ev)

    def _reduce(self, u: int) -> None:
        """Average the gradients of unit ``u`` over the ranks into this rank's fp32 shard; clear the buffer."""
        if u not in self.dirty:
            return
        self.dirty.discard(u)
        un, k = self.units[u], u % 2
        if un.size == 0:
            return
        g = self._g[k][:un.size]
        acc = self._shard_of(un, self.grad)
        self.n_reduces += 1
        if self.world == 1:
            acc.add_(g)
            g.zero_()
            return
        out = self._rs_out[:un.shard]

        def body():
            if self.reduce_dtype != g.dtype:
                dist.reduce_scatter_tensor(out, g.to(self.reduce_dtype), op=dist.ReduceOp.AVG, group=self.group)
            else:
                dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.AVG, group=self.group)
            acc.add_(out)
            g.zero_()
        if not self.cuda:
            body()
            return
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(ev)
            body()
            done = torch.cuda.Event()
            done.record()
        self._grad_free[k] = done

    def finish_backward(self) -> None:
        """After ``loss.backward()``: reduce what no hook could (units whose inputs need no gradient, such as the
        embedding) and make the compute stream wait for the side stream."""
        for u in sorted(self.dirty, reverse=True):
            self._reduce(u)
        self.in_backward = False
        self.sync()

    def sync(self) -> None:
        for k in (0, 1):
            self._finish_pending(k)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm)
        self._grad_free = [None, None]

    # ------------------------------------------------------------------ running a unit
    def run(self, u: int, fn: Callable, *xs: torch.Tensor, defer_reduce: bool = False):
        """``fn(*xs)`` with unit ``u`` gathered. ``xs`` are the tensors gradients flow through (``None`` entries are
        passed on untouched); the result is a tensor or a tuple of tensors."""
        if self._full is not None:                   # all units are materialised: nothing to gather
            return fn(*xs)
        self.ensure(u)
        grad = torch.is_grad_enabled()
        if not self.in_backward and u + 1 < len(self.units):
            self.prefetch(u + 1)
        if not grad:
            return fn(*xs)
        live = [i for i, x in enumerate(xs) if isinstance(x, torch.Tensor) and x.requires_grad]
        if live:
            wrapped = _Begin.apply(self, u, defer_reduce, *[xs[i] for i in live])
            wrapped = wrapped if isinstance(wrapped, tuple) else (wrapped,)
            xs = list(xs)
            for i, w in zip(live, wrapped):
                xs[i] = w
        out = fn(*xs)
        if isinstance(out, torch.Tensor):
            return _End.apply(self, u, out)
        outs = list(out)
        idx = [i for i, o in enumerate(outs) if isinstance(o, torch.Tensor) and o.requires_grad]
        if idx:
            res = _End.apply(self, u, *[outs[i] for i in idx])
            res = res if isinstance(res, tuple) else (res,)
            for i, r in zip(idx, res):
                outs[i] = r
        return tuple(outs)

    # ------------------------------------------------------------------ whole-model views
    def gather_full(self, out: Optional[torch.Tensor] = None, device: Optional[torch.device] = None) -> torch.Tensor:
        """Every unit gathered into one buffer in the concatenated layout the slots index."""
        self.sync()
        dev = device or self.device
        full = out if out is not None else torch.empty(self.total, dtype=self.dtype, device=dev)
        for un in self.units:
            if un.size == 0:
                continue
            src = self._shard_of(un, self.data)
            if full.device == self.device:
                dst = full[un.base: un.base + un.size]
                if self.world == 1:
                    dst.copy_(src)
                else:
                    dist.all_gather_into_tensor(dst, src, group=self.group)
            else:                                     # staged through a gathered-unit buffer
                self.ensure(un.index)
                if self.cuda:
                    torch.cuda.current_stream().synchronize()
                full[un.base: un.base + un.size].copy_(self._w[un.index % 2][:un.size])
        return full

    def scatter_full(self, full: torch.Tensor) -> None:
        """Keep this rank's piece of every unit of a full buffer (after loading or initialising weights)."""
        for un in self.units:
            lo = un.base + self.rank * un.shard
            self._shard_of(un, self.data).copy_(full[lo: lo + un.shard])
        self.invalidate()

    @contextlib.contextmanager
    def materialized(self, fill: bool = True, writeback: bool = False, device: Optional[torch.device] = None):
        """All parameters as views of one full buffer for the duration of the block (weight loading, export, weight
        synchronisation). ``device`` defaults to the training device when the buffer fits into 60 % of its free
        memory, else host memory. ``writeback`` keeps this rank's pieces of whatever the block wrote."""
        self.sync()
        dev = device
        if dev is None:
            dev = self.device
            if self.cuda:
                free, _ = torch.cuda.mem_get_info(self.device)
                if self.total * self.data.element_size() > 0.6 * free:
                    dev = torch.device("cpu")
        full = torch.empty(self.total, dtype=self.dtype, device=dev)
        if fill:
            self.gather_full(out=full)
        else:
            full.zero_()
        self._full = full
        try:
            for (name, p), slot in zip(self.params, self.slots):
                p.data = full[slot.offset: slot.offset + slot.numel].view(slot.shape)
            yield full
            if writeback:
                self.scatter_full(full)
        finally:
            for (name, p), slot, (k, o) in zip(self.params, self.slots, self._local):
                p.data = self._w_params[k][o:o + slot.numel].view(slot.shape)
            self._full = None
            self.resident = [None, None]
            self._bind_grads()

    def view(self, name: str, buf: torch.Tensor) -> torch.Tensor:
        s = self.by_name[name]
        return buf[s.offset: s.offset + s.numel].view(s.shape)

    def memory_report(self) -> Dict[str, float]:
        gib = 1 / 2**30
        es = self.data.element_size()
        return {"shard_weights_GiB": self.n_shard * es * gib, "shard_grads_GiB": self.n_shard * 4 * gib,
                "unit_buffers_GiB": 4 * self.max_unit * es * gib, "full_model_GiB": self.total * es * gib}
