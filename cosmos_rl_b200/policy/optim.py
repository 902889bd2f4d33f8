"""Optimizer and LR schedule of the policy trainers.

``FlatAdamW`` keeps fp32 master weights and Adam moments for this rank's shard of the flat parameter buffer
and updates them with one fused kernel that also rewrites the bf16 compute copy; the clip coefficient stays
on the device. Data parallel (``dp_shard``): gradients are reduce-scattered into the shard and the updated
bf16 weights all-gathered back, each once per optimizer step (optimizer-state + gradient sharding; with
180 GB of HBM per GPU the bf16 weights of the supported models stay resident, so no parameter all-gather
sits inside forward/backward). The schedule is warmup-stable-decay as in
cosmos_rl/policy/trainer/optm/__init__.py:500-620.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..ops import optim as K
from ..parallel.flat import FlatParams


def lr_factor(step: int, total_steps: int, warmup_steps, warmup_start_factor: float = 0.0,
              decay_ratio: Optional[float] = None, decay_type: Optional[str] = None,
              min_lr_factor: float = 0.0) -> float:
    """Multiplier applied to the base LR at optimizer step ``step`` (0-based)."""
    if isinstance(warmup_steps, float) and warmup_steps < 1.0:
        warmup = int(round(warmup_steps * total_steps))
    else:
        warmup = int(warmup_steps)
    if warmup > 0 and step < warmup:
        return warmup_start_factor + (1.0 - warmup_start_factor) * (step + 1) / (warmup + 1)
    if not decay_type or total_steps <= 0:
        return 1.0
    decay_steps = int(total_steps * decay_ratio) if decay_ratio is not None else max(total_steps - warmup, 1)
    stable_end = total_steps - decay_steps
    if step < stable_end:
        return 1.0
    prog = min(1.0, max(0.0, (step - stable_end + 1) / max(decay_steps, 1)))
    if decay_type == "linear":
        f = 1.0 - prog
    elif decay_type == "cosine":
        f = 0.5 * (1.0 + math.cos(math.pi * prog))
    elif decay_type == "sqrt":
        f = 1.0 - math.sqrt(prog)
    else:
        raise ValueError(f"unknown decay type {decay_type!r}")
    return min_lr_factor + (1.0 - min_lr_factor) * f


class _Quantized8:
    """An Adam moment held in 8 bits: blocks of 256 values share one fp32 scale (absmax). The first moment is stored
    as signed int8; the second moment spans many orders of magnitude inside a block, so its square root is stored
    (uint8), which halves the exponent range. The reference offers torchao's 8-bit Adam for the same purpose
    (cosmos_rl/policy/trainer/optm/__init__.py:36-41, 380-385)."""
    BLOCK = 256

    def __init__(self, n: int, device, sqrt: bool):
        self.n, self.sqrt = n, sqrt
        nb = -(-n // self.BLOCK)
        self.q = torch.zeros(nb * self.BLOCK, dtype=torch.uint8 if sqrt else torch.int8, device=device)
        self.scale = torch.zeros(nb, dtype=torch.float32, device=device)
        self.levels = 255.0 if sqrt else 127.0

    def window(self, a: int, b: int):
        """Block-aligned range that covers [a, b)."""
        return a // self.BLOCK * self.BLOCK, min(-(-b // self.BLOCK) * self.BLOCK, self.q.numel())

    def load(self, A: int, B: int) -> torch.Tensor:
        x = self.q[A:B].to(torch.float32).view(-1, self.BLOCK) * self.scale[A // self.BLOCK:B // self.BLOCK, None]
        x = x.reshape(-1)
        return x * x if self.sqrt else x

    def store(self, A: int, x: torch.Tensor) -> None:
        B = A + x.numel()
        y = (x.sqrt() if self.sqrt else x).view(-1, self.BLOCK)
        s = y.abs().amax(1) / self.levels
        self.scale[A // self.BLOCK:B // self.BLOCK] = s
        q = (y / s.clamp_min(1e-30)[:, None]).round_()
        self.q[A:B] = q.to(self.q.dtype).view(-1)

    def tensors(self, name: str):
        return [(f"{name}.q", self.q), (f"{name}.scale", self.scale)]


class FlatAdamW:
    def __init__(self, flat: FlatParams, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, dp_group: Optional[dist.ProcessGroup] = None,
                 master_dtype: torch.dtype = torch.float32, collective=None,
                 replicate_group: Optional[dist.ProcessGroup] = None,
                 tp_group: Optional[dist.ProcessGroup] = None, tp_replicated: Optional[torch.Tensor] = None,
                 norm_groups=(), sum_groups=(), state_bits: int = 32,
                 tail_replica_group: Optional[dist.ProcessGroup] = None):
        """``dp_group`` shards optimizer state (ZeRO-2 style); ``replicate_group`` is the outer data-parallel axis of
        HSDP / DDP (cosmos_rl/policy/model/gpt/parallelize.py:80-113, 426-442): ranks of it hold the same shard and
        average their reduced gradient shard before the update, so the all-reduce moves 1/dp_shard of the gradient."""
        # gradient norm under model parallelism: parameters sharded over ``tp_group`` contribute once per rank, the
        # ones every tensor-parallel rank holds (``tp_replicated``: bool mask over the flat buffer) only once;
        # ``norm_groups`` are further groups whose ranks hold disjoint parameters (pipeline stages)
        # ``sum_groups``: ranks that hold partial gradients of the SAME samples (context-parallel chunks): summed
        # ``tail_replica_group``: ranks of the dp group that hold the SAME rank-local tail (expert replicas when
        # ep < dp_shard): their tail gradients are summed, and the tail counts once per distinct copy in the norm
        self.tail_replica_group = tail_replica_group
        self.n_tail_replicas = dist.get_world_size(tail_replica_group) if tail_replica_group is not None else 1
        self.sum_groups = tuple(g for g in sum_groups if g is not None)
        self.tp_group, self.norm_groups = tp_group, tuple(norm_groups)
        self.tp_replicated = tp_replicated
        self.flat = flat
        self.replicate_group = replicate_group
        self.n_replicas = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.group = dp_group
        self.world = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.rank = dist.get_rank(dp_group) if dp_group is not None else 0
        self.collective = collective  # optional fused peer-memory reduce-scatter / all-gather provider
        self.lo, self.hi = flat.shard_range(self.rank, self.world)
        n = self.hi - self.lo
        dev = flat.device
        self.master = flat.data[self.lo:self.hi].to(torch.float32, copy=True)
        if state_bits not in (8, 32):
            raise ValueError("state_bits must be 32 or 8")
        self.state_bits = state_bits
        if state_bits == 8:                      # block-quantised moments: 2 bytes per parameter instead of 8
            self.m = self.v = None
            self.m8, self.v8 = _Quantized8(n, dev, sqrt=False), _Quantized8(n, dev, sqrt=True)
        else:
            self.m = torch.zeros(n, dtype=torch.float32, device=dev)
            self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.grad_shard = torch.zeros(n, dtype=torch.float32, device=dev) if self.world > 1 else None
        # rank-local tail (expert-parallel experts): full optimizer state here, no reduction, no publication
        self.t0, self.t1 = flat.shared_total, flat.total
        self.tail = None
        if self.t1 > self.t0:
            nt = self.t1 - self.t0
            self.tail = {"master": flat.data[self.t0:self.t1].to(torch.float32, copy=True),
                         "m": torch.zeros(nt, dtype=torch.float32, device=dev),
                         "v": torch.zeros(nt, dtype=torch.float32, device=dev)}
        self.step_count = 0
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.trainable = flat.trainable_mask()
        # frozen parameters must not even decay: the update runs over the trainable stretches of this rank's shard only
        self.segments = None
        if self.trainable is not None:
            self.segments = self._trainable_segments(self.lo, self.hi)
            self.tail_segments = self._trainable_segments(self.t0, self.t1) if self.t1 > self.t0 else []

    def _trainable_segments(self, lo: int, hi: int):
        """[(start, end)] relative to ``lo``: maximal runs of trainable parameter slots inside [lo, hi)."""
        segs = []
        for (name, p), slot in sorted(zip(self.flat.params, self.flat.slots), key=lambda t: t[1].offset):
            if not p.requires_grad:
                continue
            a, b = max(slot.offset, lo), min(slot.offset + slot.numel, hi)
            if a >= b:
                continue
            if segs and segs[-1][1] == a - lo:
                segs[-1] = (segs[-1][0], b - lo)
            else:
                segs.append((a - lo, b - lo))
        return segs

    # ------------------------------------------------------------------
    def refresh_master_from_params(self) -> None:
        """After loading weights into the bf16 buffer (HF load, weight resume)."""
        self.master.copy_(self.flat.data[self.lo:self.hi].to(torch.float32))
        if self.tail is not None:
            self.tail["master"].copy_(self.flat.data[self.t0:self.t1].to(torch.float32))

    def _reduce_grads(self) -> torch.Tensor:
        """Returns this rank's averaged gradient shard (fp32 when dp > 1, a bf16 view otherwise)."""
        g = self.flat.grad
        if self.trainable is not None:
            g.mul_(self.trainable.to(g.dtype))
        if self.world == 1:
            return g[self.lo:self.hi]
        # library path (the baseline): fp32 reduce as in FSDP2's reduce_dtype=float32, in chunks so the fp32
        # staging copy stays small
        per = self.hi - self.lo
        chunk = min(per, 1 << 26)
        for c0 in range(0, per, chunk):
            c1 = min(per, c0 + chunk)
            stage = torch.stack([g[r * per + c0: r * per + c1].to(torch.float32) for r in range(self.world)])
            dist.reduce_scatter_tensor(self.grad_shard[c0:c1], stage.view(-1), op=dist.ReduceOp.AVG, group=self.group)
        return self.grad_shard

    def step(self, lr_scale: float = 1.0, extra_norm_groups=()) -> torch.Tensor:
        """Reduce, clip, update, republish weights. Returns the global gradient norm (1-element tensor)."""
        self.step_count += 1
        fused = self.world > 1 and self.collective is not None
        if fused:
            if self.trainable is not None:
                self.flat.grad.mul_(self.trainable.to(self.flat.grad.dtype))
            sumsq = torch.zeros(1, dtype=torch.float32, device=self.flat.device)
            self.collective.reduce_scatter_sumsq(self.lo, self.hi, self.grad_shard, sumsq)
            g = self.grad_shard
        else:
            g = self._reduce_grads()
            sumsq = K.grad_sumsq([g])
        if self.sum_groups:
            g32 = g if g.dtype == torch.float32 else g.to(torch.float32)
            for grp in self.sum_groups:
                dist.all_reduce(g32, group=grp)
            if g32 is not g:
                g.copy_(g32)
            sumsq = K.grad_sumsq([g])
        if self.n_replicas > 1:
            if g.dtype != torch.float32:           # dp_shard == 1: the shard is the bf16 gradient buffer itself
                g32 = g.to(torch.float32)
                dist.all_reduce(g32, group=self.replicate_group)
                g.copy_(g32.div_(self.n_replicas))
            else:
                dist.all_reduce(g, group=self.replicate_group)
                g.div_(self.n_replicas)
            sumsq = K.grad_sumsq([g])
            if self.tail is not None:
                gt32 = self.flat.grad[self.t0:self.t1].to(torch.float32)
                dist.all_reduce(gt32, group=self.replicate_group)
                self.flat.grad[self.t0:self.t1].copy_(gt32.div_(self.n_replicas))
        if self.tail is not None:
            # experts see the tokens of every rank: their gradient already is the sum over ranks, so it takes the
            # same 1/world factor as the averaged replicated gradients; each rank adds its own experts to the norm
            gt = self.flat.grad[self.t0:self.t1]
            if self.trainable is not None:
                gt.mul_(self.trainable[self.t0:self.t1].to(gt.dtype))
            if self.tail_replica_group is not None:
                # an expert's replicas each saw the tokens of their own block of ranks: the sum covers every rank
                gt32 = gt.to(torch.float32)
                dist.all_reduce(gt32, group=self.tail_replica_group)
                gt.copy_(gt32)
            sumsq = sumsq + K.grad_sumsq([gt]) / float(self.world * self.world * self.n_tail_replicas)
        rep = None
        if self.tp_group is not None and self.tp_replicated is not None:
            rep = K.grad_sumsq([(g.float() * self.tp_replicated[self.lo:self.hi].to(torch.float32))])
            sumsq = sumsq - rep
        if self.world > 1:
            dist.all_reduce(sumsq, group=self.group)
            if rep is not None:
                dist.all_reduce(rep, group=self.group)
        if self.tp_group is not None:
            dist.all_reduce(sumsq, group=self.tp_group)
            if rep is not None:
                sumsq = sumsq + rep
        for grp in tuple(extra_norm_groups) + self.norm_groups:  # groups whose ranks hold disjoint parameters
            dist.all_reduce(sumsq, group=grp)
        norm, coef = K.clip_coef_from_sumsq(sumsq, self.max_grad_norm)
        hp = dict(lr=self.lr * lr_scale, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                  weight_decay=self.wd, step=self.step_count, grad_scale=coef)
        segs = self.segments if self.segments is not None else [(0, self.hi - self.lo)]
        if fused and self.segments is None and self.state_bits == 32:
            self.collective.adamw_publish(self.master, self.m, self.v, g, self.lo, self.hi, **hp)
        else:
            shadow = self.flat.data[self.lo:self.hi]
            for a, b in segs:
                if self.state_bits == 8:
                    self._step_quantised(a, b, g, shadow, hp)
                else:
                    K.adamw_flat(self.master[a:b], self.m[a:b], self.v[a:b], g[a:b], shadow[a:b], **hp)
            if self.world > 1:
                dist.all_gather_into_tensor(self.flat.data[:self.t0], shadow.clone(), group=self.group)
        if self.tail is not None:
            hp_t = dict(hp, grad_scale=coef / float(self.world))
            gt, dt_ = self.flat.grad[self.t0:self.t1], self.flat.data[self.t0:self.t1]
            for a, b in (self.tail_segments if self.segments is not None else [(0, self.t1 - self.t0)]):
                K.adamw_flat(self.tail["master"][a:b], self.tail["m"][a:b], self.tail["v"][a:b], gt[a:b], dt_[a:b],
                             **hp_t)
        self.last_grad_norm = norm
        return norm

    def _step_quantised(self, a: int, b: int, g, shadow, hp, chunk: int = 1 << 24) -> None:
        """[a, b) of the shard with 8-bit moments: block-aligned windows of at most ``chunk`` values are expanded to
        fp32, updated by the same kernel as the fp32 path and stored back."""
        A0, B0 = self.m8.window(a, b)
        for A in range(A0, B0, chunk):
            B = min(A + chunk, B0)
            m, v = self.m8.load(A, B), self.v8.load(A, B)
            lo, hi = max(a, A), min(b, B)
            K.adamw_flat(self.master[lo:hi], m[lo - A:hi - A], v[lo - A:hi - A], g[lo:hi], shadow[lo:hi], **hp)
            self.m8.store(A, m)
            self.v8.store(A, v)

    def zero_moments(self) -> None:
        """Clear both Adam moments everywhere they live: the fp32 shard, the 8-bit blocks, the rank-local tail."""
        if self.state_bits == 8:
            for q8 in (self.m8, self.v8):
                q8.q.zero_()
                q8.scale.zero_()
        else:
            self.m.zero_()
            self.v.zero_()
        if self.tail is not None:
            self.tail["m"].zero_()
            self.tail["v"].zero_()

    def zero_grad(self) -> None:
        self.flat.zero_grad()

    # ------------------------------------------------------------------ state (per-rank shard)
    def state_dict(self) -> Dict[str, Any]:
        sd = {"master": self.master, "m": self.m, "v": self.v, "step": self.step_count, "lo": self.lo,
              "hi": self.hi, "world": self.world}
        if self.state_bits == 8:
            sd.update(m=None, v=None, q8={k: t for k, t in self.m8.tensors("m") + self.v8.tensors("v")})
        if self.tail is not None:
            sd["tail"] = dict(self.tail)
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd["hi"] - sd["lo"] != self.hi - self.lo:
            raise ValueError("optimizer shard size changed; re-shard the checkpoint first")
        self.master.copy_(sd["master"])
        if self.state_bits == 8:
            if "q8" not in sd:
                raise ValueError("the checkpoint holds fp32 optimizer moments but the optimizer is configured for 8 bits")
            for k, t in self.m8.tensors("m") + self.v8.tensors("v"):
                t.copy_(sd["q8"][k])
        else:
            self.m.copy_(sd["m"])
            self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
        self.flat.data[self.lo:self.hi].copy_(self.master.to(self.flat.dtype))
        if self.tail is not None and "tail" in sd:
            for k in ("master", "m", "v"):
                self.tail[k].copy_(sd["tail"][k])
            self.flat.data[self.t0:self.t1].copy_(self.tail["master"].to(self.flat.dtype))

    def state_tensors(self):
        """Named tensors shipped to a new replica on elastic scale-up (policy-to-policy unicast)."""
        if self.state_bits == 8:
            out = [("optim.master", self.master)] + [(f"optim.{k}", t) for k, t in
                                                     self.m8.tensors("m") + self.v8.tensors("v")]
        else:
            out = [("optim.master", self.master), ("optim.m", self.m), ("optim.v", self.v)]
        if self.tail is not None:
            out += [(f"optim.tail.{k}", t) for k, t in self.tail.items()]
        return out
