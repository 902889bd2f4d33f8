"""Exponential moving average of the trained weights, kept on the optimizer's fp32 shard.

The reference keeps a full clone of every trainable parameter and walks the parameter list on each update
(cosmos_rl/utils/ema.py:21-130; used by the diffusion trainers: diffusers_trainer.py:130-146, nft_trainer.py:303-345,
sft_trainer.py:120-155). Here the average lives beside the sharded optimizer state: one fp32 vector of the rank's
slice of the flat parameter buffer (plus the rank-local expert tail), updated by one ``lerp_`` per trainable segment,
so its memory shrinks with the data-parallel size like the Adam moments do. ``swapped_in()`` publishes the averaged
weights into the live bf16 buffer of every rank for the duration of an export or an evaluation and restores the
trained weights afterwards.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Dict

import torch
import torch.distributed as dist


class ShardEMA:
    def __init__(self, optimizer, decay: float = 0.9999, update_step_interval: int = 1):
        if not 0.0 < decay < 1.0:
            raise ValueError(f"ema decay must be in (0, 1), got {decay}")
        self.opt, self.decay, self.interval = optimizer, float(decay), max(1, int(update_step_interval))
        self.shard = optimizer.master.clone()
        self.tail = optimizer.tail["master"].clone() if optimizer.tail is not None else None
        self.updates = 0

    def current_decay(self, optimization_step: int) -> float:
        """Warm-up: early steps average over a short window (same rule as the reference: ema.py:38-39)."""
        return min((1 + optimization_step) / (10 + optimization_step), self.decay)

    @torch.no_grad()
    def step(self, optimization_step: int) -> None:
        """Call after optimizer step number ``optimization_step`` (0-based)."""
        if (optimization_step + 1) % self.interval:
            return
        w = 1.0 - self.current_decay(optimization_step)
        o = self.opt
        for a, b in (o.segments if o.segments is not None else [(0, o.hi - o.lo)]):
            self.shard[a:b].lerp_(o.master[a:b], w)
        if self.tail is not None:
            for a, b in (o.tail_segments if o.segments is not None else [(0, o.t1 - o.t0)]):
                self.tail[a:b].lerp_(o.tail["master"][a:b], w)
        self.updates += 1

    @torch.no_grad()
    def sync_with_model(self) -> None:
        self.shard.copy_(self.opt.master)
        if self.tail is not None:
            self.tail.copy_(self.opt.tail["master"])

    @torch.no_grad()
    def _publish(self, shard: torch.Tensor, tail) -> None:
        o = self.opt
        flat = o.flat.data
        if o.world > 1:
            dist.all_gather_into_tensor(flat[:o.t0], shard.to(flat.dtype), group=o.group)
        else:
            flat[o.lo:o.hi].copy_(shard)
        if tail is not None:
            flat[o.t0:o.t1].copy_(tail)

    @contextmanager
    def swapped_in(self):
        """The live weights are the averaged ones inside the block (collective over the sharding group)."""
        self._publish(self.shard, self.tail)
        try:
            yield self
        finally:
            self._publish(self.opt.master, self.opt.tail["master"] if self.tail is not None else None)

    def state_dict(self) -> Dict[str, Any]:
        sd = {"shard": self.shard, "updates": self.updates, "decay": self.decay}
        if self.tail is not None:
            sd["tail"] = self.tail
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd["shard"].numel() != self.shard.numel():
            raise ValueError("ema state was saved with a different sharding")
        self.shard.copy_(sd["shard"])
        if self.tail is not None and "tail" in sd:
            self.tail.copy_(sd["tail"])
        self.updates = int(sd.get("updates", 0))


class FlatEMA:
    """Full-buffer variant for weights that no sharded optimizer owns (a frozen copy that trails the trained network,
    a model driven by a user's own optimizer): fp32 shadow of one flat tensor, fixed decay."""

    def __init__(self, flat_data: torch.Tensor, decay: float = 0.999, update_interval: int = 1):
        self.src = flat_data
        self.decay = decay
        self.interval = max(1, update_interval)
        self.shadow = flat_data.detach().to(torch.float32).clone()
        self.n = 0

    @torch.no_grad()
    def update(self) -> None:
        self.n += 1
        if self.n % self.interval:
            return
        d = self.decay ** self.interval
        self.shadow.mul_(d).add_(self.src.to(torch.float32), alpha=1.0 - d)

    @contextmanager
    def swapped_in(self):
        backup = self.src.clone()
        self.src.copy_(self.shadow.to(self.src.dtype))
        try:
            yield
        finally:
            self.src.copy_(backup)

    def state_dict(self) -> Dict[str, Any]:
        return {"shadow": self.shadow, "n": self.n}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.shadow.copy_(sd["shadow"])
        self.n = int(sd["n"])
