"""Parallel dimensions of one replica and the process groups derived from them.

Axis order (slowest to fastest varying rank): ``pp, dp_replicate, dp_shard, cp, tp`` — the layout of
cosmos_rl/utils/parallelism.py:82-578. Rank arithmetic (`coords_of`, `ranks_along`) needs no process group,
so the controller and the resharding planner can reason about any replica's layout.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

AXES = ("pp", "dp_replicate", "dp_shard", "cp", "tp")


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = 1
    cp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    world_size: int = 1
    pp_dynamic_shape: bool = False
    global_rank: int = 0
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    _groups: Dict[str, Optional[dist.ProcessGroup]] = field(default_factory=dict, repr=False)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_config_parallelism(cls, p, world_size: int, global_rank: int = 0, device=None) -> "ParallelDims":
        dp_shard = p.dp_shard_size
        fixed = p.tp_size * p.cp_size * p.pp_size * max(p.dp_replicate_size, 1)
        if dp_shard in (-1, 0, None):
            if world_size % fixed:
                raise ValueError(f"world size {world_size} not divisible by tp*cp*pp*dp_replicate = {fixed}")
            dp_shard = world_size // fixed
        d = cls(dp_replicate=max(p.dp_replicate_size, 1), dp_shard=dp_shard, cp=p.cp_size, tp=p.tp_size,
                pp=p.pp_size, ep=getattr(p, "ep_size", 1) or 1, world_size=world_size,
                pp_dynamic_shape=getattr(p, "pp_dynamic_shape", False), global_rank=global_rank,
                device=device or torch.device("cpu"))
        d.validate()
        return d

    def validate(self) -> None:
        for name in ("dp_replicate", "dp_shard", "cp", "tp", "pp", "ep"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")
        prod = self.dp_replicate * self.dp_shard * self.cp * self.tp * self.pp
        if prod != self.world_size:
            raise ValueError(f"dp_replicate*dp_shard*cp*tp*pp = {prod} != world size {self.world_size}")
        if self.ep > 1 and self.tp > 1:
            raise ValueError("tp must be 1 when ep > 1")
        if self.ep > 1 and (self.dp_shard * self.cp) % self.ep:
            raise ValueError("ep must divide dp_shard * cp")

    # ------------------------------------------------------------------ rank arithmetic
    def sizes(self) -> Tuple[int, ...]:
        return (self.pp, self.dp_replicate, self.dp_shard, self.cp, self.tp)

    def coords_of(self, rank: int) -> Dict[str, int]:
        out = {}
        for name, size in reversed(list(zip(AXES, self.sizes()))):
            out[name] = rank % size
            rank //= size
        return out

    def rank_of(self, coords: Dict[str, int]) -> int:
        r = 0
        for name, size in zip(AXES, self.sizes()):
            r = r * size + coords.get(name, 0)
        return r

    def ranks_along(self, axis: str, rank: Optional[int] = None) -> List[int]:
        """Global ranks of the group along ``axis`` that contains ``rank``."""
        rank = self.global_rank if rank is None else rank
        c = self.coords_of(rank)
        size = self.sizes()[AXES.index(axis)]
        return [self.rank_of({**c, axis: i}) for i in range(size)]

    @property
    def coords(self) -> Dict[str, int]:
        return self.coords_of(self.global_rank)

    @property
    def tp_coord(self) -> int:
        return self.coords["tp"]

    @property
    def dp_shard_coord(self) -> int:
        return self.coords["dp_shard"]

    @property
    def pp_coord(self) -> int:
        return self.coords["pp"]

    @property
    def cp_coord(self) -> int:
        return self.coords["cp"]

    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate * self.dp_shard > 1

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp * self.pp

    def mesh_register_fields(self) -> Tuple[List[str], List[int], List[int]]:
        """(mesh_names, ranks, group_size) in the order the controller expects."""
        c = self.coords
        return (["pp", "dp_shard", "cp", "tp"], [c["pp"], c["dp_replicate"] * self.dp_shard + c["dp_shard"], c["cp"], c["tp"]],
                [self.pp, self.dp_replicate * self.dp_shard, self.cp, self.tp])

    # ------------------------------------------------------------------ process groups
    def build_groups(self, base_ranks: Optional[List[int]] = None, backend: Optional[str] = None) -> None:
        """Create one process group per axis with size > 1. ``base_ranks`` maps this replica's local ranks
        0..world-1 to ranks of the default group (a replica may be a sub-set of a larger launch). Every
        process of the default group must call this with the same arguments (``dist.new_group`` is collective)."""
        if not dist.is_initialized() or self.world_size == 1:
            return
        base = base_ranks or list(range(self.world_size))
        me = dist.get_rank()
        for axis, size in zip(AXES, self.sizes()):
            if size == 1:
                self._groups[axis] = None
                continue
            done = set()
            for r in range(self.world_size):
                members = tuple(self.ranks_along(axis, r))
                if members in done:
                    continue
                done.add(members)
                g = dist.new_group([base[m] for m in members], backend=backend)
                if me in [base[m] for m in members]:
                    self._groups[axis] = g
                if axis == "pp":
                    # a second communicator over the same ranks: gradients between pipeline stages travel on it, so
                    # that activations and gradients between two ranks never share one communicator's message order
                    g2 = dist.new_group([base[m] for m in members], backend=backend)
                    if me in [base[m] for m in members]:
                        self._groups["pp_back"] = g2
        if self.world_size > 1:
            g = dist.new_group(base, backend=backend)
            if me in base:
                self._groups["world"] = g

    def build_ep_groups(self, base_ranks: Optional[List[int]] = None, backend: Optional[str] = None) -> None:
        """Expert parallelism inside the dp_shard axis (``ep`` divides ``dp_shard``): consecutive blocks of ``ep`` ranks
        of every dp_shard group exchange tokens (group ``"ep"``); ranks with the same position in different blocks
        hold the same experts (group ``"ep_replica"``) and sum their expert gradients. With ``ep == dp_shard`` the
        ``"ep"`` group is the dp_shard group and no replica group exists. Collective like ``build_groups``."""
        if self.ep <= 1:
            return
        if self.dp_shard % self.ep:
            raise ValueError(f"ep_size {self.ep} must divide dp_shard_size {self.dp_shard}")
        if self.ep == self.dp_shard:
            self._groups["ep"] = self._groups.get("dp_shard")
            self._groups["ep_replica"] = None
            return
        base = base_ranks or list(range(self.world_size))
        me = dist.get_rank()
        done = set()
        for r in range(self.world_size):
            line = tuple(self.ranks_along("dp_shard", r))
            if line in done:
                continue
            done.add(line)
            blocks = [line[i:i + self.ep] for i in range(0, self.dp_shard, self.ep)]
            for members in blocks:
                g = dist.new_group([base[m] for m in members], backend=backend)
                if me in [base[m] for m in members]:
                    self._groups["ep"] = g
            for j in range(self.ep):
                members = [blk[j] for blk in blocks]
                g = dist.new_group([base[m] for m in members], backend=backend)
                if me in [base[m] for m in members]:
                    self._groups["ep_replica"] = g

    @property
    def ep_coord(self) -> int:
        return self.dp_shard_coord % self.ep

    def group(self, axis: str) -> Optional[dist.ProcessGroup]:
        return self._groups.get(axis)

    def set_group(self, axis: str, group) -> None:
        self._groups[axis] = group
