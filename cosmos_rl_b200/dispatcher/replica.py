"""Replica / Atom bookkeeping on the controller.

An *atom* is one GPU process, addressed by its coordinates on the mesh axes ``["pp","dp_shard","cp","tp"]``;
a *replica* is the set of atoms of one job (``torchrun`` group). A replica becomes usable once every atom
implied by the per-axis group sizes has registered (cosmos_rl/dispatcher/replica.py:29-300).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .protocol import MESH_NAMES, RegisterRequest, Role


@dataclass
class Atom:
    ranks: List[int]
    group_size: List[int]
    global_rank: int
    host_ip: str = "127.0.0.1"
    host_name: str = "localhost"
    trace_path: Optional[str] = None

    @classmethod
    def from_request(cls, req: RegisterRequest) -> "Atom":
        return cls(list(req.ranks), list(req.group_size), req.global_rank, req.host_ip, req.host_name)

    def coord(self, axis: str) -> int:
        return self.ranks[MESH_NAMES.index(axis)]

    def size(self, axis: str) -> int:
        return self.group_size[MESH_NAMES.index(axis)]

    @property
    def world_size(self) -> int:
        n = 1
        for g in self.group_size:
            n *= g
        return n

    def key(self) -> str:
        return "_".join(str(r) for r in self.ranks)


class ReplicaStatus:
    UNINITIALIZED = "uninitialized"   # registered, weights not loaded
    READY = "ready"                   # weights loaded, idle
    RUNNING = "running"               # policy: training a step / rollout: generating
    REDUCED = "reduced"               # policy: acked the current step
    END = "end"


@dataclass
class Replica:
    name: str
    role: str
    atoms: Dict[str, Atom] = field(default_factory=dict)
    status: str = ReplicaStatus.UNINITIALIZED
    weights_loaded: bool = False
    in_mesh: bool = False
    mesh_rank: int = -1
    start_time: float = field(default_factory=time.time)
    last_heartbeat: float = field(default_factory=time.time)
    weight_step: int = 0
    acked_step: int = -1
    pending_profile: Optional[dict] = None
    ended: bool = False

    def add_atom(self, atom: Atom) -> None:
        self.atoms[atom.key()] = atom

    @property
    def expected_atoms(self) -> int:
        any_atom = next(iter(self.atoms.values()), None)
        return any_atom.world_size if any_atom else 0

    @property
    def all_atoms_arrived(self) -> bool:
        return len(self.atoms) > 0 and len(self.atoms) == self.expected_atoms

    @property
    def n_gpus(self) -> int:
        return self.expected_atoms

    def heartbeat(self) -> None:
        self.last_heartbeat = time.time()

    def silent_for(self, now: Optional[float] = None) -> float:
        return (now if now is not None else time.time()) - self.last_heartbeat

    def group_size(self, axis: str) -> int:
        any_atom = next(iter(self.atoms.values()))
        return any_atom.size(axis)

    def summary(self) -> dict:
        return {
            "name": self.name, "role": self.role, "status": self.status, "n_atoms": len(self.atoms),
            "expected_atoms": self.expected_atoms, "weights_loaded": self.weights_loaded,
            "mesh_rank": self.mesh_rank, "weight_step": self.weight_step,
            "start_time": self.start_time, "last_heartbeat": self.last_heartbeat,
            "atoms": [{"ranks": a.ranks, "group_size": a.group_size, "global_rank": a.global_rank,
                       "host_ip": a.host_ip, "trace_path": a.trace_path} for a in self.atoms.values()],
        }
