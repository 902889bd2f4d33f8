"""Elastic data parallelism across policy replicas.

Each policy replica is its own launch; gradients are averaged across replicas over a communicator that is
rebuilt whenever the controller announces a new membership (``BuildMeshCommand``). One communicator connects
the ranks with the same in-replica rank. Operations are retried after a rebuild and failures are reported to
the controller, which removes replicas that did not report (they are presumed hung) and rebuilds the mesh
(cosmos_rl/utils/distributed.py:548-852 ``HighAvailabilitylNccl``; gradient bucketing :93-206).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..utils.logging import logger
from .dyncomm import CommTimeout, DynComm, create_comm

BUCKET_ELEMS = 50 * 1024 * 1024  # 200 MB of fp32 per all-reduce


class InterReplicaComm:
    def __init__(self, api, replica_name: str, global_rank: int, device: torch.device, max_retries: int = 3,
                 op_timeout_s: Optional[float] = None):
        self.api, self.replica_name, self.global_rank, self.device = api, replica_name, global_rank, device
        self.max_retries = max_retries
        self.op_timeout_s = op_timeout_s
        self.comm: Optional[DynComm] = None
        self.mapping: Dict[str, int] = {}
        self.version = 0
        self.lock = threading.Lock()
        self.mesh_ready = threading.Event()
        self._last_uid: Optional[str] = None

    # ------------------------------------------------------------------ membership
    @property
    def world(self) -> int:
        return max(1, len(self.mapping))

    @property
    def rank(self) -> int:
        return self.mapping.get(self.replica_name, 0)

    def is_single(self) -> bool:
        return self.world <= 1

    def rebuild(self, mapping: Dict[str, int], uid: str) -> None:
        """New membership. ``uid`` (the command's uuid) makes the rendezvous key unique per rebuild."""
        with self.lock:
            if uid is not None and uid == self._last_uid:
                return                       # the same command reached us twice (membership watcher and main loop)
            self._last_uid = uid
            self.mesh_ready.clear()
            if self.comm is not None:
                self.comm.abort()
                self.comm = None
            self.mapping = dict(mapping)
            self.version += 1
            if self.replica_name not in mapping or len(mapping) <= 1:
                self.mesh_ready.set()
                return
            name = f"mesh-{uid}-r{self.global_rank}"
            self.comm = create_comm(self.api, name, self.rank, len(mapping), self.device,
                                    is_initiator=self.rank == 0, op_timeout_s=self.op_timeout_s)
            self.mesh_ready.set()

    # ------------------------------------------------------------------ collectives with retry
    def _retry(self, what: str, fn) -> None:
        for attempt in range(self.max_retries):
            if not self.mesh_ready.wait(timeout=600):
                raise CommTimeout("inter-replica mesh was never rebuilt")
            comm = self.comm
            if comm is None:
                return
            try:
                fn(comm)
                return
            except CommTimeout as e:
                logger.warning("[Policy] %s failed on attempt %d: %s", what, attempt + 1, e)
                self.mesh_ready.clear()
                try:
                    self.api.post_nccl_comm_error(self.replica_name, str(e))
                except Exception:
                    pass
                # the controller answers with a BuildMesh command; the worker loop calls rebuild()
        raise CommTimeout(f"{what} failed {self.max_retries} times")

    def all_reduce_grads(self, flat_grad: torch.Tensor) -> None:
        """Average a flat gradient buffer across replicas in fp32 buckets."""
        if self.is_single():
            return
        n = flat_grad.numel()

        def run(comm: DynComm):
            for c0 in range(0, n, BUCKET_ELEMS):
                c1 = min(n, c0 + BUCKET_ELEMS)
                buf = flat_grad[c0:c1].to(torch.float32)
                comm.all_reduce(buf)
                flat_grad[c0:c1].copy_(buf.div_(comm.size))

        self._retry("gradient all-reduce", run)

    def balance_token_count(self, tok: torch.Tensor) -> torch.Tensor:
        if self.is_single():
            return tok
        t = tok.clone().float()
        self._retry("token-count all-reduce", lambda comm: comm.all_reduce(t))
        return t / self.world

    # ------------------------------------------------------------------ full-state shipping
    def broadcast_state(self, tensors, src_rank: int) -> None:
        if self.is_single():
            return
        self._retry("state broadcast", lambda comm: [comm.broadcast(t, src_rank) for _, t in tensors])

    def send_state(self, tensors, dst_rank: int) -> None:
        self._retry("state send", lambda comm: [comm.send(t, dst_rank) for _, t in tensors])

    def recv_state(self, tensors, src_rank: int) -> None:
        self._retry("state recv", lambda comm: [comm.recv(t, src_rank) for _, t in tensors])

    def shutdown(self) -> None:
        if self.comm is not None:
            self.comm.abort()
            self.comm = None
