"""Dynamically created, abortable communicators between replicas.

Replicas are independent launches, so the communicator that connects a policy replica with a rollout
replica (or the policy replicas with each other) cannot be a sub-group of one ``torch.distributed`` world.
The reference builds them with a ctypes NCCL binding whose unique id travels through the controller
(cosmos_rl/utils/pynccl.py:546-921, cosmos_rl/utils/pynccl_wrapper.py:142-340). Here the rendezvous is a
``TCPStore`` whose address travels through the controller's key/value store, and the communicator is a
stand-alone c10d backend object (NCCL on GPUs, gloo on CPU) that is not registered as the default group.
Every operation runs under a deadline; a communicator that misses it is aborted and reported, never
waited on forever (``CommTimeout``), which is what the controller's NCCL-error consensus builds on.
"""
from __future__ import annotations

import base64
import json
import threading
import time
from datetime import timedelta
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..utils import constant
from ..utils.logging import logger
from ..utils.misc import free_port, local_ips


class CommTimeout(RuntimeError):
    pass


_REGISTRY: Dict[str, "DynComm"] = {}
_observers: List[Callable[[str, str, Dict], None]] = []


def add_phase_observer(fn: Callable[[str, str, Dict], None]) -> None:
    """``fn(comm_name, phase, info)`` is called at op enter / return / timeout / abort (hang diagnosis hook,
    cosmos_rl/utils/pynccl.py:181-207)."""
    _observers.append(fn)


def _notify(name: str, phase: str, **info) -> None:
    for fn in list(_observers):
        try:
            fn(name, phase, info)
        except Exception:
            pass


class DynComm:
    def __init__(self, name: str, store: dist.Store, rank: int, size: int, device: torch.device,
                 timeout_s: Optional[float] = None, owns_store: bool = False):
        self.name, self.rank, self.size, self.device = name, rank, size, device
        self.timeout_s = timeout_s if timeout_s is not None else constant.COSMOS_NCCL_TIMEOUT_MS / 1000.0
        self.store = store
        self.aborted = False
        td = timedelta(seconds=self.timeout_s)
        prefix = dist.PrefixStore(f"dyncomm/{name}", store)
        if device.type == "cuda":
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = td
            self.pg = dist.ProcessGroupNCCL(prefix, rank, size, opts)
            self.backend = "nccl"
        else:
            self.pg = dist.ProcessGroupGloo(prefix, rank, size, td)
            self.backend = "gloo"
        _REGISTRY[name] = self

    # ------------------------------------------------------------------ guarded execution
    def _run(self, what: str, work, timeout_s: Optional[float] = None) -> None:
        if self.aborted:
            raise CommTimeout(f"{self.name}: communicator was aborted")
        limit = timeout_s if timeout_s is not None else self.timeout_s
        _notify(self.name, "enter", op=what)
        ok = work.wait(timedelta(seconds=limit)) if work is not None else True
        if ok is False:
            _notify(self.name, "timeout", op=what)
            self.abort()
            raise CommTimeout(f"{self.name}: {what} did not finish within {limit:.0f} s")
        _notify(self.name, "return", op=what)

    def send(self, t: torch.Tensor, dst: int, tag: int = 0, timeout_s: Optional[float] = None) -> None:
        try:
            self._run(f"send->{dst}", self.pg.send([t.contiguous()], dst, tag), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def recv(self, t: torch.Tensor, src: int, tag: int = 0, timeout_s: Optional[float] = None) -> None:
        try:
            self._run(f"recv<-{src}", self.pg.recv([t], src, tag), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def broadcast(self, t: torch.Tensor, src: int, timeout_s: Optional[float] = None) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank = src
        opts.rootTensor = 0
        try:
            self._run(f"broadcast<-{src}", self.pg.broadcast([t], opts), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM, timeout_s: Optional[float] = None) -> None:
        opts = dist.AllreduceOptions()
        opts.reduceOp = op
        try:
            self._run("all_reduce", self.pg.allreduce([t], opts), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        t = torch.zeros(1, device=self.device)
        self.all_reduce(t, timeout_s=timeout_s)

    def _fail(self, e: Exception):
        if isinstance(e, CommTimeout):
            raise e
        _notify(self.name, "error", error=str(e))
        self.abort()
        raise CommTimeout(f"{self.name}: {e}") from e

    def abort(self) -> None:
        if self.aborted:
            return
        self.aborted = True
        _notify(self.name, "abort")
        try:
            if hasattr(self.pg, "abort"):
                self.pg.abort()
            elif hasattr(self.pg, "_shutdown"):
                self.pg._shutdown()
        except Exception as e:
            logger.warning("abort of %s raised: %s", self.name, e)
        _REGISTRY.pop(self.name, None)

    def destroy(self) -> None:
        self.abort()


def abort_all() -> None:
    for c in list(_REGISTRY.values()):
        c.abort()


def live_comms() -> List[str]:
    return sorted(_REGISTRY)


# ---------------------------------------------------------------------------------------------------
# rendezvous through the controller's key/value store
# ---------------------------------------------------------------------------------------------------
def create_comm(api, name: str, rank: int, size: int, device: torch.device, is_initiator: bool,
                timeout_s: float = 120.0, op_timeout_s: Optional[float] = None) -> DynComm:
    """Rank ``is_initiator`` hosts a TCPStore and publishes ``host:port`` under ``name``; the others fetch it.
    Mirrors the comm_initiator / comm_acceptor handshake of the reference."""
    td = timedelta(seconds=timeout_s)
    if is_initiator:
        port = free_port("0.0.0.0")
        store = dist.TCPStore("0.0.0.0", port, size, is_master=True, timeout=td, wait_for_workers=False)
        addr = {"hosts": local_ips(), "port": port}
        api.post_nccl_comm_initiator(name, base64.b64encode(json.dumps(addr).encode()).decode())
    else:
        raw = api.post_nccl_comm_acceptor(name, timeout_s=timeout_s)
        addr = json.loads(base64.b64decode(raw))
        store, last = None, None
        for host in addr["hosts"]:
            try:
                store = dist.TCPStore(host, addr["port"], size, is_master=False, timeout=timedelta(seconds=15))
                break
            except Exception as e:
                last = e
        if store is None:
            raise CommTimeout(f"{name}: cannot reach the rendezvous store at {addr}: {last}")
    return DynComm(name, store, rank, size, device, timeout_s=op_timeout_s, owns_store=is_initiator)
