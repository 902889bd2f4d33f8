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
import contextlib
import json
import threading
import time
from datetime import timedelta
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Union

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


# ---------------------------------------------------------------------------------------------------
# watchdog contexts: a deadline over a *block* of operations, and over the device work they enqueue
# ---------------------------------------------------------------------------------------------------
class _WatchContext:
    __slots__ = ("comms", "abort", "deadline")

    def __init__(self, deadline: float):
        self.comms: "set[DynComm]" = set()
        self.abort = False
        self.deadline = deadline


_tls = threading.local()


def _watch_stack() -> List[_WatchContext]:
    st = getattr(_tls, "stack", None)
    if st is None:
        st = _tls.stack = []
    return st


def _stream_probe(stream) -> Callable[[], bool]:
    """A callable that says whether everything enqueued on ``stream`` so far has finished. ``stream`` may be a
    CUDA stream, ``None`` (the current stream when CUDA is up, else "always finished"), or already a callable
    (host-side tests hand in a probe of their own)."""
    if callable(stream) and not hasattr(stream, "record_event"):
        return stream
    if not torch.cuda.is_available():
        return lambda: True
    ev = torch.cuda.Event()
    ev.record(stream if stream is not None else torch.cuda.current_stream())
    return ev.query


@contextlib.contextmanager
def watchdog(timeout_s: Optional[float] = None, wait_stream: bool = False, stream=None):
    """Deadline over a block of communicator calls (cosmos_rl/utils/pynccl.py:458-540 has the reference's form).

    Every ``DynComm`` used inside the block joins the context. Without ``wait_stream`` a timer aborts those
    communicators when the block is still running after ``timeout_s``, which makes a host call that is blocked
    inside the library return with an error. With ``wait_stream`` the block's host calls are only enqueues; on
    exit the context polls the stream (never a blocking synchronize) until the enqueued work has finished or the
    deadline passes, and aborts the communicators in the second case. Either way ``CommTimeout`` is raised."""
    limit = timeout_s if timeout_s is not None else constant.COSMOS_NCCL_TIMEOUT_MS / 1000.0
    ctx = _WatchContext(time.monotonic() + limit)
    stack = _watch_stack()
    stack.append(ctx)
    fired = threading.Event()

    def fire():
        fired.set()
        ctx.abort = True
        logger.error("watchdog: block exceeded %.1f s; aborting %s", limit, sorted(c.name for c in ctx.comms))
        for c in list(ctx.comms):
            c.abort()

    timer = None
    if not wait_stream:
        timer = threading.Timer(limit, fire)
        timer.daemon = True
        timer.start()
    failed = False
    try:
        yield ctx
    except BaseException:
        failed = True
        ctx.abort = True
        raise
    finally:
        if timer is not None:
            timer.cancel()
        if wait_stream and not failed:
            done = _stream_probe(stream)
            while not done():
                if time.monotonic() >= ctx.deadline:
                    fire()
                    break
                time.sleep(0.001)
        stack.remove(ctx)
        if ctx.abort:
            for c in list(ctx.comms):
                c.abort()
        if fired.is_set() and not failed:
            raise CommTimeout(f"watchdog: communicator block exceeded {limit:.1f} s and was aborted")


def bounded_drain_or_abort(stream, timeout_s: float, context: str,
                           comms: Optional[Iterable["DynComm"]] = None) -> bool:
    """Teardown helper (cosmos_rl/utils/pynccl.py:629-673): wait at most ``timeout_s`` for the work in flight on
    ``stream``. Per-operation deadlines only bound the enqueue of a collective, so a broadcast whose peer has left
    keeps spinning on the device; a plain synchronize behind it would never return. Returns True when the stream
    drained, False after aborting ``comms`` (all live communicators when omitted)."""
    done = _stream_probe(stream)
    t0 = time.monotonic()
    while not done():
        if time.monotonic() - t0 > timeout_s:
            logger.warning("[abnormal teardown] %s: device work still in flight after %.1f s; a peer has most "
                           "likely left in the middle of a collective. Aborting communicators.", context, timeout_s)
            if comms is None:
                abort_all()
            else:
                for c in list(comms):
                    c.abort()
            return False
        time.sleep(0.005)
    return True


class DynComm:
    def __init__(self, name: str, store: dist.Store, rank: int, size: int, device: torch.device,
                 timeout_s: Optional[float] = None, owns_store: bool = False):
        self.name, self.rank, self.size, self.device = name, rank, size, device
        self.timeout_s = timeout_s if timeout_s is not None else constant.COSMOS_NCCL_TIMEOUT_MS / 1000.0
        self.store = store
        self.aborted = False
        # the constructor's timeout also bounds the rendezvous through the store; operations carry their own deadline
        td = timedelta(seconds=max(self.timeout_s, 30.0))
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
        for ctx in _watch_stack():
            ctx.comms.add(self)
            limit = max(0.001, min(limit, ctx.deadline - time.monotonic()))
        _notify(self.name, "enter", op=what)
        ok = work.wait(timedelta(seconds=limit)) if work is not None else True
        if ok is False:
            _notify(self.name, "timeout", op=what)
            self.abort()
            raise CommTimeout(f"{self.name}: {what} did not finish within {limit:.0f} s")
        err = self.async_error()
        if err is not None:
            _notify(self.name, "error", op=what, error=err)
            self.abort()
            raise CommTimeout(f"{self.name}: {what} left the communicator in error state {err}")
        _notify(self.name, "return", op=what)

    def _issue(self, what: str, post: Callable[[], object], timeout_s: Optional[float]) -> None:
        """Post one operation and wait for it. The library call that posts it can itself block (a first send
        that has to connect to a peer which never arrives), and no deadline of the returned work object covers
        that, so an abort is armed before the call and cancelled when it returns
        (cosmos_rl/utils/pynccl.py:236-275)."""
        if self.aborted:
            raise CommTimeout(f"{self.name}: communicator was aborted")
        limit = timeout_s if timeout_s is not None else self.timeout_s
        lock, state = threading.Lock(), {"returned": False, "fired": False}

        def abort_blocked_call():
            with lock:
                if state["returned"]:
                    return
                state["fired"] = True
            _notify(self.name, "timeout", op=what, where="post")
            self.abort()

        timer = threading.Timer(limit, abort_blocked_call)
        timer.daemon = True
        timer.start()
        try:
            work = post()
        finally:
            with lock:
                state["returned"] = True
            timer.cancel()
        if state["fired"]:
            raise CommTimeout(f"{self.name}: posting {what} blocked for more than {limit:.0f} s")
        self._run(what, work, timeout_s)

    def async_error(self) -> Optional[str]:
        """The communicator's asynchronous error state, ``None`` when healthy (the library reports remote
        failures and aborted peers here, cosmos_rl/utils/pynccl.py:297-325). Gloo has no such state."""
        get = getattr(self.pg, "get_error", None)
        if get is None or self.aborted:
            return None
        try:
            e = get()
        except Exception as exc:                                    # a dead communicator cannot answer
            return str(exc)
        name = getattr(e, "name", str(e))
        return None if name in ("SUCCESS", "0") else name

    def send(self, t: torch.Tensor, dst: int, tag: int = 0, timeout_s: Optional[float] = None) -> None:
        try:
            self._issue(f"send->{dst}", lambda: self.pg.send([t.contiguous()], dst, tag), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def recv(self, t: torch.Tensor, src: int, tag: int = 0, timeout_s: Optional[float] = None) -> None:
        try:
            self._issue(f"recv<-{src}", lambda: self.pg.recv([t], src, tag), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def broadcast(self, t: torch.Tensor, src: int, timeout_s: Optional[float] = None) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank = src
        opts.rootTensor = 0
        try:
            self._issue(f"broadcast<-{src}", lambda: self.pg.broadcast([t], opts), timeout_s)
        except RuntimeError as e:
            self._fail(e)

    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM, timeout_s: Optional[float] = None) -> None:
        opts = dist.AllreduceOptions()
        opts.reduceOp = op
        try:
            self._issue("all_reduce", lambda: self.pg.allreduce([t], opts), timeout_s)
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
