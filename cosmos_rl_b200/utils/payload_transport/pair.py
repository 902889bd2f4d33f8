"""Rollout -> policy bulk tensors over two-rank communicators (``payload_transfer = "nccl"``).

The broker stays the control plane; the tensors move device to device. A producer parks a tensor in its send-buffer
registry and puts ``nccl:<owner>/<id>/<dtype>/<shape>`` into the rollout message. The consumer that trains on the
rollout publishes a request on the producer's request stream; the producer answers ACCEPTED or MISSING under the
transfer's response key, both sides look up (or build) the communicator of their pair, and one send / recv moves
the tensor. A request that gets no answer within the receive budget is retried and then the producer endpoint is
quarantined for a cool-down, so one wedged producer costs an episode, not the batch. The reference's transport has
the same parts (cosmos_rl/utils/payload_transport/nccl/{transport,rendezvous,comm_cache,buffer_registry,streams}.py,
docs/payload_transport/nccl.md); this one is built on ``DynComm`` (NCCL on GPUs, gloo on CPU), whose operations
carry deadlines and abort their communicator when they miss them.
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..logging import logger
from . import HealthSkipList, PayloadTransport

ACCEPTED, MISSING = b"ACCEPTED", b"MISSING"


# ------------------------------------------------------------------------------------------------- protocol (strings)
def request_stream(owner: str) -> str:
    return f"payload-req:{owner}"


def cleanup_stream(owner: str) -> str:
    return f"payload-cleanup:{owner}"


def response_key(transfer_id: str, attempt: int) -> str:
    return f"payload-resp:{transfer_id}:{attempt}"


def pair_name(owner: str, consumer: str, generation: int = 0) -> str:
    return f"payload-pair:{owner}>{consumer}:{generation}"


def make_ref(prefix: str, owner: str, tid: str, t: torch.Tensor) -> str:
    return f"{prefix}{owner}/{tid}/{str(t.dtype)[6:]}/{','.join(map(str, t.shape))}"


def parse_ref(key: str) -> Tuple[str, str, torch.dtype, List[int]]:
    owner, tid, dt, shape = key.split("/")
    return owner, tid, getattr(torch, dt), [int(s) for s in shape.split(",") if s]


# ------------------------------------------------------------------------------------------------- producer buffers
class SendBufferRegistry:
    """Tensors waiting to be fetched. Bounded: when ``capacity`` buffers are parked, ``register`` waits up to
    ``block_s`` for a slot and then drops the oldest buffer that is not being sent, so generation cannot outrun the
    fetches and fill the device. ``free`` and ``register`` are idempotent per id."""

    def __init__(self, capacity: int = 1024, block_s: float = 1.0):
        self.capacity, self.block_s = capacity, block_s
        self._items: "OrderedDict[str, Tuple[torch.Tensor, Any]]" = OrderedDict()
        self._busy: set = set()
        self._doomed: set = set()              # freed while a send was in flight: dropped when the send releases it
        self._cv = threading.Condition()
        self.evicted = self.freed = self.registered = 0

    def register(self, tid: str, tensor: torch.Tensor, ready_event=None) -> None:
        with self._cv:
            if tid in self._items:
                return
            deadline = time.monotonic() + self.block_s
            while len(self._items) >= self.capacity:
                left = deadline - time.monotonic()
                if left <= 0:
                    victim = next((k for k in self._items if k not in self._busy), None)
                    if victim is None:
                        raise RuntimeError("send-buffer registry is full and every buffer is being sent")
                    del self._items[victim]
                    self.evicted += 1
                    break
                self._cv.wait(left)
            self._items[tid] = (tensor, ready_event)
            self.registered += 1

    def acquire(self, tid: str) -> Optional[Tuple[torch.Tensor, Any]]:
        """The buffer for sending (protected from eviction until ``release``), or None when it is gone."""
        with self._cv:
            item = self._items.get(tid)
            if item is not None:
                self._busy.add(tid)
            return item

    def release(self, tid: str) -> None:
        with self._cv:
            self._busy.discard(tid)
            if tid in self._doomed:
                self._doomed.discard(tid)
                self.freed += int(self._items.pop(tid, None) is not None)
            self._cv.notify_all()

    def free(self, tid: str) -> bool:
        with self._cv:
            if tid in self._busy:                 # a send is in flight: ``release`` drops the buffer afterwards
                self._doomed.add(tid)
                return False
            gone = self._items.pop(tid, None) is not None
            self.freed += int(gone)
            self._cv.notify_all()
            return gone

    def __len__(self) -> int:
        return len(self._items)

    def __contains__(self, tid: str) -> bool:
        return tid in self._items


# ------------------------------------------------------------------------------------------------- communicator cache
class PairCommCache:
    """Two-rank communicators, built when a pair first transfers. At most ``max_live`` are kept (the least recently
    used one is aborted beyond that), at most ``max_concurrent_init`` are being built at once, and a pair whose
    communicator failed is quarantined for ``cooldown_s`` before it may be rebuilt. A dead replica only takes its own
    pairs with it."""

    def __init__(self, factory: Callable[[Any, int], Any], max_live: int = 16, max_concurrent_init: int = 2,
                 cooldown_s: float = 30.0, clock=time.monotonic):
        self.factory, self.max_live = factory, max_live
        self._live: "OrderedDict[Any, Any]" = OrderedDict()
        self._gen: Dict[Any, int] = {}
        self._lock = threading.Lock()
        self._init_slots = threading.Semaphore(max_concurrent_init)
        self._building: Dict[Any, threading.Lock] = {}
        self.health = HealthSkipList(cooldown_s, clock)
        self.built = self.evicted = 0

    def get(self, key) -> Optional[Any]:
        """The live communicator of ``key`` (built on demand, by one thread at a time per pair); None while the pair
        is quarantined."""
        with self._lock:
            build_lock = self._building.setdefault(key, threading.Lock())
        with build_lock:
            return self._get_locked(key)

    def _get_locked(self, key) -> Optional[Any]:
        with self._lock:
            comm = self._live.get(key)
            if comm is not None and not getattr(comm, "aborted", False):
                self._live.move_to_end(key)
                return comm
            if comm is not None:
                del self._live[key]
            if self.health.is_quarantined(key):
                return None
            gen = self._gen.get(key, 0)
        with self._init_slots:
            try:
                comm = self.factory(key, gen)
            except Exception as e:
                logger.warning("[payload/nccl] building the communicator of %s failed: %s", key, e)
                self.fail(key)
                return None
        victims = []
        with self._lock:
            self._live[key] = comm
            self.built += 1
            while len(self._live) > self.max_live:
                _, old = self._live.popitem(last=False)
                victims.append(old)
                self.evicted += 1
        for old in victims:
            old.abort()
        return comm

    def generation(self, key) -> int:
        with self._lock:
            return self._gen.get(key, 0)

    def set_generation(self, key, generation: int) -> None:
        """Follow the other side of the pair: it names the communicator it is about to build."""
        with self._lock:
            if self._gen.get(key, 0) == generation:
                return
            self._gen[key] = generation
            comm = self._live.pop(key, None)
        if comm is not None:
            comm.abort()

    def fail(self, key, quarantine: bool = True) -> None:
        """The pair's communicator is unusable: drop it; the next one is built under a new name."""
        with self._lock:
            comm = self._live.pop(key, None)
            self._gen[key] = self._gen.get(key, 0) + 1
            if quarantine:
                self.health.quarantine(key)
        if comm is not None:
            comm.abort()

    def close(self) -> None:
        with self._lock:
            comms, self._live = list(self._live.values()), OrderedDict()
        for c in comms:
            c.abort()

    def __len__(self) -> int:
        return len(self._live)


# ------------------------------------------------------------------------------------------------- transfer streams
class TransferStreams:
    """Low-priority CUDA streams for payload traffic, apart from the compute stream and from weight
    synchronisation; hand-over is by events. Without CUDA every helper is a no-op."""

    def __init__(self, device: Optional[torch.device], n: int = 2):
        self.cuda = device is not None and device.type == "cuda"
        self.streams = []
        if self.cuda:
            lo, _ = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, 0)
            self.streams = [torch.cuda.Stream(device, priority=lo) for _ in range(n)]
        self._next = 0

    def pick(self):
        if not self.cuda:
            return None
        self._next = (self._next + 1) % len(self.streams)
        return self.streams[self._next]

    def ready_event(self):
        """Recorded on the current (producing) stream; the transfer stream waits for it before sending."""
        if not self.cuda:
            return None
        ev = torch.cuda.Event()
        ev.record()
        return ev

    def on(self, stream, ready=None):
        import contextlib
        if not self.cuda or stream is None:
            return contextlib.nullcontext()
        if ready is not None:
            stream.wait_event(ready)
        return torch.cuda.stream(stream)

    def done_event(self, stream):
        if not self.cuda or stream is None:
            return None
        ev = torch.cuda.Event()
        ev.record(stream)
        return ev


class _KVRendezvous:
    """The two calls ``create_comm`` needs from a controller client, on top of the broker's key/value store."""

    def __init__(self, broker):
        self.broker = broker

    def post_nccl_comm_initiator(self, name: str, value: str) -> None:
        self.broker.kv_set("comm:" + name, value.encode(), ttl_s=600)

    def post_nccl_comm_acceptor(self, name: str, timeout_s: float = 60.0) -> str:
        end = time.monotonic() + timeout_s
        while time.monotonic() < end:
            raw = self.broker.kv_get("comm:" + name)
            if raw:
                return raw.decode() if isinstance(raw, (bytes, bytearray)) else raw
            time.sleep(0.01)
        raise TimeoutError(f"no rendezvous address for {name} within {timeout_s:.0f} s")


# ------------------------------------------------------------------------------------------------- the transport
class PairTransport(PayloadTransport):
    name = "nccl"
    completion_prefix = "nccl:"

    def setup(self, config=None, broker=None, device=None, owner: str = "", capacity: int = 1024,
              recv_timeout_s: Optional[float] = None, max_attempts: Optional[int] = None, max_live_comms: int = 16,
              cooldown_s: float = 30.0, **kw) -> None:
        super().setup(config, broker, device)
        custom = (getattr(config, "custom", None) or {}) if config is not None else {}
        self.owner = owner or uuid.uuid4().hex[:8]
        self.recv_timeout_s = float(recv_timeout_s if recv_timeout_s is not None else custom.get("nccl_recv_timeout", 5.0))
        self.max_attempts = int(max_attempts if max_attempts is not None else custom.get("nccl_read_max_attempts", 2))
        self.registry = SendBufferRegistry(capacity)
        self.streams = TransferStreams(device)
        self.cache = PairCommCache(self._build_comm, max_live_comms, cooldown_s=cooldown_s)
        self.endpoint_health = HealthSkipList(cooldown_s)
        self._stop = threading.Event()
        self._fetch_locks: Dict[str, threading.Lock] = {}
        self._fetch_guard = threading.Lock()
        self._threads: List[threading.Thread] = []
        self._serving = False
        self._seq = 0
        self.stats = {"sent": 0, "received": 0, "missing": 0, "cancelled": 0, "send_failed": 0}

    # ---- communicators: rank 0 = producer, rank 1 = consumer; the consumer hosts the rendezvous
    def _build_comm(self, key, generation: int):
        from ...parallel.dyncomm import create_comm
        owner, consumer, role = key
        name = pair_name(owner, consumer, generation)
        dev = self.device if self.device is not None else torch.device("cpu")
        return create_comm(_KVRendezvous(self.broker), name, 0 if role == "producer" else 1, 2, dev,
                           is_initiator=role == "consumer", timeout_s=max(10.0, 4 * self.recv_timeout_s),
                           op_timeout_s=self.recv_timeout_s)

    # ---- producer
    def publish(self, payload: torch.Tensor) -> str:
        self._ensure_serving()
        self._seq += 1
        tid = f"{self._seq}-{uuid.uuid4().hex[:8]}"
        t = payload.contiguous()
        self.registry.register(tid, t, self.streams.ready_event())
        return make_ref(self.completion_prefix, self.owner, tid, t)

    def _ensure_serving(self) -> None:
        if self._serving:
            return
        self._serving = True
        for fn, nm in ((self._serve_requests, "payload_serve"), (self._serve_cleanup, "payload_cleanup")):
            th = threading.Thread(target=fn, name=nm, daemon=True)
            th.start()
            self._threads.append(th)

    def _serve_requests(self) -> None:
        last = 0
        while not self._stop.is_set():
            try:
                msgs = self.broker.read(request_stream(self.owner), last, count=16, block_ms=100)
            except Exception as e:
                logger.warning("[payload/nccl] request read failed: %s", e)
                time.sleep(0.2)
                continue
            for mid, raw in msgs:
                last = mid
                try:
                    self._serve_one(json.loads(raw))
                except Exception as e:
                    logger.warning("[payload/nccl] serving a request failed: %s", e)

    def _serve_one(self, req: Dict[str, Any]) -> None:
        tid, consumer, attempt = req["tid"], req["consumer"], int(req.get("attempt", 0))
        item = self.registry.acquire(tid)
        key = response_key(f"{self.owner}/{tid}", attempt)
        if item is None:
            self.broker.kv_set(key, MISSING, ttl_s=60)
            self.stats["missing"] += 1
            return
        try:
            self.broker.kv_set(key, ACCEPTED, ttl_s=60)
            pair = (self.owner, consumer, "producer")
            self.cache.set_generation(pair, int(req.get("generation", 0)))
            comm = self.cache.get(pair)
            if comm is None:
                self.stats["send_failed"] += 1
                return
            tensor, ready = item
            stream = self.streams.pick()
            try:
                with self.streams.on(stream, ready):
                    comm.send(tensor, 1, timeout_s=self.recv_timeout_s)
                self.stats["sent"] += 1
            except Exception as e:
                logger.warning("[payload/nccl] send of %s to %s failed: %s", tid, consumer, e)
                self.cache.fail(pair)
                self.stats["send_failed"] += 1
        finally:
            self.registry.release(tid)

    def _serve_cleanup(self) -> None:
        last = 0
        while not self._stop.is_set():
            try:
                msgs = self.broker.read(cleanup_stream(self.owner), last, count=64, block_ms=200)
            except Exception:
                time.sleep(0.2)
                continue
            for mid, raw in msgs:
                last = mid
                for tid in json.loads(raw).get("tids", []):
                    self.registry.free(tid)

    # ---- consumer
    def sync_fetch(self, completion: str) -> Optional[torch.Tensor]:
        owner, tid, dtype, shape = parse_ref(self.cache_key(completion))
        if self.endpoint_health.is_quarantined(owner):
            return None
        # one transfer per producer at a time: the producer serves requests in order, and the receives on the pair's
        # communicator have to be posted in that same order whichever thread (prefetch or trainer) asks
        with self._fetch_guard:
            lock = self._fetch_locks.setdefault(owner, threading.Lock())
        with lock:
            return self._fetch_from(owner, tid, dtype, shape)

    def _fetch_from(self, owner: str, tid: str, dtype, shape) -> Optional[torch.Tensor]:
        if self.endpoint_health.is_quarantined(owner):
            return None
        me = self.owner
        pair = (owner, me, "consumer")
        for attempt in range(self.max_attempts):
            key = response_key(f"{owner}/{tid}", attempt)
            self.broker.kv_del(key)
            gen = self.cache.generation(pair)
            self.broker.publish(request_stream(owner), json.dumps(
                {"tid": tid, "consumer": me, "attempt": attempt, "generation": gen}).encode())
            answer = self._wait_answer(key)
            if answer == MISSING:                         # the buffer was recycled: the episode is dropped
                self.stats["missing"] += 1
                return None
            if answer != ACCEPTED:
                self.stats["cancelled"] += 1
                continue
            comm = self.cache.get(pair)
            if comm is None:
                continue
            dev = self.device if self.device is not None else torch.device("cpu")
            out = torch.empty(shape, dtype=dtype, device=dev)
            stream = self.streams.pick()
            try:
                with self.streams.on(stream):
                    comm.recv(out, 0, timeout_s=self.recv_timeout_s)
                done = self.streams.done_event(stream)
                if done is not None:
                    torch.cuda.current_stream().wait_event(done)     # the reader's stream waits, not the host
                self.stats["received"] += 1
                self.release_remote(owner, [tid])
                return out
            except Exception as e:
                logger.warning("[payload/nccl] recv of %s from %s failed (attempt %d): %s", tid, owner, attempt, e)
                self.cache.fail(pair, quarantine=False)
        self.endpoint_health.quarantine(owner)
        return None

    def _wait_answer(self, key: str) -> Optional[bytes]:
        wait = getattr(self.broker, "kv_wait", None)
        if wait is not None:
            return wait(key, self.recv_timeout_s)
        end = time.monotonic() + self.recv_timeout_s
        while time.monotonic() < end:
            v = self.broker.kv_get(key)
            if v:
                return v
            time.sleep(0.005)
        return None

    # ---- cleanup
    def release_remote(self, owner: str, tids: List[str]) -> None:
        self.broker.publish(cleanup_stream(owner), json.dumps({"tids": tids}).encode())

    def release(self, transfer_ids: List[str]) -> int:
        """Controller side: discarded rollouts. ``transfer_ids`` are cache keys (``owner/id/dtype/shape``)."""
        by_owner: Dict[str, List[str]] = {}
        for k in transfer_ids:
            owner, tid = k.split("/")[:2]
            by_owner.setdefault(owner, []).append(tid)
        for owner, tids in by_owner.items():
            self.release_remote(owner, tids)
        return len(transfer_ids)

    def shutdown(self) -> None:
        self._stop.set()
        for th in self._threads:
            th.join(timeout=1.0)
        self.cache.close()
