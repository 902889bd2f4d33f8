"""Pluggable rollout -> policy bulk-payload path (cosmos_rl/utils/payload_transport/registry.py:59-573,
strategy.py:41-170, rotation.py:47-121, prefetch_mixin.py).

Small completions travel inline in the rollout message (the default ``broker`` transport). A transport with a
``completion_prefix`` replaces the completion by a short reference string ``<prefix><transfer id>``; the policy
side resolves references in bulk on a prefetch thread before the step needs them, falls back to a blocking
single fetch on a miss, and the controller tells the producer to release resources of discarded rollouts.

Shipped transports: ``broker`` (inline), ``kv`` (tensors parked in the controller key/value store; works on any
machine), ``peer`` (tensors parked in a peer-visible device ring on the rollout GPU and pulled over NVLink by
the policy rank with plain peer loads; same box only), ``nccl`` (two-rank communicators between producer and
consumer with a request / answer handshake over the broker, ``pair.py``).
"""
from __future__ import annotations

import io
import threading
import time
import uuid
from typing import Any, Dict, Iterable, List, Optional, Tuple, Type

import torch

from ..logging import logger


class HealthSkipList:
    """Keys (endpoints, peers) quarantined for a cool-down after a failure."""

    def __init__(self, cooldown_s: float = 30.0, clock=time.monotonic):
        self.cooldown_s, self.clock = cooldown_s, clock
        self._until: Dict[Any, float] = {}

    def quarantine(self, key, cooldown: Optional[float] = None) -> None:
        self._until[key] = self.clock() + (self.cooldown_s if cooldown is None else cooldown)

    def is_quarantined(self, key) -> bool:
        t = self._until.get(key)
        if t is None:
            return False
        if self.clock() >= t:
            del self._until[key]
            return False
        return True

    def healthy(self, keys: Iterable[Any]) -> List[Any]:
        """Keys not in quarantine; if all are, every key (better a sick endpoint than none)."""
        keys = list(keys)
        ok = [k for k in keys if not self.is_quarantined(k)]
        return ok or keys

    def clear(self, key=None) -> None:
        self._until.clear() if key is None else self._until.pop(key, None)

    def __len__(self) -> int:
        return sum(1 for k in list(self._until) if self.is_quarantined(k))


class PayloadTransport:
    name: str = ""
    completion_prefix: Optional[str] = None

    def setup(self, config=None, broker=None, device=None, **kw) -> None:
        self.config, self.broker, self.device = config, broker, device

    def shutdown(self) -> None:
        pass

    # ---- producer (rollout) side
    def publish(self, payload: Any) -> Any:
        """Park ``payload`` and return what goes into the rollout message instead of it."""
        return payload

    def release(self, transfer_ids: List[str]) -> int:
        return 0

    # ---- consumer (policy) side
    def should_intercept(self, completion: Any) -> bool:
        return (self.completion_prefix is not None and isinstance(completion, str)
                and completion.startswith(self.completion_prefix))

    def cache_key(self, completion: str) -> str:
        return completion[len(self.completion_prefix):]

    def fetch_batch(self, refs: List[str]) -> Dict[str, Any]:
        out = {}
        for r in refs:
            v = self.sync_fetch(r)
            if v is not None:
                out[self.cache_key(r)] = v
        return out

    def sync_fetch(self, completion: str) -> Optional[Any]:
        return None


class BrokerTransport(PayloadTransport):
    """Inline default: nothing to park, nothing to resolve."""
    name = "broker"


def _dumps(obj) -> bytes:
    buf = io.BytesIO()
    torch.save(obj, buf)
    return buf.getvalue()


class KVTransport(PayloadTransport):
    name = "kv"
    completion_prefix = "kv://"

    def publish(self, payload):
        tid = uuid.uuid4().hex
        self.broker.kv_set("payload:" + tid, _dumps(payload), ttl_s=3600)
        return self.completion_prefix + tid

    def sync_fetch(self, completion):
        try:
            raw = self.broker.kv_get("payload:" + self.cache_key(completion))
            return None if raw is None else torch.load(io.BytesIO(raw), weights_only=False)
        except Exception as e:      # a failed fetch degrades to "skip this episode"
            logger.warning("[payload/kv] fetch of %s failed: %s", completion, e)
            return None

    def release(self, transfer_ids):
        for t in transfer_ids:
            self.broker.kv_set("payload:" + t, b"", ttl_s=0.001)
        return len(transfer_ids)


class PeerTransport(PayloadTransport):
    """Device ring on the producer GPU, exported once through the key/value store as a CUDA IPC handle; the
    consumer maps it once per producer and copies slots out with a device copy over NVLink."""
    name = "peer"
    completion_prefix = "peer://"

    def setup(self, config=None, broker=None, device=None, ring_bytes: int = 256 << 20, owner: str = "", **kw):
        super().setup(config, broker, device)
        self.owner, self.ring_bytes, self.head = owner, ring_bytes, 0
        self.ring = None
        self._maps: Dict[str, Any] = {}
        self.skip = HealthSkipList()

    def _ensure_ring(self):
        if self.ring is None:
            from ...parallel.peer import PeerBuffer
            self.ring = PeerBuffer(self.ring_bytes, self.device)
            self.broker.kv_set(f"payload-ring:{self.owner}", self.ring.export())

    def publish(self, payload: torch.Tensor):
        self._ensure_ring()
        n = payload.numel() * payload.element_size()
        n_al = (n + 255) & ~255
        if n_al > self.ring_bytes:
            raise ValueError("payload larger than the transport ring")
        if self.head + n_al > self.ring_bytes:
            self.head = 0
        off = self.head
        self.ring.tensor(torch.uint8)[off:off + n].copy_(payload.contiguous().view(torch.uint8).flatten())
        torch.cuda.current_stream().synchronize()
        self.head += n_al
        shape = ",".join(map(str, payload.shape))
        return f"{self.completion_prefix}{self.owner}/{off}/{n}/{str(payload.dtype)[6:]}/{shape}"

    def sync_fetch(self, completion):
        owner, off, n, dt, shape = self.cache_key(completion).split("/")
        if self.skip.is_quarantined(owner):
            return None
        try:
            m = self._maps.get(owner)
            if m is None:
                from ...parallel.peer import PeerMapping
                m = self._maps[owner] = PeerMapping(self.broker.kv_get(f"payload-ring:{owner}"), self.ring_bytes, self.device)
            src = m.tensor(torch.uint8)[int(off):int(off) + int(n)]
            out = torch.empty(int(n), dtype=torch.uint8, device=self.device)
            out.copy_(src)
            return out.view(getattr(torch, dt)).view([int(s) for s in shape.split(",") if s])
        except Exception as e:
            self.skip.quarantine(owner)
            logger.warning("[payload/peer] fetch from %s failed: %s", owner, e)
            return None


class PayloadTransportRegistry:
    _by_name: Dict[str, PayloadTransport] = {}

    @classmethod
    def register(cls, transport: PayloadTransport) -> None:
        cls._by_name[transport.name] = transport

    @classmethod
    def register_class(cls, transport_cls: Type[PayloadTransport]) -> None:
        cls.register(transport_cls())

    @classmethod
    def get(cls, name: str) -> PayloadTransport:
        if name not in cls._by_name:
            raise KeyError(f"unknown payload transport {name!r}; known: {sorted(cls._by_name)}")
        return cls._by_name[name]

    @classmethod
    def active_for_completion(cls, completion: Any) -> Optional[PayloadTransport]:
        for t in cls._by_name.values():
            if t.should_intercept(completion):
                return t
        return None

    @classmethod
    def handle_discarded(cls, completions: Iterable[Any]) -> int:
        """Controller side: group references of discarded rollouts by transport and release them."""
        groups: Dict[str, List[str]] = {}
        for c in completions:
            t = cls.active_for_completion(c)
            if t is not None:
                groups.setdefault(t.name, []).append(t.cache_key(c))
        return sum(cls._by_name[n].release(ids) for n, ids in groups.items())

    @classmethod
    def reset(cls) -> None:
        cls._by_name = {}
        from .pair import PairTransport
        for c in (BrokerTransport, KVTransport, PeerTransport, PairTransport):
            cls.register_class(c)


PayloadTransportRegistry.reset()


def get_payload_transfer_mode(config) -> str:
    custom = getattr(config, "custom", None) or {}
    mode = custom.get("payload_transfer", "broker")
    if mode in ("redis", "", None, "broker") and custom.get("nccl_payload_transfer"):
        return "nccl"                               # the older boolean switch of the reference
    return "broker" if mode in ("redis", "", None) else mode


class PayloadPrefetcher:
    """Resolves references of upcoming rollouts on a background thread; ``resolve`` serves from the cache, waits for a
    reference the thread is still working on (at most ``prefetch_timeout_s``; a second fetch of the same transfer
    would find its buffer already handed out) and falls back to one blocking fetch for references it never saw."""

    def __init__(self, transport: PayloadTransport, max_cached: int = 4096, prefetch_timeout_s: Optional[float] = None):
        self.t, self.max_cached = transport, max_cached
        custom = (getattr(getattr(transport, "config", None), "custom", None) or {})
        self.prefetch_timeout_s = float(prefetch_timeout_s if prefetch_timeout_s is not None
                                        else custom.get("nccl_prefetch_timeout", 30.0))
        self.cache: Dict[str, Any] = {}
        self.inflight: set = set()
        self.lock = threading.Condition()
        self.pending: List[List[str]] = []
        self.wake = threading.Event()
        self.stop_flag = threading.Event()
        self.hits = self.misses = self.failed = 0
        self.thread = threading.Thread(target=self._loop, name="payload_prefetch", daemon=True)
        self.thread.start()

    def prefetch(self, completions: List[Any]) -> int:
        refs = [c for c in completions if self.t.should_intercept(c)]
        if refs:
            with self.lock:
                self.pending.append(refs)
                self.inflight.update(self.t.cache_key(r) for r in refs)
            self.wake.set()
        return len(refs)

    def _loop(self) -> None:
        while not self.stop_flag.is_set():
            self.wake.wait(0.1)
            self.wake.clear()
            while True:
                with self.lock:
                    refs = self.pending.pop(0) if self.pending else None
                if refs is None:
                    break
                for r in refs:                      # one by one, so that a waiting ``resolve`` is served early
                    try:
                        got = self.t.fetch_batch([r])
                    except Exception as e:
                        logger.warning("[payload] prefetch of %s failed: %s", r, e)
                        got = {}
                    with self.lock:
                        self.cache.update(got)
                        self.inflight.discard(self.t.cache_key(r))
                        while len(self.cache) > self.max_cached:
                            self.cache.pop(next(iter(self.cache)))
                        self.lock.notify_all()

    def resolve(self, completion: Any) -> Any:
        if not self.t.should_intercept(completion):
            return completion
        key = self.t.cache_key(completion)
        seen = False
        with self.lock:
            end = time.monotonic() + self.prefetch_timeout_s
            while key in self.inflight and key not in self.cache:
                seen = True
                left = end - time.monotonic()
                if left <= 0:
                    break
                self.lock.wait(left)
            v = self.cache.pop(key, None)
        if v is not None:
            self.hits += 1
            return v
        self.misses += 1
        if seen:                                     # the prefetch thread tried and failed (or ran out of time)
            self.failed += 1
            return None
        v = self.t.sync_fetch(completion)
        if v is None:
            self.failed += 1
        return v

    def drain(self, timeout_s: float = 5.0) -> bool:
        end = time.time() + timeout_s
        while time.time() < end:
            with self.lock:
                if not self.pending and not self.wake.is_set():
                    return True
            time.sleep(0.005)
        return False

    def shutdown(self) -> None:
        self.stop_flag.set()
        self.wake.set()
        self.thread.join(timeout=2)


# ---------------------------------------------------------------------------------------------------
# token ids + log-probs of a completion as one tensor (what the LLM workers park with a transport)
# ---------------------------------------------------------------------------------------------------
def pack_completion(token_ids: List[List[int]], logprobs: Optional[List[List[float]]], device=None) -> torch.Tensor:
    """``[2, n, k]`` float32: plane 0 the ids (exact below 2**24), plane 1 the log-probs (zeros when absent)."""
    ids = torch.tensor(token_ids, dtype=torch.float32)
    lps = torch.tensor(logprobs, dtype=torch.float32) if logprobs else torch.zeros_like(ids)
    out = torch.stack([ids, lps])
    return out.to(device) if device is not None else out


def unpack_completion(t: torch.Tensor, with_logprobs: bool = True):
    t = t.detach().to("cpu")
    ids = t[0].to(torch.int64).tolist()
    return ids, (t[1].tolist() if with_logprobs else None)


def park_payload(transport: PayloadTransport, payload, device=None) -> int:
    """Producer side: move the per-token data of every completion of ``payload`` (an ``RLPayload``) out of the
    message. Returns the number of completions parked."""
    if transport.completion_prefix is None or not payload.completion_token_ids:
        return 0
    refs = []
    for i, ids in enumerate(payload.completion_token_ids):
        lps = payload.completion_logprobs[i] if payload.completion_logprobs else None
        refs.append(transport.publish(pack_completion(ids, lps, device)))
    payload.payload_refs = refs
    payload.extra_info = dict(payload.extra_info or {}, payload_has_logprobs=bool(payload.completion_logprobs),
                              completion_lengths=[len(x) for x in payload.completion_token_ids])
    payload.completion_token_ids = None
    payload.completion_logprobs = None
    return len(refs)


def restore_rollout(prefetcher: "PayloadPrefetcher", rollout) -> bool:
    """Consumer side: put the per-token data back into ``rollout``. False when the payload could not be fetched (the
    rollout then trains from its text, or is skipped by the caller)."""
    if not rollout.payload_ref:
        return True
    t = prefetcher.resolve(rollout.payload_ref)
    if t is None or isinstance(t, str):
        return False
    has_lp = bool((rollout.extra_info or {}).get("payload_has_logprobs", True))
    rollout.completion_token_ids, rollout.completion_logprobs = unpack_completion(t, has_lp)
    rollout.payload_ref = ""
    return True
