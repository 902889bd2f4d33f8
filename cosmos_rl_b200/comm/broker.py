"""Stream broker: append-only per-key message streams plus a small key/value store.

The reference runs a ``redis-server`` subprocess for this (cosmos_rl/utils/redis_stream.py:49-600,
cosmos_rl/dispatcher/controller.py:172-232). Here the controller hosts the broker itself:
``InProcessBroker`` lives in the controller process and is reached by workers over two HTTP routes
(``/api/stream/read`` with long-polling, ``/api/stream/publish``), so a job needs no extra daemon.
Stream semantics are those of XADD / XREAD: every message gets a monotonically increasing id and a
reader asks for messages after the last id it has seen.
"""
from __future__ import annotations

import base64
import threading
import time
from collections import defaultdict, deque
from typing import Any, Deque, Dict, List, Optional, Tuple


def command_stream(replica_name: str) -> str:
    return f"command-{replica_name}"


def rollout_stream(replica_name: str) -> str:
    return f"rollout-{replica_name}"


TEACHER_REQUEST_STREAM = "teacher-request"


class StreamBroker:
    def publish(self, stream: str, data: bytes) -> int:
        raise NotImplementedError

    def read(self, stream: str, last_id: int, count: int, block_ms: int) -> List[Tuple[int, bytes]]:
        raise NotImplementedError

    def kv_set(self, key: str, value: bytes, ttl_s: Optional[float] = None) -> None:
        raise NotImplementedError

    def kv_get(self, key: str) -> Optional[bytes]:
        raise NotImplementedError

    def kv_del(self, key: str) -> None:
        raise NotImplementedError


class InProcessBroker(StreamBroker):
    def __init__(self, maxlen: int = 100_000):
        self._streams: Dict[str, Deque[Tuple[int, bytes]]] = defaultdict(lambda: deque(maxlen=maxlen))
        self._next_id: Dict[str, int] = defaultdict(int)
        self._cv = threading.Condition()
        self._kv: Dict[str, Tuple[bytes, Optional[float]]] = {}
        self._groups: Dict[Tuple[str, str], int] = {}

    def publish(self, stream: str, data: bytes) -> int:
        with self._cv:
            self._next_id[stream] += 1
            mid = self._next_id[stream]
            self._streams[stream].append((mid, data))
            self._cv.notify_all()
            return mid

    def _after(self, stream: str, last_id: int, count: int):
        q = self._streams.get(stream)
        if not q:
            return []
        out = []
        for mid, data in q:
            if mid > last_id:
                out.append((mid, data))
                if len(out) >= count:
                    break
        return out

    def read(self, stream: str, last_id: int, count: int = 1, block_ms: int = 0):
        deadline = time.monotonic() + block_ms / 1000.0
        with self._cv:
            while True:
                out = self._after(stream, last_id, count)
                if out:
                    return out
                remaining = deadline - time.monotonic()
                if remaining <= 0:
                    return []
                self._cv.wait(timeout=remaining)

    def read_group(self, stream: str, group: str, count: int = 1, block_ms: int = 0):
        """Consumer-group read: each message is delivered to exactly one reader of the group
        (used for teacher requests, cosmos_rl/utils/redis_stream.py:287-478)."""
        deadline = time.monotonic() + block_ms / 1000.0
        with self._cv:
            while True:
                last = self._groups.get((stream, group), 0)
                out = self._after(stream, last, count)
                if out:
                    self._groups[(stream, group)] = out[-1][0]
                    return out
                remaining = deadline - time.monotonic()
                if remaining <= 0:
                    return []
                self._cv.wait(timeout=remaining)

    def length(self, stream: str) -> int:
        with self._cv:
            return len(self._streams.get(stream, ()))

    def kv_set(self, key, value, ttl_s=None):
        with self._cv:
            self._kv[key] = (value, time.monotonic() + ttl_s if ttl_s else None)
            self._cv.notify_all()

    def kv_get(self, key):
        with self._cv:
            item = self._kv.get(key)
            if item is None:
                return None
            if item[1] is not None and item[1] < time.monotonic():
                del self._kv[key]
                return None
            return item[0]

    def kv_wait(self, key: str, timeout_s: float) -> Optional[bytes]:
        deadline = time.monotonic() + timeout_s
        with self._cv:
            while True:
                item = self._kv.get(key)
                if item is not None:
                    return item[0]
                remaining = deadline - time.monotonic()
                if remaining <= 0:
                    return None
                self._cv.wait(timeout=remaining)

    def kv_del(self, key):
        with self._cv:
            self._kv.pop(key, None)


class HttpBrokerClient(StreamBroker):
    """Worker-side view of the controller-hosted broker."""

    def __init__(self, api_client):
        self.api = api_client

    def publish(self, stream, data):
        from ..utils.api_suffix import COSMOS_API_STREAM_PUBLISH_SUFFIX
        r = self.api.post(COSMOS_API_STREAM_PUBLISH_SUFFIX,
                          {"stream": stream, "data": base64.b64encode(data).decode()})
        return r.get("id", 0)

    def read(self, stream, last_id, count=1, block_ms=0):
        from ..utils.api_suffix import COSMOS_API_STREAM_READ_SUFFIX
        r = self.api.get(COSMOS_API_STREAM_READ_SUFFIX,
                         {"stream": stream, "last_id": last_id, "count": count, "block_ms": block_ms},
                         timeout=block_ms / 1000.0 + 30.0)
        return [(m["id"], base64.b64decode(m["data"])) for m in r.get("messages", [])]

    def read_group(self, stream, group, count=1, block_ms=0):
        from ..utils.api_suffix import COSMOS_API_STREAM_READ_SUFFIX
        r = self.api.get(COSMOS_API_STREAM_READ_SUFFIX,
                         {"stream": stream, "group": group, "count": count, "block_ms": block_ms},
                         timeout=block_ms / 1000.0 + 30.0)
        return [(m["id"], base64.b64decode(m["data"])) for m in r.get("messages", [])]

    def kv_set(self, key, value, ttl_s=None):
        from ..utils.api_suffix import COSMOS_API_KV_SUFFIX
        self.api.post(COSMOS_API_KV_SUFFIX, {"key": key, "value": base64.b64encode(value).decode(), "ttl_s": ttl_s})

    def kv_get(self, key):
        from ..utils.api_suffix import COSMOS_API_KV_SUFFIX
        r = self.api.get(COSMOS_API_KV_SUFFIX, {"key": key})
        v = r.get("value")
        return base64.b64decode(v) if v is not None else None

    def kv_del(self, key):
        from ..utils.api_suffix import COSMOS_API_KV_SUFFIX
        self.api.post(COSMOS_API_KV_SUFFIX, {"key": key, "delete": True})


class RedisBroker(StreamBroker):  # pragma: no cover - needs a redis server
    """Adapter for deployments that already run Redis (``redis = "<port>"`` in the job file)."""

    def __init__(self, host: str, port: int):
        import redis  # gated: not part of the base image
        self.r = redis.Redis(host=host, port=port)

    def publish(self, stream, data):
        mid = self.r.xadd(stream, {"d": data})
        return int(mid.decode().split("-")[0])

    def read(self, stream, last_id, count=1, block_ms=0):
        res = self.r.xread({stream: f"{last_id}-0" if last_id else "0-0"}, count=count, block=block_ms or None)
        out = []
        for _, msgs in res or []:
            for mid, fields in msgs:
                out.append((int(mid.decode().split("-")[0]), fields[b"d"]))
        return out

    def kv_set(self, key, value, ttl_s=None):
        self.r.set(key, value, ex=int(ttl_s) if ttl_s else None)

    def kv_get(self, key):
        return self.r.get(key)

    def kv_del(self, key):
        self.r.delete(key)
