"""HTTP service: ``enqueue`` stores the request and returns a uuid at once, a pool of scoring threads runs the
requested handlers, ``pull`` returns the scores (or 202 while pending), ``push`` lets an external scorer deposit
scores under a uuid, ``ping`` reports liveness and the handlers loaded
(reward_service/cosmos_rl_reward/launcher/reward_serve.py:58-229). Scores expire after ``ttl_s``."""
from __future__ import annotations

import argparse
import queue
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, HTTPException, Request      # module level: route annotations are resolved by name
from fastapi.responses import JSONResponse

from ..utils.logging import logger
from . import protocol as P
from .handler import BaseRewardHandler, RewardHandlerRegistry


class ScoreStore:
    def __init__(self, ttl_s: float = 3600.0):
        self.ttl_s, self.lock = ttl_s, threading.Lock()
        self.items: Dict[str, Dict[str, Any]] = {}

    def put(self, key: str, reward: str, value: Dict[str, Any]) -> None:
        with self.lock:
            self.items.setdefault(key, {"t": time.time(), "scores": {}})["scores"][reward] = value

    def get(self, key: str, rewards: List[str]) -> Optional[Dict[str, Any]]:
        now = time.time()
        with self.lock:
            for k in [k for k, v in self.items.items() if now - v["t"] > self.ttl_s]:
                del self.items[k]
            it = self.items.get(key)
            if it is None or any(r not in it["scores"] for r in rewards):
                return None
            return {r: it["scores"][r] for r in rewards}


class RewardService:
    def __init__(self, rewards: List[str], num_workers: int = 2, device: str = "cpu", ttl_s: float = 3600.0,
                 handler_options: Optional[Dict[str, Dict[str, Any]]] = None):
        opts = handler_options or {}
        self.handlers: Dict[str, BaseRewardHandler] = {
            r: RewardHandlerRegistry.create(r, device=device, **opts.get(r, {})) for r in rewards}
        self.store = ScoreStore(ttl_s)
        self.tasks: "queue.Queue" = queue.Queue()
        self.pending: Dict[str, List[str]] = {}
        self.stop = threading.Event()
        self.workers = [threading.Thread(target=self._work, name=f"reward-{i}", daemon=True) for i in range(num_workers)]
        for w in self.workers:
            w.start()

    def enqueue(self, blob: bytes) -> str:
        rewards, meta, media = P.decode_request(blob)
        unknown = [r for r in rewards if r not in self.handlers]
        if unknown:
            raise KeyError(f"rewards not served here: {unknown}; serving {sorted(self.handlers)}")
        key = uuid.uuid4().hex
        self.pending[key] = rewards
        for r in rewards:
            self.tasks.put((key, r, media, meta))
        return key

    def _work(self) -> None:
        while not self.stop.is_set():
            try:
                key, r, media, meta = self.tasks.get(timeout=0.2)
            except queue.Empty:
                continue
            try:
                self.store.put(key, r, self.handlers[r].calculate_reward(media, meta))
            except Exception as e:  # noqa: BLE001  (a failing handler must not take the worker down)
                logger.exception("reward %s failed", r)
                self.store.put(key, r, {"error": str(e), "type": r})

    def pull(self, key: str, rewards: Optional[List[str]] = None) -> Optional[Dict[str, Any]]:
        return self.store.get(key, rewards or self.pending.get(key, []) or list(self.handlers))

    def close(self) -> None:
        self.stop.set()


def build_app(service: RewardService):
    app = FastAPI()

    @app.post(P.ENQUEUE)
    async def enqueue(request: Request):
        try:
            return {"uuid": service.enqueue(await request.body())}
        except (ValueError, KeyError) as e:
            raise HTTPException(status_code=400, detail=str(e))

    @app.post(P.PULL)
    async def pull(body: Dict[str, Any]):
        res = service.pull(body["uuid"], body.get("reward_fns"))
        if res is None:
            return JSONResponse({"status": "pending"}, status_code=202)
        return {"status": "done", "scores": res}

    @app.post(P.PUSH)
    async def push(body: Dict[str, Any]):
        service.store.put(body["uuid"], body["reward_fn"], {"scores": body["scores"], "type": body["reward_fn"]})
        return {"ok": True}

    @app.post(P.PING)
    async def ping():
        return {"ok": True, "rewards": sorted(service.handlers), "queued": service.tasks.qsize()}

    return app


def main(argv=None) -> None:
    import uvicorn
    ap = argparse.ArgumentParser(description="reward service")
    ap.add_argument("--rewards", nargs="+", default=["sharpness"], help=f"any of {RewardHandlerRegistry.known()}")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--workers", type=int, default=2)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    uvicorn.run(build_app(RewardService(a.rewards, a.workers, a.device)), host=a.host, port=a.port, log_level="warning")


if __name__ == "__main__":
    main()
