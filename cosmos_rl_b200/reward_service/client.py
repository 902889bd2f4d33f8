"""Client of the reward service: enqueue, then poll ``pull`` until the scores are there
(reward_service/cosmos_rl_reward/utils/client.py, example/image_client.py)."""
from __future__ import annotations

import time
from typing import Any, Dict, List, Optional

import torch

from . import protocol as P


class RewardClient:
    def __init__(self, url: str, timeout_s: float = 60.0, poll_s: float = 0.05):
        self.url, self.timeout_s, self.poll_s = url.rstrip("/"), timeout_s, poll_s

    def enqueue(self, reward_fns: List[str], metadata: Dict[str, Any], media: Optional[torch.Tensor] = None) -> str:
        import requests
        r = requests.post(self.url + P.ENQUEUE, data=P.encode_request(reward_fns, metadata, media),
                          headers={"Content-Type": "application/octet-stream"}, timeout=self.timeout_s)
        r.raise_for_status()
        return r.json()["uuid"]

    def pull(self, key: str, reward_fns: Optional[List[str]] = None, block: bool = True) -> Optional[Dict[str, Any]]:
        import requests
        t0 = time.time()
        while True:
            r = requests.post(self.url + P.PULL, json={"uuid": key, "reward_fns": reward_fns}, timeout=self.timeout_s)
            if r.status_code == 200:
                return r.json()["scores"]
            if r.status_code != 202:
                r.raise_for_status()
            if not block:
                return None
            if time.time() - t0 > self.timeout_s:
                raise TimeoutError(f"scores for {key} not ready after {self.timeout_s:.0f} s")
            time.sleep(self.poll_s)

    def score(self, reward_fns: List[str], metadata: Dict[str, Any], media: Optional[torch.Tensor] = None) -> Dict[str, Any]:
        return self.pull(self.enqueue(reward_fns, metadata, media), reward_fns)

    def ping(self) -> Dict[str, Any]:
        import requests
        r = requests.post(self.url + P.PING, timeout=self.timeout_s)
        r.raise_for_status()
        return r.json()
