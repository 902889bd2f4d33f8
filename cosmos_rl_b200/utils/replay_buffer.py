"""Trajectory store on a shared file system: large rollout products (latents, sampler traces, action-chunk transitions,
pixel observations) are written once by the rollout worker and read by the policy worker; only a small id travels
through the controller (cosmos_rl/utils/replay_buffer.py:40-218 does this for VLA trajectories).

Writes go to a temporary name in the same folder and are renamed into place, so a reader never sees a partial file;
ids are random, so writers on several nodes need no coordination. ``cleanup`` removes entries nobody fetched (a trainer
that died between a rollout and its step)."""
from __future__ import annotations

import os
import time
import uuid
from typing import Any, Iterable, Optional

import torch


class ReplayBuffer:
    def __init__(self, buffer_dir: str):
        self.dir = buffer_dir
        os.makedirs(self.dir, exist_ok=True)

    def _path(self, key: str) -> str:
        if not key or any(c in key for c in "/\\.") or len(key) > 64:
            raise ValueError(f"bad trajectory id {key!r}")
        return os.path.join(self.dir, key + ".pt")

    def save(self, item: Any, key: Optional[str] = None) -> str:
        key = key or uuid.uuid4().hex
        path = self._path(key)
        tmp = f"{path}.tmp{os.getpid()}"
        torch.save(item, tmp)
        os.replace(tmp, path)
        return key

    def load(self, key: str, wait_s: float = 0.0) -> Any:
        """``wait_s``: a shared file system may show the file a moment after the id arrived."""
        path = self._path(key)
        deadline = time.time() + wait_s
        while not os.path.exists(path):
            if time.time() >= deadline:
                raise KeyError(f"trajectory {key} is not in {self.dir}")
            time.sleep(0.05)
        return torch.load(path, map_location="cpu", weights_only=False)

    def __contains__(self, key: str) -> bool:
        return os.path.exists(self._path(key))

    def delete(self, keys: Iterable[str]) -> int:
        n = 0
        for k in keys:
            try:
                os.unlink(self._path(k))
                n += 1
            except (FileNotFoundError, ValueError):
                pass
        return n

    def __len__(self) -> int:
        return sum(1 for f in os.listdir(self.dir) if f.endswith(".pt"))

    def cleanup(self, max_age_s: float) -> int:
        """Remove entries (and abandoned temporaries) older than ``max_age_s``."""
        now, n = time.time(), 0
        for f in os.listdir(self.dir):
            p = os.path.join(self.dir, f)
            try:
                if (f.endswith(".pt") or ".pt.tmp" in f) and now - os.path.getmtime(p) > max_age_s:
                    os.unlink(p)
                    n += 1
            except FileNotFoundError:
                pass
        return n


def buffer_dir_of(config) -> Optional[str]:
    """``[custom] replay_buffer_dir`` of the job file, else ``COSMOS_REPLAY_BUFFER_DIR``; None keeps trajectories in the
    memory of the process that made them (colocated jobs)."""
    d = (getattr(config, "custom", None) or {}).get("replay_buffer_dir") if config is not None else None
    return d or os.environ.get("COSMOS_REPLAY_BUFFER_DIR") or None
