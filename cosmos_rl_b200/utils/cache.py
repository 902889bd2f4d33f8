"""Disk cache for pre-processed dataset samples (``enable_dataset_cache``).

Tokenising a conversation or running an image processor costs far more than reading the result back, and SFT visits
every sample once per epoch. ``DiskCache`` keeps one file per sample index (``torch.save``), spread over sub-folders
of at most ``files_per_dir`` files, written in the background through a temporary name so that a reader never sees a
half-written file. When the writers fall behind, new entries are dropped instead of queued: the cache is an
optimisation and must never hold a training step back. The reference has the same facility
(cosmos_rl/utils/cache.py:25-95, used by cosmos_rl/policy/worker/sft_worker.py:70-190).
"""
from __future__ import annotations

import os
import shutil
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Optional

import torch

from .logging import logger


class DiskCache:
    def __init__(self, path: str, files_per_dir: int = 10000, writers: int = 4, max_pending: int = 64):
        self.path, self.files_per_dir, self.max_pending = path, files_per_dir, max_pending
        os.makedirs(path, exist_ok=True)
        self._pool: Optional[ThreadPoolExecutor] = ThreadPoolExecutor(max_workers=writers, thread_name_prefix="disk_cache")
        self._pending = 0
        self._lock = threading.Lock()
        self.hits = self.misses = self.dropped = 0

    def _file(self, idx: int) -> str:
        d = os.path.join(self.path, str(int(idx) // self.files_per_dir))
        os.makedirs(d, exist_ok=True)
        return os.path.join(d, f"{int(idx)}.pt")

    def set(self, idx: int, obj: Any) -> bool:
        """Queue ``obj`` for writing; False when the writers are saturated (the entry is skipped) or the cache is closed."""
        if self._pool is None:
            return False
        with self._lock:
            if self._pending >= self.max_pending:
                self.dropped += 1
                return False
            self._pending += 1
        path = self._file(idx)

        def write():
            tmp = f"{path}.{os.getpid()}.{threading.get_ident()}.tmp"
            try:
                torch.save(obj, tmp)
                os.replace(tmp, path)
            except Exception as e:  # noqa: BLE001  (a failed write only costs a later re-computation)
                logger.warning("[cache] writing %s failed: %s", path, e)
                try:
                    os.remove(tmp)
                except OSError:
                    pass
            finally:
                with self._lock:
                    self._pending -= 1
        self._pool.submit(write)
        return True

    def get(self, idx: int) -> Optional[Any]:
        path = self._file(idx)
        if not os.path.exists(path):
            self.misses += 1
            return None
        try:
            obj = torch.load(path, weights_only=False)
        except Exception as e:  # noqa: BLE001
            logger.warning("[cache] reading %s failed: %s", path, e)
            self.misses += 1
            return None
        self.hits += 1
        return obj

    def flush(self) -> None:
        """Wait for the queued writes (tests, and before a process hands the folder to another one)."""
        pool = self._pool
        if pool is not None:
            pool.shutdown(wait=True)
            self._pool = ThreadPoolExecutor(max_workers=4, thread_name_prefix="disk_cache")

    def clear(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None
        shutil.rmtree(self.path, ignore_errors=True)
