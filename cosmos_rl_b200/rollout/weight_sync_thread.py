"""Asynchronous weight synchronisation for a rollout replica: a background thread with its own CUDA stream
receives new weights into a *buffer* copy of the parameters while generation continues on the live copy;
``sync_buffer_to_live`` swaps the newest complete buffer in between two generation batches
(cosmos_rl/rollout/worker/weight_sync.py:94-971: WeightSyncThread, sync_buffer_to_live, fence / drain).

Versions are monotone: the live copy only ever jumps forward to the newest buffered version (intermediate
versions that were superseded before adoption are skipped)."""
from __future__ import annotations

import queue
import threading
from typing import Callable, Optional

import torch


class WeightSyncThread:
    def __init__(self, live_flat: torch.Tensor, receive_fn: Callable[[torch.Tensor, object], None]):
        """``receive_fn(buffer, request)`` fills ``buffer`` with the weights named by ``request`` (a peer pull,
        a collective receive ...); it runs on this thread's stream."""
        self.live = live_flat
        self.buffer = torch.empty_like(live_flat)
        self.receive_fn = receive_fn
        self.stream = torch.cuda.Stream() if live_flat.is_cuda else None
        self.requests: "queue.Queue" = queue.Queue()
        self.buf_version = -1
        self.live_version = -1
        self.lock = threading.Lock()
        self.ready = threading.Event()
        self.stop_flag = threading.Event()
        self.error: Optional[BaseException] = None
        self.thread = threading.Thread(target=self._loop, name="weight_sync", daemon=True)
        self.thread.start()

    def submit(self, version: int, request=None) -> None:
        self.requests.put((version, request))

    def _loop(self) -> None:
        while not self.stop_flag.is_set():
            try:
                version, request = self.requests.get(timeout=0.1)
            except queue.Empty:
                continue
            # drop-to-latest: only the newest queued request is worth receiving
            while not self.requests.empty():
                version, request = self.requests.get_nowait()
            try:
                with self.lock:
                    if self.stream is not None:
                        with torch.cuda.stream(self.stream):
                            self.receive_fn(self.buffer, request)
                        self.stream.synchronize()
                    else:
                        self.receive_fn(self.buffer, request)
                    self.buf_version = version
                self.ready.set()
            except BaseException as e:  # surfaced to the main loop by sync_buffer_to_live
                self.error = e
                self.ready.set()

    def sync_buffer_to_live(self) -> int:
        """Adopt the newest buffered weights if they are newer than the live ones. Called between batches."""
        if self.error is not None:
            err, self.error = self.error, None
            raise err
        with self.lock:
            if self.buf_version > self.live_version:
                self.live.copy_(self.buffer)
                self.live_version = self.buf_version
        return self.live_version

    def fence(self, timeout_s: float = 600.0) -> bool:
        """Wait (bounded) until every submitted request has been received."""
        import time
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            if self.requests.empty() and not self.lock.locked():
                return True
            time.sleep(0.005)
        return False

    def stop(self) -> None:
        self.stop_flag.set()
        self.thread.join(timeout=5)
