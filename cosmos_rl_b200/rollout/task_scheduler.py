"""Asynchronous rollout generation (``rollout.mode = "async"``): a producer-consumer scheduler between the worker's
control loop and the generation engine.

The reference drives vLLM's AsyncLLM with one coroutine per payload and a semaphore of ``max_concurrent_requests``
(cosmos_rl/rollout/worker/asynchronous/rollout_task_scheduler.py:51-871, cosmos_rl/rollout/vllm_rollout/
vllm_rollout_async.py:41-347). The engine here batches continuously inside one call, so concurrency is expressed the
way that engine wants it: the generation thread takes up to ``max_concurrent_requests`` queued payloads per engine
call and the control loop never blocks on generation - it keeps fetching prompts, answering commands and reporting
finished rollouts while a batch decodes. ``paused()`` fences the engine for weight updates: it returns once the batch
in flight has finished and holds new batches back until the block exits.
"""
from __future__ import annotations

import queue
import threading
import time
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Sequence

from ..utils.logging import logger


@dataclass
class RolloutTask:
    idx: int
    payload: Any
    is_validation: bool = False
    submitted_at: float = field(default_factory=time.time)


@dataclass
class CompletedRollout:
    idx: int
    payload: Any
    result: Any
    is_validation: bool = False
    error: Optional[BaseException] = None
    latency_s: float = 0.0


class RolloutTaskScheduler:
    """``generate(payloads, is_validation) -> results`` is called on the scheduler's thread with 1 to
    ``max_concurrent_requests`` payloads of one kind (training or validation)."""

    def __init__(self, generate: Callable[[Sequence[Any], bool], Sequence[Any]], max_concurrent_requests: int = 10,
                 poll_s: float = 0.01):
        if max_concurrent_requests < 1:
            raise ValueError("max_concurrent_requests must be positive")
        self.generate, self.max_batch, self.poll_s = generate, int(max_concurrent_requests), poll_s
        self.tasks: "queue.Queue[RolloutTask]" = queue.Queue()
        self.done: "queue.Queue[CompletedRollout]" = queue.Queue()
        self._running, self._paused, self._idle = threading.Event(), threading.Event(), threading.Event()
        self._idle.set()
        self._gate = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._held: Optional[RolloutTask] = None        # first task of the other kind, kept for the next batch
        self.stats = {"batches": 0, "tasks": 0, "errors": 0, "busy_s": 0.0}

    # ------------------------------------------------------------------ producer side
    def put_rollout(self, task: RolloutTask) -> None:
        self.tasks.put(task)

    def get(self, block: bool = False, timeout: Optional[float] = None) -> Optional[CompletedRollout]:
        try:
            return self.done.get(block=block, timeout=timeout)
        except queue.Empty:
            return None

    def get_all(self) -> List[CompletedRollout]:
        out = []
        while True:
            c = self.get()
            if c is None:
                return out
            out.append(c)

    def pending(self) -> int:
        return self.tasks.qsize() + (1 if self._held is not None else 0) + (0 if self._idle.is_set() else 1)

    def is_idle(self) -> bool:
        return self._idle.is_set() and self.tasks.empty() and self._held is None

    # ------------------------------------------------------------------ life cycle
    def start(self) -> None:
        if self._thread is not None:
            return
        self._running.set()
        self._thread = threading.Thread(target=self._loop, name="rollout-task-scheduler", daemon=True)
        self._thread.start()

    def stop(self, wait_for_queue: bool = True, timeout_s: float = 600.0) -> None:
        """Finish what is queued (or only the batch in flight) and end the thread."""
        if self._thread is None:
            return
        deadline = time.time() + timeout_s
        if wait_for_queue:
            self.resume()
            while not self.is_idle() and time.time() < deadline:
                time.sleep(self.poll_s)
        self._running.clear()
        self._thread.join(max(0.0, deadline - time.time()))
        self._thread = None

    def pause(self, wait_for_active_tasks: bool = True, timeout_s: float = 600.0) -> bool:
        with self._gate:
            self._paused.set()
        return self._idle.wait(timeout_s) if wait_for_active_tasks else True

    def resume(self) -> None:
        self._paused.clear()

    @contextmanager
    def paused(self, wait_for_active_tasks: bool = True):
        """No engine call runs inside the block (weight updates, validation on the control thread)."""
        was = self._paused.is_set()
        if not self.pause(wait_for_active_tasks):
            logger.warning("[Rollout] the batch in flight did not finish before the pause timeout")
        try:
            yield self
        finally:
            if not was:
                self.resume()

    # ------------------------------------------------------------------ consumer side
    def _next_batch(self) -> List[RolloutTask]:
        batch: List[RolloutTask] = []
        if self._held is not None:
            batch.append(self._held)
            self._held = None
        while len(batch) < self.max_batch:
            try:
                t = self.tasks.get(timeout=self.poll_s if not batch else 0.0)
            except queue.Empty:
                break
            if batch and t.is_validation != batch[0].is_validation:
                self._held = t
                break
            batch.append(t)
        return batch

    def _loop(self) -> None:
        while self._running.is_set():
            if self._paused.is_set():
                time.sleep(self.poll_s)
                continue
            with self._gate:                    # pause() takes the same lock: a batch is either claimed before the
                if self._paused.is_set():       # pause flag goes up (and pause waits for it) or not started at all
                    continue
                batch = self._next_batch()
                if batch:
                    self._idle.clear()
            if not batch:
                continue
            t0 = time.time()
            try:
                results = list(self.generate([t.payload for t in batch], batch[0].is_validation))
                if len(results) != len(batch):
                    raise RuntimeError(f"engine returned {len(results)} results for {len(batch)} payloads")
                err = None
            except BaseException as e:          # noqa: BLE001 (reported per task; the control loop decides)
                logger.error("[Rollout] generation of %d payloads failed: %s", len(batch), e)
                results, err = [None] * len(batch), e
                self.stats["errors"] += 1
            now = time.time()
            for t, r in zip(batch, results):
                self.done.put(CompletedRollout(t.idx, t.payload, r, t.is_validation, err, now - t.submitted_at))
            self.stats["batches"] += 1
            self.stats["tasks"] += len(batch)
            self.stats["busy_s"] += now - t0
            self._idle.set()
        self._idle.set()
