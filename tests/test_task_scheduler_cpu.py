"""Asynchronous rollout scheduler: batching, pause fence, error reporting, shutdown."""
import threading
import time

import pytest

from cosmos_rl_b200.rollout.task_scheduler import RolloutTask, RolloutTaskScheduler


def _collect(s, n, timeout=5.0):
    out, t0 = [], time.time()
    while len(out) < n and time.time() - t0 < timeout:
        c = s.get(block=True, timeout=0.05)
        if c is not None:
            out.append(c)
    return out


def test_batches_up_to_the_concurrency_limit_and_keeps_kinds_apart():
    calls = []

    def gen(payloads, is_validation):
        calls.append((list(payloads), is_validation))
        time.sleep(0.02)
        return [p * 10 for p in payloads]

    s = RolloutTaskScheduler(gen, max_concurrent_requests=3)
    for i in range(7):
        s.put_rollout(RolloutTask(i, i, is_validation=(i == 4)))
    s.start()
    done = _collect(s, 7)
    s.stop()
    assert sorted((c.idx, c.result) for c in done) == [(i, i * 10) for i in range(7)]
    assert all(len(p) <= 3 for p, _ in calls)
    assert ([4], True) in calls and all(4 not in p for p, v in calls if not v)     # validation goes in its own call
    assert s.stats["tasks"] == 7 and s.is_idle()


def test_pause_waits_for_the_batch_in_flight_and_holds_new_ones_back():
    started, release = threading.Event(), threading.Event()
    calls = []

    def gen(payloads, is_validation):
        calls.append(list(payloads))
        started.set()
        release.wait(5)
        return payloads

    s = RolloutTaskScheduler(gen, max_concurrent_requests=1)
    s.start()
    s.put_rollout(RolloutTask(0, "a"))
    assert started.wait(5)
    s.put_rollout(RolloutTask(1, "b"))
    threading.Timer(0.2, release.set).start()
    t0 = time.time()
    with s.paused():
        assert time.time() - t0 >= 0.15 and calls == [["a"]]          # returned only after "a" finished
        time.sleep(0.1)
        assert calls == [["a"]] and s.pending() == 1                   # "b" is held back inside the block
    assert [c.idx for c in _collect(s, 2)] == [0, 1]
    s.stop()


def test_engine_errors_are_reported_per_task_and_the_thread_survives():
    def gen(payloads, is_validation):
        if "bad" in payloads:
            raise RuntimeError("boom")
        return payloads

    s = RolloutTaskScheduler(gen, max_concurrent_requests=1)
    s.start()
    s.put_rollout(RolloutTask(0, "bad"))
    s.put_rollout(RolloutTask(1, "ok"))
    done = {c.idx: c for c in _collect(s, 2)}
    s.stop()
    assert isinstance(done[0].error, RuntimeError) and done[0].result is None
    assert done[1].error is None and done[1].result == "ok" and s.stats["errors"] == 1
    with pytest.raises(ValueError):
        RolloutTaskScheduler(gen, 0)
