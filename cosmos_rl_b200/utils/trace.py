"""Structured trace lines ``[Trace] worker=... thread=... op=... start=... end=...`` and their parser
(cosmos_rl/utils/trace.py:83-330; grammar docs/profiler/trace_format.rst)."""
from __future__ import annotations

import contextlib
import os
import re
import threading
import time
from typing import Dict, Iterable, Iterator, List, Optional

from .logging import logger

_ENABLED = os.environ.get("COSMOS_TRACE", "0") not in ("0", "", "false")
_worker = threading.local()
LINE = re.compile(r"\[Trace\] worker=(?P<worker>\S+) thread=(?P<thread>\S+) op=(?P<op>\S+) "
                  r"start=(?P<start>[0-9.]+) end=(?P<end>[0-9.]+)(?P<rest>.*)")


def set_enabled(flag: bool) -> None:
    global _ENABLED
    _ENABLED = flag


def set_worker(name: str) -> None:
    _worker.name = name


def format_line(worker: str, thread: str, op: str, start: float, end: float, **attrs) -> str:
    extra = "".join(f" {k}={v}" for k, v in attrs.items())
    return f"[Trace] worker={worker} thread={thread} op={op} start={start:.6f} end={end:.6f}{extra}"


@contextlib.contextmanager
def trace_op(op: str, **attrs):
    """Time a block and log one trace line (no-op unless COSMOS_TRACE=1 or ``set_enabled(True)``)."""
    if not _ENABLED:
        yield
        return
    t0 = time.time()
    try:
        yield
    finally:
        logger.info(format_line(getattr(_worker, "name", "main"), threading.current_thread().name, op, t0,
                                time.time(), **attrs))


def parse_lines(lines: Iterable[str]) -> Iterator[Dict]:
    for ln in lines:
        m = LINE.search(ln)
        if not m:
            continue
        d = m.groupdict()
        rec = {"worker": d["worker"], "thread": d["thread"], "op": d["op"], "start": float(d["start"]),
               "end": float(d["end"])}
        for kv in d["rest"].split():
            if "=" in kv:
                k, v = kv.split("=", 1)
                rec[k] = v
        yield rec


def summarize(records: Iterable[Dict]) -> Dict[str, Dict[str, float]]:
    """Per (worker, op): count, total, mean and max duration in seconds."""
    out: Dict[str, Dict[str, float]] = {}
    for r in records:
        key = f"{r['worker']}:{r['op']}"
        s = out.setdefault(key, {"count": 0, "total": 0.0, "max": 0.0})
        dur = r["end"] - r["start"]
        s["count"] += 1
        s["total"] += dur
        s["max"] = max(s["max"], dur)
    for s in out.values():
        s["mean"] = s["total"] / max(1, s["count"])
    return out
