"""Heartbeats from a child process (cosmos_rl/comm/base.py:487-576): it keeps posting while the worker's main
interpreter is busy inside native code, and the kernel sends it SIGKILL when the worker dies (``PR_SET_PDEATHSIG``), so
a crashed worker stops reporting and the controller reaps it after ``COSMOS_HEARTBEAT_TIMEOUT``."""
from __future__ import annotations

import multiprocessing as mp
import os
import signal
import time
from typing import List


def _die_with_parent() -> None:
    try:
        import ctypes
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        libc.prctl(1, signal.SIGKILL)           # PR_SET_PDEATHSIG
    except Exception:  # noqa: BLE001  (non-Linux: the parent-pid check below still ends the loop)
        pass


def _loop(urls: List[str], replica_name: str, interval_s: float, parent_pid: int, suffix: str) -> None:
    _die_with_parent()
    import requests
    while os.getppid() == parent_pid:
        for u in urls:
            try:
                if requests.post(u + suffix, json={"replica_name": replica_name}, timeout=10.0).status_code == 200:
                    break
            except Exception:  # noqa: BLE001  (try the next controller address, then the next beat)
                continue
        time.sleep(interval_s)


def start_heartbeat_process(urls: List[str], replica_name: str, interval_s: float) -> mp.Process:
    from ..utils.api_suffix import COSMOS_API_HEARTBEAT_SUFFIX
    ctx = mp.get_context("spawn")               # never fork a process that may hold a CUDA context
    p = ctx.Process(target=_loop, args=(list(urls), replica_name, float(interval_s), os.getpid(),
                                        COSMOS_API_HEARTBEAT_SUFFIX), daemon=True, name="heartbeat")
    p.start()
    return p
