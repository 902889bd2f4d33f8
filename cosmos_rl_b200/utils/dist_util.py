"""Process-group helpers: initialisation for CPU (gloo) or GPU (nccl + gloo) worlds and a shutdown that
cannot hang (cosmos_rl/utils/distributed.py:57-84 initialises ``cuda:nccl,cpu:gloo``; the reference's
shutdown aborts every communicator before destroying the group, cosmos_rl/utils/pynccl.py:609-676)."""
from __future__ import annotations

import gc
import os
import sys
import threading
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist

from .logging import logger


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> None:
    if dist.is_initialized():
        return
    if "RANK" not in os.environ:
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    cuda = torch.cuda.is_available()
    backend = backend or ("cuda:nccl,cpu:gloo" if cuda else "gloo")
    kw = {}
    if cuda:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend, timeout=timedelta(seconds=timeout_s), **kw)


def safe_destroy(timeout_s: float = 20.0, exit_code: int = 0) -> None:
    """Destroy the default process group, but never wait longer than ``timeout_s``: communicators that were
    captured into CUDA graphs (or that lost a peer) can block in their destructor; in that case the process
    ends with ``os._exit`` once everything it had to print is flushed."""
    if not dist.is_initialized():
        return
    gc.collect()
    if torch.cuda.is_available():
        from ..parallel.dyncomm import bounded_drain_or_abort
        if not bounded_drain_or_abort(None, timeout_s, "process-group teardown"):
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(exit_code)
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(timeout_s)
    if t.is_alive():
        logger.warning("process-group teardown did not finish in %.0f s; exiting without it", timeout_s)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(exit_code)


def host_id() -> str:
    """Identity of the machine this process runs on: host name plus the kernel's boot id (two processes that agree on
    it can exchange CUDA IPC handles; two that do not must talk through a network transport). ``COSMOS_HOST_ID``
    overrides it (tests that stand in several machines on one)."""
    forced = os.environ.get("COSMOS_HOST_ID")
    if forced:
        return forced
    import socket
    boot = ""
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            boot = f.read().strip()
    except OSError:
        pass
    return f"{socket.gethostname()}:{boot}"


def group_on_one_host(group=None) -> bool:
    """True when every rank of ``group`` (default: the world) runs on the same machine."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return True
    ids = [None] * dist.get_world_size(group)
    dist.all_gather_object(ids, host_id(), group=group)
    return len(set(ids)) == 1


def __getattr__(name: str):
    # the reference's name for the fault-tolerant communicator between policy replicas
    if name == "HighAvailabilitylNccl":
        from ..parallel.inter_replica import InterReplicaComm
        return InterReplicaComm
    raise AttributeError(name)
