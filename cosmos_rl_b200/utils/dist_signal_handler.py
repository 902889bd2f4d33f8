"""Signals seen by ANY rank become visible to ALL ranks (cosmos_rl/utils/dist_signal_handler.py:30-110): a scheduler
sends SIGUSR1 / SIGTERM to one process of a job, every rank has to act on it at the same step.

    with DistributedSignalHandler(["SIGUSR1"]) as h:
        for step in ...:
            train_step()
            if any(h.signals_received()):      # one small all-gather; the same answer on every rank
                save_checkpoint(); break

The policy worker of this package does the same through ``policy/worker/rl_worker.py: agree_force_save``."""
from __future__ import annotations

import signal
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class DistributedSignalHandler:
    def __init__(self, sig: Sequence = ("SIGTERM",), processes: Optional[list] = None, group=None):
        self.signals = [getattr(signal, s) if isinstance(s, str) else s for s in sig]
        self.processes = processes or []        # child processes the signal is passed on to
        self.group = group
        self._received = False
        self._previous = {}
        self.released = True

    def _on_signal(self, signum, frame) -> None:
        self._received = True
        for p in self.processes:
            try:
                p.send_signal(signum)
            except Exception:  # noqa: BLE001  (a child that is gone needs no signal)
                pass

    def __enter__(self) -> "DistributedSignalHandler":
        self._received, self.released = False, False
        for s in self.signals:
            self._previous[s] = signal.getsignal(s)
            signal.signal(s, self._on_signal)
        return self

    def signals_received(self) -> List[bool]:
        """One flag per rank (this rank's own when there is no process group)."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self.group) == 1:
            return [self._received]
        backend = dist.get_backend(self.group)
        dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        mine = torch.tensor([int(self._received)], dtype=torch.int32, device=dev)
        out = [torch.zeros_like(mine) for _ in range(dist.get_world_size(self.group))]
        dist.all_gather(out, mine, group=self.group)
        return [bool(int(t.item())) for t in out]

    def release(self) -> bool:
        if self.released:
            return False
        for s, prev in self._previous.items():
            signal.signal(s, prev)
        self.released = True
        return True

    def __exit__(self, *exc) -> None:
        self.release()
