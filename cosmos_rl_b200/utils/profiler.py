"""torch.profiler wrapper with a static schedule from the job file and a dynamic mode switched on at run
time through the controller (``cosmos-cli profile set`` -> ``POST /api/set_profile`` -> the next
``DataFetchCommand`` carries the request) (cosmos_rl/utils/profiler.py:29-254)."""
from __future__ import annotations

import gzip
import os
import shutil
from typing import Optional

import torch

from .logging import logger


class CosmosProfiler:
    def __init__(self, config, replica_name: str, global_rank: int, api=None):
        self.config = config
        self.replica_name, self.rank, self.api = replica_name, global_rank, api
        sub = config.profiler.sub_profiler_config
        self.static = bool(config.profiler.enable_profiler and sub.do_profile)
        self.sub = sub
        self.prof: Optional[torch.profiler.profile] = None
        self.remaining = 0
        self.n_traces = 0
        self.out_dir = os.path.join(config.train.output_dir, "profile_trace", f"{replica_name}_{global_rank}")
        if self.static and self.rank in sub.rank_filter:
            self._start(sub.wait_steps, sub.warmup_steps, sub.active_steps, sub)

    def _start(self, wait: int, warmup: int, active: int, opts) -> None:
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        os.makedirs(self.out_dir, exist_ok=True)
        self.prof = torch.profiler.profile(
            activities=acts, schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active, repeat=1),
            record_shapes=getattr(opts, "record_shape", False), profile_memory=getattr(opts, "profile_memory", False),
            with_stack=getattr(opts, "with_stack", False), with_modules=getattr(opts, "with_modules", False),
            on_trace_ready=self._save)
        self.prof.start()
        self.remaining = wait + warmup + active

    def start_dynamic(self, command) -> None:
        """Start a capture requested at run time (fields of the DataFetch command)."""
        if self.prof is not None or self.rank not in (command.rank_filter or [0]):
            return
        self._start(0, 0, max(1, command.active_steps), command)

    def _save(self, prof) -> None:
        path = os.path.join(self.out_dir, f"{self.n_traces}_trace.json")
        prof.export_chrome_trace(path)
        with open(path, "rb") as f, gzip.open(path + ".gz", "wb") as g:
            shutil.copyfileobj(f, g)
        os.remove(path)
        self.n_traces += 1
        logger.info("[Profiler] trace saved to %s.gz", path)
        if self.api is not None:
            try:
                self.api.set_trace_path(self.replica_name, path + ".gz", self.rank)
            except Exception as e:
                logger.warning("could not report trace path: %s", e)

    def step(self) -> bool:
        """Advance one training step; True when a capture finished with this step."""
        if self.prof is None:
            return False
        self.prof.step()
        self.remaining -= 1
        if self.remaining <= 0:
            self.prof.stop()
            self.prof = None
            return True
        return False
