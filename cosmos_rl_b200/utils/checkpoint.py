"""Training checkpoints: per-rank files, completion markers, async save, pruning and resume scanning.

Layout (same as cosmos_rl/utils/checkpoint.py:50-852):
``<output_dir>/checkpoints/step_<N>/policy/{model,optimizer,scheduler,extra_info}_rank_<r>.pth`` plus
``.rank_<r>_complete`` written after every file of the rank is on disk; a step directory is valid for
resume only when its marker set is complete. ``best/`` is a symlink to the best-scoring step.
"""
from __future__ import annotations

import concurrent.futures
import glob
import json
import os
import re
import shutil
import threading
from typing import Any, Dict, List, Optional

import torch

from .logging import logger
from .misc import rng_state, set_rng_state


def restore_rng(extra_info: Dict[str, Any]) -> None:
    st = extra_info.get("rng_state")
    if st:
        try:
            set_rng_state(st)
        except Exception as e:  # device count / generator layout changed
            logger.warning("could not restore RNG state: %s", e)


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


class CheckpointManager:
    def __init__(self, config, global_rank: int = 0, world_size: Optional[int] = None, role: str = "policy"):
        self.config = config
        self.rank = global_rank
        self.world_size = world_size
        self.role = role
        ck = config.train.ckpt
        self.save_mode = ck.save_mode
        self.max_keep = ck.max_keep
        self.root = os.path.join(config.train.output_dir, "checkpoints")
        self.pool = concurrent.futures.ThreadPoolExecutor(max_workers=4) if self.save_mode == "async" else None
        self.pending: List[concurrent.futures.Future] = []
        self.s3_client = None       # an injected client (tests); boto3's default client otherwise
        self.best_score: Optional[float] = None
        self._lock = threading.Lock()

    # ------------------------------------------------------------------ paths
    def step_dir(self, step: int) -> str:
        return os.path.join(self.root, f"step_{step}", self.role)

    def _marker(self, step: int, rank: Optional[int] = None) -> str:
        return os.path.join(self.step_dir(step), f".rank_{self.rank if rank is None else rank}_complete")

    # ------------------------------------------------------------------ save
    def save(self, step: int, model_state, optimizer_state, scheduler_state, extra_info: Dict[str, Any],
             is_final: bool = False, world_size: Optional[int] = None) -> None:
        d = self.step_dir(step)
        os.makedirs(d, exist_ok=True)
        extra = dict(extra_info)
        extra["rng_state"] = rng_state()
        extra["world_size"] = world_size or self.world_size or 1
        # state is moved to host memory first so training can continue while files are written
        items = {"model": _to_cpu(model_state), "optimizer": _to_cpu(optimizer_state),
                 "scheduler": _to_cpu(scheduler_state), "extra_info": extra}
        if self.rank == 0:
            with open(os.path.join(d, "cosmos_config"), "w") as f:
                json.dump(self.config.to_dict(), f)

        def write():
            for name, obj in items.items():
                tmp = os.path.join(d, f"{name}_rank_{self.rank}.pth.tmp")
                torch.save(obj, tmp)
                os.replace(tmp, os.path.join(d, f"{name}_rank_{self.rank}.pth"))
            with open(self._marker(step), "w") as f:
                f.write("ok")
            ck = self.config.train.ckpt
            from .upload import upload_folder_to_s3, wants_s3
            if wants_s3(ck, is_final):          # this rank's files (and rank 0's config) of the step folder
                upload_folder_to_s3(d, ck.s3_bucket, os.path.join(ck.s3_prefix, "checkpoints", f"step_{step}", self.role),
                                    client=self.s3_client)
            self._prune()

        if self.pool is not None and not is_final:
            self.pending.append(self.pool.submit(write))
        else:
            write()

    def wait(self) -> None:
        for f in self.pending:
            f.result()
        self.pending = []

    def finalize(self) -> None:
        self.wait()
        if self.pool is not None:
            self.pool.shutdown(wait=True)
            self.pool = None

    # ------------------------------------------------------------------ scan / prune
    def steps_on_disk(self) -> List[int]:
        out = []
        for p in glob.glob(os.path.join(self.root, "step_*")):
            m = re.fullmatch(r"step_(\d+)", os.path.basename(p))
            if m:
                out.append(int(m.group(1)))
        return sorted(out)

    def is_complete(self, step: int) -> bool:
        d = self.step_dir(step)
        markers = glob.glob(os.path.join(d, ".rank_*_complete"))
        if not markers:
            return False
        extra_files = glob.glob(os.path.join(d, "extra_info_rank_*.pth"))
        want = len(extra_files)
        try:
            info = torch.load(os.path.join(d, "extra_info_rank_0.pth"), weights_only=False)
            want = int(info.get("world_size", want))
        except Exception:
            pass
        return len(markers) >= max(want, 1)

    def latest_valid_step(self) -> Optional[int]:
        for s in reversed(self.steps_on_disk()):
            if self.is_complete(s):
                return s
        return None

    def _prune(self) -> None:
        if self.rank != 0 or self.max_keep is None or self.max_keep <= 0:
            return
        with self._lock:
            steps = self.steps_on_disk()
            complete = [s for s in steps if self.is_complete(s)]
            best = self._best_step()
            for s in complete[: max(0, len(complete) - self.max_keep)]:
                if s == best:
                    continue
                shutil.rmtree(os.path.join(self.root, f"step_{s}"), ignore_errors=True)

    def _best_step(self) -> Optional[int]:
        link = os.path.join(self.root, "best")
        if os.path.islink(link):
            m = re.search(r"step_(\d+)", os.readlink(link))
            return int(m.group(1)) if m else None
        return None

    def report_validation_score(self, step: int, score: float) -> None:
        """Keep ``best`` pointing at the step with the highest validation score."""
        if self.rank != 0:
            return
        if self.best_score is None or score > self.best_score:
            self.best_score = score
            link = os.path.join(self.root, "best")
            tmp = link + ".tmp"
            if os.path.lexists(tmp):
                os.remove(tmp)
            os.symlink(f"step_{step}", tmp)
            os.replace(tmp, link)

    # ------------------------------------------------------------------ load
    def load(self, step: int, device) -> Dict[str, Any]:
        d = self.step_dir(step)
        out = {}
        for name in ("model", "optimizer", "scheduler", "extra_info"):
            out[name] = torch.load(os.path.join(d, f"{name}_rank_{self.rank}.pth"), map_location=device,
                                   weights_only=False)
        return out

    def load_latest(self, device) -> Optional[Dict[str, Any]]:
        resume = self.config.train.resume
        if isinstance(resume, str) and resume not in ("True", "true"):
            m = re.search(r"step_(\d+)", resume)
            if m and os.path.isdir(resume):
                self.root = os.path.dirname(resume.rstrip("/").split("/step_")[0] + "/x")
                step = int(m.group(1))
                return self.load(step, device)
        step = self.latest_valid_step()
        if step is None:
            return None
        return self.load(step, device)
