"""Report sinks of the controller: every finished training step hands ``(report, step)`` to the sinks named in
``logging.logger`` (cosmos_rl/utils/report/wandb_logger.py:31-110; console lines in dispatcher/status.py)."""
from __future__ import annotations

import json
import os
import time
from typing import Any, Callable, Dict, List


class JsonlLogger:
    """Appends one JSON object per step to ``<output_dir>/metrics.jsonl`` (always available, no service needed)."""

    def __init__(self, config):
        self.path = os.path.join(config.train.output_dir, "metrics.jsonl")
        os.makedirs(config.train.output_dir, exist_ok=True)

    def __call__(self, report: Dict[str, Any], step: int) -> None:
        row = {"step": step, "time": time.time(), **{k: v for k, v in report.items() if isinstance(v, (int, float, str))}}
        with open(self.path, "a") as f:
            f.write(json.dumps(row) + "\n")


class WandbLogger:
    """Weights & Biases sink; ``WANDB_MODE=offline`` works without network. Initialised lazily on the first report."""

    def __init__(self, config):
        self.config, self.run = config, None

    def _init(self):
        try:
            import wandb
        except ImportError as e:
            raise RuntimeError('logging.logger contains "wandb" but the wandb package is not installed') from e
        lg = self.config.logging
        self.run = wandb.init(project=lg.project_name, group=lg.group_name, name=lg.experiment_name,
                              dir=self.config.train.output_dir, config=self.config.model_dump(), resume="allow")
        return self.run

    def __call__(self, report: Dict[str, Any], step: int) -> None:
        run = self.run or self._init()
        run.log({k: v for k, v in report.items() if isinstance(v, (int, float))}, step=step)


SINKS: Dict[str, Callable] = {"jsonl": JsonlLogger, "wandb": WandbLogger}


def build_report_hooks(config) -> List[Callable]:
    """Sinks for the names in ``logging.logger`` ("console" is the controller's own log line)."""
    hooks = []
    for name in config.logging.logger:
        if name == "console":
            continue
        if name not in SINKS:
            raise ValueError(f"unknown logger {name!r}; known: console, {', '.join(sorted(SINKS))}")
        hooks.append(SINKS[name](config))
    return hooks
