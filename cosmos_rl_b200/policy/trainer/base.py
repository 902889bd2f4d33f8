"""Trainer registry and interface (cosmos_rl/policy/trainer/base.py:105-255)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, List, Optional, Type


class TrainerRegistry:
    _trainers: Dict[str, Type["Trainer"]] = {}

    @classmethod
    def register(cls, trainer_type: str):
        def deco(c):
            cls._trainers[trainer_type] = c
            return c
        return deco

    @classmethod
    def get_trainer_cls(cls, trainer_type: str) -> Type["Trainer"]:
        if trainer_type not in cls._trainers:
            cls._load_builtin()
        if trainer_type not in cls._trainers:
            raise KeyError(f"unknown trainer type {trainer_type!r}; known: {sorted(cls._trainers)}")
        return cls._trainers[trainer_type]

    @classmethod
    def known(cls) -> List[str]:
        cls._load_builtin()
        return sorted(cls._trainers)

    @classmethod
    def _load_builtin(cls) -> None:
        """Import the trainers that ship with the package (each registers itself on import)."""
        import importlib
        for m in ("sft_trainer", "dpo_trainer", "grpo_trainer", "diffusion_trainer", "vla_trainer"):
            importlib.import_module(f"{__package__}.{m}")


class Trainer(ABC):
    """Keys every trainer reports after a step (aggregated and logged by the controller)."""
    REPORT_KEYS = ("train/loss_avg", "train/loss_max", "train/learning_rate", "train/iteration_time",
                   "train/grad_norm")

    @abstractmethod
    def step_training(self, *a, **kw) -> Dict[str, Any]: ...

    def step_validation(self, *a, **kw) -> Dict[str, Any]:
        return {}

    def before_weight_sync(self) -> None:
        """Called before the weights are handed to a rollout replica (LoRA folds its adapters in)."""

    def after_weight_sync(self) -> None:
        pass

    @abstractmethod
    def export_safetensors(self, output_dir: str, **kw) -> None: ...

    @abstractmethod
    def model_load_from_hf(self) -> None: ...

    @abstractmethod
    def model_resume_from_checkpoint(self) -> bool: ...

    @abstractmethod
    def save_checkpoint(self, step: int, total_steps: int, **kw) -> None: ...
