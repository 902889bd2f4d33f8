"""Outer loops for trainers whose rollouts hold many trainable transitions (embodied episodes, multi-turn
trajectories): ``begin -> per rollout (whole, or in chunks of transitions) -> finalize``
(cosmos_rl/policy/trainer/trajectory_mixin.py:39-200). The mixin only orders the phases; the loss, gradient
accumulation and metrics belong to the composing trainer. Put it leftmost so its ``step_training`` wins:

    class MyTrainer(TrajectoryExpansionMixin, Trainer):
        chunk_size = 8                      # None = one call per rollout
        def _train_one_chunk(self, rollout, chunk, *a, **kw): ...
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

PACKER_METHODS = ("num_transitions", "iter_transitions", "iter_chunks", "iter_rollouts")


class TrajectoryExpansionMixin:
    chunk_size: Optional[int] = None

    def step_training(self, rollouts: Sequence[Any], *args: Any, **kwargs: Any) -> Dict[str, Any]:
        packer = getattr(self, "data_packer", None)
        missing = [m for m in PACKER_METHODS if not hasattr(packer, m)]
        if missing:
            raise TypeError(f"{type(self).__name__}.data_packer ({type(packer).__name__}) does not implement the "
                            f"trajectory packer methods {missing}")
        if self.chunk_size is not None and self.chunk_size < 1:
            raise ValueError("chunk_size must be None or >= 1")
        state = self._begin_training_step(rollouts, *args, **kwargs)
        for ro in packer.iter_rollouts(rollouts):
            if self.chunk_size is None:
                self._train_one_rollout(ro, state, *args, **kwargs)
            else:
                for chunk in packer.iter_chunks([ro], self.chunk_size):
                    self._train_one_chunk(ro, chunk, state, *args, **kwargs)
        return self._finalize_training_step(rollouts, state, *args, **kwargs)

    # ------------------------------------------------------------------ hooks
    def _begin_training_step(self, rollouts, *args, **kwargs) -> Any:
        return {}

    def _train_one_rollout(self, rollout, state, *args, **kwargs) -> None:
        raise NotImplementedError(f"{type(self).__name__} has chunk_size=None and must override _train_one_rollout")

    def _train_one_chunk(self, rollout, chunk: List[Dict[str, Any]], state, *args, **kwargs) -> None:
        raise NotImplementedError(f"{type(self).__name__} has chunk_size={self.chunk_size} and must override "
                                  f"_train_one_chunk")

    def _finalize_training_step(self, rollouts, state, *args, **kwargs) -> Dict[str, Any]:
        return {}
