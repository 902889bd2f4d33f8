"""Rollout backend ``gym``: the "prompt" is an episode seed, the "completions" are ``n_generation`` episodes played
by the current policy (cosmos_rl/tools/gym_example/gym_rollout_backend.py). Built on the four generation hooks."""
from __future__ import annotations

from typing import Any, List

import torch

from ...rollout.base import RolloutBase, RolloutRegistry, RolloutResult
from ...rollout.generation_mixin import RolloutGenerationMixin
from .gym_policy import GymMLPConfig, GymPolicy
from .gym_rollout import GymRolloutEngine


@RolloutRegistry.register("gym")
class GymRolloutBackend(RolloutGenerationMixin, RolloutBase):
    def __init__(self, config, parallel_dims, device, tokenizer=None, **kw):
        super().__init__(config, parallel_dims, device)
        self.model = None
        self.engine = None

    def init_engine(self, load_format: str = "dummy", shared_model=None, **kw) -> None:
        c = self.config.custom.get("gym", {})
        self.model = shared_model if shared_model is not None else GymPolicy(GymMLPConfig.from_dict(c)).to(self.device)
        self.engine = GymRolloutEngine(self.model, env_name=c.get("env_name", "cartpole"),
                                       num_envs=int(c.get("num_envs", 8)), max_steps=int(c.get("max_steps", 200)),
                                       use_subprocess=bool(c.get("subprocess_env", False)), device=self.device)

    def get_underlying_model(self):
        return self.model

    def _collate_batch(self, samples: List[int], is_validation: bool):
        n = self.config.validation.n_generation if is_validation else self.config.rollout.n_generation
        return [s * 1000003 + g for s in samples for g in range(n)], n     # distinct episode per generation

    def _generate(self, batch, is_validation: bool):
        seeds, n = batch
        return self.engine.run(seeds, greedy=is_validation), n

    def _postprocess(self, payloads, raw, is_validation: bool) -> List[RolloutResult]:
        trajs, n = raw
        return [RolloutResult(prompt=p.prompt, completions=trajs[i * n:(i + 1) * n]) for i, p in enumerate(payloads)]
