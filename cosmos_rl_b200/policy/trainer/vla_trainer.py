"""GRPO for action-token policies, trainer type ``vla_grpo`` (cosmos_rl/policy/trainer/vla_trainer/): an episode is
expanded into one language-model sample per control step (prompt = observation tokens, completion = action tokens,
behaviour log-probs as recorded by the rollout) and every step inherits the episode's group-relative advantage; the
packed GRPO step of the language-model trainer does the rest."""
from __future__ import annotations

from typing import Any, Dict, List

from ...dispatcher.data.schema import Rollout
from .base import TrainerRegistry
from .grpo_trainer import GRPOTrainer


def expand_episode(ro: Rollout, max_steps_per_episode: int = 0) -> List[Rollout]:
    steps = ro.completion["steps"]
    if max_steps_per_episode and len(steps) > max_steps_per_episode:
        stride = len(steps) / max_steps_per_episode                  # evenly spaced sub-sample of a long episode
        steps = [steps[int(i * stride)] for i in range(max_steps_per_episode)]
    return [Rollout(prompt=s["obs_tokens"], prompt_idx=ro.prompt_idx, completion=s["action_tokens"], reward=ro.reward,
                    advantage=ro.advantage, weight_version=ro.weight_version,
                    completion_token_ids=[[t] for t in s["action_tokens"]],
                    completion_logprobs=[[l] for l in s["logprobs"]]) for s in steps]


@TrainerRegistry.register("vla_grpo")
class VLATrainer(GRPOTrainer):
    def step_training(self, rollouts: List[Rollout], *args, **kw) -> Dict[str, Any]:
        cap = int(self.config.custom.get("vla", {}).get("train_steps_per_episode", 0))
        flat = [s for ro in rollouts for s in expand_episode(ro, cap)]
        report = super().step_training(flat, *args, **kw)
        report["train/episode_return"] = sum(r.reward for r in rollouts) / max(1, len(rollouts))
        report["train/transitions"] = float(len(flat))
        return report
