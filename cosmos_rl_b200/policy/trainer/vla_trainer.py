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


@TrainerRegistry.register("openvla_grpo")
class OpenVLAGRPOTrainer(GRPOTrainer):
    """GRPO for the image-conditioned action-token policy (``models/openvla.py`` with the ``openvla`` rollout backend):
    every control step of an episode is one sample whose prompt carries the step's pixels, whose completion is the
    action tokens, scored under the softmax over the action bins (the distribution the rollout sampled from), with the
    episode's group-relative advantage."""

    def __init__(self, config, parallel_dims, **kw):
        super().__init__(config, parallel_dims, **kw)
        if type(self.model).__name__ != "OpenVLA":
            raise ValueError(f"openvla_grpo needs an openvla model, got {type(self.model).__name__}")
        self.model.action_only_logprobs = True

    def step_training(self, rollouts: List[Rollout], *args, **kw) -> Dict[str, Any]:
        from ...rollout.diffusion_rollout import LatentStore
        cap = int(self.config.custom.get("vla", {}).get("train_steps_per_episode", 0))
        flat: List[Rollout] = []
        for ro in rollouts:
            item = LatentStore.get(ro.completion)
            steps = item["steps"]
            if cap and len(steps) > cap:
                stride = len(steps) / cap                                # evenly spaced sub-sample of a long episode
                steps = [steps[int(i * stride)] for i in range(cap)]
            for s in steps:
                prompt = {"input_ids": list(item["prompt_ids"]), "pixel_values": s["pixel_values"].float()[None]}
                flat.append(Rollout(prompt=prompt, prompt_idx=ro.prompt_idx, completion=list(s["action_tokens"]),
                                    reward=ro.reward, advantage=ro.advantage, weight_version=ro.weight_version,
                                    completion_token_ids=[[t] for t in s["action_tokens"]],
                                    completion_logprobs=[[l] for l in s["logprobs"]]))
        report = super().step_training(flat, *args, **kw)
        LatentStore.release([ro.completion for ro in rollouts])
        report["train/episode_return"] = sum(r.reward for r in rollouts) / max(1, len(rollouts))
        report["train/transitions"] = float(len(flat))
        return report
