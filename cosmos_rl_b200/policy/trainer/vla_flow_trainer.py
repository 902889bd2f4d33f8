"""Trainers of policies with a flow-matching action expert (``models/vla_flow.py``), trainer types ``flow_vla_grpo`` and
``flow_vla_sft`` (the reference trains PI0.5 with the same two objectives: behaviour cloning by flow matching and RL on
the transition log-probabilities of an SDE sampler, cosmos_rl/policy/model/pi05/__init__.py). They reuse the flat
parameter buffer, the sharded AdamW and the checkpoint manager of the language-model trainers.

RL: every action chunk of an episode is one sample: the prompt tokens and state it was drawn for, the recorded SDE
transitions, and the episode's group-relative advantage. The loss is the clipped likelihood ratio of every recorded
transition under the current weights (``FlowVLA.flow_grpo_loss``).
SFT: a batch row is ``{"obs_tokens": [...], "state": [...], "actions": [[...] * action_dim] * horizon}`` with actions
already normalised to [-1, 1]."""
from __future__ import annotations

import time
from typing import Any, Dict, List

import torch

from ...rollout.diffusion_rollout import LatentStore
from ...rollout.vla_flow_rollout import flow_vla_options
from .base import TrainerRegistry
from .diffusion_trainer import _DiffusionBase


class _FlowVLABase(_DiffusionBase):
    def __init__(self, config, parallel_dims, device=None, **kw):
        super().__init__(config, parallel_dims, device=device, **kw)
        self.vla_opts = flow_vla_options(config)
        if type(self.model).__name__ != "FlowVLA":
            raise ValueError(f"trainer type {config.train.train_policy.trainer_type!r} needs a flow_vla model, got "
                             f"{type(self.model).__name__}")
        self.model.backbone.gradient_checkpointing = bool(config.policy.model_gradient_checkpointing)


@TrainerRegistry.register("flow_vla_grpo")
class FlowVLAGRPOTrainer(_FlowVLABase):
    def step_training(self, rollouts, current_step: int = 0, total_steps: int = 0, remain_samples_num: int = 0,
                      do_save: bool = False, **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        self.total_steps = total_steps or self.total_steps
        tp, o = self.config.train.train_policy, self.vla_opts
        samples = []                                     # (chunk, advantage) over every episode of the batch
        cap = int(o.get("train_chunks_per_episode", 0))
        for r in rollouts:
            chunks = LatentStore.get(r.completion)["chunks"]
            if cap and len(chunks) > cap:                # evenly spaced sub-sample of a long episode
                stride = len(chunks) / cap
                chunks = [chunks[int(i * stride)] for i in range(cap)]
            samples += [(c, float(r.advantage)) for c in chunks]
        if not samples:
            raise ValueError("flow_vla_grpo got episodes without recorded transitions (validation rollouts?)")
        mb = max(1, tp.mini_batch)
        clip = float(tp.epsilon_high)
        self.flat.zero_grad()
        losses, clips = [], []
        dev = self.device
        for s in range(0, len(samples), mb):
            part = samples[s:s + mb]
            prompts = [c["obs_tokens"] for c, _ in part]
            state = torch.stack([c["state"] for c, _ in part]).to(dev) if part[0][0]["state"] is not None else None
            ro = {"timesteps": part[0][0]["timesteps"],
                  "states": torch.stack([c["states"] for c, _ in part]).to(dev),
                  "next_states": torch.stack([c["next_states"] for c, _ in part]).to(dev),
                  "logprobs": torch.stack([c["logprobs"] for c, _ in part]).to(dev)}
            adv = torch.tensor([a for _, a in part], dtype=torch.float32, device=dev)
            loss, m = self.model.flow_grpo_loss(prompts, ro, adv, state, noise_level=o["noise_level"], clip=clip)
            (loss * len(part) / len(samples)).backward()
            losses.append(float(loss.detach()))
            clips.append(m["clip_frac"])
        norm = self.optimizer_step()
        self.train_step = current_step or self.train_step + 1
        LatentStore.release([r.completion for r in rollouts])
        if do_save:
            self.save_checkpoint(self.train_step, total_steps, remain_samples_num, self.train_step >= total_steps)
        return self._report(losses, norm, t0, clip_frac=sum(clips) / max(1, len(clips)),
                            episode_return=sum(r.reward for r in rollouts) / max(1, len(rollouts)),
                            transitions=float(len(samples)))


@TrainerRegistry.register("flow_vla_sft")
class FlowVLASFTTrainer(_FlowVLABase):
    def step_training(self, batch: List[Dict[str, Any]], total_steps: int = 0, train_step: int = 0, do_save: bool = False,
                      **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        self.total_steps = total_steps or self.total_steps
        mb = max(1, self.config.train.train_policy.mini_batch)
        self.flat.zero_grad()
        losses = []
        for s in range(0, len(batch), mb):
            part = batch[s:s + mb]
            prompts = [list(b["obs_tokens"]) for b in part]
            state = torch.tensor([b["state"] for b in part], dtype=torch.float32, device=self.device) \
                if part[0].get("state") is not None and self.model.args.state_dim else None
            actions = torch.tensor([b["actions"] for b in part], dtype=torch.float32, device=self.device)
            loss = self.model.bc_loss(prompts, actions, state)
            (loss * len(part) / len(batch)).backward()
            losses.append(float(loss.detach()))
        norm = self.optimizer_step()
        self.train_step = train_step or self.train_step + 1
        if do_save:
            self.save_checkpoint(self.train_step, total_steps, is_final=self.train_step >= total_steps)
        return self._report(losses, norm, t0)
