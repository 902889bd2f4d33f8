"""Trainer of the control example, registered as trainer type ``gym_pg``: composes the trajectory mixin in rollout
mode (one forward/backward per episode, gradients accumulated, one optimizer step per batch of episodes)
(cosmos_rl/tools/gym_example/gym_trainer.py)."""
from __future__ import annotations

import os
import time
from typing import Any, Dict, Optional

import torch

from ...policy.trainer.base import Trainer, TrainerRegistry
from ...policy.trainer.trajectory_mixin import TrajectoryExpansionMixin
from ...utils.logging import logger
from .gym_algo import compute_returns, pg_loss
from .gym_data_packer import GymDataPacker
from .gym_policy import GymMLPConfig, GymPolicy


@TrainerRegistry.register("gym_pg")
class GymTrainer(TrajectoryExpansionMixin, Trainer):
    chunk_size = None

    def __init__(self, config, parallel_dims, device=None, data_packer=None, **kw):
        self.config, self.parallel_dims = config, parallel_dims
        self.device = device or torch.device("cpu")
        c = config.custom.get("gym", {})
        torch.manual_seed(config.train.seed or 0)
        self.model = GymPolicy(GymMLPConfig.from_dict(c)).to(self.device)
        self.gamma = float(c.get("gamma", 0.99))
        self.entropy_coef = float(c.get("entropy_coef", 0.01))
        lr = config.train.optm_lr if isinstance(config.train.optm_lr, float) else float(config.train.optm_lr[0])
        self.optimizer = torch.optim.Adam(self.model.parameters(), lr=lr)
        self.data_packer = data_packer or GymDataPacker()
        self.data_packer.setup(config, None)
        self.ckpt_manager = None
        self.train_step = 0

    # ------------------------------------------------------------------ trajectory hooks
    def _begin_training_step(self, rollouts, *a, **kw):
        self.optimizer.zero_grad(set_to_none=True)
        n = sum(self.data_packer.num_transitions(r) for r in rollouts)
        return {"t0": time.perf_counter(), "n_transitions": max(1, n), "losses": [], "returns": [], "entropy": []}

    def _train_one_rollout(self, rollout, state, *a, **kw):
        x = self.data_packer.get_policy_input(rollout.prompt, rollout.completion)
        obs, act, rew = (x[k].to(self.device) for k in ("observations", "actions", "rewards"))
        if rew.numel() == 0:
            return
        ret = compute_returns(rew, self.gamma)
        logp, ent, val = self.model.log_prob_entropy_value(obs, act)
        loss, m = pg_loss(logp, ent, val, ret / 10.0, entropy_coef=self.entropy_coef)
        (loss * rew.numel() / state["n_transitions"]).backward()     # transition-weighted mean over the batch
        state["losses"].append(float(loss.detach())); state["returns"].append(float(rew.sum())); state["entropy"].append(m["entropy"])

    def _finalize_training_step(self, rollouts, state, current_step: int = 0, total_steps: int = 0, *a, **kw):
        norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.config.train.optm_grad_norm_clip or 1e9)
        self.optimizer.step()
        self.train_step = current_step or self.train_step + 1
        mean = lambda v: sum(v) / max(1, len(v))
        return {"train/loss_avg": mean(state["losses"]), "train/loss_max": max(state["losses"], default=0.0),
                "train/learning_rate": self.optimizer.param_groups[0]["lr"], "train/grad_norm": float(norm),
                "train/iteration_time": time.perf_counter() - state["t0"],
                "train/episode_return": mean(state["returns"]), "train/entropy": mean(state["entropy"])}

    # ------------------------------------------------------------------ persistence
    def weight_resume(self) -> bool:
        path = os.path.join(self.config.train.output_dir, "gym_policy.pt")
        if self.config.train.resume and os.path.exists(path):
            self.model.load_state_dict(torch.load(path, map_location=self.device))
            return True
        return False

    def model_load_from_hf(self) -> None:
        logger.info("[GymTrainer] the control policy is initialised from the seed; nothing to load")

    def model_resume_from_checkpoint(self) -> bool:
        return self.weight_resume()

    def save_checkpoint(self, step: int, total_steps: int, *a, **kw) -> None:
        os.makedirs(self.config.train.output_dir, exist_ok=True)
        torch.save(self.model.state_dict(), os.path.join(self.config.train.output_dir, "gym_policy.pt"))

    def export_safetensors(self, output_dir: str, **kw) -> None:
        from safetensors.torch import save_file
        os.makedirs(output_dir, exist_ok=True)
        save_file({k: v.detach().cpu().contiguous() for k, v in self.model.state_dict().items()},
                  os.path.join(output_dir, "model.safetensors"))
