"""A custom GRPO trainer: extend ``GRPOTrainer``, override the hooks you need, register the class under a new
``trainer_type`` and name it in the job file (``[train.train_policy] trainer_type = "custom_grpo"``); launch as usual
with a script that imports this module (cosmos_rl/tools/custom_example/custom_grpo_trainer.py, README.md).

Hooks: ``compute_logprobs(hidden, batch)``, ``loss_fn(logprob, old_logprob, batch, ...)``, ``lr_scale(step)`` and, for
anything else, ``step_training`` itself. This example adds an entropy bonus and a length penalty to the objective and
a stepwise learning-rate schedule."""
from __future__ import annotations

from typing import Any, Dict

import torch

from cosmos_rl_b200.policy.trainer.base import TrainerRegistry
from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer


@TrainerRegistry.register("custom_grpo")
class CustomGRPOTrainer(GRPOTrainer):
    def __init__(self, config, parallel_dims, **kw):
        super().__init__(config, parallel_dims, **kw)
        opts = config.custom.get("custom_grpo", {})
        self.entropy_bonus = float(opts.get("entropy_bonus", 0.0))
        self.length_penalty = float(opts.get("length_penalty", 0.0))
        self.lr_drop_every = int(opts.get("lr_drop_every", 0))

    def loss_fn(self, logprob, old_logprob, b: Dict[str, Any], ref_logprob=None, entropy=None, total_tokens=None):
        loss, metrics = super().loss_fn(logprob, old_logprob, b, ref_logprob=ref_logprob, entropy=entropy,
                                        total_tokens=total_tokens)
        n = total_tokens if total_tokens is not None else torch.tensor(float(max(1, logprob.numel())), device=logprob.device)
        if self.entropy_bonus and entropy is not None:
            bonus = entropy.sum() / n
            loss = loss - self.entropy_bonus * bonus
            metrics["entropy_bonus"] = bonus.detach()
        if self.length_penalty:
            # a differentiable stand-in for "shorter is better": the policy's own log-likelihood mass of long samples
            lens = torch.bincount(b["seq_ids_sel"], minlength=int(b["cu_seqlens"].numel() - 1)).float()
            pen = (lens[b["seq_ids_sel"]] * logprob).sum() / n / max(1.0, float(lens.max()))
            loss = loss + self.length_penalty * pen
            metrics["length_penalty"] = pen.detach()
        return loss, metrics

    def lr_scale(self, step: int) -> float:
        base = super().lr_scale(step)
        return base * (0.5 ** (step // self.lr_drop_every)) if self.lr_drop_every else base
