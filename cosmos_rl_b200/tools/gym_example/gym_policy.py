"""A small MLP policy for control tasks: categorical head for discrete actions, Gaussian (mean, state-independent
log-std) for continuous ones (cosmos_rl/tools/gym_example/gym_policy.py is the reference's counterpart)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn


@dataclass
class GymMLPConfig:
    obs_dim: int = 4
    action_dim: int = 2
    discrete: bool = True
    hidden: int = 64
    n_hidden: int = 2
    model_type: str = "gym_mlp"

    @classmethod
    def from_dict(cls, d) -> "GymMLPConfig":
        return cls(**{k: v for k, v in dict(d).items() if k in cls.__dataclass_fields__})


class GymPolicy(nn.Module):
    def __init__(self, cfg: GymMLPConfig):
        super().__init__()
        self.args = cfg
        dims = [cfg.obs_dim] + [cfg.hidden] * cfg.n_hidden
        layers = []
        for a, b in zip(dims, dims[1:]):
            layers += [nn.Linear(a, b), nn.Tanh()]
        self.body = nn.Sequential(*layers)
        self.head = nn.Linear(dims[-1], cfg.action_dim)
        self.value = nn.Linear(dims[-1], 1)
        if not cfg.discrete:
            self.log_std = nn.Parameter(torch.zeros(cfg.action_dim))

    def distribution(self, obs: torch.Tensor):
        h = self.body(obs)
        out = self.head(h)
        if self.args.discrete:
            return torch.distributions.Categorical(logits=out), self.value(h).squeeze(-1)
        return torch.distributions.Normal(out, self.log_std.exp()), self.value(h).squeeze(-1)

    @torch.no_grad()
    def act(self, obs: torch.Tensor, greedy: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        dist, _ = self.distribution(obs)
        if greedy:
            a = dist.probs.argmax(-1) if self.args.discrete else dist.mean
        else:
            a = dist.sample()
        lp = dist.log_prob(a)
        return a, lp if self.args.discrete else lp.sum(-1)

    def log_prob_entropy_value(self, obs: torch.Tensor, actions: torch.Tensor):
        dist, v = self.distribution(obs)
        if self.args.discrete:
            return dist.log_prob(actions.long()), dist.entropy(), v
        return dist.log_prob(actions).sum(-1), dist.entropy().sum(-1), v
