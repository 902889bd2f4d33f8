"""Policy-gradient arithmetic for the control example: discounted returns-to-go and the REINFORCE loss with a learned
value baseline and an entropy bonus (the reference ships a toy return-weighted regression here,
cosmos_rl/tools/gym_example/gym_algo.py; this one is an actual policy gradient so the example can be seen to learn)."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


def compute_returns(rewards: torch.Tensor, gamma: float) -> torch.Tensor:
    """Discounted return-to-go of one episode: ``G_t = r_t + gamma * G_{t+1}``."""
    out = torch.empty_like(rewards)
    g = 0.0
    for t in range(rewards.numel() - 1, -1, -1):
        g = float(rewards[t]) + gamma * g
        out[t] = g
    return out


def pg_loss(logp: torch.Tensor, entropy: torch.Tensor, values: torch.Tensor, returns: torch.Tensor,
            value_coef: float = 0.5, entropy_coef: float = 0.01) -> Tuple[torch.Tensor, Dict[str, float]]:
    adv = returns - values.detach()
    adv = (adv - adv.mean()) / (adv.std() + 1e-6) if adv.numel() > 1 else adv
    policy = -(logp * adv).mean()
    value = torch.nn.functional.mse_loss(values, returns)
    ent = entropy.mean()
    loss = policy + value_coef * value - entropy_coef * ent
    return loss, {"policy_loss": float(policy.detach()), "value_loss": float(value.detach()),
                  "entropy": float(ent.detach())}
