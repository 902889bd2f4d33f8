"""Flow-matching arithmetic shared by the diffusion trainers and the diffusion rollout backend.

Convention (rectified flow): ``x_t = (1 - t) x_0 + t eps`` with t in [0, 1], t = 1 pure noise; the network predicts the
velocity ``v = eps - x_0``, so ``x_0 = x_t - t v``. Sampling integrates from t = 1 down to 0.

* ``flow_matching_loss``: supervised objective (cosmos_rl/policy/trainer/diffusers_trainer/sft_trainer.py).
* ``nft_loss``: DiffusionNFT, reward-weighted positive / implicit-negative regression around the behaviour policy
  (cosmos_rl/policy/trainer/diffusers_trainer/nft_trainer.py:528-650).
* ``sde_step`` / ``sde_logprob``: the stochastic sampler FlowGRPO needs to have per-step likelihoods
  (docs/wfm/overview.rst:44-60 lists the algorithm family).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Tuple

import torch


def _bc(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return t.view(-1, *([1] * (like.dim() - 1))).to(like.dtype)


def sample_timesteps(n: int, scheme: str = "logit_normal", shift: float = 1.0, generator=None, device=None) -> torch.Tensor:
    """t in (0, 1). ``logit_normal``: sigmoid of a standard normal (mass in the middle of the path); ``shift`` > 1
    moves mass towards the noisy end as resolution grows: ``t' = shift t / (1 + (shift - 1) t)``."""
    if scheme == "uniform":
        t = torch.rand(n, generator=generator, device=device)
    elif scheme == "logit_normal":
        t = torch.sigmoid(torch.randn(n, generator=generator, device=device))
    else:
        raise ValueError(f"unknown timestep scheme {scheme!r}")
    t = shift * t / (1 + (shift - 1) * t)
    return t.clamp(1e-4, 1 - 1e-4)


def add_noise(x0: torch.Tensor, t: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    tb = _bc(t, x0)
    return (1 - tb) * x0 + tb * noise


def flow_matching_loss(model: Callable, x0: torch.Tensor, text, text_mask=None, t: Optional[torch.Tensor] = None,
                       noise: Optional[torch.Tensor] = None, scheme: str = "logit_normal", shift: float = 1.0
                       ) -> torch.Tensor:
    t = sample_timesteps(x0.shape[0], scheme, shift, device=x0.device) if t is None else t
    noise = torch.randn_like(x0) if noise is None else noise
    v = model(add_noise(x0, t, noise), t, text, text_mask)
    return (v.float() - (noise - x0).float()).pow(2).mean()


def timestep_grid(steps: int, shift: float = 1.0, device=None) -> torch.Tensor:
    """steps + 1 times from 1 down to 0 (shifted like the training distribution)."""
    t = torch.linspace(1.0, 0.0, steps + 1, device=device)
    return shift * t / (1 + (shift - 1) * t)


@torch.no_grad()
def euler_sample(model: Callable, noise: torch.Tensor, text, text_mask=None, steps: int = 20, shift: float = 1.0,
                 guidance: float = 1.0, null_text=None) -> torch.Tensor:
    """Deterministic sampler. ``guidance`` > 1 with ``null_text`` enables classifier-free guidance."""
    x = noise
    ts = timestep_grid(steps, shift, noise.device)
    for i in range(steps):
        t = ts[i].expand(x.shape[0])
        v = model(x, t, text, text_mask).float()
        if guidance != 1.0 and null_text is not None:
            v0 = model(x, t, null_text, None).float()
            v = v0 + guidance * (v - v0)
        x = (x.float() + (ts[i + 1] - ts[i]) * v).to(noise.dtype)
    return x


def sde_coeffs(t: float, t_next: float, noise_level: float) -> Tuple[float, float]:
    """(sigma_t, std of the transition) of the reverse-time SDE that has the same marginals as the flow ODE:
    ``dx = [v + sigma^2 / (2 t) (x + (1 - t) v)] dt + sigma dw`` with ``sigma_t = a sqrt(t / (1 - t))``; 1 - t is floored
    so the first step from pure noise stays finite."""
    sigma = noise_level * math.sqrt(t / max(1.0 - t, 0.05))
    return sigma, sigma * math.sqrt(abs(t_next - t))


def sde_mean(x: torch.Tensor, v: torch.Tensor, t: float, t_next: float, noise_level: float) -> torch.Tensor:
    sigma, _ = sde_coeffs(t, t_next, noise_level)
    drift = v + (sigma * sigma / (2.0 * t)) * (x + (1.0 - t) * v)
    return x + (t_next - t) * drift


def sde_logprob(x_next: torch.Tensor, mean: torch.Tensor, std: float) -> torch.Tensor:
    """Per-sample log density of the Gaussian transition, averaged over latent elements (keeps ratios well scaled)."""
    z = (x_next.float() - mean.float()) / std
    return (-0.5 * z * z - math.log(std) - 0.5 * math.log(2 * math.pi)).flatten(1).mean(1)


@torch.no_grad()
def sde_sample(model: Callable, noise: torch.Tensor, text, text_mask=None, steps: int = 10, shift: float = 1.0,
               noise_level: float = 0.7, generator=None) -> Dict[str, torch.Tensor]:
    """Stochastic sampler that records what FlowGRPO trains on: the state before each step, the state after it and
    the behaviour log-probability. The last step is deterministic (std would be 0 at t = 0)."""
    x = noise.float()
    ts = timestep_grid(steps, shift, noise.device).tolist()
    xs, nxt, lps = [], [], []
    for i in range(steps):
        t, tn = ts[i], ts[i + 1]
        v = model(x.to(noise.dtype), torch.full((x.shape[0],), t, device=x.device), text, text_mask).float()
        if i == steps - 1:
            x = x + (tn - t) * v
            break
        mean = sde_mean(x, v, t, tn, noise_level)
        _, std = sde_coeffs(t, tn, noise_level)
        x_new = mean + std * torch.randn(x.shape, generator=generator, device=x.device)
        xs.append(x); nxt.append(x_new); lps.append(sde_logprob(x_new, mean, std))
        x = x_new
    return {"x0": x.to(noise.dtype), "states": torch.stack(xs, 1), "next_states": torch.stack(nxt, 1),
            "logprobs": torch.stack(lps, 1), "timesteps": torch.tensor(ts, device=x.device)}


def nft_loss(v: torch.Tensor, v_old: torch.Tensor, v_ref: torch.Tensor, xt: torch.Tensor, x0: torch.Tensor,
             t: torch.Tensor, advantages: torch.Tensor, beta: float, adv_clip: float, kl_beta: float
             ) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """DiffusionNFT. With r = clip(A / (2 A_max) + 1/2, 0, 1) the "probability of being a good sample":

        v+ = beta v + (1 - beta) v_old          (positive branch, pulled towards the data of good samples)
        v- = (1 + beta) v_old - beta v          (implicit negative branch, mirrored around the behaviour policy)
        loss = A_max / beta * [ r ||x0(v+) - x0||^2 / w+  +  (1 - r) ||x0(v-) - x0||^2 / w- ]  +  kl_beta ||v - v_ref||^2

    where w+- are the detached mean absolute errors of each sample (self-normalised regression)."""
    tb = _bc(t, x0)
    dims = tuple(range(1, x0.dim()))
    r = (advantages.clamp(-adv_clip, adv_clip) / adv_clip / 2.0 + 0.5).clamp(0, 1).to(v.dtype)
    v, v_old, v_ref = v.float(), v_old.float(), v_ref.float()
    x0f, xtf = x0.float(), xt.float()

    def branch(vb):
        err = xtf - tb.float() * vb - x0f
        w = err.detach().abs().mean(dim=dims, keepdim=True).clamp_min(1e-5)
        return (err * err / w).mean(dim=dims)

    pos = branch(beta * v + (1 - beta) * v_old)
    neg = branch((1 + beta) * v_old - beta * v)
    per_sample = (r * pos + (1 - r) * neg) / beta
    policy = (per_sample * adv_clip).mean()
    kl = (v - v_ref).pow(2).mean(dim=dims).mean()
    return policy + kl_beta * kl, {"policy_loss": policy.detach(), "kl_loss": kl.detach(),
                                   "old_deviation": (v - v_old).pow(2).mean().detach()}


def old_policy_decay(step: int, kind: str = "ramp") -> float:
    """EMA factor of the behaviour ("old") weights after optimizer step ``step``: 0 copies the new weights at once
    (on-policy), values near 1 let the behaviour policy trail. ``ramp`` starts on-policy and grows to 0.5 over the
    first 100 steps, which keeps early training stable and later rollouts usable for several updates."""
    if kind == "copy":
        return 0.0
    if kind == "ramp":
        return min(0.5, 0.005 * step)
    if kind == "slow":
        return min(0.999, 0.001 * step)
    raise ValueError(f"unknown decay kind {kind!r}")
