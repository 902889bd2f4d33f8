"""Higher-order samplers and noise parametrisations for the diffusion / flow trainers.

``policy/diffusion.py`` integrates the learned velocity with Euler steps (and an SDE variant for FlowGRPO). The
world-model stack of the reference ships a family of solvers and two pre-conditionings
(cosmos_rl/policy/model/wfm/sampler/__init__.py:170-460 Runge-Kutta and multistep steps, :799-880 EDM and
rectified-flow scalings). Written out here on this package's convention (``x_t = (1 - t) x0 + t noise``, the network
predicts ``v = noise - x0``, sampling runs t from 1 to 0):

* one-step Runge-Kutta integrators of the probability-flow ODE: ``euler`` (order 1), ``midpoint`` and ``heun``
  (order 2, two network calls per step), ``kutta3`` (order 3, three calls);
* a two-step Adams-Bashforth integrator (``ab2``: order 2 at ONE call per step, re-using the previous velocity; variable
  step sizes);
* the data-prediction exponential integrator (``exp2``): in log-SNR time ``lambda = log((1 - t) / t)`` the ODE for a
  data predictor is linear in x, so its linear part is integrated exactly and only the predicted ``x0`` is
  extrapolated from the previous step. Second order, one call per step, and stable at very few steps;
* EDM pre-conditioning (``c_skip, c_out, c_in, c_noise`` and the loss weight) and the rectified-flow scaling that maps
  between ``sigma`` and ``t``, plus the log-normal sigma sampler of EDM training.

``sample(model, noise, text, ..., solver="heun")`` is the entry point; classifier-free guidance as in ``euler_sample``.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Tuple

import torch

from .diffusion import timestep_grid

Velocity = Callable[[torch.Tensor, torch.Tensor], torch.Tensor]      # (x, t scalar tensor) -> v


# ---------------------------------------------------------------------------------------------------
# one-step integrators: x(t_next) from x(t)
# ---------------------------------------------------------------------------------------------------
def step_euler(f: Velocity, x, t, t_next):
    return x + (t_next - t) * f(x, t)


def step_midpoint(f: Velocity, x, t, t_next):
    h = t_next - t
    return x + h * f(x + 0.5 * h * f(x, t), t + 0.5 * h)


def step_heun(f: Velocity, x, t, t_next):
    h = t_next - t
    k1 = f(x, t)
    k2 = f(x + h * k1, t_next)
    return x + 0.5 * h * (k1 + k2)


def step_kutta3(f: Velocity, x, t, t_next):
    h = t_next - t
    k1 = f(x, t)
    k2 = f(x + 0.5 * h * k1, t + 0.5 * h)
    k3 = f(x - h * k1 + 2.0 * h * k2, t_next)
    return x + h * (k1 + 4.0 * k2 + k3) / 6.0


ONE_STEP: Dict[str, Tuple[Callable, int]] = {          # name -> (step function, network calls per step)
    "euler": (step_euler, 1), "midpoint": (step_midpoint, 2), "heun": (step_heun, 2), "kutta3": (step_kutta3, 3)}
MULTI_STEP = ("ab2", "exp2")


def is_solver_supported(name: str) -> bool:
    return name in ONE_STEP or name in MULTI_STEP


def integrate(f: Velocity, x: torch.Tensor, ts: torch.Tensor, solver: str = "heun") -> torch.Tensor:
    """Integrate ``dx/dt = f(x, t)`` along the grid ``ts`` (any monotone grid; sampling uses 1 -> 0)."""
    if solver in ONE_STEP:
        step = ONE_STEP[solver][0]
        for i in range(len(ts) - 1):
            x = step(f, x, ts[i], ts[i + 1])
        return x
    if solver == "ab2":
        v_prev, h_prev = None, None
        for i in range(len(ts) - 1):
            h = ts[i + 1] - ts[i]
            v = f(x, ts[i])
            if v_prev is None:
                x = x + h * v                                   # the first step has no history
            else:
                r = h / h_prev                                  # variable-step Adams-Bashforth 2
                x = x + h * ((1 + 0.5 * r) * v - 0.5 * r * v_prev)
            v_prev, h_prev = v, h
        return x
    if solver == "exp2":
        return _exp2(f, x, ts)
    raise ValueError(f"unknown solver {solver!r}; known: {sorted(ONE_STEP) + list(MULTI_STEP)}")


def _exp2(f: Velocity, x: torch.Tensor, ts: torch.Tensor) -> torch.Tensor:
    """Data-prediction exponential integrator. With ``x0_hat = x - t v`` and ``lambda = log((1 - t) / t)``:
    ``x(t') = (t' / t) x(t) + (1 - t') (1 - exp(-dl)) x0_tilde`` for a constant ``x0_tilde`` over the step
    (exact for a perfect data predictor), where ``dl = lambda' - lambda``; second order comes from extrapolating
    ``x0_hat`` linearly in lambda from the previous step. The last step to t = 0 returns the data prediction."""
    lam = lambda t: torch.log((1 - t).clamp_min(1e-12) / t.clamp_min(1e-12))
    x0_prev, dl_prev = None, None
    for i in range(len(ts) - 1):
        t, tn = ts[i], ts[i + 1]
        x0 = x - t * f(x, t)
        if float(tn) <= 0.0:
            return x0
        if float(t) >= 1.0:                                     # lambda = -inf at pure noise: a plain first-order step
            x = tn * (x - x0) / t + x0 if float(t) > 0 else x0  # keeps the noise direction, moves along the chord
            x0_prev, dl_prev = x0, None
            continue
        dl = lam(tn) - lam(t)
        x0_use = x0
        if x0_prev is not None and dl_prev is not None:
            x0_use = x0 + 0.5 * (dl / dl_prev) * (x0 - x0_prev)
        x = (tn / t) * x + (1 - tn) * (1 - torch.exp(-dl)) * x0_use
        x0_prev, dl_prev = x0, dl
    return x


@torch.no_grad()
def sample(model: Callable, noise: torch.Tensor, text, text_mask=None, steps: int = 20, shift: float = 1.0,
           guidance: float = 1.0, null_text=None, solver: str = "heun") -> torch.Tensor:
    """Deterministic sampling with the chosen solver; ``steps`` grid intervals (``calls_per_step`` network calls each)."""
    def f(x, t):
        tt = t.expand(x.shape[0]) if t.dim() == 0 else t
        v = model(x.to(noise.dtype), tt, text, text_mask).float()
        if guidance != 1.0 and null_text is not None:
            v0 = model(x.to(noise.dtype), tt, null_text, None).float()
            v = v0 + guidance * (v - v0)
        return v
    ts = timestep_grid(steps, shift, noise.device)
    return integrate(f, noise.float(), ts, solver).to(noise.dtype)


def calls_per_step(solver: str) -> int:
    return ONE_STEP[solver][1] if solver in ONE_STEP else 1


# ---------------------------------------------------------------------------------------------------
# parametrisations
# ---------------------------------------------------------------------------------------------------
class EDMScaling:
    """Pre-conditioning of Karras et al.: ``D(x; sigma) = c_skip x + c_out F(c_in x, c_noise)``."""

    def __init__(self, sigma_data: float = 0.5):
        self.sigma_data = sigma_data

    def __call__(self, sigma: torch.Tensor):
        sd2, s2 = self.sigma_data ** 2, sigma ** 2
        c_skip = sd2 / (s2 + sd2)
        c_out = sigma * self.sigma_data / (s2 + sd2).sqrt()
        c_in = 1.0 / (s2 + sd2).sqrt()
        c_noise = 0.25 * sigma.log()
        return c_skip, c_out, c_in, c_noise

    def loss_weight(self, sigma: torch.Tensor) -> torch.Tensor:
        return (sigma ** 2 + self.sigma_data ** 2) / (sigma * self.sigma_data) ** 2


class RectifiedFlowScaling:
    """The flow path seen through EDM's glasses: ``t = sigma / (sigma + 1)`` (so ``x_t = (1 - t)(x0 + sigma noise)``),
    a velocity network turned into a denoiser ``D = x_t - t v``, and the loss weight ``(1 + sigma)^2 / sigma^2`` that
    makes the denoising loss equal the velocity loss."""

    def __init__(self, t_scale: float = 1.0):
        self.t_scale = t_scale

    @staticmethod
    def sigma_to_t(sigma: torch.Tensor) -> torch.Tensor:
        return sigma / (sigma + 1.0)

    @staticmethod
    def t_to_sigma(t: torch.Tensor) -> torch.Tensor:
        return t / (1.0 - t)

    def __call__(self, sigma: torch.Tensor):
        t = self.sigma_to_t(sigma)
        return torch.ones_like(t), -t, 1.0 - t, t * self.t_scale      # c_skip, c_out, c_in (on x0 + sigma noise), c_noise

    def loss_weight(self, sigma: torch.Tensor) -> torch.Tensor:
        return (1.0 + sigma) ** 2 / sigma ** 2


class LogNormalSigma:
    """``log sigma ~ N(p_mean, p_std^2)``, clipped to ``[sigma_min, sigma_max]`` (EDM's training distribution)."""

    def __init__(self, p_mean: float = -1.2, p_std: float = 1.2, sigma_min: float = 0.002, sigma_max: float = 80.0):
        self.p_mean, self.p_std, self.sigma_min, self.sigma_max = p_mean, p_std, sigma_min, sigma_max

    def sample(self, n: int, generator=None, device=None) -> torch.Tensor:
        z = torch.randn(n, generator=generator, device=device)
        return (self.p_mean + self.p_std * z).exp().clamp(self.sigma_min, self.sigma_max)


def karras_sigmas(steps: int, sigma_min: float = 0.002, sigma_max: float = 80.0, rho: float = 7.0) -> torch.Tensor:
    """``steps + 1`` noise levels from ``sigma_max`` down to 0 on Karras' rho-spaced grid."""
    i = torch.arange(steps, dtype=torch.float64)
    s = (sigma_max ** (1 / rho) + i / max(steps - 1, 1) * (sigma_min ** (1 / rho) - sigma_max ** (1 / rho))) ** rho
    return torch.cat([s, s.new_zeros(1)]).float()
