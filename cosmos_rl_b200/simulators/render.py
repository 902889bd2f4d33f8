"""Software rasteriser for the render-free control tasks: a camera-like image of the state, drawn with tensor
operations, so image-conditioned policies (``models/openvla.py``) can run in closed loop without a graphics stack.
The pictures follow the classic renderings: cart-pole is a cart on a track with the pole hinged on it, the pendulum a
rod around the centre; colours are fixed so a featurizer sees stable statistics."""
from __future__ import annotations

import math
from typing import Sequence

import torch


def _segment(img: torch.Tensor, x0: float, y0: float, x1: float, y1: float, width: float, colour: Sequence[int]) -> None:
    """Draw a thick line segment (image coordinates, y down) into ``img [S, S, 3]`` uint8."""
    S = img.shape[0]
    ys, xs = torch.meshgrid(torch.arange(S, dtype=torch.float32), torch.arange(S, dtype=torch.float32), indexing="ij")
    dx, dy = x1 - x0, y1 - y0
    L2 = max(dx * dx + dy * dy, 1e-9)
    t = (((xs - x0) * dx + (ys - y0) * dy) / L2).clamp(0.0, 1.0)
    dist2 = (xs - (x0 + t * dx)) ** 2 + (ys - (y0 + t * dy)) ** 2
    img[dist2 <= (width / 2.0) ** 2] = torch.tensor(colour, dtype=torch.uint8)


def render_cartpole(obs: Sequence[float], size: int = 56) -> torch.Tensor:
    """``obs = [x, x_dot, theta, theta_dot]``; the track spans x in [-2.4, 2.4]; theta = 0 is upright."""
    img = torch.full((size, size, 3), 255, dtype=torch.uint8)
    s = size / 56.0
    ground = 40.0 * s
    _segment(img, 0.0, ground, size - 1.0, ground, 1.5 * s, (0, 0, 0))
    cx = (float(obs[0]) + 2.4) / 4.8 * (size - 1)
    _segment(img, cx - 6 * s, ground - 3 * s, cx + 6 * s, ground - 3 * s, 6 * s, (40, 40, 200))
    th = float(obs[2])
    length = 26.0 * s
    _segment(img, cx, ground - 6 * s, cx + length * math.sin(th), ground - 6 * s - length * math.cos(th), 3 * s,
             (200, 120, 40))
    return img


def render_pendulum(obs: Sequence[float], size: int = 56) -> torch.Tensor:
    """``obs = [cos(theta), sin(theta), theta_dot]``; theta = 0 points up."""
    img = torch.full((size, size, 3), 255, dtype=torch.uint8)
    c = (size - 1) / 2.0
    length = 0.4 * size
    _segment(img, c, c, c + length * float(obs[1]), c - length * float(obs[0]), 0.08 * size, (200, 60, 60))
    _segment(img, c, c, c, c, 0.1 * size, (0, 0, 0))
    return img


RENDERERS = {"cartpole": render_cartpole, "CartPole-v1": render_cartpole, "pendulum": render_pendulum,
             "Pendulum-v1": render_pendulum}


def render_state(env_name: str, obs: Sequence[float], size: int = 56) -> torch.Tensor:
    if env_name not in RENDERERS:
        raise KeyError(f"no software renderer for {env_name!r}; known: {sorted(RENDERERS)}")
    return RENDERERS[env_name](obs, size)
