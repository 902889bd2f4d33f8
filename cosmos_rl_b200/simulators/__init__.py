"""Environment back-ends of embodied rollouts. Render-free control tasks are built in; the third-party robot
simulators the reference wraps (LIBERO, ManiSkill, RoboTwin, BEHAVIOR-1K: cosmos_rl/simulators/{libero,maniskill,
robotwin,b1k}) render through EGL / Vulkan and cannot run on a compute-only GPU box, so their names resolve to an
error that says so instead of an import failure deep inside a job."""
from __future__ import annotations

from .classic_control import ENV_TYPES, BatchedControlEnv, CartPoleEnv, PendulumEnv  # noqa: F401
from .env_manager import EnvManager  # noqa: F401

RENDERED = ("libero", "maniskill", "robotwin", "b1k")


class SimulatorUnavailable(RuntimeError):
    pass


def get_env_cls(name: str):
    if name in ENV_TYPES:
        return BatchedControlEnv
    if name.lower() in RENDERED:
        raise SimulatorUnavailable(f"simulator {name!r} renders through a graphics API (EGL / Vulkan), which a "
                                   f"compute-only GPU box does not have; render-free tasks: {sorted(ENV_TYPES)}")
    raise KeyError(f"unknown environment {name!r}; known: {sorted(ENV_TYPES)} (+ rendered: {list(RENDERED)})")
