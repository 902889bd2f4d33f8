"""Render-free control environments (cart-pole balancing, pendulum swing-up) with the step/reset interface of
Gymnasium's classic-control suite, written from the equations of motion, and a batched wrapper with the
``reset(env_ids)`` / ``step(env_ids, actions)`` / ``chunk_step`` interface the embodied rollout loop drives
(cosmos_rl/simulators/libero/env_wrapper.py:175-312 is the rendered counterpart; the reference's own CPU demo uses
these two tasks, tools/gym_example/README.md:17-60)."""
from __future__ import annotations

import math
import pickle
import random
from typing import Any, Dict, List, Optional, Sequence, Tuple


class CartPoleEnv:
    """Pole on a cart, force of +-10 N per step (action 0 = left, 1 = right), Euler integration at 50 Hz. The
    episode ends when the pole leaves +-12 degrees or the cart leaves +-2.4 m; reward 1 per step."""
    obs_dim, action_dim, discrete = 4, 2, True
    gravity, m_cart, m_pole, half_len, force, tau = 9.8, 1.0, 0.1, 0.5, 10.0, 0.02
    theta_limit, x_limit = 12 * 2 * math.pi / 360, 2.4

    def __init__(self, max_steps: int = 500):
        self.max_steps = max_steps
        self.rng = random.Random(0)
        self.state = [0.0] * 4
        self.t = 0

    def reset(self, seed: Optional[int] = None) -> Tuple[List[float], Dict]:
        if seed is not None:
            self.rng = random.Random(seed)
        self.state = [self.rng.uniform(-0.05, 0.05) for _ in range(4)]
        self.t = 0
        return list(self.state), {}

    def step(self, action) -> Tuple[List[float], float, bool, bool, Dict]:
        x, xd, th, thd = self.state
        f = self.force if int(action) == 1 else -self.force
        ct, st = math.cos(th), math.sin(th)
        total = self.m_cart + self.m_pole
        pml = self.m_pole * self.half_len
        tmp = (f + pml * thd * thd * st) / total
        tha = (self.gravity * st - ct * tmp) / (self.half_len * (4.0 / 3.0 - self.m_pole * ct * ct / total))
        xa = tmp - pml * tha * ct / total
        self.state = [x + self.tau * xd, xd + self.tau * xa, th + self.tau * thd, thd + self.tau * tha]
        self.t += 1
        x, _, th, _ = self.state
        terminated = abs(x) > self.x_limit or abs(th) > self.theta_limit
        return list(self.state), 1.0, terminated, self.t >= self.max_steps, {}


class PendulumEnv:
    """Torque-limited pendulum (|u| <= 2); observation (cos, sin, angular velocity); reward
    -(angle^2 + 0.1 velocity^2 + 0.001 u^2); never terminates, truncated at ``max_steps``."""
    obs_dim, action_dim, discrete = 3, 1, False
    max_speed, max_torque, dt, g, m, l = 8.0, 2.0, 0.05, 10.0, 1.0, 1.0

    def __init__(self, max_steps: int = 200):
        self.max_steps = max_steps
        self.rng = random.Random(0)
        self.th, self.thd, self.t = 0.0, 0.0, 0

    def _obs(self) -> List[float]:
        return [math.cos(self.th), math.sin(self.th), self.thd]

    def reset(self, seed: Optional[int] = None):
        if seed is not None:
            self.rng = random.Random(seed)
        self.th, self.thd, self.t = self.rng.uniform(-math.pi, math.pi), self.rng.uniform(-1.0, 1.0), 0
        return self._obs(), {}

    def step(self, action):
        u = float(action[0] if isinstance(action, (list, tuple)) else action)
        u = min(max(u, -self.max_torque), self.max_torque)
        ang = ((self.th + math.pi) % (2 * math.pi)) - math.pi
        cost = ang * ang + 0.1 * self.thd * self.thd + 0.001 * u * u
        thd = self.thd + (3 * self.g / (2 * self.l) * math.sin(self.th) + 3.0 / (self.m * self.l ** 2) * u) * self.dt
        self.thd = min(max(thd, -self.max_speed), self.max_speed)
        self.th += self.thd * self.dt
        self.t += 1
        return self._obs(), -cost, False, self.t >= self.max_steps, {}


ENV_TYPES = {"cartpole": CartPoleEnv, "CartPole-v1": CartPoleEnv, "pendulum": PendulumEnv, "Pendulum-v1": PendulumEnv}


class BatchedControlEnv:
    """``num_envs`` independent environments addressed by id. Finished environments ignore further steps (their
    observation is frozen, reward 0), so a batch can be stepped until every member is done."""

    def __init__(self, cfg: Any, num_envs: int):
        get = (lambda k, d=None: cfg.get(k, d)) if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
        self.env_name = get("env_name", "cartpole")
        self.max_steps = int(get("max_steps", 200))
        cls = ENV_TYPES[self.env_name]
        self.envs = [cls(self.max_steps) for _ in range(num_envs)]
        self.obs: List[List[float]] = [[0.0] * cls.obs_dim for _ in range(num_envs)]
        self.done = [True] * num_envs
        self.returns = [0.0] * num_envs
        self.lengths = [0] * num_envs
        self.obs_dim, self.action_dim, self.discrete = cls.obs_dim, cls.action_dim, cls.discrete

    def reset(self, env_ids: Sequence[int], seeds: Optional[Sequence[int]] = None) -> List[List[float]]:
        for j, i in enumerate(env_ids):
            self.obs[i], _ = self.envs[i].reset(None if seeds is None else int(seeds[j]))
            self.done[i], self.returns[i], self.lengths[i] = False, 0.0, 0
        return [list(self.obs[i]) for i in env_ids]

    def step(self, env_ids: Sequence[int], actions: Sequence) -> Dict[str, List]:
        obs, rew, term, trunc = [], [], [], []
        for i, a in zip(env_ids, actions):
            if self.done[i]:
                obs.append(list(self.obs[i])); rew.append(0.0); term.append(True); trunc.append(False)
                continue
            o, r, te, tr, _ = self.envs[i].step(a)
            self.obs[i] = o
            self.returns[i] += r
            self.lengths[i] += 1
            self.done[i] = te or tr
            obs.append(list(o)); rew.append(r); term.append(te); trunc.append(tr)
        return {"observations": obs, "rewards": rew, "terminated": term, "truncated": trunc}

    def chunk_step(self, env_ids: Sequence[int], action_chunks: Sequence[Sequence]) -> Dict[str, List]:
        """Apply a chunk of actions per environment (action-chunking policies); rewards are summed over the chunk."""
        n = len(action_chunks[0]) if action_chunks else 0
        total = [0.0] * len(env_ids)
        out: Dict[str, List] = {}
        for k in range(n):
            out = self.step(env_ids, [c[k] for c in action_chunks])
            total = [t + r for t, r in zip(total, out["rewards"])]
        out["rewards"] = total
        return out

    def get_env_states(self, env_ids: Sequence[int]) -> List[Dict[str, Any]]:
        return [{"done": self.done[i], "return": self.returns[i], "length": self.lengths[i]} for i in env_ids]

    # state hand-over across a simulator restart (the manager stops simulators while the policy trains)
    def get_state(self) -> bytes:
        return pickle.dumps({"envs": [e.__dict__ for e in self.envs], "obs": self.obs, "done": self.done,
                             "returns": self.returns, "lengths": self.lengths})

    def load_state(self, blob: bytes) -> None:
        st = pickle.loads(blob)
        for e, d in zip(self.envs, st["envs"]):
            e.__dict__.update(d)
        self.obs, self.done, self.returns, self.lengths = st["obs"], st["done"], st["returns"], st["lengths"]

    def close(self) -> None:
        pass
