"""Drives a batched environment with the policy for whole episodes and returns tensor trajectories
(cosmos_rl/tools/gym_example/gym_rollout.py)."""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import torch

from ...simulators import EnvManager, get_env_cls
from ...utils.trace import trace_op
from .gym_policy import GymPolicy


class GymRolloutEngine:
    def __init__(self, policy: GymPolicy, env_name: str = "cartpole", num_envs: int = 8, max_steps: int = 200,
                 use_subprocess: bool = False, device=None):
        self.policy, self.device = policy, device or torch.device("cpu")
        self.num_envs, self.max_steps = num_envs, max_steps
        self.env = EnvManager({"num_envs": num_envs, "env_name": env_name, "max_steps": max_steps}, 0,
                              get_env_cls(env_name), use_subprocess=use_subprocess)

    def run(self, seeds: Sequence[int], greedy: bool = False) -> List[Dict[str, Any]]:
        """One episode per seed (at most ``num_envs`` at a time). Each trajectory: observations [L, obs], actions
        [L] or [L, act], rewards [L], log-probs [L], episode_length, terminated."""
        out: List[Dict[str, Any]] = []
        self.env.start_simulator()
        for s0 in range(0, len(seeds), self.num_envs):
            chunk = list(seeds[s0:s0 + self.num_envs])
            ids = list(range(len(chunk)))
            with trace_op("gym_episode_batch", n=len(chunk)):
                obs = self.env.reset(ids, chunk)
                traj = [{"observations": [], "actions": [], "rewards": [], "logprobs": [], "terminated": False}
                        for _ in ids]
                live = list(ids)
                for _ in range(self.max_steps):
                    if not live:
                        break
                    o = torch.tensor([obs[i] for i in live], dtype=torch.float32, device=self.device)
                    a, lp = self.policy.act(o, greedy)
                    acts = a.tolist()
                    res = self.env.step(live, acts)
                    nxt = []
                    for j, i in enumerate(live):
                        t = traj[i]
                        t["observations"].append(obs[i]); t["actions"].append(acts[j])
                        t["rewards"].append(res["rewards"][j]); t["logprobs"].append(float(lp[j]))
                        obs[i] = res["observations"][j]
                        if res["terminated"][j] or res["truncated"][j]:
                            t["terminated"] = bool(res["terminated"][j])
                        else:
                            nxt.append(i)
                    live = nxt
            for t in traj:
                t["episode_length"] = len(t["rewards"])
                out.append(t)
        return out

    def close(self) -> None:
        self.env.stop_simulator()
