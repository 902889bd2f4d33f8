"""Rollout backend ``vla``: action-token policies in closed loop with an environment
(cosmos_rl/rollout/vla_rollout/: OpenVLA-style discretised actions; environments through simulators/env_manager.py).

One "prompt" is an initial condition (``{"seed": n}``), one "completion" a whole episode. At every control step the
observation is turned into tokens, the language-model policy generates ``action_dim`` tokens through the paged
generation engine, the tokens are decoded into a continuous action (256 uniform bins per dimension, as OpenVLA's
action tokenizer does) and the batched environment is stepped. The episode stores, per step, the observation tokens,
the action tokens and their behaviour log-probs, which is all the GRPO trainer needs."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..simulators import EnvManager, get_env_cls
from .b200_rollout import B200Rollout
from .base import RolloutRegistry, RolloutResult
from .engine import SamplingParams


class ActionTokenizer:
    """Uniform bins over ``[low, high]`` per action dimension. Any vocabulary id decodes (id mod n_bins), so sampling
    needs no logit mask and the recorded log-probs are exact."""

    def __init__(self, low: Sequence[float], high: Sequence[float], n_bins: int = 256, discrete: bool = False):
        self.low, self.high, self.n_bins, self.discrete = list(low), list(high), n_bins, discrete

    def decode(self, tokens: Sequence[int]) -> Any:
        if self.discrete:                       # one token chooses among `high[0] + 1` discrete actions
            return int(tokens[0]) % (int(self.high[0]) + 1)
        out = []
        for t, lo, hi in zip(tokens, self.low, self.high):
            b = int(t) % self.n_bins
            out.append(lo + (b + 0.5) / self.n_bins * (hi - lo))
        return out

    def encode(self, action: Sequence[float]) -> List[int]:
        return [min(self.n_bins - 1, max(0, int((a - lo) / (hi - lo) * self.n_bins)))
                for a, lo, hi in zip(action, self.low, self.high)]


class ObservationTokenizer:
    """State observations -> tokens: each dimension is clipped to its range and binned; dimension i uses the id block
    ``[offset + i * n_bins, offset + (i + 1) * n_bins)`` so the model can tell dimensions apart."""

    def __init__(self, low: Sequence[float], high: Sequence[float], n_bins: int = 256, offset: int = 1024):
        self.low, self.high, self.n_bins, self.offset = list(low), list(high), n_bins, offset

    def encode(self, obs: Sequence[float]) -> List[int]:
        ids = []
        for i, (x, lo, hi) in enumerate(zip(obs, self.low, self.high)):
            b = int((min(max(x, lo), hi) - lo) / (hi - lo) * (self.n_bins - 1))
            ids.append(self.offset + i * self.n_bins + b)
        return ids


ENV_SPECS = {
    "cartpole": dict(obs_low=[-2.4, -3.0, -0.21, -3.0], obs_high=[2.4, 3.0, 0.21, 3.0], act_low=[0], act_high=[1],
                     discrete=True),
    "pendulum": dict(obs_low=[-1, -1, -8], obs_high=[1, 1, 8], act_low=[-2.0], act_high=[2.0], discrete=False),
}


def vla_options(config) -> Dict[str, Any]:
    d = dict(env_name="cartpole", max_steps=100, num_envs=16, n_bins=256, subprocess_env=False)
    d.update(config.custom.get("vla", {}))
    return d


@RolloutRegistry.register("vla")
class VLARollout(B200Rollout):
    def init_engine(self, load_format: str = "dummy", shared_model=None, seed: Optional[int] = None, **kw) -> None:
        super().init_engine(load_format, shared_model=shared_model, seed=seed, **kw)
        o = self.opts = vla_options(self.config)
        spec = ENV_SPECS[o["env_name"]]
        self.actions = ActionTokenizer(spec["act_low"], spec["act_high"], o["n_bins"], spec["discrete"])
        self.observations = ObservationTokenizer(spec["obs_low"], spec["obs_high"], o["n_bins"])
        self.env = EnvManager({"num_envs": o["num_envs"], "env_name": o["env_name"], "max_steps": o["max_steps"]},
                              0, get_env_cls(o["env_name"]), use_subprocess=bool(o["subprocess_env"]))

    def _seed_of(self, prompt) -> int:
        p = prompt["prompt"] if isinstance(prompt, dict) and "prompt" in prompt else prompt
        p = json.loads(p) if isinstance(p, str) else p
        return int(p["seed"] if isinstance(p, dict) else p)

    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        n = self.config.validation.n_generation if is_validation else self.config.rollout.n_generation
        seeds = [self._seed_of(p.prompt) * 1000003 + g for p in payloads for g in range(n)]
        episodes: List[Dict[str, Any]] = []
        sp = SamplingParams.from_config(self.config, validation=is_validation)
        sp.n, sp.stop_token_ids = 1, ()
        sp.max_tokens = 1 if self.actions.discrete else len(self.actions.low)
        self.env.start_simulator()
        E = self.opts["num_envs"]
        for s0 in range(0, len(seeds), E):
            chunk = seeds[s0:s0 + E]
            ids = list(range(len(chunk)))
            obs = self.env.reset(ids, chunk)
            eps = [{"steps": [], "rewards": []} for _ in ids]
            live = list(ids)
            for _ in range(self.opts["max_steps"]):
                if not live:
                    break
                prompts = [self.observations.encode(obs[i]) for i in live]
                outs = self.engine.generate(prompts, sp)
                acts = [self.actions.decode(o[0].token_ids) for o in outs]
                res = self.env.step(live, acts)
                nxt = []
                for j, i in enumerate(live):
                    eps[i]["steps"].append({"obs_tokens": prompts[j], "action_tokens": list(outs[j][0].token_ids),
                                            "logprobs": list(outs[j][0].logprobs)})
                    eps[i]["rewards"].append(res["rewards"][j])
                    obs[i] = res["observations"][j]
                    if not (res["terminated"][j] or res["truncated"][j]):
                        nxt.append(i)
                live = nxt
            for e in eps:
                e["episode_length"] = len(e["rewards"])
                episodes.append(e)
        self.env.stop_simulator()
        return [RolloutResult(prompt=p.prompt, completions=episodes[i * n:(i + 1) * n]) for i, p in enumerate(payloads)]


def episode_return(completion, reference=None, **kw) -> float:
    return float(sum(completion["rewards"]))
