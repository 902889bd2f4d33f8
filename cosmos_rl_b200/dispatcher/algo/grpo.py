"""Rule-based RL algorithms: reward aggregation and group-relative advantages
(cosmos_rl/dispatcher/algo/grpo.py:38-47, cosmos_rl/dispatcher/algo/base.py)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

_ALGOS: Dict[str, type] = {}


def register_rule_based_algo(name: str, cls: Optional[type] = None):
    def deco(c):
        _ALGOS[name] = c
        return c
    return deco(cls) if cls is not None else deco


def get_rule_based_algo(name: str) -> type:
    if name not in _ALGOS:
        raise KeyError(f"unknown rule-based algo {name!r}; known: {sorted(_ALGOS)}")
    return _ALGOS[name]


class RuleBasedAlgo:
    def compute_reward(self, to_be_evaluated, reference, prompt=None, **kw) -> float:
        raise NotImplementedError

    def compute_advantage(self, rewards: Sequence[float]) -> List[float]:
        raise NotImplementedError


@register_rule_based_algo("grpo")
class GRPO(RuleBasedAlgo):
    """reward = weighted sum of reward functions; advantage = (r - mean) / (std + 1e-6) within the prompt's
    group, or r - mean when ``unbiased_advantage``."""

    def __init__(self, reward_fn: Callable, unbiased: bool = False, filter_reward_fn: Optional[Callable] = None):
        self.reward_fn = reward_fn
        self.filter_reward_fn = filter_reward_fn
        self.unbiased = unbiased

    def compute_reward(self, to_be_evaluated, reference, prompt=None, **kw):
        return self.reward_fn(to_be_evaluated, reference, prompt=prompt, **kw)

    def compute_filter_reward(self, to_be_evaluated, reference, prompt=None, **kw):
        if self.filter_reward_fn is None:
            return None
        return self.filter_reward_fn(to_be_evaluated, reference, prompt=prompt, **kw)

    def compute_advantage(self, rewards):
        r = np.asarray(rewards, dtype=np.float64)
        if r.size == 0:
            return []
        centered = r - r.mean()
        if self.unbiased:
            return centered.tolist()
        return (centered / (r.std() + 1e-6)).tolist()
