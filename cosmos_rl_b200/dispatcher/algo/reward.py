"""Built-in reward functions and the weighted reward combiner
(cosmos_rl/dispatcher/algo/reward.py:93-496). A reward function has the signature
``fn(to_be_evaluated, reference, prompt=None, **kwargs) -> float | (float, dict)``."""
from __future__ import annotations

import re
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

_REWARDS: Dict[str, Callable] = {}


def register_reward_fn(name: str):
    def deco(fn):
        _REWARDS[name] = fn
        return fn
    return deco


def get_reward_fn(name: str) -> Callable:
    if name not in _REWARDS:
        raise KeyError(f"unknown reward function {name!r}; known: {sorted(_REWARDS)}")
    return _REWARDS[name]


def _text(x) -> str:
    if isinstance(x, str):
        return x
    if isinstance(x, dict):
        return str(x.get("content", ""))
    if isinstance(x, (list, tuple)) and x and isinstance(x[-1], dict):
        return str(x[-1].get("content", ""))
    return str(x)


@register_reward_fn("format")
def format_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    """1.0 when the completion has the ``<think>...</think><answer>...</answer>`` structure."""
    s = _text(to_be_evaluated)
    return 1.0 if re.fullmatch(r"\s*<think>.*?</think>\s*<answer>.*?</answer>\s*", s, re.DOTALL) else 0.0


@register_reward_fn("single_choice")
def single_choice_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    s = _text(to_be_evaluated)
    m = re.search(r"<answer>(.*?)</answer>", s, re.DOTALL)
    ans = (m.group(1) if m else s).strip()
    return 1.0 if reference is not None and ans.lower() == str(reference).strip().lower() else 0.0


@register_reward_fn("boxed_math")
def boxed_math_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    s = _text(to_be_evaluated)
    m = re.findall(r"\\boxed\{([^{}]*)\}", s)
    if not m or reference is None:
        return 0.0
    norm = lambda t: re.sub(r"[\s,$]", "", str(t))
    return 1.0 if norm(m[-1]) == norm(reference) else 0.0


@register_reward_fn("gsm8k")
def gsm8k_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    s = _text(to_be_evaluated)
    nums = re.findall(r"-?\d[\d,]*\.?\d*", s)
    if not nums or reference is None:
        return 0.0
    ref = re.findall(r"-?\d[\d,]*\.?\d*", str(reference))
    if not ref:
        return 0.0
    try:
        return 1.0 if float(nums[-1].replace(",", "")) == float(ref[-1].replace(",", "")) else 0.0
    except ValueError:
        return 0.0


@register_reward_fn("overlong")
def overlong_reward(to_be_evaluated, reference=None, prompt=None, *, length: Optional[int] = None,
                    max_length: int = 0, buffer_length: int = 0, penalty_factor: float = 1.0, **kw) -> float:
    """DAPO soft overlong punishment: linear penalty inside the last ``buffer_length`` tokens."""
    if length is None or buffer_length <= 0 or max_length <= 0:
        return 0.0
    expected = max_length - buffer_length
    exceed = length - expected
    return min(-exceed / buffer_length * penalty_factor, 0.0) if exceed > 0 else 0.0


@register_reward_fn("even_token_fraction")
def even_token_fraction(to_be_evaluated, reference=None, prompt=None, *, token_ids: Optional[Sequence[int]] = None,
                        **kw) -> float:
    """Synthetic benchmark reward: the fraction of response token ids that are even."""
    ids = token_ids
    if ids is None:
        if isinstance(to_be_evaluated, (list, tuple)):
            ids = to_be_evaluated
        else:
            ids = [int(t) for t in re.findall(r"\d+", _text(to_be_evaluated))]
    if not ids:
        return 0.0
    return sum(1 for t in ids if int(t) % 2 == 0) / len(ids)


class Reward:
    """Weighted sum of named (or user supplied) reward functions."""

    def __init__(self, spec: Union[str, List[str], Dict[str, float], None] = None,
                 explicit_fns: Optional[List[Callable]] = None):
        self.fns: List[Tuple[Callable, float]] = []
        if explicit_fns:
            self.fns = [(f, 1.0) for f in explicit_fns]
        elif spec:
            if isinstance(spec, str):
                spec = [spec]
            if isinstance(spec, (list, tuple)):
                spec = {n: 1.0 for n in spec}
            self.fns = [(get_reward_fn(n), float(w)) for n, w in spec.items()]

    def __call__(self, to_be_evaluated, reference, prompt=None, **kw) -> float:
        total = 0.0
        for fn, w in self.fns:
            r = fn(to_be_evaluated, reference, prompt=prompt, **kw)
            if isinstance(r, tuple):
                r = r[0]
            total += w * float(r)
        return total

    def batch(self, to_be_evaluated: List[Any], reference, prompt=None, **kw) -> List[float]:
        """``group_reward_calculation``: every function is called once with all completions of a prompt and returns
        one value per completion, optionally ``(values, per-completion dicts)`` (cosmos_rl/dispatcher/algo/reward.py:
        396-427). Useful when scoring shares work across the group (one verifier call, one judge request)."""
        total = [0.0] * len(to_be_evaluated)
        for fn, w in self.fns:
            vals = fn(to_be_evaluated, reference, prompt=prompt, **kw)
            if isinstance(vals, tuple) and len(vals) == 2:
                vals = vals[0]
            if not isinstance(vals, (list, tuple)) or len(vals) != len(to_be_evaluated):
                raise ValueError("with group_reward_calculation a reward function returns one value per completion")
            for i, v in enumerate(vals):
                total[i] += w * float(v)
        return total
