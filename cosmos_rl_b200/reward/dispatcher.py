"""Reward computation for finished generations (cosmos_rl/reward/dispatcher.py:27-264,
reward/local_calculator.py:27-360, reward/base.py:22-169).

The rollout worker enqueues one task per prompt (its n completions); a worker pool computes rewards,
group-relative advantages, DAPO validity (a group whose filter rewards are all equal carries no signal and
is dropped) and the shared-prefix mask (completions of one group that start with the same long prefix but
got different rewards: the prefix tokens are excluded from the loss). Finished payloads are collected with
``dequeue``.
"""
from __future__ import annotations

import concurrent.futures
import queue
import threading
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from ..dispatcher.algo.grpo import GRPO
from ..dispatcher.algo.reward import Reward, get_reward_fn
from ..dispatcher.data.schema import RLPayload


def shared_prefix_ignore(token_lists: Sequence[Sequence[int]], rewards: Sequence[float], min_tokens: int) -> List[int]:
    """For each completion: length of the longest prefix (>= ``min_tokens``) it shares with a completion of the
    same group that received a different reward."""
    n = len(token_lists)
    out = [0] * n
    for i in range(n):
        for j in range(n):
            if i == j or rewards[i] == rewards[j]:
                continue
            a, b = token_lists[i], token_lists[j]
            k = 0
            m = min(len(a), len(b))
            while k < m and a[k] == b[k]:
                k += 1
            if k >= min_tokens:
                out[i] = max(out[i], k)
    return out


class LocalRewardCalculator:
    def __init__(self, config, reward_fns: Optional[List[Callable]] = None,
                 filter_reward_fns: Optional[List[Callable]] = None, validation: bool = False):
        self.config = config
        tp = config.train.train_policy
        spec = config.validation.reward_function if validation and config.validation.reward_function else \
            getattr(tp, "reward_function", None)
        self.reward = Reward(spec, explicit_fns=reward_fns)
        self.filter_reward = Reward(getattr(tp, "filter_reward_metric", None), explicit_fns=filter_reward_fns) \
            if (filter_reward_fns or getattr(tp, "filter_reward_metric", None)) else None
        self.algo = GRPO(self.reward, unbiased=getattr(tp, "unbiased_advantage", False),
                         filter_reward_fn=self.filter_reward)
        self.variant = getattr(tp, "variant", "grpo")
        self.min_prefix = getattr(tp, "min_filter_prefix_tokens", None)
        self.bypass = bool(getattr(tp, "bypass_reward", False))
        self.grouped = bool(getattr(tp, "group_reward_calculation", False))
        self.overlong = getattr(tp, "overlong_reward", None)
        self.max_response = config.rollout.max_response_length
        self.adv_low = getattr(tp, "advantage_low", -1e9)
        self.adv_high = getattr(tp, "advantage_high", 1e9)

    def compute(self, payload: RLPayload) -> RLPayload:
        comps = payload.completions or []
        toks = [[p[0] for p in c] for c in payload.completion_token_ids] if payload.completion_token_ids else None
        if self.bypass:
            payload.rewards = [0.0] * len(comps)
            payload.advantages = [0.0] * len(comps)
            payload.filter_rewards = [0.0] * len(comps)
            payload.valid = True
            return payload
        rewards, filt = [], []
        grouped = None
        if self.grouped and comps and hasattr(self.algo.reward_fn, "batch"):
            grouped = self.algo.reward_fn.batch(list(comps), payload.reference_answer, prompt=payload.prompt,
                                                **({"token_ids": toks} if toks else {}))
        for i, c in enumerate(comps):
            kw = {"token_ids": toks[i]} if toks else {}
            r = float(grouped[i]) if grouped is not None else float(
                self.algo.compute_reward(c, payload.reference_answer, prompt=payload.prompt, **kw))
            if self.overlong is not None and self.overlong.enable_overlong_penalty and toks:
                from ..dispatcher.algo.reward import overlong_reward
                r += overlong_reward(c, length=len(toks[i]), max_length=self.max_response,
                                     buffer_length=self.overlong.buffer_length,
                                     penalty_factor=self.overlong.penalty_factor)
            rewards.append(r)
            f = self.algo.compute_filter_reward(c, payload.reference_answer, prompt=payload.prompt, **kw)
            filt.append(float(f) if f is not None else r)
        advs = [min(max(a, self.adv_low), self.adv_high) for a in self.algo.compute_advantage(rewards)]
        payload.rewards, payload.advantages, payload.filter_rewards = rewards, advs, filt
        payload.valid = True
        if self.variant == "dapo" and len(set(filt)) <= 1:
            payload.valid = False   # dynamic sampling: no learning signal in this group
        if self.min_prefix and toks:
            payload.n_ignore_prefix_tokens = shared_prefix_ignore(toks, rewards, self.min_prefix)
        return payload


class RemoteRewardCalculator:
    """Scores completions through the HTTP reward service (``train_policy.use_remote_reward``): the completions of a
    prompt go out as one media tensor, every configured reward function returns one score per completion, and the
    reward is ``clip(scale * sum_f weight_f * clip_f(score_f))`` (cosmos_rl/reward/remote_calculator.py:41-436; the
    service address comes from the environment there as well: REMOTE_REWARD_ENQUEUE_URL / _FETCH_URL)."""

    def __init__(self, config, url: Optional[str] = None, timeout_s: float = 600.0, validation: bool = False):
        import os
        from ..reward_service.client import RewardClient
        url = url or os.environ.get("REMOTE_REWARD_URL") or os.environ.get("REMOTE_REWARD_ENQUEUE_URL", "")
        if not url:
            raise ValueError("use_remote_reward needs the service address in REMOTE_REWARD_URL")
        for suffix in ("/api/reward/enqueue", "/api/reward/pull"):
            if url.endswith(suffix):
                url = url[:-len(suffix)]
        self.config, self.url = config, url
        self.rr = config.train.train_policy.remote_reward
        if not self.rr.reward_fns:
            raise ValueError("train.train_policy.remote_reward.reward_fns names no reward function")
        self.client = RewardClient(url, timeout_s=timeout_s)
        self.local = LocalRewardCalculator(config, reward_fns=[lambda *a, **k: 0.0], validation=validation)

    @staticmethod
    def media_of(completions) -> "torch.Tensor":
        """One tensor [n, ...] from the completions of a prompt: tensors, dicts that carry ``media`` or the handle of a
        stored sample (diffusion rollouts keep their latents in the process-local store)."""
        import torch
        items = []
        for c in completions:
            if isinstance(c, dict) and "latent_id" in c:
                from ..rollout.diffusion_rollout import LatentStore
                c = LatentStore.get(c)["x0"]
            elif isinstance(c, dict) and "media" in c:
                c = c["media"]
            items.append(torch.as_tensor(c).detach().float().cpu())
        return torch.stack(items)

    def compute(self, payload: RLPayload) -> RLPayload:
        rr = self.rr
        comps = payload.completions or []
        meta = {"prompt": payload.prompt if isinstance(payload.prompt, str) else None, "prompt_idx": payload.prompt_idx}
        res = self.client.score([f.name for f in rr.reward_fns], meta, self.media_of(comps))
        total = [0.0] * len(comps)
        for f in rr.reward_fns:
            scores = res[f.name]["scores"]
            vals = scores[f.score_key] if f.score_key else next(iter(scores.values()))
            if len(vals) != len(comps):
                raise ValueError(f"reward {f.name!r} returned {len(vals)} scores for {len(comps)} completions")
            for i, v in enumerate(vals):
                total[i] += f.weight * min(max(float(v), f.clip_min), f.clip_max)
        rewards = [min(max(t * rr.scale, rr.reward_clip_min), rr.reward_clip_max) for t in total]
        payload.rewards = rewards
        payload.advantages = [min(max(a, self.local.adv_low), self.local.adv_high)
                              for a in self.local.algo.compute_advantage(rewards)]
        payload.filter_rewards = list(rewards)
        payload.valid = True
        return payload


def make_reward_calculator(config, reward_fns=None, filter_reward_fns=None, validation: bool = False):
    """Local rule-based rewards, or the remote service when the (validation) policy asks for it."""
    tp = config.train.train_policy
    remote = config.validation.use_remote_reward if validation else getattr(tp, "use_remote_reward", False)
    if remote:
        return RemoteRewardCalculator(config, validation=validation)
    if validation:
        return LocalRewardCalculator(config, reward_fns, validation=True)
    return LocalRewardCalculator(config, reward_fns, filter_reward_fns)


class RewardDispatcher:
    def __init__(self, calculator, num_workers: int = 2):
        self.calc = calculator
        self.pool = concurrent.futures.ThreadPoolExecutor(max_workers=max(1, num_workers),
                                                          thread_name_prefix="reward")
        self.pending: "queue.Queue[concurrent.futures.Future]" = queue.Queue()
        self.n_inflight = 0
        self.lock = threading.Lock()

    def enqueue_rewards_cal(self, payloads: List[RLPayload], is_validation: bool = False, step: int = 0) -> None:
        for p in payloads:
            with self.lock:
                self.n_inflight += 1
            self.pending.put(self.pool.submit(self.calc.compute, p))

    def dequeue(self, block: bool = False, timeout: Optional[float] = None) -> List[RLPayload]:
        """Payloads whose rewards are done, in submission order (stops at the first unfinished one unless
        ``block``)."""
        out: List[RLPayload] = []
        while True:
            try:
                fut = self.pending.queue[0] if not block else self.pending.get(timeout=timeout)
            except (IndexError, queue.Empty):
                break
            if not block:
                if not fut.done():
                    break
                self.pending.get_nowait()
            out.append(fut.result())
            with self.lock:
                self.n_inflight -= 1
            if block and self.pending.empty():
                break
        return out

    def is_empty(self) -> bool:
        return self.n_inflight == 0

    def shutdown(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)
