"""Colocated mode: policy and rollout share the same GPUs and the same parameter tensors.

``ColocatedGRPO`` is the in-process form of the GRPO loop (the reference's colocated worker with its
in-process controller: cosmos_rl/colocated/rl_worker.py:41-229, colocated/controller.py:74-552): the
rollout engine generates on the policy model's own bf16 weights, so publishing new weights after the
optimizer step costs nothing but a version bump and CUDA-graph reuse.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from ..config import Config
from ..dispatcher.algo.grpo import GRPO
from ..dispatcher.algo.reward import Reward
from ..dispatcher.data.schema import Rollout
from ..parallel.dims import ParallelDims
from ..policy.trainer.base import TrainerRegistry
from ..policy.trainer import grpo_trainer  # noqa: F401  (registers "grpo")
from ..rollout.engine import RolloutEngine, SamplingParams


class ColocatedGRPO:
    def __init__(self, config: Config, parallel_dims: Optional[ParallelDims] = None, device=None,
                 reward_fns: Optional[List[Callable]] = None, max_num_seqs: Optional[int] = None, **trainer_kw):
        self.config = config
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.dims = parallel_dims or ParallelDims(world_size=1, device=self.device)
        self.dims.device = self.device
        tp = config.train.train_policy
        self.trainer = TrainerRegistry.get_trainer_cls(tp.trainer_type)(config, self.dims, device=self.device,
                                                                        **trainer_kw)
        self.trainer.weight_resume()
        r = config.rollout
        self.sampling = SamplingParams.from_config(config)
        n_seqs = max_num_seqs or max(8, r.batch_size * r.n_generation)
        self.engine = RolloutEngine(
            self.trainer.model, max_num_seqs=n_seqs, max_model_len=config.policy.model_max_length,
            page_size=config.b200.rollout_page_size, use_cuda_graph=config.b200.cuda_graph_decode,
            seed=(r.seed or 0) + 7919 * int(getattr(self.dims, "global_rank", 0) or 0))
        reward = Reward(tp.reward_function, explicit_fns=reward_fns)
        self.algo = GRPO(reward, unbiased=tp.unbiased_advantage)
        self.step_idx = 0
        self.weight_version = 0
        self.last_timing: Dict[str, float] = {}

    # ------------------------------------------------------------------
    def rollout(self, prompts: Sequence, references: Optional[Sequence] = None) -> List[Rollout]:
        self.trainer.before_weight_sync()              # LoRA: the engine reads the base weights with adapters folded in
        try:
            outs = self.engine.generate(prompts, self.sampling)
        finally:
            self.trainer.after_weight_sync()
        rollouts: List[Rollout] = []
        for pi, comps in enumerate(outs):
            ref = references[pi] if references is not None else None
            p = prompts[pi]
            p_list = p.tolist() if torch.is_tensor(p) else list(p)
            rewards = [self.algo.compute_reward(c.token_ids, ref, prompt=p_list, token_ids=c.token_ids) for c in comps]
            advs = self.algo.compute_advantage(rewards)
            for c, rw, adv in zip(comps, rewards, advs):
                rollouts.append(Rollout(prompt=p_list, prompt_idx=pi, completion=c.token_ids, reward=rw,
                                        advantage=adv, weight_version=self.weight_version,
                                        completion_token_ids=[[t] for t in c.token_ids],
                                        completion_logprobs=[[l] for l in c.logprobs]))
        return rollouts

    def step(self, prompts: Sequence, references: Optional[Sequence] = None, total_steps: int = 1 << 30
             ) -> Dict[str, Any]:
        """One full GRPO step: generate, score, train, publish weights."""
        t0 = time.perf_counter()
        rollouts = self.rollout(prompts, references)
        t1 = time.perf_counter()
        self.step_idx += 1
        report = self.trainer.step_training(rollouts, self.step_idx, total_steps)
        # the engine reads the very tensors the optimizer just rewrote: publishing is a version bump
        self.weight_version = self.step_idx
        self.engine.weight_version = self.weight_version
        t2 = time.perf_counter()
        n_tok = sum(len(r.prompt) + len(r.completion) for r in rollouts)
        report.update({"rollout/time": t1 - t0, "train/time": t2 - t1, "step/tokens": float(n_tok),
                       "rollout/reward_mean": sum(r.reward for r in rollouts) / max(1, len(rollouts)),
                       "weight_sync/ms": 0.0})
        self.last_timing = {"rollout_s": t1 - t0, "train_s": t2 - t1}
        return report
