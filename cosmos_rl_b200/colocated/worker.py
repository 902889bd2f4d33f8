"""Colocated RL worker: policy and rollout share one process and one set of GPUs; the controller logic runs
in the same process too (no HTTP, no broker daemon), so a whole job is `ColocatedRLControlWorker(...).run()`
(cosmos_rl/colocated/rl_worker.py:41-229, cosmos_rl/colocated/controller.py:74-552).

The loop is driven by the same Controller object as the disaggregated mode (prompt hand-out with weight
versions, rollout buffer, step scheduling, checkpoint cadence), reached through ``LocalAPIClient``; only the
transport differs. Weight synchronisation is a version bump because the engine generates on the trainer's own
parameter tensors.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

from ..comm.broker import command_stream, rollout_stream
from ..config import Config
from ..dispatcher import command as cmd
from ..dispatcher.api.client import LocalAPIClient
from ..dispatcher.controller import Controller
from ..dispatcher.data import CosmosDataset, WorkerDataFetcher
from ..dispatcher.data.schema import RLPayload, Rollout
from ..dispatcher.protocol import RegisterRequest, Role
from ..data.packer import BaseDataPacker
from ..parallel.dims import ParallelDims
from ..policy.trainer import diffusion_trainer, grpo_trainer, vla_flow_trainer, vla_trainer  # noqa: F401
from ..policy.trainer.base import TrainerRegistry
from ..reward.dispatcher import make_reward_calculator
from ..rollout import (b200_rollout, diffusion_rollout, hf_rollout, openvla_rollout, vla_flow_rollout,  # noqa: F401
                       vla_rollout)                       # (registers the built-in backends)
from ..rollout.base import RolloutRegistry
from ..utils.logging import logger


class ColocatedRLControlWorker:
    def __init__(self, config: Config, dataset, val_dataset=None, reward_fns: Optional[List[Callable]] = None,
                 data_packer=None, device: Optional[torch.device] = None, custom_logger_fns=None, tokenizer=None):
        self.config = config
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.controller = Controller(config, dataset=dataset, val_dataset=val_dataset,
                                     custom_logger_fns=custom_logger_fns)
        self.api = LocalAPIClient(self.controller)
        self.dims = ParallelDims(world_size=1, device=self.device)
        tp = config.train.train_policy
        self.trainer = TrainerRegistry.get_trainer_cls(tp.trainer_type)(config, self.dims, device=self.device,
                                                                        data_packer=data_packer, tokenizer=tokenizer)
        # custom workloads register their own trainer type and rollout backend (non-LLM policies, environments)
        backend = config.rollout.backend
        model_cls = type(self.trainer.model)
        if backend == "b200" and model_cls.__name__ == "HFModel":
            backend = "hf"
        elif backend == "b200" and not getattr(model_cls, "paged_engine", True):
            backend = "recompute"
        self.rollout = RolloutRegistry.get(backend)(config, self.dims, self.device, tokenizer=tokenizer)
        self.rollout.init_engine(shared_model=self.trainer.model)
        if hasattr(self.trainer, "attach_rollout"):
            self.trainer.attach_rollout(self.rollout)
        mt = getattr(getattr(self.trainer.model, "args", None), "model_type", "hfmodel")
        self.packer = data_packer or BaseDataPacker.get_default(mt)()
        self.packer.setup(config, tokenizer)
        self.fetcher = WorkerDataFetcher(config, CosmosDataset.wrap(dataset, config))
        self.rewards = make_reward_calculator(config, reward_fns)
        self.policy_name, self.rollout_name = "colocated-policy", "colocated-rollout"
        self.weight_version = 0
        self._cmd_pos = {self.policy_name: 0, self.rollout_name: 0}
        self._rollout_pos = 0
        self.reports: List[Dict[str, Any]] = []

    def _register(self) -> None:
        for name, role in ((self.policy_name, Role.POLICY), (self.rollout_name, Role.ROLLOUT)):
            self.controller.register(RegisterRequest(replica_name=name, role=role,
                                                     mesh_names=["pp", "dp_shard", "cp", "tp"], ranks=[0, 0, 0, 0],
                                                     group_size=[1, 1, 1, 1], global_rank=0))

    def _commands(self, name: str) -> List[cmd.Command]:
        msgs = self.controller.broker.read(command_stream(name), self._cmd_pos[name], 64, 0)
        if msgs:
            self._cmd_pos[name] = msgs[-1][0]
        return [cmd.Command.depack(d) for _, d in msgs]

    # ------------------------------------------------------------------ one pass of each side
    def _rollout_pass(self) -> bool:
        """Generate for one batch of prompts; returns False when the prompt stream has ended."""
        for c in self._commands(self.rollout_name):
            if isinstance(c, cmd.RolloutToRolloutBroadcastCommand) and c.weight_step is not None:
                self.weight_version = c.weight_step
            if isinstance(c, cmd.StopCommand):
                return False
        batch, is_end = self.api.get_next_prompt(self.config.rollout.batch_size)
        if not batch:
            return not is_end
        payloads = [self.fetcher.fill(p) for _, p in batch]
        sync = getattr(self.trainer, "before_weight_sync", None)      # LoRA: generate with the adapters folded in
        if sync is not None:
            sync()
        try:
            results = self.rollout.rollout_generation(payloads, self.packer)
        finally:
            if sync is not None:
                self.trainer.after_weight_sync()
        for p, r in zip(payloads, results):
            p.completions = r.completions
            p.completed_conversations = r.completed_conversations
            if r.completion_token_ids is not None:
                p.completion_token_ids = [[[t] for t in toks] for toks in r.completion_token_ids]
                p.completion_logprobs = [[[l] for l in lps] for lps in r.completion_logprobs]
            if r.extra_info is not None:
                p.extra_info = r.extra_info
            p.weight_version = self.weight_version
            self.rewards.compute(p)
        self.api.post_rollout_completion(self.rollout_name, payloads, is_end=is_end)
        return not is_end

    def _policy_pass(self) -> bool:
        """Execute pending policy commands; returns True when training is over."""
        done = False
        for c in self._commands(self.policy_name):
            if isinstance(c, cmd.WeightResumeCommand):
                if self.trainer.weight_resume():
                    self.api.post_resume_info(getattr(self.trainer, "resume_extra_info", {}))
            elif isinstance(c, cmd.DataFetchCommand):
                msgs = self.controller.broker.read(rollout_stream(self.policy_name), self._rollout_pos, c.items_count, 0)
                self._rollout_pos = msgs[-1][0] if msgs else self._rollout_pos
                rollouts = [self.fetcher.fill(Rollout.model_validate_json(d)) for _, d in msgs]
                report = self.trainer.step_training(rollouts, c.global_step, c.total_steps, c.remain_samples_num,
                                                    do_save=c.do_save)
                self.reports.append(report)
                self.api.post_train_ack(self.policy_name, c.global_step, c.total_steps, False, report)
                done = done or c.replica_should_stop()
            elif isinstance(c, cmd.TrainingCompleteCommand):
                if c.do_save:
                    self.trainer.save_checkpoint(c.final_step, c.checkpoint_total_steps, c.remain_samples_num, True)
                done = True
        return done

    def run(self, max_iterations: int = 1 << 30) -> List[Dict[str, Any]]:
        self._register()
        more = True
        for _ in range(max_iterations):
            if self._policy_pass():
                break
            if more:
                more = self._rollout_pass()
                continue
            # prompts are exhausted: keep serving policy commands until the controller has none left
            if not self.controller.broker.read(command_stream(self.policy_name), self._cmd_pos[self.policy_name], 1, 0):
                break
        if getattr(self.trainer, "ckpt_manager", None) is not None:
            self.trainer.ckpt_manager.finalize()
        self.controller.unregister(self.policy_name)
        self.controller.unregister(self.rollout_name)
        return self.reports
