"""Supervised fine-tuning trainer: token cross-entropy on packed sequences through the fused lm_head kernel,
token-balanced across data-parallel ranks (cosmos_rl/policy/trainer/llm_trainer/sft_trainer.py:49-553)."""
from __future__ import annotations

import time
from typing import Any, Dict, List, Sequence

import torch
import torch.distributed as dist

from ...utils.sequence_packing import pack_sequences, token_budget_batches
from ..loss import sft_ce_loss
from .base import TrainerRegistry
from .llm_trainer import LLMTrainer


@TrainerRegistry.register("sft")
class SFTTrainer(LLMTrainer):
    def _pack(self, samples: List[Dict[str, Any]]) -> Dict[str, Any]:
        seqs = [s["input_ids"] for s in samples]
        # mask[i] = 1 where token i+1 is a label to learn
        masks = [[1 if (i + 1 < len(s["label_ids"]) and s["label_ids"][i + 1] != -100) else 0
                  for i in range(len(s["input_ids"]))] for s in samples]
        b = pack_sequences(seqs, masks, device=self.device,
                           pad_multiple=self.pack_multiple())
        b = self.cp_shard(b)
        sel = (b["label_ids"] >= 0).nonzero(as_tuple=True)[0]
        b["sel"], b["labels_sel"] = sel, b["label_ids"][sel]
        if any(s.get("mm") for s in samples):
            from ...data.packer import merge_mm
            b["mm"] = merge_mm([s.get("mm") for s in samples])
        return b

    def _batches(self, processed: List[Dict[str, Any]]) -> List[List[int]]:
        tp = self.config.train.train_policy
        budget = getattr(tp, "load_balanced_max_tokens_for_batch", None)
        if budget:
            return token_budget_batches([len(s["input_ids"]) for s in processed], budget)
        mb = max(1, tp.mini_batch)
        if self.parallel_dims.pp > 1:           # the packed batches are the micro-batches of the pipeline schedule
            mb = max(1, self.config.policy.parallelism.pp_micro_batch_size)
        return [list(range(i, min(i + mb, len(processed)))) for i in range(0, len(processed), mb)]

    def _loss_of(self, total_tokens):
        def loss_of(hidden, i, b):
            lp, _ = self.model.logprobs(hidden[b["sel"]], b["labels_sel"], 1.0)
            return sft_ce_loss(lp, total_tokens)
        return loss_of

    def step_training(self, global_batch: Sequence[Any], total_steps: int, train_step: int, save_freq: int = 0,
                      do_save: bool = False, **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        self.total_steps = total_steps
        max_len = self.config.policy.model_max_length
        processed = [self.data_packer.sft_process_sample(s) for s in global_batch]
        for p in processed:
            if not p.get("mm"):                 # image placeholder tokens must stay in step with the pixel inputs
                p["input_ids"], p["label_ids"] = p["input_ids"][:max_len], p["label_ids"][:max_len]
        packed = [self._pack([processed[i] for i in idxs]) for idxs in self._batches(processed)]
        tok = torch.tensor(float(sum(b["n_scored"] for b in packed)), device=self.device)
        dp = self.parallel_dims.dp_shard
        if dp > 1 and getattr(self.config.train.train_policy, "balance_dp_token", True):
            dist.all_reduce(tok, group=self.parallel_dims.group("dp_shard"))
            tok = tok / dp
        inter = getattr(self, "inter_replica", None)
        if inter is not None:
            tok = inter.balance_token_count(tok)
        self.model.train()
        self.optimizer.zero_grad()
        losses = self.run_batches_train(packed, self._loss_of(tok.clamp_min(1.0)))
        if inter is not None:
            inter.all_reduce_grads(self.flat.grad)
        norm = self.optimizer_step()
        self.train_step = train_step
        if do_save:
            self.save_checkpoint(train_step, total_steps, is_final=train_step >= total_steps)
        loss_sum = self.pp_sum(torch.stack(losses).sum() if losses else torch.zeros((), device=self.device))
        if self.parallel_dims.cp > 1:                       # every cp rank saw a part of every sequence
            dist.all_reduce(loss_sum, group=self.parallel_dims.group("cp"))
        return {"train/loss_avg": float(loss_sum), "train/loss_max": float(loss_sum),
                "train/learning_rate": self.optimizer.lr * self.lr_scale(max(train_step - 1, 0)),
                "train/iteration_time": time.perf_counter() - t0, "train/grad_norm": float(norm),
                "train/n_tokens": float(sum(len(p["input_ids"]) for p in processed))}

    @torch.no_grad()
    def step_validation(self, batch: Sequence[Any], **kw) -> Dict[str, Any]:
        self.model.eval()
        processed = [self.data_packer.sft_process_sample(s) for s in batch]
        packed = [self._pack([processed[i] for i in idxs]) for idxs in self._batches(processed)]
        tok = torch.tensor(float(sum(b["n_scored"] for b in packed)), device=self.device).clamp_min(1.0)
        loss = self.pp_sum(torch.tensor(float(sum(float(x) for x in self.run_batches_nograd(packed, self._loss_of(tok)))),
                                        device=self.device))
        if self.parallel_dims.cp > 1:
            dist.all_reduce(loss, group=self.parallel_dims.group("cp"))
        return {"val/loss": float(loss)}

    def __init__(self, config, parallel_dims, **kw):
        self.inter_replica = kw.pop("inter_replica", None)
        super().__init__(config, parallel_dims, **kw)
