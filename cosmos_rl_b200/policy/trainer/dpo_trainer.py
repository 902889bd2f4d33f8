"""Direct preference optimisation on (prompt, chosen, rejected) triples: sequence log-probs of both
completions under the policy and under the frozen reference (the initial weights, kept on the host),
``-logsigmoid(beta * margin)`` (cosmos_rl/policy/trainer/llm_trainer/dpo_trainer.py:34-475). Prompts of a
vision-language model carry their pixel inputs (multimodal preference data such as MMPR): the data packer returns them
with the tokens and both completions of a pair are scored against the same images."""
from __future__ import annotations

import time
from typing import Any, Dict, List, Sequence

import torch

from ...utils.sequence_packing import pack_sequences
from ..loss import dpo_loss
from .base import TrainerRegistry
from .llm_trainer import LLMTrainer


@TrainerRegistry.register("dpo")
class DPOTrainer(LLMTrainer):
    def __init__(self, config, parallel_dims, **kw):
        self.inter_replica = kw.pop("inter_replica", None)
        super().__init__(config, parallel_dims, **kw)
        if parallel_dims.cp > 1 or parallel_dims.pp > 1:
            raise NotImplementedError("the DPO trainer supports dp_shard / dp_replicate / tp; use cp_size = pp_size = 1")
        self.beta = float(config.custom.get("dpo_beta", 0.1))

    def needs_reference(self) -> bool:
        return True

    def _encode(self, sample) -> Dict[str, Any]:
        pk = self.data_packer
        p = pk.get_rollout_input(sample["prompt"])
        out = {}
        for key in ("chosen", "rejected"):
            pi = pk.get_policy_input(sample["prompt"], sample[key])
            out[key] = (pi.input_ids, pi.logprob_masks, getattr(pi, "mm", None))    # mm: the prompt's pixel inputs
        return out

    def _seq_logprobs(self, pairs: List[Dict[str, Any]]) -> torch.Tensor:
        """[2 * n] sequence log-probs ordered chosen_0, rejected_0, chosen_1, ..."""
        seqs, masks, mms = [], [], []
        for e in pairs:
            for key in ("chosen", "rejected"):
                seqs.append(e[key][0])
                masks.append(e[key][1])
                mms.append(e[key][2])
        b = pack_sequences(seqs, masks, device=self.device)
        if getattr(self.model, "is_vlm", False):
            # vision-language preference pairs: both completions of a pair carry the prompt's images, so the pixel
            # inputs are stacked once per packed sequence, in packing order
            from ...data.packer import merge_mm
            self.model.mm_inputs = merge_mm(mms)
        sel = (b["label_ids"] >= 0).nonzero(as_tuple=True)[0]
        hidden = self.model(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"])
        lp, _ = self.model.logprobs(hidden[sel], b["label_ids"][sel], 1.0)
        return torch.zeros(len(seqs), device=self.device).index_add_(0, b["seq_ids"][sel], lp.float())

    def step_training(self, batch: Sequence[Dict[str, Any]], total_steps: int, train_step: int, do_save=False, **kw):
        t0 = time.perf_counter()
        self.total_steps = total_steps
        enc = [self._encode(s) for s in batch]
        mb = max(1, getattr(self.config.train.train_policy, "mini_batch", 2))
        chunks = [enc[i:i + mb] for i in range(0, len(enc), mb)]
        if self.reference_state is None:
            self.reference_state = self.flat.data.to("cpu", copy=True)
        cur = self.flat.data.to("cpu", copy=True)
        self.flat.data.copy_(self.reference_state.to(self.device))
        self._weights_changed()
        with torch.no_grad():
            ref = [self._seq_logprobs(c) for c in chunks]
        self.flat.data.copy_(cur.to(self.device))
        self._weights_changed()
        self.model.train()
        self.optimizer.zero_grad()
        losses, accs = [], []
        for c, r in zip(chunks, ref):
            lp = self._seq_logprobs(c)
            loss, m = dpo_loss(lp[0::2], lp[1::2], r[0::2], r[1::2], self.beta)
            (loss * len(c) / len(enc)).backward()
            losses.append(loss.detach())
            accs.append(m["reward_acc"])
        if self.inter_replica is not None:
            self.inter_replica.all_reduce_grads(self.flat.grad)
        norm = self.optimizer_step()
        self.train_step = train_step
        if do_save:
            self.save_checkpoint(train_step, total_steps, is_final=train_step >= total_steps)
        lt = torch.stack(losses)
        return {"train/loss_avg": float(lt.mean()), "train/loss_max": float(lt.max()),
                "train/learning_rate": self.optimizer.lr * self.lr_scale(max(train_step - 1, 0)),
                "train/iteration_time": time.perf_counter() - t0, "train/grad_norm": float(norm),
                "train/reward_acc": float(torch.stack(accs).mean())}
