"""GRPO trainer: turns a batch of rollouts into packed micro-batches, runs forward/backward through the
fused log-prob kernel and the GRPO loss, and applies one (or several) optimizer steps
(cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:977-1931).

Phases of a step: [reference log-probs when kl_beta != 0] -> [old log-probs when the batch is optimised in
several chunks or mu_iterations > 1] -> training. Mini-batches are built by count (``mini_batch``) or by
token budget (``max_token_len_per_mini_batch``) and always packed (no padding reaches the GPU).
"""
from __future__ import annotations

import math

import time
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ...dispatcher.data.schema import Rollout
from ...utils.logging import logger
from ...utils.sequence_packing import pack_sequences, token_budget_batches
from ..loss import GrpoLossConfig, grpo_loss
from .base import TrainerRegistry
from .llm_trainer import LLMTrainer


class _Sample:
    __slots__ = ("ids", "mask", "advantage", "reward", "rollout_lp", "n_scored", "mm", "teacher_lp", "teacher_topk")

    def __init__(self, ids, mask, advantage, reward, rollout_lp, mm=None, teacher_lp=None, teacher_topk=None):
        self.ids, self.mask, self.advantage, self.reward, self.rollout_lp = ids, mask, advantage, reward, rollout_lp
        self.n_scored = int(sum(mask))
        self.mm = mm            # vision inputs of a vision-language sample
        self.teacher_lp = teacher_lp   # per scored token, from the distillation teacher
        self.teacher_topk = teacher_topk   # (ids [n_scored][k], log-probs [n_scored][k]) of the teacher's k best tokens


def discounted_suffix_sum(x: torch.Tensor, seq_ids: torch.Tensor, gamma: float) -> torch.Tensor:
    """``y[i] = x[i] + gamma * y[i + 1]`` inside every run of equal ``seq_ids`` (tokens of one sequence are contiguous).
    Vectorised: cumulative sums for gamma == 1, a scaled cumulative sum in float64 while ``gamma ** longest_run`` stays
    above 1e-6 (the scaling costs that many digits), a plain backward loop beyond that."""
    n = x.numel()
    if n == 0:
        return x
    ids = seq_ids.to(torch.long)
    start = torch.ones(n, dtype=torch.bool, device=x.device)
    start[1:] = ids[1:] != ids[:-1]
    seg = torch.cumsum(start.to(torch.long), 0) - 1                      # run index of every element
    first = torch.nonzero(start, as_tuple=True)[0]                       # first element of every run
    rel = torch.arange(n, device=x.device) - first[seg]                  # position inside the run
    longest = int(rel.max()) + 1
    xd = x.double()
    if gamma == 1.0:
        w = xd
    elif gamma ** longest > 1e-6:        # late elements lose log10(gamma ** -rel) digits in the scaled sum
        w = xd * torch.pow(torch.tensor(gamma, dtype=torch.float64, device=x.device), rel.double())
    else:
        vals, out, acc = x.tolist(), [0.0] * n, 0.0
        st = start.tolist()
        for i in range(n - 1, -1, -1):
            acc = vals[i] + (gamma * acc if (i + 1 < n and not st[i + 1]) else 0.0)
            out[i] = acc
        return torch.tensor(out, dtype=x.dtype, device=x.device)
    c = torch.cumsum(w, 0)
    total = torch.zeros(first.numel(), dtype=torch.float64, device=x.device).index_add_(0, seg, w)
    before = c - w - (c - w)[first][seg]                                  # sum of the run's earlier elements
    suffix = total[seg] - before
    if gamma != 1.0:
        suffix = suffix / torch.pow(torch.tensor(gamma, dtype=torch.float64, device=x.device), rel.double())
    return suffix.to(x.dtype)


@TrainerRegistry.register("grpo")
class GRPOTrainer(LLMTrainer):
    def __init__(self, config, parallel_dims, **kw):
        super().__init__(config, parallel_dims, **kw)
        self.tp_cfg = config.train.train_policy
        self.loss_cfg = GrpoLossConfig.from_config(self.tp_cfg)
        self.temperature = float(self.tp_cfg.temperature)
        if self.tp_cfg.kl_beta != 0.0:
            self._reference_pending = True
        self.inter_replica = kw.get("inter_replica")  # elastic data parallelism across policy replicas

    # ------------------------------------------------------------------ data
    def _prepare(self, rollouts: Sequence[Rollout]) -> List[_Sample]:
        out = []
        for r in rollouts:
            comp = r.completion
            if r.completed_conversation:
                comp = r.completed_conversation        # multi-turn: the packer scores every assistant turn
            elif r.completion_token_ids:
                comp = [pos[0] for pos in r.completion_token_ids]
            pi = self.data_packer.get_policy_input(r.prompt, comp, r.n_ignore_prefix_tokens)
            lp = None
            if r.completion_logprobs:
                lp = [pos[0] for pos in r.completion_logprobs][r.n_ignore_prefix_tokens:]
            max_len = self.config.policy.model_max_length
            mm = getattr(pi, "mm", None)
            if mm:                                  # image placeholders must stay in step with the pixel inputs
                max_len = max(max_len, len(pi.input_ids))
            ids, mask = pi.input_ids[:max_len], pi.logprob_masks[:max_len]
            if len(ids) < len(pi.input_ids):
                mask[-1] = 0
            tlp = None
            if r.teacher_logprobs:
                tlp = [pos[0] for pos in r.teacher_logprobs][r.n_ignore_prefix_tokens:]
            topk = None
            if r.teacher_topk_ids and r.teacher_topk_logprobs:
                topk = (r.teacher_topk_ids[r.n_ignore_prefix_tokens:], r.teacher_topk_logprobs[r.n_ignore_prefix_tokens:])
            out.append(_Sample(ids, mask, float(r.advantage), float(r.reward), lp, mm, tlp, topk))
        return out

    def _mini_batches(self, samples: List[_Sample]) -> List[List[int]]:
        budget = self.tp_cfg.max_token_len_per_mini_batch
        if budget:
            return token_budget_batches([len(s.ids) for s in samples], budget * self.parallel_dims.cp)
        mb = max(1, self.tp_cfg.mini_batch)
        if self.parallel_dims.pp > 1:           # the packed batches are the micro-batches of the pipeline schedule
            mb = max(1, self.config.policy.parallelism.pp_micro_batch_size)
        return [list(range(i, min(i + mb, len(samples)))) for i in range(0, len(samples), mb)]

    def _pack(self, samples: List[_Sample]) -> Dict[str, Any]:
        pad_mult = self.pack_multiple()
        b = pack_sequences([s.ids for s in samples], [s.mask for s in samples], device=self.device,
                           pad_multiple=1 if pad_mult == 1 else pad_mult)
        rlp_full = None
        if all(s.rollout_lp is not None and len(s.rollout_lp) == s.n_scored for s in samples):
            flat = [x for s in samples for x in s.rollout_lp]
            rlp_full = torch.zeros(b["label_ids"].numel(), dtype=torch.float32, device=self.device)
            rlp_full[(b["label_ids"] >= 0)] = torch.tensor(flat, dtype=torch.float32, device=self.device)
        tlp_full = None
        if self.config.distillation.enable:
            # teacher log-probs per scored token; samples without a teacher result are excluded from the KL term
            tlp_full = torch.full((b["label_ids"].numel(),), float("nan"), dtype=torch.float32, device=self.device)
            scored = (b["label_ids"] >= 0).nonzero(as_tuple=True)[0]
            pos = 0
            for s_ in samples:
                if s_.teacher_lp is not None and len(s_.teacher_lp) == s_.n_scored:
                    tlp_full[scored[pos:pos + s_.n_scored]] = torch.tensor(s_.teacher_lp, dtype=torch.float32,
                                                                            device=self.device)
                pos += s_.n_scored
        k = int(self.config.distillation.top_k) if self.config.distillation.enable else 0
        tk_ids = tk_lp = None
        if k > 0:
            # the teacher's k best tokens per scored position (ids -1 where a sample came without a teacher result)
            T_all = b["label_ids"].numel()
            tk_ids = torch.full((T_all, k), -1, dtype=torch.long, device=self.device)
            tk_lp = torch.zeros(T_all, k, dtype=torch.float32, device=self.device)
            scored = (b["label_ids"] >= 0).nonzero(as_tuple=True)[0]
            pos = 0
            for s_ in samples:
                tk = s_.teacher_topk
                if tk is not None and len(tk[0]) == s_.n_scored and s_.n_scored and len(tk[0][0]) == k:
                    rows = scored[pos:pos + s_.n_scored]
                    tk_ids[rows] = torch.tensor(tk[0], dtype=torch.long, device=self.device)
                    tk_lp[rows] = torch.tensor(tk[1], dtype=torch.float32, device=self.device)
                pos += s_.n_scored
        cu_full = b["cu_seqlens"]
        b = self.cp_shard(b)
        if any(s.mm for s in samples):
            from ...data.packer import merge_mm
            b["mm"] = merge_mm([s.mm for s in samples])
        sel = (b["label_ids"] >= 0).nonzero(as_tuple=True)[0]
        b["sel"] = sel
        b["labels_sel"] = b["label_ids"][sel]
        b["seq_ids_sel"] = b["seq_ids"][sel]
        adv = torch.tensor([s.advantage for s in samples], dtype=torch.float32, device=self.device)
        b["adv_tok"] = adv[b["seq_ids_sel"]]
        b["seq_rewards"] = torch.tensor([s.reward for s in samples], dtype=torch.float32, device=self.device)
        if rlp_full is not None:
            if self.parallel_dims.cp > 1:
                from ...parallel.context_parallel import split_for_cp
                rlp_full = split_for_cp(rlp_full, cu_full, self.parallel_dims.cp, self.parallel_dims.cp_coord,
                                        zigzag=self.config.b200.cp_mode == "ring-zigzag")
            b["rollout_lp"] = rlp_full[sel]
        if tlp_full is not None:
            if self.parallel_dims.cp > 1:
                from ...parallel.context_parallel import split_for_cp
                tlp_full = split_for_cp(tlp_full, cu_full, self.parallel_dims.cp, self.parallel_dims.cp_coord,
                                        zigzag=self.config.b200.cp_mode == "ring-zigzag")
            b["teacher_lp"] = tlp_full[sel]
        if tk_ids is not None:
            if self.parallel_dims.cp > 1:
                from ...parallel.context_parallel import split_for_cp
                tk_ids = split_for_cp(tk_ids, cu_full, self.parallel_dims.cp, self.parallel_dims.cp_coord,
                                        zigzag=self.config.b200.cp_mode == "ring-zigzag")
                tk_lp = split_for_cp(tk_lp, cu_full, self.parallel_dims.cp, self.parallel_dims.cp_coord,
                                        zigzag=self.config.b200.cp_mode == "ring-zigzag")
            b["teacher_topk_ids"], b["teacher_topk_lp"] = tk_ids[sel], tk_lp[sel]
        return b

    def teacher_kl_advantages(self, logprob: torch.Tensor, b: Dict[str, Any]):
        """On-policy distillation: every scored token gets ``-kl_penalty_coef * (log p_student - log p_teacher)`` (the
        per-token reverse-KL estimate on the sampled token) added to its advantage, optionally as a discounted sum over
        the rest of its sequence (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:692-860). Returns the new
        per-token advantages and the mean divergence."""
        d = self.config.distillation
        t = b["teacher_lp"]
        have = ~torch.isnan(t)
        div = torch.where(have, logprob.detach().float() - torch.nan_to_num(t), torch.zeros_like(t))
        kl_adv = -d.kl_penalty_coef * div
        if d.kl_discount_factor != 0.0:
            kl_adv = discounted_suffix_sum(kl_adv, b["seq_ids_sel"], float(d.kl_discount_factor))
        return b["adv_tok"] + kl_adv, div.sum() / have.sum().clamp_min(1)

    def teacher_topk_jsd_advantages(self, b: Dict[str, Any]):
        """Top-k distillation (``distillation.top_k > 0``): the divergence of a token is the generalised Jensen-Shannon
        divergence between teacher and student restricted to the teacher's k most likely tokens,
        ``beta * KL(t || m) + (1 - beta) * KL(s || m)`` with ``m = beta * t + (1 - beta) * s``; ``beta = 0`` is the
        forward KL ``sum t (log t - log s)`` and ``beta = 1`` the reverse one. It is subtracted from the advantages
        like the single-token estimate (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:716-787)."""
        d = self.config.distillation
        s, t, ids = b["student_topk_lp"], b["teacher_topk_lp"], b["teacher_topk_ids"]
        have = ids[:, 0] >= 0
        beta = float(d.jsd_beta)
        if beta == 0.0:
            div = t.exp() * (t - s)
        elif beta == 1.0:
            div = s.exp() * (s - t)
        else:
            m = torch.logaddexp(s + math.log1p(-beta), t + math.log(beta))
            div = beta * t.exp() * (t - m) + (1.0 - beta) * s.exp() * (s - m)
        div = torch.where(have, div.sum(-1), torch.zeros_like(div[:, 0]))
        kl_adv = -d.kl_penalty_coef * div
        if d.kl_discount_factor != 0.0:
            kl_adv = discounted_suffix_sum(kl_adv, b["seq_ids_sel"], float(d.kl_discount_factor))
        return b["adv_tok"] + kl_adv, div.sum() / have.sum().clamp_min(1)

    @torch.no_grad()
    def _student_topk_logprobs(self, hidden_sel: torch.Tensor, ids: torch.Tensor, chunk: int = 2048) -> torch.Tensor:
        """Student log-probs at the teacher's top-k ids, [n, k] fp32; full-vocabulary logits exist for ``chunk`` rows
        at a time only."""
        out = torch.zeros(ids.shape, dtype=torch.float32, device=ids.device)
        for i in range(0, ids.shape[0], chunk):
            lg = self.model.logits(hidden_sel[i:i + chunk]).float() / self.temperature
            out[i:i + chunk] = torch.log_softmax(lg, -1).gather(1, ids[i:i + chunk].clamp_min(0))
        return out

    # ------------------------------------------------------------------ hooks a custom trainer may override
    def compute_logprobs(self, hidden: torch.Tensor, b: Dict[str, Any]):
        """(per-token log-probs, entropies) of the scored tokens of a packed batch from the final hidden states."""
        hs = hidden[b["sel"]]
        if "teacher_topk_ids" in b and "student_topk_lp" not in b:
            # advantage shaping only (no gradient): taken once, from the weights the batch is first scored with
            b["student_topk_lp"] = self._student_topk_logprobs(hs.detach(), b["teacher_topk_ids"])
        return self.model.logprobs(hs, b["labels_sel"], self.temperature)

    def loss_fn(self, logprob, old_logprob, b: Dict[str, Any], ref_logprob=None, entropy=None, total_tokens=None):
        """(scalar loss, metrics) of one packed batch; the default is the configured GRPO / DAPO / GSPO objective
        (cosmos_rl/tools/custom_example/README.md lists the same override points)."""
        adv, teacher_kl, kl_name = b["adv_tok"], None, "teacher_kl_reversed"
        if "student_topk_lp" in b:
            adv, teacher_kl = self.teacher_topk_jsd_advantages(b)
            kl_name = f"teacher_jsd_top{b['teacher_topk_ids'].shape[1]}"
        elif "teacher_lp" in b:
            adv, teacher_kl = self.teacher_kl_advantages(logprob, b)
        loss, metrics = grpo_loss(logprob, old_logprob, adv, b["seq_ids_sel"], int(b["cu_seqlens"].numel() - 1),
                                  self.loss_cfg, ref_logprob=ref_logprob, rollout_logprob=b.get("rollout_lp"),
                                  entropy=entropy, seq_rewards=b["seq_rewards"], total_tokens=total_tokens)
        if teacher_kl is not None:
            metrics[kl_name] = teacher_kl.detach()
        return loss, metrics

    def _logprobs_of(self, hidden, b: Dict[str, Any]):
        return self.compute_logprobs(hidden, b)

    def _forward_logprobs(self, b: Dict[str, Any]):
        hidden = self.model(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"])
        return self._logprobs_of(hidden, b)

    @torch.no_grad()
    def _compute_logprobs_nograd(self, batches: List[Dict[str, Any]]) -> List[torch.Tensor]:
        """Per-batch log-probs without gradients (on the last stage only under pipeline parallelism)."""
        return self.run_batches_nograd(batches, lambda h, i, b: self._logprobs_of(h, b)[0].detach())

    # ------------------------------------------------------------------ reference policy (KL)
    def _swap_flat(self, other: torch.Tensor) -> torch.Tensor:
        cur = self.flat.data.to("cpu", copy=True)
        self.flat.data.copy_(other.to(self.device))
        self._weights_changed()
        return cur

    def _reference_logprobs(self, batches):
        if self.reference_state is None:
            self.reference_state = self.flat.data.to("cpu", copy=True)
        cur = self._swap_flat(self.reference_state)
        try:
            return self._compute_logprobs_nograd(batches)
        finally:
            self.flat.data.copy_(cur.to(self.device))
            self._weights_changed()

    def needs_reference(self) -> bool:
        return self.tp_cfg.kl_beta != 0.0

    def reference_reset(self) -> None:
        """Make the current weights the new reference (every ``reference_reset_interval`` steps)."""
        self.reference_state = self.flat.data.to("cpu", copy=True)
        self.reference_step = self.train_step
        if self.tp_cfg.reset_optimizer_with_reference:
            self.optimizer.zero_moments()

    # ------------------------------------------------------------------ the step
    def step_training(self, rollouts: Sequence[Rollout], current_step: int, total_steps: int,
                      remain_samples_num: int = 0, do_save: bool = False, **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        if self.device.type == "cuda":
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        self.total_steps = total_steps
        if self.parallel_dims.cp > 1 and (self.loss_cfg.loss_type != "token-mean" or self.loss_cfg.variant == "gspo"):
            raise NotImplementedError("context parallelism supports the token-mean loss (per-sequence reductions would "
                                      "need sums across the cp ranks)")
        samples = self._prepare(rollouts)
        n = len(samples)
        per_opt = self.tp_cfg.batch_size_per_optimize or n
        mu = max(1, self.tp_cfg.mu_iterations)
        chunks = [list(range(i, min(i + per_opt, n))) for i in range(0, n, per_opt)]
        need_old = len(chunks) > 1 or mu > 1
        use_rollout_lp = self.tp_cfg.use_rollout_logprobs_for_loss
        losses: List[torch.Tensor] = []
        metrics_acc: Dict[str, List[torch.Tensor]] = {}
        grad_norms: List[torch.Tensor] = []
        dp_world = self.parallel_dims.dp_shard
        self.model.train()

        # pack once; the same packed mini-batches serve every phase
        chunk_batches = []
        for ch in chunks:
            sub = [samples[i] for i in ch]
            chunk_batches.append([self._pack([sub[i] for i in idxs]) for idxs in self._mini_batches(sub)])
        self.resolve_recompute(max(int(b["input_ids"].numel()) for bs in chunk_batches for b in bs))

        ref_lps = old_lps = None
        if self.tp_cfg.kl_beta != 0.0:
            ref_lps = [self._reference_logprobs(bs) for bs in chunk_batches]
        if need_old and not use_rollout_lp:
            old_lps = [self._compute_logprobs_nograd(bs) for bs in chunk_batches]

        for it in range(mu):
            for ci, batches in enumerate(chunk_batches):
                tok = torch.tensor(float(sum(b["n_scored"] for b in batches)), device=self.device)
                if self.tp_cfg.balance_dp_token and dp_world > 1:
                    dist.all_reduce(tok, group=self.parallel_dims.group("dp_shard"))
                    tok = tok / dp_world
                if self.inter_replica is not None and self.tp_cfg.balance_dp_token:
                    tok = self.inter_replica.balance_token_count(tok)
                self.optimizer.zero_grad()
                n_seq_total = max(1, sum(len(x["seq_rewards"]) for x in batches))

                def loss_of(hidden, bi, b, ci=ci, tok=tok, n_seq_total=n_seq_total):
                    lp, ent = self._logprobs_of(hidden, b)
                    if use_rollout_lp and "rollout_lp" in b:
                        old = b["rollout_lp"]
                    elif old_lps is not None:
                        old = old_lps[ci][bi]
                    else:
                        old = lp.detach()
                    loss, m = self.loss_fn(lp, old, b, ref_logprob=ref_lps[ci][bi] if ref_lps is not None else None,
                                           entropy=ent,
                                           total_tokens=tok if self.loss_cfg.loss_type == "token-mean" else None)
                    if self.loss_cfg.loss_type != "token-mean":
                        loss = loss * (len(b["seq_rewards"]) / n_seq_total)
                    for k, v in m.items():
                        metrics_acc.setdefault(k, []).append(v.detach())
                    return loss

                losses.extend(self.run_batches_train(batches, loss_of))
                if self.inter_replica is not None:
                    self.inter_replica.all_reduce_grads(self.flat.grad)
                grad_norms.append(self.optimizer_step())
            # mu-iterations re-use the same old log-probs
        self.train_step = current_step

        if self.tp_cfg.reference_reset_interval and current_step % self.tp_cfg.reference_reset_interval == 0 \
                and self.tp_cfg.kl_beta != 0.0:
            self.reference_reset()
        if do_save:
            self.save_checkpoint(current_step, total_steps, remain_samples_num,
                                 is_final=current_step >= total_steps)

        if self.device.type == "cuda":
            ev1.record()
            ev1.synchronize()
            iter_time = ev0.elapsed_time(ev1) / 1e3
        else:
            iter_time = time.perf_counter() - t0
        loss_t = torch.stack(losses) if losses else torch.zeros(1, device=self.device)
        n_mb = max(1, len(losses) // max(1, len(chunks) * mu))
        loss_sum = self.pp_sum(loss_t.sum().clone())             # only the last pipeline stage has the losses
        report = {
            "train/loss_avg": float(loss_sum / max(1, len(chunks) * mu)),
            "train/loss_max": float(loss_t.max() * n_mb),
            "train/learning_rate": self.optimizer.lr * self.lr_scale(max(self.train_step - 1, 0)),
            "train/iteration_time": iter_time,
            "train/grad_norm": float(torch.stack(grad_norms).mean()) if grad_norms else 0.0,
            "train/n_tokens": float(sum(len(s.ids) for s in samples)),
        }
        for k, v in metrics_acc.items():
            report[f"train/{k}"] = float(torch.stack(v).mean())
        if self.pipeline is not None:
            # loss-side metrics exist on the last stage only; the replica's reporter is its first rank
            pp_group = self.parallel_dims.group("pp")
            last = dist.get_process_group_ranks(pp_group)[-1]
            box = [{k: v for k, v in report.items() if k.startswith("train/") and k not in (
                "train/iteration_time", "train/learning_rate", "train/grad_norm", "train/n_tokens")}]
            dist.broadcast_object_list(box, src=last, group=pp_group)
            report.update(box[0])
        if self.config.logging.report_mfu and self.device.type == "cuda":
            from ...utils.misc import peak_flops
            ntok = sum(len(s.ids) for s in samples)
            avg_len = ntok / max(1, len(samples))
            _, flops_per_tok = self.model.get_nparams_and_flops(int(avg_len))
            report["train/mfu"] = flops_per_tok * ntok * mu / iter_time / peak_flops("bf16")
        return report
