"""Policy-gradient and supervised losses on packed per-token log-probabilities.

All functions take flat tensors over the *scored* tokens of a mini-batch (completion positions of all
sequences, concatenated) plus ``seq_ids [n_tok]`` mapping each token to its sequence, so per-sequence
reductions are segment sums instead of a Python loop over ``cu_seqlens``
(semantics of cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:67-353; DPO: dpo_trainer.py:34-45;
SFT CE with token balancing: sft_trainer.py:49-110).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


def _seg_sum(x: torch.Tensor, seq_ids: torch.Tensor, n_seq: int) -> torch.Tensor:
    return torch.zeros(n_seq, dtype=x.dtype, device=x.device).index_add_(0, seq_ids, x)


@dataclass
class GrpoLossConfig:
    epsilon_low: float = 0.2
    epsilon_high: float = 0.2
    lower_bound_ratio: float = 3.0
    kl_beta: float = 0.0
    unbiased_kl_estimate: bool = False
    loss_type: str = "token-mean"      # token-mean | seq-mean-token-sum | seq-mean-token-mean | token-sum
    unbiased_loss_max_tokens: Optional[int] = None
    variant: str = "grpo"              # grpo | dapo | gspo
    aipo_rho: Optional[float] = None
    use_decoupled_loss: bool = False
    behav_imp_weight_cap: Optional[float] = None
    off_policy_masking_delta: Optional[float] = None
    entropy_coeff: float = 0.0
    positive_nll_coef: Optional[float] = None

    @classmethod
    def from_config(cls, tp) -> "GrpoLossConfig":
        return cls(**{k: getattr(tp, k) for k in cls.__dataclass_fields__ if hasattr(tp, k)})


def _per_token_terms_torch(lp, old, A, seq_ids, n_seq, tok_per_seq, cfg, ref_logprob, rollout_logprob, mask=None):
    """Op-by-op per-token surrogate + KL (every variant; the oracle of the fused kernel). ``mask`` (off-policy
    sequence masking) multiplies the surrogate only: a masked sequence keeps its KL penalty and its place in the
    denominators (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:253-287)."""
    diff = lp - old
    if cfg.variant == "gspo":
        seq_diff = (_seg_sum(diff, seq_ids, n_seq) / tok_per_seq).clamp(max=10.0)
        # sequence-level ratio, gradient flows through every token of the sequence
        ratio = torch.exp(seq_diff)[seq_ids]
    else:
        ratio = torch.exp(diff.clamp(-20.0, 20.0))

    if cfg.aipo_rho is not None:
        per_tok = -torch.clamp(ratio, max=cfg.aipo_rho) * A
        clip_frac = (ratio > cfg.aipo_rho).float().mean()
    else:
        l1 = ratio * A
        l2 = ratio.clamp(1.0 - cfg.epsilon_low, 1.0 + cfg.epsilon_high) * A
        clip1 = -torch.minimum(l1, l2)
        clip_frac = (l2 < l1).float().mean()
        if cfg.variant == "gspo":
            per_tok = clip1
        else:
            l3 = -cfg.lower_bound_ratio * A
            per_tok = torch.where(A < 0, torch.minimum(l3, clip1), clip1)

    if cfg.use_decoupled_loss and rollout_logprob is not None:
        w = torch.exp(old - rollout_logprob.float()).detach()
        if cfg.behav_imp_weight_cap is not None:
            w = torch.where(w > cfg.behav_imp_weight_cap, torch.zeros_like(w), w)
        per_tok = per_tok * w

    if mask is not None:
        per_tok = per_tok * mask

    kl = torch.zeros_like(lp)
    if cfg.kl_beta != 0.0 and ref_logprob is not None:
        r = (ref_logprob.float() - lp).clamp(-20.0, 20.0)
        if cfg.unbiased_kl_estimate:
            # importance-weighted k3: the weight stays differentiable and the product is clamped
            kl = (torch.exp(diff) * (torch.exp(r) - r - 1.0)).clamp(-10.0, 10.0)
        else:
            kl = (torch.exp(r) - r - 1.0).clamp(-10.0, 10.0)
        per_tok = per_tok + cfg.kl_beta * kl

    return per_tok, kl, clip_frac.detach(), ratio.detach().mean()


class _FusedGrpoTerms(torch.autograd.Function):
    """One kernel for surrogate, KL, their derivative w.r.t. the current log-prob and the metric sums."""

    @staticmethod
    def forward(ctx, lp, old, A, ref, roll, mask, cfg):
        from ..ops import native
        n = lp.numel()
        out = torch.empty(3, n, dtype=torch.float32, device=lp.device)
        stats = torch.empty(3, dtype=torch.float32, device=lp.device)
        decoupled = bool(cfg.use_decoupled_loss and roll is not None)
        cap = cfg.behav_imp_weight_cap
        P = lambda t: native.ptr(t) if t is not None else None
        native.check(native.lib().b200_grpo_loss(
            P(lp), P(old), P(ref if cfg.kl_beta != 0.0 else None), P(roll if decoupled else None), P(A), P(mask), n,
            cfg.epsilon_low, cfg.epsilon_high, cfg.lower_bound_ratio, 1, cfg.kl_beta,
            int(cfg.unbiased_kl_estimate), int(cfg.aipo_rho is not None), float(cfg.aipo_rho or 0.0), int(decoupled),
            int(cap is not None), float(cap or 0.0), P(out[0]), P(out[1]), P(out[2]), P(stats), native.stream()),
            "grpo_loss")
        ctx.save_for_backward(out[1])
        ctx.mark_non_differentiable(stats)
        return out[0], out[2].detach(), stats

    @staticmethod
    def backward(ctx, g_per, g_kl, g_stats):
        (dlp,) = ctx.saved_tensors
        return g_per * dlp, None, None, None, None, None, None


USE_FUSED_KERNEL = True


def _fusable(lp: torch.Tensor, cfg: "GrpoLossConfig") -> bool:
    return USE_FUSED_KERNEL and lp.is_cuda and cfg.variant != "gspo"


def grpo_loss(logprob: torch.Tensor, old_logprob: torch.Tensor, advantages: torch.Tensor, seq_ids: torch.Tensor,
              n_seq: int, cfg: GrpoLossConfig, ref_logprob: Optional[torch.Tensor] = None,
              rollout_logprob: Optional[torch.Tensor] = None, entropy: Optional[torch.Tensor] = None,
              seq_rewards: Optional[torch.Tensor] = None, total_tokens: Optional[torch.Tensor] = None,
              ) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """``advantages`` is per token (sequence advantage broadcast). Returns (scalar loss, metrics).

    ``total_tokens`` overrides the denominator of ``token-mean`` (token count balanced across data-parallel
    ranks and replicas)."""
    lp = logprob.float()
    old = old_logprob.float()
    A = advantages.float()
    ntok = lp.numel()
    tok_per_seq = _seg_sum(torch.ones_like(lp), seq_ids, n_seq).clamp_min(1.0)
    mask = torch.ones_like(lp)

    if cfg.off_policy_masking_delta is not None:
        # drop negative-advantage sequences whose behaviour policy drifted too far from the current one
        src = rollout_logprob.float() if rollout_logprob is not None else old
        drift = _seg_sum((src - lp).detach(), seq_ids, n_seq) / tok_per_seq
        seq_adv = _seg_sum(A, seq_ids, n_seq) / tok_per_seq
        drop = (seq_adv < 0) & (drift > cfg.off_policy_masking_delta)
        mask = (~drop)[seq_ids].float()

    if _fusable(lp, cfg):
        f32 = lambda t: None if t is None else t.float().contiguous()
        per_tok, kl, stats = _FusedGrpoTerms.apply(lp.contiguous(), old.contiguous(), A.contiguous(),
                                                   f32(ref_logprob), f32(rollout_logprob), mask, cfg)
        clip_frac, ratio_mean = stats[0] / ntok, stats[1] / ntok
    else:
        per_tok, kl, clip_frac, ratio_mean = _per_token_terms_torch(lp, old, A, seq_ids, n_seq, tok_per_seq, cfg,
                                                                    ref_logprob, rollout_logprob, mask)

    # the mask is already inside per_tok (surrogate only); every denominator counts all scored tokens
    if cfg.loss_type == "token-mean":
        denom = total_tokens if total_tokens is not None else float(max(ntok, 1))
        loss = per_tok.sum() / denom
    elif cfg.loss_type == "token-sum":
        loss = per_tok.sum()
    elif cfg.loss_type == "seq-mean-token-sum":
        loss = _seg_sum(per_tok, seq_ids, n_seq).mean()
    elif cfg.loss_type == "seq-mean-token-mean":
        cap = cfg.unbiased_loss_max_tokens
        div = tok_per_seq if (cap is None or cap <= 0) else torch.full_like(tok_per_seq, float(cap))
        loss = (_seg_sum(per_tok, seq_ids, n_seq) / div).mean()
    else:
        raise ValueError(f"unknown loss_type {cfg.loss_type!r}")

    metrics: Dict[str, torch.Tensor] = {"kl": kl.sum() / float(max(ntok, 1)),
                                        "clip_frac": clip_frac, "ratio_mean": ratio_mean}
    if entropy is not None:
        ent_mean = entropy.float().sum() / float(max(ntok, 1))
        metrics["entropy"] = ent_mean.detach()
        if cfg.entropy_coeff != 0.0:
            loss = loss - cfg.entropy_coeff * ent_mean
    if cfg.positive_nll_coef and seq_rewards is not None:
        pos = (seq_rewards > 0)[seq_ids].float()
        if pos.sum() > 0:
            loss = loss + cfg.positive_nll_coef * (-(lp * pos).sum() / pos.sum())
    return loss, metrics


def dpo_loss(policy_chosen_lp, policy_rejected_lp, ref_chosen_lp, ref_rejected_lp, beta: float = 0.1,
             label_smoothing: float = 0.0):
    """Sequence-level DPO: ``-logsigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))``."""
    logits = (policy_chosen_lp - policy_rejected_lp) - (ref_chosen_lp - ref_rejected_lp)
    ls = torch.nn.functional.logsigmoid
    losses = -ls(beta * logits) * (1 - label_smoothing) - ls(-beta * logits) * label_smoothing
    chosen_rewards = beta * (policy_chosen_lp - ref_chosen_lp).detach()
    rejected_rewards = beta * (policy_rejected_lp - ref_rejected_lp).detach()
    return losses.mean(), {"reward_acc": (chosen_rewards > rejected_rewards).float().mean(),
                           "reward_margin": (chosen_rewards - rejected_rewards).mean()}


def sft_ce_loss(logprob: torch.Tensor, total_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token cross-entropy from label log-probs; ``total_tokens`` is the (dp-balanced) global token count."""
    denom = total_tokens if total_tokens is not None else torch.tensor(float(max(logprob.numel(), 1)),
                                                                        device=logprob.device)
    return -logprob.float().sum() / denom
