"""Trainers of diffusion / flow models on the DiT family, registered as trainer types ``diffusion_sft``,
``diffusion_nft`` and ``flow_grpo`` (cosmos_rl/policy/trainer/diffusers_trainer/{sft_trainer,nft_trainer}.py,
policy/trainer/wfm_trainer.py). They reuse the flat parameter buffer, the sharded AdamW and the checkpoint manager of
the language-model trainers; only batches and losses differ."""
from __future__ import annotations

import time
from typing import Any, Dict, List, Optional

import torch

from ...parallel.flat import FlatParams
from ...rollout.diffusion_rollout import LatentStore, diffusion_options
from .. import diffusion as D
from .. import loss as L
from .base import TrainerRegistry
from .llm_trainer import LLMTrainer


class _DiffusionBase(LLMTrainer):
    def __init__(self, config, parallel_dims, device=None, **kw):
        super().__init__(config, parallel_dims, device=device, **kw)
        self.opts = diffusion_options(config)
        LatentStore.configure(config)
        self.model.gradient_checkpointing = bool(config.policy.model_gradient_checkpointing)

    def _replica(self) -> torch.nn.Module:
        """A frozen copy of the network with its own flat buffer (behaviour / reference weights)."""
        from ...models.base import ModelRegistry
        with torch.device("meta"):
            m = ModelRegistry.build_model(self.hf_config)
        m._flat = FlatParams(m, self.param_dtype, self.device, with_grad=False)
        m._flat.data.copy_(self.flat.data)
        for p in m.parameters():
            p.requires_grad_(False)
        return m.eval()

    def _report(self, losses: List[float], norm, t0: float, **extra) -> Dict[str, Any]:
        mean = sum(losses) / max(1, len(losses))
        rep = {"train/loss_avg": mean, "train/loss_max": max(losses, default=0.0),
               "train/learning_rate": self.optimizer.lr * self.lr_scale(self.train_step),
               "train/grad_norm": float(norm), "train/iteration_time": time.perf_counter() - t0}
        rep.update({f"train/{k}": float(v) for k, v in extra.items()})
        return rep


@TrainerRegistry.register("diffusion_sft")
class DiffusionSFTTrainer(_DiffusionBase):
    """Flow-matching fine-tuning on (latent, text embedding) pairs."""

    def step_training(self, batch: List[Dict[str, Any]], total_steps: int = 0, train_step: int = 0, do_save: bool = False,
                      **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        self.total_steps = total_steps or self.total_steps
        dt = self.param_dtype
        mb = max(1, self.config.train.train_policy.mini_batch)
        self.flat.zero_grad()
        losses = []
        for s in range(0, len(batch), mb):
            part = batch[s:s + mb]
            x0 = torch.stack([torch.as_tensor(b["latents"], dtype=torch.float32) for b in part]).to(self.device, dt)
            text = torch.stack([torch.as_tensor(b["text_embeds"], dtype=torch.float32) for b in part]).to(self.device, dt)
            loss = D.flow_matching_loss(self.model, x0, text, None, scheme=self.opts["timestep_scheme"],
                                        shift=self.opts["shift"])
            (loss * len(part) / len(batch)).backward()
            losses.append(float(loss.detach()))
        norm = self.optimizer_step()
        self.train_step = train_step or self.train_step + 1
        if do_save:
            self.save_checkpoint(self.train_step, total_steps, is_final=self.train_step >= total_steps)
        return self._report(losses, norm, t0)


class _DiffusionRLBase(_DiffusionBase):
    def _gather(self, rollouts):
        items = [LatentStore.get(r.completion) for r in rollouts]
        adv = torch.tensor([r.advantage for r in rollouts], dtype=torch.float32, device=self.device)
        return items, adv


@TrainerRegistry.register("diffusion_nft")
class DiffusionNFTTrainer(_DiffusionRLBase):
    """DiffusionNFT: forward-process RL without sampler likelihoods. Keeps two frozen copies of the weights: the
    behaviour policy (trailing average of the trained weights; rollouts are drawn from it) and the reference the KL
    term pulls towards."""

    def __init__(self, config, parallel_dims, device=None, **kw):
        super().__init__(config, parallel_dims, device=device, **kw)
        if config.train.train_policy.kl_beta <= 0.0:
            raise ValueError("diffusion_nft needs train.train_policy.kl_beta > 0")
        self.old = self.ref = self._rollout = None

    def model_load_from_hf(self) -> None:
        super().model_load_from_hf()
        self.old, self.ref = self._replica(), self._replica()
        if self._rollout is not None:
            self._rollout.behaviour = self.old

    def attach_rollout(self, rollout) -> None:
        """Colocated mode: samples come from the behaviour weights, not from the weights being optimised."""
        self._rollout = rollout
        if self.old is not None:
            rollout.behaviour = self.old

    def step_training(self, rollouts, current_step: int = 0, total_steps: int = 0, remain_samples_num: int = 0,
                      do_save: bool = False, **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        self.total_steps = total_steps or self.total_steps
        o, tp = self.opts, self.config.train.train_policy
        items, adv = self._gather(rollouts)
        dt = self.param_dtype
        B, K = len(items), int(o["train_timesteps"])
        mb = max(1, tp.mini_batch)
        adv_clip = float(tp.advantage_high) if tp.advantage_high < 1e8 else 5.0
        self.flat.zero_grad()
        losses, stats = [], {"policy_loss": 0.0, "kl_loss": 0.0, "old_deviation": 0.0}
        n_terms = 0
        for s in range(0, B, mb):
            part = items[s:s + mb]
            x0 = torch.stack([it["x0"] for it in part]).to(self.device, dt)
            text = torch.stack([it["text"] for it in part]).to(self.device, dt)
            mask = torch.stack([it["text_mask"] for it in part]).to(self.device)
            for _ in range(K):
                t = D.sample_timesteps(x0.shape[0], o["timestep_scheme"], o["shift"], device=self.device)
                xt = D.add_noise(x0, t, torch.randn_like(x0))
                with torch.no_grad():
                    v_old, v_ref = self.old(xt, t, text, mask), self.ref(xt, t, text, mask)
                loss, m = D.nft_loss(self.model(xt, t, text, mask), v_old, v_ref, xt, x0, t, adv[s:s + mb],
                                     float(o["nft_beta"]), adv_clip, float(tp.kl_beta))
                (loss * x0.shape[0] / (B * K)).backward()
                losses.append(float(loss.detach()))
                for k in stats:
                    stats[k] += float(m[k])
                n_terms += 1
        norm = self.optimizer_step()
        self.train_step = current_step or self.train_step + 1
        decay = D.old_policy_decay(self.train_step, o["old_decay"])
        self.old._flat.data.mul_(decay).add_(self.flat.data, alpha=1.0 - decay)
        LatentStore.release([r.completion for r in rollouts])
        if do_save:
            self.save_checkpoint(self.train_step, total_steps, remain_samples_num, self.train_step >= total_steps)
        return self._report(losses, norm, t0, old_decay=decay, **{k: v / max(1, n_terms) for k, v in stats.items()})


@TrainerRegistry.register("flow_grpo")
class FlowGRPOTrainer(_DiffusionRLBase):
    """FlowGRPO: the sampler is the reverse-time SDE, every denoising step is a Gaussian action whose likelihood ratio
    is clipped as in GRPO (each step plays the role a token plays for a language model)."""

    def step_training(self, rollouts, current_step: int = 0, total_steps: int = 0, remain_samples_num: int = 0,
                      do_save: bool = False, **kw) -> Dict[str, Any]:
        t0 = time.perf_counter()
        self.total_steps = total_steps or self.total_steps
        o, tp = self.opts, self.config.train.train_policy
        items, adv = self._gather(rollouts)
        if "states" not in items[0]:
            raise ValueError('flow_grpo needs custom.diffusion.sampler = "sde" (per-step likelihoods)')
        dt = self.param_dtype
        B = len(items)
        ts = items[0]["timesteps"].tolist()
        S = items[0]["states"].shape[0]
        mb = max(1, tp.mini_batch)
        cfg = L.GrpoLossConfig(epsilon_low=tp.epsilon_low, epsilon_high=tp.epsilon_high, loss_type="token-mean")
        self.flat.zero_grad()
        losses, clip = [], []
        for s in range(0, B, mb):
            part = items[s:s + mb]
            text = torch.stack([it["text"] for it in part]).to(self.device, dt)
            mask = torch.stack([it["text_mask"] for it in part]).to(self.device)
            n = len(part)
            for i in range(S):
                x = torch.stack([it["states"][i] for it in part]).to(self.device)
                xn = torch.stack([it["next_states"][i] for it in part]).to(self.device)
                old_lp = torch.stack([it["logprobs"][i] for it in part]).to(self.device)
                v = self.model(x.to(dt), torch.full((n,), ts[i], device=self.device), text, mask).float()
                mean = D.sde_mean(x, v, ts[i], ts[i + 1], o["noise_level"])
                _, std = D.sde_coeffs(ts[i], ts[i + 1], o["noise_level"])
                # mean-over-elements log-probs: scale back so the ratio is the per-element geometric mean
                lp = D.sde_logprob(xn, mean, std)
                loss, m = L.grpo_loss(lp, old_lp, adv[s:s + mb], torch.arange(n, device=self.device), n, cfg)
                (loss * n / (B * S)).backward()
                losses.append(float(loss.detach())); clip.append(float(m["clip_frac"]))
        norm = self.optimizer_step()
        self.train_step = current_step or self.train_step + 1
        LatentStore.release([r.completion for r in rollouts])
        if do_save:
            self.save_checkpoint(self.train_step, total_steps, remain_samples_num, self.train_step >= total_steps)
        return self._report(losses, norm, t0, clip_frac=sum(clip) / max(1, len(clip)))
