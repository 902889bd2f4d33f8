"""Vision-language-action policy with a flow-matching action expert.

The reference's PI0.5 policy pairs a vision-language backbone with a second, smaller transformer (the action expert)
that turns noise into a chunk of continuous actions by integrating a learned velocity field, conditioned on what the
backbone made of the observation and the instruction (cosmos_rl/policy/model/pi05/__init__.py:1-1408,
``PaliGemmaWithExpertModel`` in ``model_utils.py``); RL fine-tuning explores by sampling that flow as an SDE and
trains on the transition log-probabilities. The same construction out of this package's parts:

* backbone: any decoder of the GPT family or a native vision-language model (:mod:`qwen2_5_vl`, :mod:`internvl`,
  :mod:`qwen3_vl_moe`); its final hidden states over the packed prompt are the context;
* action expert: a :class:`DiT` over the ``horizon`` action tokens of a chunk (self-attention among them,
  cross-attention to the context, timestep modulation) with the proprioceptive state folded into the timestep
  embedding;
* behaviour cloning is the flow-matching loss of ``policy/diffusion.py`` on action chunks; acting integrates the flow
  with any solver of ``policy/diffusion_solvers.py``; exploration for RL is ``sde_sample`` (states, next states and
  behaviour log-probabilities per step), and ``flow_grpo_loss`` is the clipped ratio objective on those transitions.

Differences from PI0.5 that matter to a user: the expert reads the backbone's LAST hidden states through
cross-attention instead of sharing every layer's keys and values with it, and nothing here loads PaliGemma weights.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..policy import diffusion as D
from .base import BaseModel, ModelRegistry, WeightMapper
from .dit import DiT, DiTArgs


@dataclass
class FlowVLAArgs:
    action_dim: int = 7
    horizon: int = 8                      # actions per chunk
    state_dim: int = 0                    # proprioceptive state (0 = none)
    expert_dim: int = 512
    expert_layers: int = 6
    expert_heads: int = 4
    expert_head_dim: int = 128
    expert_ffn: int = 2048
    freeze_backbone: bool = False
    backbone: Optional[Dict[str, Any]] = None     # the backbone's own config (HF form); None when it is passed in
    model_type: str = "flow_vla"

    @classmethod
    def from_hf_config(cls, c, **over) -> "FlowVLAArgs":
        d = {k: v for k, v in dict(c).items() if k in cls.__dataclass_fields__}
        d.update(over)
        return cls(**d)

    def to_hf_config(self) -> Dict[str, Any]:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d["architectures"] = ["FlowVLA"]
        return d


class FlowVLAWeightMapper(WeightMapper):
    """Checkpoints of this family are stored under the framework's own parameter names (``backbone.*``, ``expert.*``,
    ``state_in.*``)."""

    def hf_names(self, local: str) -> List[str]:
        return [local]


@ModelRegistry.register(FlowVLAWeightMapper)
class FlowVLA(BaseModel):
    paged_engine = False                  # acting integrates a flow: no token-by-token decoding

    @staticmethod
    def supported_model_types():
        return ["flow_vla"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        args = FlowVLAArgs.from_hf_config(hf_config)
        if not args.backbone:
            raise ValueError("a flow_vla config needs the backbone's config under 'backbone'")
        bkw = {k: v for k, v in kw.items() if k in ("tp_size", "tp_rank") and v not in (None, 1, 0)}
        if bkw.get("tp_size", 1) > 1:
            raise NotImplementedError("the flow-matching action policy trains with data parallelism only")
        return cls(ModelRegistry.build_model(args.backbone), args)

    def __init__(self, backbone: nn.Module, args: FlowVLAArgs):
        super().__init__()
        self.args, self.backbone = args, backbone
        ctx_dim = backbone.args.dim
        self.expert = DiT(DiTArgs(in_channels=args.action_dim, patch_size=(1, 1, 1), dim=args.expert_dim,
                                  n_layers=args.expert_layers, n_heads=args.expert_heads, head_dim=args.expert_head_dim,
                                  ffn_dim=args.expert_ffn, text_dim=ctx_dim, freq_dim=256))
        self.state_in = nn.Sequential(nn.Linear(args.state_dim, ctx_dim), nn.SiLU(), nn.Linear(ctx_dim, ctx_dim)) \
            if args.state_dim > 0 else None
        if args.freeze_backbone:
            for p in self.backbone.parameters():
                p.requires_grad_(False)

    def init_weights(self, seed: int = 0) -> None:
        self.backbone.init_weights(seed)
        self.expert.init_weights(seed + 1)
        if self.state_in is not None:
            g = torch.Generator().manual_seed(seed + 2)
            with torch.no_grad():
                for p in self.state_in.parameters():
                    p.copy_((torch.randn(p.shape, generator=g) * 0.02).to(p.dtype)) if p.dim() > 1 else p.zero_()

    init_weights_on_device = init_weights

    def shard_parts(self, flat):
        """Weight-sync parts: every tensor whole (the family runs data parallel only)."""
        from ..parallel.reshard import whole_parts
        return whole_parts(flat)

    # ------------------------------------------------------------------ context
    def context(self, prompts: Sequence[Sequence[int]], state: Optional[torch.Tensor] = None, mm: Optional[Dict] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Backbone pass over the packed prompts -> (context ``[B, L, D]`` padded per sample, mask ``[B, L]``); the
        proprioceptive state, when there is one, becomes one more context token per sample."""
        dev = next(self.backbone.parameters()).device
        lens = [len(p) for p in prompts]
        ids = torch.tensor([t for p in prompts for t in p], dtype=torch.long, device=dev)
        cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        if getattr(self.backbone, "is_vlm", False):
            self.backbone.mm_inputs = mm or {}
        pos = self.backbone.get_position_ids(cu, int(ids.numel()))
        with torch.set_grad_enabled(torch.is_grad_enabled() and not self.args.freeze_backbone):
            h = self.backbone(ids, pos, cu, max(lens))
        extra = 1 if self.state_in is not None else 0
        L = max(lens) + extra
        ctx = h.new_zeros(len(prompts), L, h.shape[-1])
        mask = torch.zeros(len(prompts), L, dtype=torch.bool, device=dev)
        for i, (a, b) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
            ctx[i, :b - a] = h[a:b]
            mask[i, :b - a] = True
        if extra:
            s = self.state_in(state.to(h.dtype))
            idx = torch.tensor(lens, device=dev)
            ctx[torch.arange(len(prompts)), idx] = s
            mask[torch.arange(len(prompts)), idx] = True
        return ctx, mask

    # ------------------------------------------------------------------ the velocity field over action chunks
    def velocity_fn(self, ctx: torch.Tensor, mask: torch.Tensor) -> Callable:
        """``f(a_t [B, horizon, action_dim], t [B], ...) -> v`` in the calling convention of ``policy/diffusion.py``."""
        def f(a_t, t, text=None, text_mask=None):
            z = a_t.transpose(1, 2)[..., None, None]                      # [B, A, horizon, 1, 1]
            v = self.expert(z.to(ctx.dtype), t, ctx, mask)
            return v[..., 0, 0].transpose(1, 2)
        return f

    def bc_loss(self, prompts, actions: torch.Tensor, state=None, mm=None, t=None, noise=None) -> torch.Tensor:
        """Flow-matching behaviour cloning: ``actions [B, horizon, action_dim]`` (normalised to about unit scale)."""
        ctx, mask = self.context(prompts, state, mm)
        return D.flow_matching_loss(self.velocity_fn(ctx, mask), actions.to(ctx.dtype), None, None, t=t, noise=noise)

    @torch.no_grad()
    def act(self, prompts, state=None, mm=None, steps: int = 10, solver: str = "euler", generator=None) -> torch.Tensor:
        """One action chunk per prompt by integrating the flow from noise (deterministic given the noise)."""
        from ..policy.diffusion_solvers import sample
        ctx, mask = self.context(prompts, state, mm)
        a = self.args
        noise = torch.randn(len(prompts), a.horizon, a.action_dim, generator=generator).to(ctx.device, ctx.dtype)
        return sample(self.velocity_fn(ctx, mask), noise, None, None, steps=steps, solver=solver)

    @torch.no_grad()
    def explore(self, prompts, state=None, mm=None, steps: int = 10, noise_level: float = 0.7, generator=None
                ) -> Dict[str, torch.Tensor]:
        """Stochastic action chunks for RL: ``x0`` (the actions), and per SDE step the state, the next state and the
        behaviour log-probability."""
        ctx, mask = self.context(prompts, state, mm)
        a = self.args
        noise = torch.randn(len(prompts), a.horizon, a.action_dim, generator=generator).to(ctx.device, ctx.dtype)
        return D.sde_sample(self.velocity_fn(ctx, mask), noise, None, None, steps=steps, noise_level=noise_level,
                            generator=generator)

    def flow_grpo_loss(self, prompts, rollout: Dict[str, torch.Tensor], advantages: torch.Tensor, state=None, mm=None,
                       noise_level: float = 0.7, clip: float = 0.2) -> Tuple[torch.Tensor, Dict[str, float]]:
        """Clipped-ratio policy gradient on the recorded SDE transitions: for every step the current policy's transition
        density of the recorded next state against the behaviour density, weighted by the sample's advantage."""
        ctx, mask = self.context(prompts, state, mm)
        f = self.velocity_fn(ctx, mask)
        ts = rollout["timesteps"].tolist()
        states, nxt, old = rollout["states"], rollout["next_states"], rollout["logprobs"]
        adv = advantages.to(old.device, torch.float32)
        total, clipped = 0.0, 0.0
        K = states.shape[1]
        for k in range(K):
            t, tn = ts[k], ts[k + 1]
            x = states[:, k]
            v = f(x.to(ctx.dtype), torch.full((x.shape[0],), t, device=x.device)).float()
            mean = D.sde_mean(x.float(), v, t, tn, noise_level)
            _, std = D.sde_coeffs(t, tn, noise_level)
            ratio = (D.sde_logprob(nxt[:, k], mean, std) - old[:, k]).exp()
            un, cl = ratio * adv, ratio.clamp(1 - clip, 1 + clip) * adv
            total = total - torch.minimum(un, cl).mean() / K
            clipped += float(((ratio - 1).abs() > clip).float().mean()) / K
        return total, {"clip_frac": clipped}


def normalize_actions(a: torch.Tensor, low: torch.Tensor, high: torch.Tensor) -> torch.Tensor:
    """Map actions from ``[low, high]`` per dimension to ``[-1, 1]`` (what the flow is trained on)."""
    return 2.0 * (a - low) / (high - low).clamp_min(1e-8) - 1.0


def denormalize_actions(a: torch.Tensor, low: torch.Tensor, high: torch.Tensor) -> torch.Tensor:
    return (a.clamp(-1.0, 1.0) + 1.0) * 0.5 * (high - low) + low


def _tiny_backbone() -> Dict[str, Any]:
    from .gpt import ARCHS as GPT_ARCHS
    return GPT_ARCHS["tiny-qwen2"].to_hf_config()


ARCHS = {
    # pendulum-sized: 1 action dimension, chunks of 4 actions, the 3 observation values as proprioceptive state
    "tiny-flow-vla": FlowVLAArgs(action_dim=1, horizon=4, state_dim=3, expert_dim=64, expert_layers=2, expert_heads=2,
                                 expert_head_dim=32, expert_ffn=128, backbone=_tiny_backbone()),
}
