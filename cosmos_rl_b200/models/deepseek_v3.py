"""DeepSeek-V3 family: multi-head latent attention (low-rank q and joint kv compression with a decoupled RoPE
key), dense feed-forward in the first blocks, then MoE blocks with a sigmoid router, group-limited top-k, a
load-balancing bias that is updated outside of autograd, and always-on shared experts
(model of cosmos_rl/policy/model/deepseek_v3/__init__.py and its weight mapper; routing of
cosmos_rl/policy/kernel/moe/moe.py:563-635).

Parameters use the stacked-expert layout of ``qwen3_moe`` so the grouped tcgen05 GEMM, the expert-parallel
exchange and the rank-local optimizer tail apply unchanged. Attention runs through the packed varlen kernel with V
padded to the q/k head width (nope + rope); the latent cache form is not used in training.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import ModelRegistry
from .gpt import GPT, FeedForward, GPTArgs, _linear, _rope_theta
from .qwen3_moe import MoEFeedForward, Qwen3MoEWeightMapper


@dataclass
class DeepseekV3Args(GPTArgs):
    q_lora_rank: Optional[int] = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    rope_interleave: bool = True
    rope_scaling: Optional[Dict[str, Any]] = None      # yarn: factor, beta_fast, beta_slow, mscale, mscale_all_dim, ...
    n_experts: int = 256
    n_shared_experts: int = 1
    top_k: int = 8
    n_group: int = 8
    topk_group: int = 4
    moe_ffn_dim: int = 2048
    first_k_dense: int = 3
    routed_scaling_factor: float = 2.5
    norm_topk_prob: bool = True
    aux_loss_coeff: float = 0.0
    ep_size: int = 1
    ep_rank: int = 0

    @classmethod
    def from_hf_config(cls, c, **over) -> "DeepseekV3Args":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        rp = g("rope_parameters") or g("rope_scaling")
        if rp is not None and not isinstance(rp, dict):
            rp = dict(rp)
        scaling = rp if rp and rp.get("rope_type", rp.get("type", "default")) not in ("default", None) else None
        a = cls(vocab_size=g("vocab_size"), dim=g("hidden_size"), n_layers=g("num_hidden_layers"),
                n_heads=g("num_attention_heads"), n_kv_heads=g("num_attention_heads"),
                head_dim=g("qk_nope_head_dim") + g("qk_rope_head_dim"), ffn_dim=g("intermediate_size"),
                norm_eps=g("rms_norm_eps", 1e-6), rope_theta=_rope_theta(g, 1e4), qkv_bias=bool(g("attention_bias", False)),
                qk_norm=False, tie_word_embeddings=bool(g("tie_word_embeddings", False)),
                max_seq_len=g("max_position_embeddings", 4096), model_type="deepseek_v3",
                q_lora_rank=g("q_lora_rank"), kv_lora_rank=g("kv_lora_rank"), qk_nope_head_dim=g("qk_nope_head_dim"),
                qk_rope_head_dim=g("qk_rope_head_dim"), v_head_dim=g("v_head_dim"),
                rope_interleave=bool(g("rope_interleave", True)), rope_scaling=scaling,
                n_experts=g("n_routed_experts"), n_shared_experts=g("n_shared_experts", 0) or 0,
                top_k=g("num_experts_per_tok"), n_group=g("n_group", 1) or 1, topk_group=g("topk_group", 1) or 1,
                moe_ffn_dim=g("moe_intermediate_size"), first_k_dense=g("first_k_dense_replace", 0) or 0,
                routed_scaling_factor=float(g("routed_scaling_factor", 1.0)),
                norm_topk_prob=bool(g("norm_topk_prob", True)))
        for k, v in over.items():
            setattr(a, k, v)
        a.__post_init__()
        return a

    def to_hf_config(self) -> Dict[str, Any]:
        d = super().to_hf_config()
        rp = dict(self.rope_scaling) if self.rope_scaling else {"rope_type": "default"}
        rp.setdefault("rope_theta", self.rope_theta)
        d.update({"architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3",
                  "q_lora_rank": self.q_lora_rank, "kv_lora_rank": self.kv_lora_rank,
                  "qk_nope_head_dim": self.qk_nope_head_dim, "qk_rope_head_dim": self.qk_rope_head_dim,
                  "v_head_dim": self.v_head_dim, "rope_interleave": self.rope_interleave, "rope_parameters": rp,
                  "n_routed_experts": self.n_experts, "n_shared_experts": self.n_shared_experts,
                  "num_experts_per_tok": self.top_k, "n_group": self.n_group, "topk_group": self.topk_group,
                  "moe_intermediate_size": self.moe_ffn_dim, "first_k_dense_replace": self.first_k_dense,
                  "routed_scaling_factor": self.routed_scaling_factor, "norm_topk_prob": self.norm_topk_prob,
                  "num_key_value_heads": self.n_heads})
        return d


ARCHS = {
    "deepseek-v3": DeepseekV3Args(
        vocab_size=129280, dim=7168, n_layers=61, n_heads=128, n_kv_heads=128, head_dim=192, ffn_dim=18432,
        rope_theta=1e4, model_type="deepseek_v3", max_seq_len=163840,
        rope_scaling={"rope_type": "yarn", "factor": 40.0, "beta_fast": 32.0, "beta_slow": 1.0, "mscale": 1.0,
                      "mscale_all_dim": 1.0, "original_max_position_embeddings": 4096}),
    "tiny-deepseek-v3": DeepseekV3Args(
        vocab_size=32000, dim=256, n_layers=3, n_heads=4, n_kv_heads=4, head_dim=48, ffn_dim=512, rope_theta=1e4,
        model_type="deepseek_v3", q_lora_rank=96, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16,
        v_head_dim=32, n_experts=8, n_shared_experts=1, top_k=2, n_group=2, topk_group=1, moe_ffn_dim=128,
        first_k_dense=1),
}


# ---------------------------------------------------------------------------------------------- rotary embedding
def _yarn_mscale(scale: float, m: float = 1.0) -> float:
    return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0


def rope_tables(a: DeepseekV3Args, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin ``[T, rope_dim / 2]`` in fp32; YaRN blends interpolated and extrapolated frequencies per dimension
    and scales the tables by the attention factor."""
    d = a.qk_rope_head_dim
    idx = torch.arange(0, d, 2, dtype=torch.float32, device=positions.device) / d
    inv = 1.0 / (a.rope_theta ** idx)
    factor_att = 1.0
    rs = a.rope_scaling
    if rs and rs.get("rope_type", rs.get("type")) == "yarn":
        factor = float(rs["factor"])
        orig = rs.get("original_max_position_embeddings") or a.max_seq_len
        bf, bs = float(rs.get("beta_fast") or 32.0), float(rs.get("beta_slow") or 1.0)
        corr = lambda n_rot: d * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(a.rope_theta))
        lo, hi = corr(bf), corr(bs)
        if rs.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, d - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(d // 2, dtype=torch.float32, device=positions.device) - lo) / (hi - lo)).clamp(0, 1)
        extra = 1.0 - ramp
        inv = (inv / factor) * (1 - extra) + inv * extra
        ms, msa = rs.get("mscale"), rs.get("mscale_all_dim")
        factor_att = rs.get("attention_factor") or (
            _yarn_mscale(factor, ms) / _yarn_mscale(factor, msa) if ms and msa else _yarn_mscale(factor))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang) * factor_att, torch.sin(ang) * factor_att


def softmax_scale(a: DeepseekV3Args) -> float:
    s = (a.qk_nope_head_dim + a.qk_rope_head_dim) ** -0.5
    rs = a.rope_scaling
    if rs and rs.get("mscale_all_dim"):
        m = _yarn_mscale(float(rs["factor"]), float(rs["mscale_all_dim"]))
        s *= m * m
    return s


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleave: bool) -> torch.Tensor:
    """x [T, h, d]. ``interleave``: checkpoint stores the pairs as (x0, x1), (x2, x3), ...; they are brought to the
    half-split form first (q and k get the same permutation, so q.k is unchanged)."""
    if interleave:
        x = x.unflatten(-1, (-1, 2)).transpose(-1, -2).flatten(-2)
    x1, x2 = x.float().chunk(2, dim=-1)
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


# ---------------------------------------------------------------------------------------------- attention
class MLAttention(nn.Module):
    def __init__(self, a: DeepseekV3Args):
        super().__init__()
        assert a.tp_size == 1, "latent attention is not tensor-parallel here; use dp_shard / ep"
        self.a = a
        self.h = a.n_heads
        self.dn, self.dr, self.dv = a.qk_nope_head_dim, a.qk_rope_head_dim, a.v_head_dim
        self.eps = a.norm_eps
        dq = self.dn + self.dr
        if a.q_lora_rank:
            self.q_a_proj = nn.Linear(a.dim, a.q_lora_rank, bias=a.qkv_bias)
            self.q_a_layernorm = nn.Parameter(torch.ones(a.q_lora_rank))
            self.q_b_proj = nn.Linear(a.q_lora_rank, self.h * dq, bias=False)
        else:
            self.q_proj = nn.Linear(a.dim, self.h * dq, bias=False)
        self.kv_a_proj_with_mqa = nn.Linear(a.dim, a.kv_lora_rank + self.dr, bias=a.qkv_bias)
        self.kv_a_layernorm = nn.Parameter(torch.ones(a.kv_lora_rank))
        self.kv_b_proj = nn.Linear(a.kv_lora_rank, self.h * (self.dn + self.dv), bias=False)
        self.o_proj = nn.Linear(self.h * self.dv, a.dim, bias=a.qkv_bias)
        self.scale = softmax_scale(a)

    def project_qkv(self, x, positions):
        """q, k ``[T, h, dn + dr]`` (RoPE applied to the last dr), v ``[T, h, dv]``."""
        a, T, h = self.a, x.shape[0], self.h
        if a.q_lora_rank:
            ql = _linear(x, self.q_a_proj.weight, self.q_a_proj.bias)
            q = _linear(F.rms_norm(ql, self.q_a_layernorm, self.eps)[0], self.q_b_proj.weight)
        else:
            q = _linear(x, self.q_proj.weight)
        q = q.view(T, h, self.dn + self.dr)
        ckv = _linear(x, self.kv_a_proj_with_mqa.weight, self.kv_a_proj_with_mqa.bias)
        c, k_pe = ckv.split([a.kv_lora_rank, self.dr], dim=-1)
        kv = _linear(F.rms_norm(c.contiguous(), self.kv_a_layernorm, self.eps)[0], self.kv_b_proj.weight)
        kv = kv.view(T, h, self.dn + self.dv)
        k_nope, v = kv.split([self.dn, self.dv], dim=-1)
        cos, sin = rope_tables(a, positions)
        q_pe = _rotate(q[..., self.dn:], cos, sin, a.rope_interleave)
        k_pe = _rotate(k_pe.reshape(T, 1, self.dr), cos, sin, a.rope_interleave)
        q = torch.cat([q[..., :self.dn], q_pe], dim=-1)
        k = torch.cat([k_nope, k_pe.expand(T, h, self.dr)], dim=-1)
        return q, k, v

    def forward(self, x, positions, cu_seqlens, max_seqlen, tp=None):
        q, k, v = self.project_qkv(x, positions)
        pad = q.shape[-1] - self.dv
        vp = torch.nn.functional.pad(v, (0, pad)) if pad > 0 else v
        o = F.varlen_attention(q.contiguous(), k.contiguous(), vp.contiguous(), cu_seqlens, max_seqlen, self.scale)
        o = o[..., :self.dv].reshape(x.shape[0], self.h * self.dv)
        return _linear(o, self.o_proj.weight, self.o_proj.bias)


# ---------------------------------------------------------------------------------------------- MoE
class DeepseekMoE(MoEFeedForward):
    """Sigmoid scores; the top ``topk_group`` of ``n_group`` expert groups are kept (group score = sum of its two best
    biased scores), then the top-k experts among them; weights are the unbiased scores, renormalised and scaled. The
    bias only steers the choice and is moved by ``update_bias`` from the measured load, never by the gradient."""

    def __init__(self, a: DeepseekV3Args):
        super().__init__(a)
        self.n_group, self.topk_group, self.route_scale = a.n_group, a.topk_group, a.routed_scaling_factor
        self.gate.e_score_correction_bias = nn.Parameter(torch.zeros(a.n_experts), requires_grad=False)
        self.shared = None
        if a.n_shared_experts > 0:
            sa = GPTArgs(vocab_size=a.vocab_size, dim=a.dim, n_layers=1, n_heads=a.n_heads, n_kv_heads=a.n_kv_heads,
                         head_dim=a.head_dim, ffn_dim=a.moe_ffn_dim * a.n_shared_experts)
            self.shared = FeedForward(sa)
        self.last_load: Optional[torch.Tensor] = None

    def route(self, x):
        logits = torch.nn.functional.linear(x.float(), self.gate.weight.float())
        scores = torch.sigmoid(logits)
        biased = scores + self.gate.e_score_correction_bias.float()[None, :]
        T, E, G = scores.shape[0], self.E, self.n_group
        if G > 1:
            grp = biased.view(T, G, E // G).topk(min(2, E // G), dim=-1).values.sum(-1)
            keep = torch.zeros_like(grp, dtype=torch.bool).scatter_(1, grp.topk(self.topk_group, dim=-1).indices, True)
            biased = biased.masked_fill(~keep[:, :, None].expand(T, G, E // G).reshape(T, E), 0.0)
        idx = biased.topk(self.k, dim=-1).indices
        w = scores.gather(1, idx)
        if self.renorm:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * self.route_scale
        with torch.no_grad():
            self.last_load = torch.bincount(idx.flatten(), minlength=E).float()
        if self.aux_coeff > 0 and torch.is_grad_enabled():
            p = scores / (scores.sum(-1, keepdim=True) + 1e-20)
            self.last_aux_loss = self.aux_coeff * E * ((self.last_load / idx.numel()) * p.mean(0)).sum()
        counts = self.last_load.to(torch.int32) if x.is_cuda else None
        return w, idx.to(torch.int32), counts, logits

    @torch.no_grad()
    def update_bias(self, rate: float, load: Optional[torch.Tensor] = None) -> None:
        """Auxiliary-loss-free balancing: raise the bias of under-loaded experts and lower it for over-loaded ones by
        a fixed step. ``load`` is the per-expert token count summed over the data-parallel ranks (default: last
        forward of this rank)."""
        load = self.last_load if load is None else load
        if load is None:
            return
        self.gate.e_score_correction_bias.add_(rate * torch.sign(load.mean() - load).to(self.gate.e_score_correction_bias.dtype))

    def forward(self, x, tp=None):
        y = super().forward(x, tp)
        return y + self.shared(x) if self.shared is not None else y


class DeepseekV3Block(nn.Module):
    def __init__(self, a: DeepseekV3Args, layer_idx: int):
        super().__init__()
        self.eps = a.norm_eps
        self.input_layernorm = nn.Parameter(torch.ones(a.dim))
        self.self_attn = MLAttention(a)
        self.post_attention_layernorm = nn.Parameter(torch.ones(a.dim))
        self.is_moe = layer_idx >= a.first_k_dense
        self.mlp = DeepseekMoE(a) if self.is_moe else FeedForward(a)

    def forward(self, h, res, positions, cu_seqlens, max_seqlen, tp=None, recompute: str = "none"):
        if res is None:
            x, res = F.rms_norm(h, self.input_layernorm, self.eps)[0], h
        else:
            x, res = F.rms_norm(h, self.input_layernorm, self.eps, residual=res)
        h = self.self_attn(x, positions, cu_seqlens, max_seqlen)
        x, res = F.rms_norm(h, self.post_attention_layernorm, self.eps, residual=res)
        return self.mlp(x), res


class DeepseekV3WeightMapper(Qwen3MoEWeightMapper):
    RENAME = dict(Qwen3MoEWeightMapper.RENAME, **{"self_attn.q_a_layernorm": "self_attn.q_a_layernorm.weight",
                                                 "self_attn.kv_a_layernorm": "self_attn.kv_a_layernorm.weight"})

    def hf_names(self, local: str) -> List[str]:
        if local.endswith("mlp.gate.e_score_correction_bias"):
            return ["model." + self._shift(local)]
        local = local.replace(".mlp.shared.", ".mlp.shared_experts.")
        return super().hf_names(local)

    def _shift(self, name: str) -> str:
        if self.layer_offset and name.startswith("layers."):
            idx, rest = name[len("layers."):].split(".", 1)
            return f"layers.{int(idx) + self.layer_offset}.{rest}"
        return name


@ModelRegistry.register(DeepseekV3WeightMapper)
class DeepseekV3(GPT):
    paged_engine = False    # latent attention has no paged KV path in the generation engine: rollouts recompute

    def __init__(self, args: DeepseekV3Args):
        super().__init__(args)
        lo, hi = args.stage_layers()
        self.layers = nn.ModuleList([DeepseekV3Block(args, i) for i in range(lo, hi)])

    @staticmethod
    def supported_model_types():
        return ["deepseek_v3"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(DeepseekV3Args.from_hf_config(hf_config, **kw))

    def moe_layers(self) -> List[DeepseekMoE]:
        return [l.mlp for l in self.layers if l.is_moe]

    def set_ep_group(self, group) -> None:
        for m in self.moe_layers():
            m.ep_group = group

    def aux_loss(self) -> Optional[torch.Tensor]:
        losses = [m.last_aux_loss for m in self.moe_layers() if m.last_aux_loss is not None]
        return torch.stack(losses).sum() if losses else None

    def update_router_bias(self, rate: float = 1e-3, group=None) -> None:
        """Call once per optimizer step (after the backward pass): the bias update of every MoE block."""
        import torch.distributed as dist
        for m in self.moe_layers():
            load = m.last_load
            if load is not None and group is not None:
                load = load.clone()
                dist.all_reduce(load, group=group)
            m.update_bias(rate, load)

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        a = self.args
        n = sum(p.numel() for p in self.parameters())
        routed = sum(p.numel() for name, p in self.named_parameters() if name.endswith("w_gate_up") or name.endswith("w_down"))
        embed = sum(p.numel() for name, p in self.named_parameters() if "embed_tokens" in name)
        n_moe = max(0, a.n_layers - a.first_k_dense)
        active = n - routed - embed + n_moe * a.top_k * 3 * a.dim * a.moe_ffn_dim
        return n, 6 * active + 12 * a.n_layers * a.n_heads * a.head_dim * seq_len

    def shard_parts(self, flat):
        """Weight-sync parts: stacked experts as per-expert rectangles (each expert-parallel rank publishes its own
        experts), everything else as full or fused rectangles."""
        from .qwen3_moe import Qwen3MoE
        return Qwen3MoE.shard_parts(self, flat)

    def export_items(self):
        """(hf name, tensor) pairs: stacked experts and fused gate/up are split back."""
        mapper = DeepseekV3WeightMapper({"model_type": "deepseek_v3"})
        mapper.layer_offset = self.layer_offset
        a = self.args
        from .hf_io import _split_fused
        out = []
        for name, p in self.named_parameters():
            if name.endswith("w_gate_up") or name.endswith("w_down"):
                El = p.shape[0]
                for i, (e, names) in enumerate(mapper.expert_names(name, El, a.ep_rank * El)):
                    out.extend(zip(names, p[i].detach().chunk(len(names), dim=0)))
            else:
                out.extend(_split_fused(name, p.detach(), mapper, a.to_hf_config(), a.n_heads, a.n_kv_heads, a.head_dim))
        return out
