"""Qwen3-MoE (e.g. Qwen3-30B-A3B): GQA attention with per-head q/k RMSNorm and a top-k routed
mixture-of-experts feed-forward in every block (cosmos_rl/policy/model/qwen3_moe/__init__.py:287-887).

Experts are stored stacked (``w_gate_up [E_local, 2I, H]``, ``w_down [E_local, H, I]``) so the grouped
tcgen05 GEMMs see one tensor; the HF checkpoint's per-expert tensors are assembled into / split out of the
stacks by the weight mapper. Expert parallelism shards the expert dimension; tokens travel to the rank that
owns their expert and back.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as tF

from ..ops import functional as F
from ..ops import moe as M
from .base import ModelRegistry, WeightMapper
from .gpt import GPT, Attention, GPTArgs, GPTWeightMapper, _linear, _rope_theta


@dataclass
class Qwen3MoEArgs(GPTArgs):
    n_experts: int = 128
    top_k: int = 8
    moe_ffn_dim: int = 768
    norm_topk_prob: bool = True
    aux_loss_coeff: float = 0.0
    ep_size: int = 1
    ep_rank: int = 0

    @classmethod
    def from_hf_config(cls, c, **over) -> "Qwen3MoEArgs":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        a = cls(vocab_size=g("vocab_size"), dim=g("hidden_size"), n_layers=g("num_hidden_layers"),
                n_heads=g("num_attention_heads"), n_kv_heads=g("num_key_value_heads"), head_dim=g("head_dim"),
                ffn_dim=g("intermediate_size", 0) or 0, norm_eps=g("rms_norm_eps", 1e-6),
                rope_theta=_rope_theta(g, 1e6), qkv_bias=bool(g("attention_bias", False)), qk_norm=True,
                tie_word_embeddings=bool(g("tie_word_embeddings", False)),
                max_seq_len=g("max_position_embeddings", 40960), model_type="qwen3_moe",
                n_experts=g("num_experts") or g("num_local_experts"), top_k=g("num_experts_per_tok"), moe_ffn_dim=g("moe_intermediate_size"),
                norm_topk_prob=bool(g("norm_topk_prob", False)))
        for k, v in over.items():
            setattr(a, k, v)
        a.__post_init__()
        return a

    def to_hf_config(self) -> Dict[str, Any]:
        d = super().to_hf_config()
        d.update({"architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "num_experts": self.n_experts,
                  "num_experts_per_tok": self.top_k, "moe_intermediate_size": self.moe_ffn_dim,
                  "norm_topk_prob": self.norm_topk_prob, "intermediate_size": self.ffn_dim or self.moe_ffn_dim})
        return d


ARCHS = {
    "qwen3-30b-a3b": Qwen3MoEArgs(vocab_size=151936, dim=2048, n_layers=48, n_heads=32, n_kv_heads=4, head_dim=128,
                                  ffn_dim=6144, rope_theta=1e6, qkv_bias=False, qk_norm=True, model_type="qwen3_moe",
                                  n_experts=128, top_k=8, moe_ffn_dim=768, max_seq_len=40960),
    "tiny-qwen3-moe": Qwen3MoEArgs(vocab_size=32000, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64,
                                   ffn_dim=512, rope_theta=1e6, qkv_bias=False, qk_norm=True, model_type="qwen3_moe",
                                   n_experts=8, top_k=2, moe_ffn_dim=128),
}


class MoEFeedForward(nn.Module):
    def __init__(self, a: Qwen3MoEArgs):
        super().__init__()
        assert a.n_experts % a.ep_size == 0
        self.E, self.k, self.I = a.n_experts, a.top_k, a.moe_ffn_dim
        self.ep_size, self.ep_rank = a.ep_size, a.ep_rank
        self.E_local = a.n_experts // a.ep_size
        self.renorm = a.norm_topk_prob
        self.aux_coeff = a.aux_loss_coeff
        self.gate = nn.Linear(a.dim, a.n_experts, bias=False)
        self.w_gate_up = nn.Parameter(torch.empty(self.E_local, 2 * self.I, a.dim))
        self.w_down = nn.Parameter(torch.empty(self.E_local, a.dim, self.I))
        self.ep_group: Optional[dist.ProcessGroup] = None
        self.peer_a2a = None       # parallel.peer_a2a.PeerAllToAll: token exchange over NVLink peer memory
        self.fused_ep = None       # parallel.ep_fused.FusedEPForward: inference path, dispatch fused into the GEMM
        self.last_aux_loss: Optional[torch.Tensor] = None

    def route(self, x: torch.Tensor):
        logits = _linear(x, self.gate.weight).float()      # router in fp32
        counts = torch.zeros(self.E, dtype=torch.int32, device=x.device) if x.is_cuda else None
        if x.is_cuda and not (torch.is_grad_enabled() and self.gate.weight.requires_grad):
            probs, idx = M.route_topk(logits, self.k, self.renorm, counts)
            return probs, idx, counts, logits
        # differentiable path: same math with autograd through the probabilities
        p = torch.softmax(logits, dim=-1)
        topv, topi = torch.topk(p, self.k, dim=-1)
        if self.renorm:
            topv = topv / topv.sum(-1, keepdim=True)
        if self.aux_coeff > 0:
            frac = torch.zeros(self.E, device=x.device).index_add_(
                0, topi.flatten(), torch.ones(topi.numel(), device=x.device)) / topi.numel()
            self.last_aux_loss = self.aux_coeff * self.E * (frac * p.mean(0)).sum()
        return topv, topi.to(torch.int32), None, logits

    def forward(self, x: torch.Tensor, tp=None) -> torch.Tensor:
        probs, idx, counts, _ = self.route(x)
        if self.ep_size == 1:
            return M.moe_experts(x, probs, idx, self.w_gate_up, self.w_down, counts)
        if (self.fused_ep is not None and x.is_cuda and not torch.is_grad_enabled()
                and x.shape[0] * self.k <= self.fused_ep.max_send):
            # inference: dispatch fused into the first grouped GEMM, no host read of the split sizes
            return self.fused_ep.forward(x, probs, idx, self.w_gate_up, self.w_down)
        return self._forward_ep(x, probs, idx)

    # ------------------------------------------------------------------ expert parallel (library all-to-all)
    def _forward_ep(self, x, probs, idx):
        """Tokens go to the rank owning their expert (all_to_all_single with split sizes), are processed by the
        local experts and come back; the statement of the reference's Megatron all-to-all dispatcher
        (cosmos_rl/policy/kernel/megatron_moe/token_dispatcher.py:808-1201)."""
        T, H = x.shape
        k, ep, El = self.k, self.ep_size, self.E_local
        flat_e = idx.flatten().long()
        order = torch.argsort(flat_e, stable=True)
        tok = order // k
        send_x = x[tok]
        dest = flat_e[order] // El
        send_counts = torch.bincount(dest, minlength=ep)
        peer = self.peer_a2a if (self.peer_a2a is not None and x.is_cuda) else None
        if peer is not None:
            # full split-size matrix (row s = what rank s sends to each rank): both sides derive row offsets from it
            allc = [torch.empty_like(send_counts) for _ in range(ep)]
            dist.all_gather(allc, send_counts, group=self.ep_group)
            mat = torch.stack(allc).tolist()
            sc, rc = mat[self.ep_rank], [mat[s][self.ep_rank] for s in range(ep)]
        else:
            mat = None
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.ep_group)
            sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv_e = torch.empty(sum(rc), dtype=torch.long, device=x.device)
        recv_x = _A2A.apply(send_x, peer, sc, rc, self.ep_group, mat)
        dist.all_to_all_single(recv_e, (flat_e[order] % El).contiguous(), rc, sc, group=self.ep_group)
        ones = torch.ones(recv_x.shape[0], 1, dtype=torch.float32, device=x.device)
        y = M.moe_experts(recv_x, ones, recv_e[:, None].to(torch.int32), self.w_gate_up, self.w_down)
        matT = [list(r) for r in zip(*mat)] if mat is not None else None
        back = _A2A.apply(y, peer, rc, sc, self.ep_group, matT)
        w = probs.flatten()[order].to(back.dtype)[:, None]
        out = torch.zeros(T, H, dtype=back.dtype, device=x.device).index_add_(0, tok, back * w)
        return out


class _A2A(torch.autograd.Function):
    """Rows sorted by destination rank out, rows sorted by source rank back. ``peer`` (a ``PeerAllToAll``) moves the
    payload with the peer-memory push kernel; without it the library collective does. ``mat[s][d]`` is the split-size
    matrix of the forward direction (only needed by the peer path)."""

    @staticmethod
    def forward(ctx, x, peer, send_counts, recv_counts, group, mat=None):
        ctx.sc, ctx.rc, ctx.group, ctx.peer, ctx.mat = send_counts, recv_counts, group, peer, mat
        if peer is not None:
            return peer.exchange(x.contiguous(), send_counts, mat)
        out = torch.empty(sum(recv_counts), x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), recv_counts, send_counts, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        if ctx.peer is not None:
            matT = [list(r) for r in zip(*ctx.mat)]
            return ctx.peer.exchange(g.contiguous(), ctx.rc, matT), None, None, None, None, None
        out = torch.empty(sum(ctx.sc), g.shape[1], dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), ctx.sc, ctx.rc, group=ctx.group)
        return out, None, None, None, None, None


class Qwen3MoEBlock(nn.Module):
    def __init__(self, a: Qwen3MoEArgs):
        super().__init__()
        self.eps = a.norm_eps
        self.input_layernorm = nn.Parameter(torch.ones(a.dim))
        self.self_attn = Attention(a)
        self.post_attention_layernorm = nn.Parameter(torch.ones(a.dim))
        self.mlp = MoEFeedForward(a)

    def _attn_part(self, h, res, positions, cu_seqlens, max_seqlen, tp):
        if res is None:
            x, _ = F.rms_norm(h, self.input_layernorm, self.eps)
            res = h
        else:
            x, res = F.rms_norm(h, self.input_layernorm, self.eps, residual=res)
        h = self.self_attn(x, positions, cu_seqlens, max_seqlen, tp)
        return F.rms_norm(h, self.post_attention_layernorm, self.eps, residual=res)

    def forward(self, h, res, positions, cu_seqlens, max_seqlen, tp=None, recompute: str = "none"):
        x, res = self._attn_part(h, res, positions, cu_seqlens, max_seqlen, tp)
        return self.mlp(x, tp), res


class Qwen3MoEWeightMapper(GPTWeightMapper):
    def hf_names(self, local: str) -> List[str]:
        if local.endswith("mlp.gate.weight"):
            return ["model." + local]
        return super().hf_names(local)

    def expert_names(self, local: str, n_experts: int, e0: int) -> List[Tuple[int, List[str]]]:
        """For a stacked expert parameter: [(global expert id, hf names in row order)] of its local experts."""
        stem = local.rsplit(".", 1)[0]
        if self.layer_offset and stem.startswith("layers."):
            i, rest = stem[len("layers."):].split(".", 1)
            stem = f"layers.{int(i) + self.layer_offset}.{rest}"
        prefix = "model." + stem + ".experts."
        parts = ("gate_proj", "up_proj") if local.endswith("w_gate_up") else ("down_proj",)
        return [(e0 + i, [f"{prefix}{e0 + i}.{p}.weight" for p in parts]) for i in range(n_experts)]

    def load_param(self, name, p, read, available, tp, r) -> bool:
        if not (name.endswith("w_gate_up") or name.endswith("w_down")):
            return False
        El = p.shape[0]
        e0 = getattr(self, "ep_rank", 0) * El
        for i, (e, names) in enumerate(self.expert_names(name, El, e0)):
            t = torch.cat([read(n) for n in names], dim=0)
            p[i].copy_(t.to(p.dtype))
        return True


@ModelRegistry.register(Qwen3MoEWeightMapper)
class Qwen3MoE(GPT):
    def __init__(self, args: Qwen3MoEArgs):
        super().__init__(args)
        self.layers = nn.ModuleList([Qwen3MoEBlock(args) for _ in range(args.n_layers)])

    @staticmethod
    def supported_model_types():
        return ["qwen3_moe"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(Qwen3MoEArgs.from_hf_config(hf_config, **kw))

    def set_ep_group(self, group) -> None:
        for layer in self.layers:
            layer.mlp.ep_group = group

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        super().init_weights(seed, std)
        if self.args.ep_size > 1:
            # every rank draws the same stream: give the experts this rank owns their own values
            g = torch.Generator(device="cpu").manual_seed(seed * 1000003 + 17 + self.args.ep_rank)
            with torch.no_grad():
                for name, p in self.named_parameters():
                    if name.endswith("w_gate_up") or name.endswith("w_down"):
                        p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std).to(p.dtype))

    def aux_loss(self) -> Optional[torch.Tensor]:
        losses = [l.mlp.last_aux_loss for l in self.layers if l.mlp.last_aux_loss is not None]
        return torch.stack(losses).sum() if losses else None

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        a = self.args
        n = sum(p.numel() for p in self.parameters())
        dense = sum(p.numel() for name, p in self.named_parameters() if "w_gate_up" not in name and "w_down" not in name
                    and "embed_tokens" not in name)
        active = dense + a.n_layers * a.top_k * 3 * a.dim * a.moe_ffn_dim
        return n, 6 * active + 12 * a.n_layers * a.n_heads * a.head_dim * seq_len

    def export_items(self):
        """(hf name, tensor) pairs: stacked experts are split back into per-expert tensors."""
        mapper = Qwen3MoEWeightMapper({"model_type": "qwen3_moe"})
        a = self.args
        from .hf_io import _split_fused
        out = []
        for name, p in self.named_parameters():
            if name.endswith("w_gate_up") or name.endswith("w_down"):
                El = p.shape[0]
                for i, (e, names) in enumerate(mapper.expert_names(name, El, a.ep_rank * El)):
                    pieces = p[i].detach().chunk(len(names), dim=0)
                    out.extend(zip(names, pieces))
            else:
                out.extend(_split_fused(name, p.detach(), mapper, a.to_hf_config(), a.n_heads // a.tp_size,
                                        max(1, a.n_kv_heads // a.tp_size), a.head_dim))
        return out

    def shard_parts(self, flat):
        """Weight-sync parts: the dense parameters as in the dense decoder, experts as per-expert rectangles."""
        from ..parallel.reshard import Part, gpt_parts
        from .base import ModelRegistry
        mapper = ModelRegistry.mapper(self.args.model_type)({"model_type": self.args.model_type})
        mapper.layer_offset = getattr(self, "layer_offset", 0)
        a = self.args
        dense = [(n, p) for n, p in flat.params if not (n.endswith("w_gate_up") or n.endswith("w_down"))]
        view = copy.copy(flat)
        view.params = dense
        parts = gpt_parts(self, view)
        for name, p in flat.params:
            if not (name.endswith("w_gate_up") or name.endswith("w_down")):
                continue
            slot = flat.by_name[name]
            El, rows, cols = p.shape
            for i, (e, names) in enumerate(mapper.expert_names(name, El, a.ep_rank * El)):
                per = rows // len(names)
                for j, hf in enumerate(names):
                    parts.append(Part(hf, 0, per, 0, cols, slot.offset + (i * rows + j * per) * cols, cols,
                                      bool(p.requires_grad)))
        return parts
