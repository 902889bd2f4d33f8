"""Dense decoder-only transformer (Llama / Qwen2 / Qwen2.5 / Qwen3 families).

Same model family as cosmos_rl/policy/model/gpt/__init__.py:119-813, laid out for this framework:
* q/k/v and gate/up are stored fused (``qkv_proj``, ``gate_up_proj``): one GEMM each, and the parameter
  layout is exactly what the rollout engine consumes, so colocated rollouts share the policy's tensors and
  separated rollouts receive rectangular slices.
* activations are packed ``[T, H]`` (no padding); attention takes ``cu_seqlens``.
* the model returns the final hidden states; log-probabilities come from the fused lm_head kernel
  (``logprobs``), logits are only materialised by ``logits`` for generation.
Tensor parallelism: column-parallel qkv / gate_up, row-parallel o / down, vocabulary-parallel embedding and
lm_head; the collectives are issued through :mod:`cosmos_rl_b200.parallel.tp`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as tF
from torch.utils.checkpoint import checkpoint

from ..ops import functional as F
from .base import BaseModel, ModelRegistry, WeightMapper


@dataclass
class GPTArgs:
    vocab_size: int = 32000
    dim: int = 256
    n_layers: int = 2
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: Optional[int] = None
    ffn_dim: int = 688
    norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qkv_bias: bool = True
    qk_norm: bool = False
    tie_word_embeddings: bool = False
    max_seq_len: int = 4096
    model_type: str = "qwen2"
    tp_size: int = 1
    tp_rank: int = 0
    pp_size: int = 1        # pipeline stages: a stage owns a contiguous range of blocks (+ embedding / head)
    pp_rank: int = 0
    pp_chunks: int = 1      # model chunks per pipeline rank (interleaved schedule): chunk c of rank r is virtual stage
                            # c * pp_size + r of pp_size * pp_chunks virtual stages
    pp_embed_weight: float = 0.0    # cost of the embedding (first stage) and of final norm + lm_head (last stage)
    pp_head_weight: float = 0.0     # in units of one block, for the layer split; -1 = from the shapes

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.dim // self.n_heads

    def stage_layers(self) -> Tuple[int, int]:
        """[lo, hi) block indices of this pipeline stage (earlier stages take the remainder)."""
        bounds = self.stage_bounds()
        return bounds[self.pp_rank], bounds[self.pp_rank + 1]

    def chunk_layers(self) -> List[Tuple[int, int]]:
        """[lo, hi) block indices of every model chunk this rank holds (one chunk unless ``pp_chunks > 1``)."""
        if self.pp_chunks <= 1:
            return [self.stage_layers()]
        bounds = self.stage_bounds(self.pp_size * self.pp_chunks)
        return [(bounds[c * self.pp_size + self.pp_rank], bounds[c * self.pp_size + self.pp_rank + 1])
                for c in range(self.pp_chunks)]

    def stage_bounds(self, n_stages: Optional[int] = None) -> List[int]:
        """Block index where every stage starts (plus n_layers). Without weights: an even split. With
        ``pp_embed_weight`` / ``pp_head_weight`` the first / last stage are charged that many block-equivalents, so
        they get fewer blocks (the reference balances its DeepSeek stages by per-layer weights in the same spirit,
        cosmos_rl/utils/pipelining/pipelining_utils.py:36-110); every stage keeps at least one block."""
        n, pp = self.n_layers, (n_stages or self.pp_size)
        head = self.pp_head_weight
        if head < 0:        # lm_head GEMM against one block's GEMMs (attention projections + SwiGLU), per token
            per_block = self.dim * (self.n_heads + 2 * self.n_kv_heads) * self.head_dim \
                + self.n_heads * self.head_dim * self.dim + 3 * self.dim * self.ffn_dim
            head = self.vocab_size * self.dim / per_block
        embed = max(0.0, self.pp_embed_weight)
        if pp == 1 or (head == 0 and embed == 0):
            base, rem = divmod(n, pp)
            return [r * base + min(r, rem) for r in range(pp)] + [n]
        target = (n + head + embed) / pp
        bounds, done = [0], 0
        for r in range(pp - 1):
            want = target * (r + 1) - embed            # blocks that should sit before the end of stage r
            k = int(round(want)) - done
            k = max(1, min(k, n - done - (pp - 1 - r)))     # at least one block here and on every later stage
            done += k
            bounds.append(done)
        return bounds + [n]

    @classmethod
    def from_hf_config(cls, c, **over) -> "GPTArgs":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        mt = g("model_type", "qwen2")
        theta = _rope_theta(g, 1e4)
        a = cls(
            vocab_size=g("vocab_size"), dim=g("hidden_size"), n_layers=g("num_hidden_layers"),
            n_heads=g("num_attention_heads"), n_kv_heads=g("num_key_value_heads") or g("num_attention_heads"),
            head_dim=g("head_dim"), ffn_dim=g("intermediate_size"), norm_eps=g("rms_norm_eps", 1e-6),
            rope_theta=theta,
            qkv_bias=bool(g("attention_bias", mt == "qwen2")), qk_norm=(mt == "qwen3"),
            tie_word_embeddings=bool(g("tie_word_embeddings", False)),
            max_seq_len=g("max_position_embeddings", 4096), model_type=mt)
        for k, v in over.items():
            setattr(a, k, v)
        a.__post_init__()
        return a

    def to_hf_config(self) -> Dict[str, Any]:
        arch = {"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "llama": "LlamaForCausalLM"}
        return {
            "architectures": [arch.get(self.model_type, "Qwen2ForCausalLM")], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.dim, "num_hidden_layers": self.n_layers,
            "num_attention_heads": self.n_heads, "num_key_value_heads": self.n_kv_heads, "head_dim": self.head_dim,
            "intermediate_size": self.ffn_dim, "rms_norm_eps": self.norm_eps, "rope_theta": self.rope_theta,
            "attention_bias": self.qkv_bias, "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_seq_len, "hidden_act": "silu", "torch_dtype": "bfloat16",
        }


# named benchmark architectures (random-init; shapes of the public checkpoints)
ARCHS: Dict[str, GPTArgs] = {
    "tiny-qwen2": GPTArgs(vocab_size=32000, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=688,
                          rope_theta=1e6, qkv_bias=True, model_type="qwen2"),
    "tiny-qwen2-d128": GPTArgs(vocab_size=32000, dim=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128,
                               ffn_dim=1024, rope_theta=1e6, qkv_bias=True, model_type="qwen2"),
    "qwen2.5-7b": GPTArgs(vocab_size=152064, dim=3584, n_layers=28, n_heads=28, n_kv_heads=4, ffn_dim=18944,
                          rope_theta=1e6, qkv_bias=True, model_type="qwen2", max_seq_len=32768),
    "qwen3-32b": GPTArgs(vocab_size=151936, dim=5120, n_layers=64, n_heads=64, n_kv_heads=8, head_dim=128,
                         ffn_dim=25600, rope_theta=1e6, qkv_bias=False, qk_norm=True, model_type="qwen3",
                         max_seq_len=40960),
    "llama3-8b": GPTArgs(vocab_size=128256, dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim=14336,
                         rope_theta=5e5, qkv_bias=False, model_type="llama", max_seq_len=8192),
}


def _rope_theta(g, default: float) -> float:
    """``rope_theta`` of a config.json: top level (transformers 4) or inside ``rope_parameters`` (transformers 5)."""
    rp = g("rope_parameters") or g("rope_scaling") or {}
    t = g("rope_theta") or (rp.get("rope_theta") if isinstance(rp, dict) else getattr(rp, "rope_theta", None))
    return float(t or default)


def _linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = F.linear_maybe_fp8(x, w, b)
    lora = getattr(w, "_lora", None)       # policy.lora.LoraRef: low-rank path of an adapted projection
    return y if lora is None else lora.apply(x, y)


class Attention(nn.Module):
    def __init__(self, a: GPTArgs):
        super().__init__()
        assert a.n_heads % a.tp_size == 0, "attention heads must divide by tp"
        self.hq = a.n_heads // a.tp_size
        self.hkv = max(1, a.n_kv_heads // a.tp_size)
        self.d = a.head_dim
        self.theta = a.rope_theta
        self.qk_norm = a.qk_norm
        self.eps = a.norm_eps
        self.qkv_proj = nn.Linear(a.dim, (self.hq + 2 * self.hkv) * self.d, bias=a.qkv_bias)
        self.o_proj = nn.Linear(self.hq * self.d, a.dim, bias=False)
        if a.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(self.d))
            self.k_norm = nn.Parameter(torch.ones(self.d))

    def project_qkv(self, x: torch.Tensor, positions: torch.Tensor):
        """x [T, H] -> q [T, hq, d], k, v [T, hkv, d] with RoPE (and per-head q/k norm) applied."""
        return self.split_qkv(_linear(x, self.qkv_proj.weight, self.qkv_proj.bias), positions)

    mrope_section = None    # rotary frequencies per position stream (time, height, width) of multimodal models

    def split_qkv(self, qkv: torch.Tensor, positions: torch.Tensor):
        T = qkv.shape[0]
        hq, hkv, d = self.hq, self.hkv, self.d
        if positions.dim() == 2:
            # multimodal rotary positions [3, T]: every frequency follows the stream of its section
            from .qwen2_5_vl import apply_rotary, mrope_cos_sin
            q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
            if self.qk_norm:
                q = F.rms_norm(q.reshape(T * hq, d), self.q_norm, self.eps)[0]
                k = F.rms_norm(k.reshape(T * hkv, d), self.k_norm, self.eps)[0]
            cos, sin = mrope_cos_sin(positions, d, self.theta, self.mrope_section or [d // 2],
                                     getattr(self, "mrope_interleaved", False))
            q, k = apply_rotary(q.reshape(T, hq, d), k.reshape(T, hkv, d), cos, sin)
            return q.contiguous(), k.contiguous(), v.reshape(T, hkv, d)
        if self.qk_norm:
            q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
            qw, kw = self.q_norm, self.k_norm
            tp = getattr(self, "tp_for_replicated", None)
            if tp is not None and torch.is_grad_enabled():
                # replicated weights applied to this rank's heads only: their gradient is summed over the TP ranks
                qw, kw = tp.copy_to_region(qw), tp.copy_to_region(kw)
            q = F.rms_norm(q.reshape(T * hq, d), qw, self.eps)[0].view(T, hq, d)
            k = F.rms_norm(k.reshape(T * hkv, d), kw, self.eps)[0].view(T, hkv, d)
            q, k = F.apply_rope(q, k, positions, self.theta)
            return q, k, v.reshape(T, hkv, d)
        qkv = F.rope_qkv_(qkv, positions, hq, hkv, d, self.theta)
        q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
        return q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))

    cp = None    # ContextParallel, set by GPT.attach_context_parallel: tokens are this rank's chunk of every sequence

    def forward(self, x, positions, cu_seqlens, max_seqlen, tp=None):
        """``x`` is [T, H], or this rank's [T / tp, H] rows under sequence parallelism (the column-parallel projection
        gathers the sequence, the row-parallel one scatters it again)."""
        self.tp_for_replicated = tp
        if tp is not None:
            q, k, v = self.split_qkv(tp.col_linear(x, self.qkv_proj.weight, self.qkv_proj.bias), positions)
        else:
            q, k, v = self.project_qkv(x, positions)
        if self.cp is not None:
            o = self.cp.attention(q, k, v, cu_seqlens, max_seqlen)
        else:
            o = F.varlen_attention(q, k, v, cu_seqlens, max_seqlen)
        o = o.reshape(q.shape[0], -1)
        return tp.row_linear(o, self.o_proj.weight) if tp is not None else _linear(o, self.o_proj.weight)


class FeedForward(nn.Module):
    def __init__(self, a: GPTArgs):
        super().__init__()
        assert a.ffn_dim % a.tp_size == 0
        self.I = a.ffn_dim // a.tp_size
        self.gate_up_proj = nn.Linear(a.dim, 2 * self.I, bias=False)
        self.down_proj = nn.Linear(self.I, a.dim, bias=False)

    def forward(self, x, tp=None):
        if tp is None:
            return _linear(F.swiglu(_linear(x, self.gate_up_proj.weight)), self.down_proj.weight)
        return tp.row_linear(F.swiglu(tp.col_linear(x, self.gate_up_proj.weight)), self.down_proj.weight)


class GPTBlock(nn.Module):
    def __init__(self, a: GPTArgs):
        super().__init__()
        self.eps = a.norm_eps
        self.input_layernorm = nn.Parameter(torch.ones(a.dim))
        self.self_attn = Attention(a)
        self.post_attention_layernorm = nn.Parameter(torch.ones(a.dim))
        self.mlp = FeedForward(a)

    def _attn_part(self, h, res, positions, cu_seqlens, max_seqlen, tp):
        w_in, w_post = self.input_layernorm, self.post_attention_layernorm
        if tp is not None:
            w_in, w_post = tp.shared_weight(w_in), tp.shared_weight(w_post)
        if res is None:
            x, _ = F.rms_norm(h, w_in, self.eps)
            res = h
        else:
            x, res = F.rms_norm(h, w_in, self.eps, residual=res)
        h = self.self_attn(x, positions, cu_seqlens, max_seqlen, tp)
        x, res = F.rms_norm(h, w_post, self.eps, residual=res)
        return x, res

    def forward(self, h, res, positions, cu_seqlens, max_seqlen, tp=None, recompute: str = "none"):
        """(h, res) is the un-added residual pair: the stream value is h + res (res None on the first block).

        ``recompute="selective"`` keeps the output of the gate/up GEMM (the expensive one) and recomputes only
        the attention half of the block (12 % of its forward FLOPs) and the SwiGLU product in backward, instead
        of re-running the whole block as full activation checkpointing does."""
        if recompute in ("selective", "swiglu") and torch.is_grad_enabled():
            if recompute == "swiglu":      # keep the attention half's activations, recompute only the SwiGLU product
                x, res = self._attn_part(h, res, positions, cu_seqlens, max_seqlen, tp)
            else:
                x, res = checkpoint(self._attn_part, h, res, positions, cu_seqlens, max_seqlen, tp,
                                    use_reentrant=False)
            gu = tp.col_linear(x, self.mlp.gate_up_proj.weight) if tp is not None else \
                _linear(x, self.mlp.gate_up_proj.weight)
            act = checkpoint(F.swiglu, gu, use_reentrant=False)
            h = tp.row_linear(act, self.mlp.down_proj.weight) if tp is not None else \
                _linear(act, self.mlp.down_proj.weight)
            return h, res
        x, res = self._attn_part(h, res, positions, cu_seqlens, max_seqlen, tp)
        h = self.mlp(x, tp)
        return h, res


class GPTWeightMapper(WeightMapper):
    """HF stores q_proj/k_proj/v_proj and gate_proj/up_proj separately; this framework fuses them."""

    FUSED = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}
    RENAME = {"input_layernorm": "input_layernorm.weight", "post_attention_layernorm": "post_attention_layernorm.weight",
              "self_attn.q_norm": "self_attn.q_norm.weight", "self_attn.k_norm": "self_attn.k_norm.weight",
              "norm": "norm.weight"}

    layer_offset = 0    # first block index of this pipeline stage
    layer_map = None    # block index in the whole model per local block (several chunks per rank); wins over the offset

    def hf_names(self, local: str) -> List[str]:
        """HF parameter names a local parameter is assembled from (in row order)."""
        name = local
        if name.startswith("layers.") and (self.layer_offset or self.layer_map):
            idx, rest = name[len("layers."):].split(".", 1)
            g = self.layer_map[int(idx)] if self.layer_map else int(idx) + self.layer_offset
            name = f"layers.{g}.{rest}"
        for k, v in self.RENAME.items():
            if name == k or name.endswith("." + k):
                name = name[: len(name) - len(k)] + v
                break
        if not name.startswith("lm_head"):
            name = "model." + name
        for fused, parts in self.FUSED.items():
            if f".{fused}." in name:
                return [name.replace(fused, p) for p in parts]
        return [name]


@ModelRegistry.register(GPTWeightMapper)
class GPT(BaseModel):
    def __init__(self, args: GPTArgs):
        super().__init__()
        self.args = args
        a = args
        assert a.vocab_size % a.tp_size == 0 or a.tp_size == 1
        self.v_local = a.vocab_size // a.tp_size if a.tp_size > 1 else a.vocab_size
        ranges = a.chunk_layers()
        # local block i is block layer_map[i] of the whole model; with one chunk that is layer_offset + i
        self.layer_map = [g for lo, hi in ranges for g in range(lo, hi)]
        self.layer_offset = ranges[0][0] if len(ranges) == 1 else 0
        self.chunk_bounds = [0]
        for lo, hi in ranges:
            self.chunk_bounds.append(self.chunk_bounds[-1] + hi - lo)
        self.is_first_stage, self.is_last_stage = a.pp_rank == 0, a.pp_rank == a.pp_size - 1
        assert a.pp_size == 1 or not a.tie_word_embeddings, "tied embeddings live on both ends of a pipeline"
        self.embed_tokens = nn.Embedding(self.v_local, a.dim) if self.is_first_stage else None
        self.layers = nn.ModuleList([GPTBlock(a) for _ in self.layer_map])
        self.norm = nn.Parameter(torch.ones(a.dim)) if self.is_last_stage else None
        if a.tie_word_embeddings or not self.is_last_stage:
            self.lm_head = None
        else:
            self.lm_head = nn.Linear(a.dim, self.v_local, bias=False)
        self.gradient_checkpointing = False
        self.param_sharder = None       # ShardedFlatParams under parameter-sharded data parallelism
        self.tp = None  # set by parallel.tp.TensorParallel when tp_size > 1

    # ------------------------------------------------------------------ registry hooks
    @staticmethod
    def supported_model_types():
        return ["llama", "qwen2", "qwen3"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(GPTArgs.from_hf_config(hf_config, **kw))

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Random init from a seed; identical on every rank given the same seed."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            with torch.no_grad():
                if p.dim() == 1 and ("norm" in name):
                    p.fill_(1.0)
                elif p.dim() == 1:
                    p.zero_()
                else:
                    p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std).to(p.dtype))

    def init_weights_on_device(self, seed: int = 0, std: float = 0.02) -> None:
        """Fast random init directly on the parameter's device (benchmark-sized models)."""
        g = torch.Generator(device=self.norm.device).manual_seed(seed)
        for name, p in self.named_parameters():
            with torch.no_grad():
                if p.dim() == 1 and ("norm" in name):
                    p.fill_(1.0)
                elif p.dim() == 1:
                    p.zero_()
                else:
                    p.normal_(0.0, std, generator=g)

    # ------------------------------------------------------------------ forward
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            return self.tp.vocab_parallel_embed(input_ids, self.embed_tokens.weight)
        return self.embed_tokens(input_ids)

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, cu_seqlens: torch.Tensor,
                max_seqlen: int) -> torch.Tensor:
        """Packed forward: ``input_ids [T]`` -> final hidden states ``[T, H]`` (after the last norm).

        Under sequence parallelism the token axis is padded to the rank multiple with a dummy sequence, every block
        works on this rank's rows, and the final hidden states are gathered (and un-padded) before they are returned."""
        if self.param_sharder is not None:
            return self._forward_sharded(input_ids, position_ids, cu_seqlens, max_seqlen)
        if len(self.chunk_bounds) > 2:
            raise RuntimeError("a model built with pp_chunks > 1 runs chunk by chunk (forward_chunk) under the "
                               "interleaved pipeline schedule")
        return self._forward_layers(input_ids, position_ids, cu_seqlens, max_seqlen, self.layers,
                                    self.is_first_stage, self.is_last_stage)

    def forward_chunk(self, chunk: int, x: torch.Tensor, position_ids: torch.Tensor, cu_seqlens: torch.Tensor,
                      max_seqlen: int) -> torch.Tensor:
        """One model chunk of this rank (interleaved pipeline schedule): chunk 0 of the first rank embeds ``x``
        (token ids), the last chunk of the last rank applies the final norm; every other boundary carries the hidden
        states."""
        lo, hi = self.chunk_bounds[chunk], self.chunk_bounds[chunk + 1]
        n_chunks = len(self.chunk_bounds) - 1
        return self._forward_layers(x, position_ids, cu_seqlens, max_seqlen, self.layers[lo:hi],
                                    self.is_first_stage and chunk == 0, self.is_last_stage and chunk == n_chunks - 1)

    def _forward_layers(self, input_ids, position_ids, cu_seqlens, max_seqlen, layers, embeds: bool, finishes: bool):
        sp = self.tp is not None and self.tp.sequence_parallel
        T = input_ids.shape[0]
        if sp:
            if not (embeds and finishes):
                raise NotImplementedError("sequence parallelism is not combined with pipeline stages")
            mult = self.tp.row_multiple(input_ids.is_cuda)
            pad = (-T) % mult
            if pad:
                input_ids = torch.nn.functional.pad(input_ids, (0, pad))
                position_ids = torch.cat([position_ids, torch.arange(pad, device=position_ids.device,
                                                                     dtype=position_ids.dtype)])
                cu_seqlens = torch.cat([cu_seqlens, cu_seqlens.new_tensor([T + pad])])
                max_seqlen = max(int(max_seqlen), pad)
        h = self.embed(input_ids) if embeds else input_ids                # later stages receive hidden states
        res = None
        for layer in layers:
            if self.gradient_checkpointing in ("selective", "swiglu") and torch.is_grad_enabled():
                h, res = layer(h, res, position_ids, cu_seqlens, max_seqlen, self.tp,
                               recompute=self.gradient_checkpointing)
            elif self.gradient_checkpointing and torch.is_grad_enabled():
                h, res = checkpoint(layer, h, res, position_ids, cu_seqlens, max_seqlen, self.tp, use_reentrant=False)
            else:
                h, res = layer(h, res, position_ids, cu_seqlens, max_seqlen, self.tp)
        if not finishes:
            return h + res if res is not None else h                        # one tensor crosses the stage boundary
        norm_w = self.tp.shared_weight(self.norm) if self.tp is not None else self.norm
        out, _ = F.rms_norm(h, norm_w, self.args.norm_eps, residual=res)
        if sp:
            out = self.tp.gather_rows(out)[:T]
        return out

    def _forward_sharded(self, input_ids, position_ids, cu_seqlens, max_seqlen) -> torch.Tensor:
        """The same forward with parameter-sharded data parallelism: every unit (embedding, block, final norm + head)
        runs inside ``param_sharder.run``, which gathers its weights and hooks its backward."""
        sh, gc = self.param_sharder, self.gradient_checkpointing
        h = sh.run(0, lambda: self.embed_tokens(input_ids)) if self.is_first_stage else input_ids
        res = None
        for i, layer in enumerate(self.layers):
            def block(h, res, layer=layer):
                if gc in ("selective", "swiglu") and torch.is_grad_enabled():
                    return layer(h, res, position_ids, cu_seqlens, max_seqlen, None, recompute=gc)
                if gc and torch.is_grad_enabled():
                    return checkpoint(layer, h, res, position_ids, cu_seqlens, max_seqlen, None, use_reentrant=False)
                return layer(h, res, position_ids, cu_seqlens, max_seqlen, None)
            h, res = sh.run(1 + i, block, h, res)
        return sh.run(len(self.layers) + 1,
                      lambda h, res: F.rms_norm(h, self.norm, self.args.norm_eps, residual=res)[0], h, res)

    def _head_unit(self):
        """(unit that holds the output head, whether its gradient reduction waits for a later use of the unit)."""
        sh = self.param_sharder
        if self.lm_head is None:                      # tied: the head is the embedding; reduce before the blocks run
            return sh.unit_of_param["embed_tokens.weight"], False
        return sh.unit_of_param["lm_head.weight"], True

    def attach_context_parallel(self, cp) -> None:
        """Inputs of ``forward`` become this rank's chunk of every sequence (``ContextParallel.shard``), with global
        position ids and local ``cu_seqlens``; only the attention layers communicate."""
        for layer in self.layers:
            layer.self_attn.cp = cp

    def logprobs(self, hidden: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0):
        """Per-token log-prob of ``labels`` and entropy from hidden states, through the fused lm_head kernel."""
        if self.tp is not None:
            return self.tp.vocab_parallel_logprob(hidden, self.lm_head_weight, labels, temperature)
        if self.param_sharder is not None:
            u, defer = self._head_unit()
            return self.param_sharder.run(
                u, lambda h: F.fused_logprob(h, self.lm_head_weight, labels, temperature), hidden, defer_reduce=defer)
        return F.fused_logprob(hidden, self.lm_head_weight, labels, temperature)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        if self.param_sharder is not None:
            u, defer = self._head_unit()
            return self.param_sharder.run(u, lambda h: _linear(h, self.lm_head_weight), hidden, defer_reduce=defer)
        out = _linear(hidden, self.lm_head_weight)
        return self.tp.gather_vocab(out) if self.tp is not None else out

    # ------------------------------------------------------------------ accounting
    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        """(parameter count, training FLOPs per token = 6N + attention term), cosmos_rl/policy/model/gpt/__init__.py:689-713."""
        a = self.args
        n = sum(p.numel() for p in self.parameters()) * a.tp_size
        n_embed = a.vocab_size * a.dim
        flops = 6 * (n - n_embed) + 12 * a.n_layers * a.n_heads * a.head_dim * seq_len
        return n, flops

    def check_tp_compatible(self, tp_size: int) -> None:
        a = self.args
        if a.n_heads % tp_size or a.ffn_dim % tp_size or (a.n_kv_heads % tp_size and tp_size % a.n_kv_heads):
            raise ValueError(f"tp_size={tp_size} incompatible with heads={a.n_heads}/{a.n_kv_heads}, ffn={a.ffn_dim}")

    def check_cp_compatible(self, cp_size: int, tp_size: int) -> None:
        if self.args.n_heads % (cp_size * tp_size):
            raise ValueError("n_heads must be divisible by cp_size * tp_size")

    def get_position_ids(self, cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
        pos = torch.arange(total, device=cu_seqlens.device)
        starts = torch.repeat_interleave(cu_seqlens[:-1], (cu_seqlens[1:] - cu_seqlens[:-1]))
        return pos - starts
