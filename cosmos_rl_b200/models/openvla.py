"""Native OpenVLA: one or two image featurizers -> MLP projector -> Llama decoder, actions as the last 256 token ids.

The reference wraps the published remote-code model (cosmos_rl/policy/model/vla/__init__.py:63-999 around
``openvla/modeling_prismatic.py``). Here the decoder IS :class:`GPT` (packed sequences, the fused kernels, tensor
parallelism, weight sync); on top of it:

* the featurizers: plain vision transformers in the layout of the ``timm`` checkpoints the published weights carry
  (patch convolution, learned positions, optional class and register tokens in front, pre-LayerNorm blocks with a fused
  qkv projection, optional per-channel layer scale, GELU MLP). The patch tokens are taken after the SECOND-TO-LAST block,
  unnormalised, as the published model does; with two featurizers (DINOv2 + SigLIP) the input carries six channels, each
  featurizer reads its three, and the two patch sequences are concatenated along the channel axis;
* the projector: ``Linear -> GELU -> Linear`` for one featurizer, ``Linear(4x) -> GELU -> Linear -> GELU -> Linear`` for
  the fused pair;
* the patch embeddings stand right after the first (BOS) token of every prompt; prompts carry ``image_token_id``
  placeholders there (``build_prompt``) and :meth:`embed` scatters the projected patches onto them;
* actions: dimension d of an action is one token; bin b of ``n_action_bins`` uniform bins over [-1, 1] is token
  ``vocab - 1 - b`` of the un-padded vocabulary; decoding maps a token to its bin centre and un-normalises with the data
  set's 1st / 99th percentiles (``norm_stats``), encoding is the inverse (:class:`ActionBins`);
* the OFT additions that are plain modules: a proprioceptive-state projector (one more prompt embedding) and an L1
  regression head that reads the decoder's hidden states at the action positions (:class:`L1ActionHead`).

``mm_inputs["pixel_values"]`` is ``[images, 3 * featurizers, S, S]`` for the whole packed batch, in prompt order.
Not carried over: the last block, the final norm and the pooling head of each featurizer are never run, so they are
not instantiated and an export leaves them out (the published loader accepts their absence only with
``strict=False``); FiLM conditioning and the diffusion head of OFT.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import ModelRegistry
from .gpt import GPT, GPTArgs, GPTWeightMapper, _linear
from .qwen2_5_vl import _as_dict


@dataclass
class ViTArgs:
    embed_dim: int = 1024
    depth: int = 24
    num_heads: int = 16
    mlp_dim: int = 4096
    image_size: int = 224
    patch_size: int = 14
    class_token: bool = True
    reg_tokens: int = 0
    pos_embed_has_cls: bool = False      # positions cover the class token too (plain ViT) or the patches only
    layer_scale: bool = False
    act: str = "gelu"                    # "gelu" | "gelu_tanh"
    eps: float = 1e-6

    @classmethod
    def from_dict(cls, d) -> "ViTArgs":
        d = _as_dict(d)
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


# geometry of the featurizers the published checkpoints name (``timm_model_ids`` of the config)
TIMM_GEOMETRY: Dict[str, Dict[str, Any]] = {
    "vit_large_patch14_reg4_dinov2.lvd142m": dict(embed_dim=1024, depth=24, num_heads=16, mlp_dim=4096, class_token=True,
                                                  reg_tokens=4, layer_scale=True),
    "vit_so400m_patch14_siglip_224": dict(embed_dim=1152, depth=27, num_heads=16, mlp_dim=4304, class_token=False),
    "vit_so400m_patch14_siglip_384": dict(embed_dim=1152, depth=27, num_heads=16, mlp_dim=4304, class_token=False),
    "vit_large_patch14_clip_224.openai": dict(embed_dim=1024, depth=24, num_heads=16, mlp_dim=4096, class_token=True,
                                              pos_embed_has_cls=True),
}


@dataclass
class OpenVLAArgs(GPTArgs):
    towers: List[ViTArgs] = field(default_factory=list)
    image_token_id: int = 32000          # the pad token of the published tokenizer: never part of a real prompt
    n_action_bins: int = 256
    pad_to_multiple_of: int = 64         # rows added to the embedding table; the action ids count from the un-padded end
    norm_stats: Dict[str, Any] = field(default_factory=dict)
    proprio_dim: int = 0                 # > 0: the OFT state projector
    action_head: bool = False            # the OFT L1 regression head
    action_dim: int = 7
    action_chunk: int = 1
    text_model_type: str = "llama"
    timm_model_ids: List[str] = field(default_factory=list)

    @classmethod
    def from_hf_config(cls, c, **over) -> "OpenVLAArgs":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        text = _as_dict(g("text_config") or {})
        base = GPTArgs.from_hf_config(dict(text, model_type=text.get("model_type", "llama")))
        a = cls(**{k: getattr(base, k) for k in GPTArgs.__dataclass_fields__})
        a.text_model_type, a.model_type = base.model_type, "openvla"
        ids = list(g("timm_model_ids") or [])
        sizes = list(g("image_sizes") or [224] * max(1, len(ids)))
        acts = list(g("timm_override_act_layers") or [None] * len(ids))
        if g("vision_towers"):
            a.towers = [ViTArgs.from_dict(t) for t in g("vision_towers")]
        else:
            if not ids:
                raise ValueError("an openvla config needs timm_model_ids or explicit vision_towers")
            if not g("use_fused_vision_backbone", len(ids) > 1):
                ids = ids[:1]
            for i, name in enumerate(ids):
                if name not in TIMM_GEOMETRY:
                    raise ValueError(f"unknown featurizer {name!r}: give its geometry under 'vision_towers' "
                                     f"(known: {sorted(TIMM_GEOMETRY)})")
                kw = dict(TIMM_GEOMETRY[name], image_size=int(sizes[i]))
                if i < len(acts) and acts[i]:
                    kw["act"] = acts[i]
                a.towers.append(ViTArgs(**kw))
        a.timm_model_ids = ids
        for k in ("image_token_id", "n_action_bins", "pad_to_multiple_of", "proprio_dim", "action_head", "action_dim",
                  "action_chunk"):
            if g(k) is not None:
                setattr(a, k, g(k))
        a.norm_stats = dict(g("norm_stats") or {})
        for k, v in over.items():
            setattr(a, k, v)
        a.__post_init__()
        return a

    def to_hf_config(self) -> Dict[str, Any]:
        saved, self.model_type = self.model_type, self.text_model_type
        try:
            text = GPTArgs.to_hf_config(self)
        finally:
            self.model_type = saved
        text.pop("architectures", None)
        return {"architectures": ["OpenVLAForActionPrediction"], "model_type": "openvla", "text_config": text,
                "timm_model_ids": list(self.timm_model_ids), "image_sizes": [t.image_size for t in self.towers],
                "use_fused_vision_backbone": len(self.towers) > 1,
                "vision_towers": [{k: getattr(t, k) for k in t.__dataclass_fields__} for t in self.towers],
                "image_token_id": self.image_token_id, "n_action_bins": self.n_action_bins,
                "pad_to_multiple_of": self.pad_to_multiple_of, "norm_stats": self.norm_stats,
                "proprio_dim": self.proprio_dim, "action_head": self.action_head, "action_dim": self.action_dim,
                "action_chunk": self.action_chunk, "pad_token_id": self.image_token_id, "torch_dtype": "bfloat16"}


# ---------------------------------------------------------------------------------------------------
# featurizer
# ---------------------------------------------------------------------------------------------------
class ViTBlock(nn.Module):
    def __init__(self, v: ViTArgs):
        super().__init__()
        D = v.embed_dim
        self.heads, self.d, self.eps, self.tanh = v.num_heads, D // v.num_heads, v.eps, v.act == "gelu_tanh"
        self.norm1 = nn.LayerNorm(D, eps=v.eps)
        self.qkv = nn.Linear(D, 3 * D, bias=True)
        self.proj = nn.Linear(D, D, bias=True)
        self.norm2 = nn.LayerNorm(D, eps=v.eps)
        self.fc1 = nn.Linear(D, v.mlp_dim, bias=True)
        self.fc2 = nn.Linear(v.mlp_dim, D, bias=True)
        self.ls1 = nn.Parameter(torch.ones(D)) if v.layer_scale else None
        self.ls2 = nn.Parameter(torch.ones(D)) if v.layer_scale else None

    def forward(self, x: torch.Tensor, cu: torch.Tensor, max_len: int) -> torch.Tensor:
        N = x.shape[0]
        h = torch.nn.functional.layer_norm(x, (x.shape[-1],), self.norm1.weight, self.norm1.bias, self.eps)
        q, k, v = _linear(h, self.qkv.weight, self.qkv.bias).view(N, 3, self.heads, self.d).unbind(1)
        o = F.full_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, max_len, max_len)
        o = _linear(o.reshape(N, -1), self.proj.weight, self.proj.bias)
        x = x + (o * self.ls1 if self.ls1 is not None else o)
        h = torch.nn.functional.layer_norm(x, (x.shape[-1],), self.norm2.weight, self.norm2.bias, self.eps)
        h = torch.nn.functional.gelu(_linear(h, self.fc1.weight, self.fc1.bias), approximate="tanh" if self.tanh else "none")
        h = _linear(h, self.fc2.weight, self.fc2.bias)
        return x + (h * self.ls2 if self.ls2 is not None else h)


class ViTFeaturizer(nn.Module):
    """Patch tokens after block ``depth - 2`` (the last block is never needed, so it is not built)."""

    def __init__(self, v: ViTArgs):
        super().__init__()
        self.v = v
        self.grid = v.image_size // v.patch_size
        D = v.embed_dim
        self.patch_embed = nn.Linear(3 * v.patch_size * v.patch_size, D, bias=True)          # the convolution
        self.cls_token = nn.Parameter(torch.zeros(1, D)) if v.class_token else None
        self.reg_token = nn.Parameter(torch.zeros(v.reg_tokens, D)) if v.reg_tokens else None
        n_pos = self.grid * self.grid + (1 if (v.class_token and v.pos_embed_has_cls) else 0)
        self.pos_embed = nn.Parameter(torch.zeros(n_pos, D))
        self.blocks = nn.ModuleList([ViTBlock(v) for _ in range(v.depth - 1)])

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels [B, 3, S, S]`` -> ``[B, (S / patch)^2, embed_dim]``."""
        v = self.v
        B, C, S, _ = pixels.shape
        p, g = v.patch_size, S // v.patch_size
        if g != self.grid:
            raise ValueError(f"the featurizer was built for {v.image_size}-pixel images, got {S}")
        x = pixels.to(self.patch_embed.weight.dtype).view(B, C, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B * g * g, -1)
        x = _linear(x, self.patch_embed.weight, self.patch_embed.bias).view(B, g * g, -1)
        prefix = []
        if self.cls_token is not None:
            prefix.append(self.cls_token.expand(B, 1, -1))
        if v.class_token and v.pos_embed_has_cls:
            x = torch.cat([prefix.pop(), x], dim=1) + self.pos_embed[None]
        else:
            x = x + self.pos_embed[None]
        if self.reg_token is not None:
            prefix.append(self.reg_token.expand(B, -1, -1))
        if prefix:
            x = torch.cat(prefix + [x], dim=1)
        n = x.shape[1]
        n_prefix = n - g * g
        x = x.reshape(B * n, -1)
        cu = torch.arange(0, (B + 1) * n, n, dtype=torch.int32, device=x.device)
        for blk in self.blocks:
            x = blk(x, cu, n)
        return x.view(B, n, -1)[:, n_prefix:]


class VisionBackbone(nn.Module):
    def __init__(self, towers: Sequence[ViTArgs]):
        super().__init__()
        if not 1 <= len(towers) <= 2:
            raise ValueError("one featurizer, or two fused ones")
        self.featurizer = ViTFeaturizer(towers[0])
        self.fused_featurizer = ViTFeaturizer(towers[1]) if len(towers) == 2 else None
        self.embed_dim = sum(t.embed_dim for t in towers)
        if self.fused_featurizer is not None and self.fused_featurizer.grid != self.featurizer.grid:
            raise ValueError("fused featurizers must produce the same number of patches")

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        if self.fused_featurizer is None:
            return self.featurizer(pixels[:, :3])
        return torch.cat([self.featurizer(pixels[:, :3]), self.fused_featurizer(pixels[:, 3:6])], dim=2)


class Projector(nn.Module):
    def __init__(self, fused: bool, vision_dim: int, llm_dim: int):
        super().__init__()
        if fused:
            self.fc1 = nn.Linear(vision_dim, 4 * vision_dim, bias=True)
            self.fc2 = nn.Linear(4 * vision_dim, llm_dim, bias=True)
            self.fc3 = nn.Linear(llm_dim, llm_dim, bias=True)
        else:
            self.fc1 = nn.Linear(vision_dim, llm_dim, bias=True)
            self.fc2 = nn.Linear(llm_dim, llm_dim, bias=True)
            self.fc3 = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = torch.nn.functional.gelu(_linear(x, self.fc1.weight, self.fc1.bias))
        x = _linear(x, self.fc2.weight, self.fc2.bias)
        if self.fc3 is not None:
            x = _linear(torch.nn.functional.gelu(x), self.fc3.weight, self.fc3.bias)
        return x


class ProprioProjector(nn.Module):
    """Robot state -> one embedding in the decoder's space (cosmos_rl/policy/model/vla/openvla_oft/modeling_prismatic.py:62-81)."""

    def __init__(self, llm_dim: int, proprio_dim: int):
        super().__init__()
        self.fc1 = nn.Linear(proprio_dim, llm_dim, bias=True)
        self.fc2 = nn.Linear(llm_dim, llm_dim, bias=True)

    def forward(self, s: torch.Tensor) -> torch.Tensor:
        return self.fc2(torch.nn.functional.gelu(self.fc1(s)))


class L1ActionHead(nn.Module):
    """Continuous actions from the decoder's hidden states at the ``action_chunk * action_dim`` action positions: the
    ``action_dim`` states of one control step are concatenated, then LayerNorm -> Linear -> ReLU -> two pre-norm
    residual blocks -> LayerNorm -> Linear to ``action_dim``; trained with an L1 loss against normalised actions."""

    def __init__(self, llm_dim: int, action_dim: int, hidden: Optional[int] = None, n_blocks: int = 2):
        super().__init__()
        hidden = hidden or llm_dim
        self.action_dim = action_dim
        self.norm_in = nn.LayerNorm(llm_dim * action_dim)
        self.fc_in = nn.Linear(llm_dim * action_dim, hidden)
        self.blocks = nn.ModuleList([nn.Sequential(nn.LayerNorm(hidden), nn.Linear(hidden, hidden), nn.ReLU())
                                     for _ in range(n_blocks)])
        self.norm_out = nn.LayerNorm(hidden)
        self.fc_out = nn.Linear(hidden, action_dim)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """``h [B, chunk * action_dim, llm_dim]`` -> ``[B, chunk, action_dim]``."""
        B, n, D = h.shape
        x = h.reshape(B, n // self.action_dim, self.action_dim * D)
        x = torch.relu(self.fc_in(self.norm_in(x)))
        for blk in self.blocks:
            x = x + blk(x)
        return self.fc_out(self.norm_out(x))

    def l1_loss(self, h: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return (self(h).float() - target.float()).abs().mean()


# ---------------------------------------------------------------------------------------------------
# actions <-> tokens
# ---------------------------------------------------------------------------------------------------
class ActionBins:
    """Uniform bins over [-1, 1]; bin ``b`` (1-based, ``numpy.digitize`` convention) is token ``vocab - b`` where
    ``vocab`` is the tokenizer's un-padded size, so the bins occupy the LAST ids of the vocabulary. Decoding returns
    the bin centre (255 centres for 256 edges) and un-normalises dimensions whose mask is set with the data set's
    q01 / q99 (cosmos_rl/policy/model/vla/openvla/modeling_prismatic.py:574-625)."""

    def __init__(self, vocab_size: int, n_bins: int = 256, norm_stats: Optional[Dict[str, Any]] = None):
        self.vocab, self.n_bins = vocab_size, n_bins
        self.edges = torch.linspace(-1.0, 1.0, n_bins, device="cpu")      # models are built under the meta device
        self.centers = (self.edges[:-1] + self.edges[1:]) / 2.0
        self.norm_stats = norm_stats or {}

    def _stats(self, key: Optional[str]):
        if not self.norm_stats:
            return None
        if key is None:
            if len(self.norm_stats) != 1:
                raise ValueError(f"several data sets' statistics are loaded, name one of {sorted(self.norm_stats)}")
            key = next(iter(self.norm_stats))
        if key not in self.norm_stats:
            raise KeyError(f"no statistics for {key!r}; known: {sorted(self.norm_stats)}")
        s = self.norm_stats[key]
        return s.get("action", s)

    def action_dim(self, key: Optional[str] = None) -> int:
        s = self._stats(key)
        if s is None:
            raise ValueError("the action dimension comes from norm_stats, which this model does not carry")
        return len(s["q01"])

    def normalize(self, actions: torch.Tensor, key: Optional[str] = None) -> torch.Tensor:
        s = self._stats(key)
        if s is None:
            return actions
        lo, hi = torch.tensor(s["q01"], dtype=torch.float32), torch.tensor(s["q99"], dtype=torch.float32)
        mask = torch.tensor(s.get("mask", [True] * len(s["q01"])), dtype=torch.bool)
        norm = 2.0 * (actions - lo) / (hi - lo).clamp_min(1e-8) - 1.0
        return torch.where(mask, norm, actions)

    def unnormalize(self, norm: torch.Tensor, key: Optional[str] = None) -> torch.Tensor:
        s = self._stats(key)
        if s is None:
            return norm
        lo, hi = torch.tensor(s["q01"], dtype=torch.float32), torch.tensor(s["q99"], dtype=torch.float32)
        mask = torch.tensor(s.get("mask", [True] * len(s["q01"])), dtype=torch.bool)
        return torch.where(mask, 0.5 * (norm + 1.0) * (hi - lo) + lo, norm)

    def encode(self, actions: torch.Tensor, key: Optional[str] = None) -> torch.Tensor:
        """Actions (data-set units) -> token ids, same shape."""
        x = self.normalize(actions.float(), key).clamp(-1.0, 1.0)
        b = torch.bucketize(x, self.edges, right=True)              # numpy.digitize: 1 .. n_bins
        return self.vocab - b

    def decode(self, tokens: torch.Tensor, key: Optional[str] = None) -> torch.Tensor:
        b = (self.vocab - tokens.long() - 1).clamp(0, self.centers.numel() - 1)
        return self.unnormalize(self.centers[b], key)


def build_prompt(text_ids: Sequence[int], n_patches: int, image_token_id: int, extra: int = 0) -> List[int]:
    """``[bos] + placeholders for the patches (+ ``extra`` further embeddings such as the state) + the rest``: the
    layout the published model builds by splicing the patch embeddings in after the first token."""
    ids = list(text_ids)
    return ids[:1] + [image_token_id] * (n_patches + extra) + ids[1:]


# ---------------------------------------------------------------------------------------------------
class OpenVLAWeightMapper(GPTWeightMapper):
    """Checkpoint names of the published model: ``language_model.{model.*, lm_head.*}``, ``projector.fc{1,2,3}``,
    ``vision_backbone.{featurizer,fused_featurizer}.*`` in timm's naming (``patch_embed.proj`` is a convolution,
    ``pos_embed`` / ``cls_token`` / ``reg_token`` carry a leading batch axis, layer scale is ``ls{1,2}.scale_factor``)."""
    BLOCK = {"fc1": "mlp.fc1", "fc2": "mlp.fc2", "qkv": "attn.qkv", "proj": "attn.proj", "ls1": "ls1.scale_factor",
             "ls2": "ls2.scale_factor"}

    def hf_names(self, local: str) -> List[str]:
        if local.startswith("visual."):
            tower, _, rest = local[len("visual."):].partition(".")
            head, _, tail = rest.partition(".")
            if head == "patch_embed":
                rest = "patch_embed.proj." + tail
            elif head == "blocks":
                idx, _, leaf = tail.partition(".")
                f, _, wb = leaf.partition(".")
                rest = f"blocks.{idx}." + self.BLOCK.get(f, f) + ("." + wb if wb else "")
            return [f"vision_backbone.{tower}.{rest}"]
        if local.startswith(("projector.", "proprio_projector.", "action_head.")):
            return [local]
        return ["language_model." + n for n in super().hf_names(local)]

    def load_param(self, name, p, read, available, tp, r) -> bool:
        from .hf_io import _tp_slice
        hf = self.hf_names(name)
        if not all(h in available for h in hf):
            return False
        cfg = _as_dict(_as_dict(getattr(self, "config", None) or {}).get("text_config") or {})
        parts = []
        for h in hf:
            t = read(h)
            if name.startswith(("visual.", "projector.", "proprio_projector.", "action_head.")):
                t = t.reshape(p.shape) if t.numel() == p.numel() else t
            else:
                t = _tp_slice(h, t, tp, r, cfg)
            parts.append(t)
        t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != model shape {tuple(p.shape)}")
        p.copy_(t.to(p.dtype))
        return True

    def export_tensor(self, name: str, t: torch.Tensor) -> torch.Tensor:
        if not name.startswith("visual."):
            return t
        towers = _as_dict(getattr(self, "config", None) or {}).get("vision_towers") or []
        idx = 1 if ".fused_featurizer." in "." + name else 0
        if name.endswith("patch_embed.weight"):              # stored as a 2-D convolution
            ps = int(_as_dict(towers[idx]).get("patch_size", 14)) if idx < len(towers) else 14
            return t.reshape(t.shape[0], 3, ps, ps)
        if name.endswith((".pos_embed", ".cls_token", ".reg_token")):
            return t.reshape(1, *t.shape)
        return t


@ModelRegistry.register(OpenVLAWeightMapper)
class OpenVLA(GPT):
    is_vlm = True
    paged_engine = False     # rollouts re-run the packed forward (no vision prefill in the paged engine)

    def __init__(self, args: OpenVLAArgs):
        saved, args.model_type = args.model_type, args.text_model_type       # the decoder is built as its own family
        try:
            super().__init__(args)
        finally:
            args.model_type = saved
        first = self.is_first_stage
        self.visual = VisionBackbone(args.towers) if first else None
        self.projector = Projector(len(args.towers) > 1, sum(t.embed_dim for t in args.towers), args.dim) if first else None
        self.proprio_projector = ProprioProjector(args.dim, args.proprio_dim) if (first and args.proprio_dim) else None
        self.action_head = L1ActionHead(args.dim, args.action_dim) if (args.action_head and self.is_last_stage) else None
        self.mm_inputs: Dict[str, Any] = {}
        self.bins = ActionBins(args.vocab_size - args.pad_to_multiple_of, args.n_action_bins, args.norm_stats)

    @staticmethod
    def supported_model_types():
        return ["openvla"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(OpenVLAArgs.from_hf_config(hf_config, **kw))

    @property
    def n_patches(self) -> int:
        g = self.args.towers[0].image_size // self.args.towers[0].patch_size
        return g * g

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        super().init_weights(seed)
        g = torch.Generator(device="cpu").manual_seed(seed + 17)
        with torch.no_grad():
            for top in ("visual", "projector", "proprio_projector", "action_head"):
                mod = getattr(self, top, None)
                for name, p in (mod.named_parameters() if mod is not None else ()):
                    leaf = name.rsplit(".", 1)[-1]
                    if leaf in ("ls1", "ls2"):
                        p.fill_(0.1)
                    elif p.dim() == 1 and "norm" in name:
                        p.fill_(1.0) if leaf == "weight" else p.zero_()
                    elif p.dim() == 1:
                        p.zero_()
                    else:
                        p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std).to(p.dtype))

    init_weights_on_device = init_weights

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = super().embed(input_ids)
        mm = self.mm_inputs or {}
        px = mm.get("pixel_values")
        if px is None or px.numel() == 0:
            return h
        feats = self.projector(self.visual(px.to(h.device)))                       # [images, patches, dim]
        if self.proprio_projector is not None and mm.get("proprio") is not None:
            state = self.proprio_projector(mm["proprio"].to(h.device, feats.dtype))
            feats = torch.cat([feats, state[:, None]], dim=1)
        feats = feats.reshape(-1, feats.shape[-1])
        mask = input_ids == self.args.image_token_id
        if int(mask.sum()) != feats.shape[0]:
            raise ValueError(f"{int(mask.sum())} placeholder tokens but {feats.shape[0]} vision embeddings")
        return h.masked_scatter(mask[:, None], feats.to(h.dtype))

    def decode_actions(self, tokens: torch.Tensor, unnorm_key: Optional[str] = None) -> torch.Tensor:
        return self.bins.decode(tokens.cpu(), unnorm_key)

    # ------------------------------------------------------------------ the policy over action tokens
    @property
    def action_token_range(self) -> Tuple[int, int]:
        """``[lo, hi)``: the ids of the action bins (the last ``n_action_bins`` of the un-padded vocabulary)."""
        hi = self.args.vocab_size - self.args.pad_to_multiple_of
        return hi - self.args.n_action_bins, hi

    def action_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Logits over the action bins only (``[N, n_action_bins]``, column j = token ``lo + j``): RL samples and scores
        actions under this restricted distribution, so no probability mass sits on text tokens."""
        lo, hi = self.action_token_range
        return _linear(hidden, self.lm_head_weight[lo:hi]).float()

    def logprobs(self, hidden: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0):
        """With ``action_only_logprobs`` set (the action-token RL trainer does): log-probability and entropy under the
        softmax over the action bins; otherwise the decoder's full-vocabulary path."""
        if not getattr(self, "action_only_logprobs", False):
            return super().logprobs(hidden, labels, temperature)
        lo, hi = self.action_token_range
        lsm = torch.log_softmax(self.action_logits(hidden) / float(temperature), dim=-1)
        idx = (labels.long() - lo).clamp(0, hi - lo - 1)
        return lsm.gather(1, idx[:, None])[:, 0], -(lsm.exp() * lsm).sum(-1)

    def shard_parts(self, flat):
        """The decoder's parts plus every other tensor whole (featurizers, projectors and the action head are
        replicated over tensor-parallel ranks)."""
        from ..parallel.reshard import Part, gpt_parts
        mapper = OpenVLAWeightMapper({"model_type": "openvla"})
        mapper.layer_offset, mapper.layer_map = self.layer_offset, self.layer_map
        extra = ("visual.", "projector.", "proprio_projector.", "action_head.")
        dec = copy.copy(flat)
        dec.params = [(n, p) for n, p in flat.params if not n.startswith(extra)]
        parts = gpt_parts(self, dec)
        for name, p in flat.params:
            if name.startswith(extra):
                slot = flat.by_name[name]
                rows, cols = (1, p.numel()) if p.dim() == 1 else (p.shape[0], p.numel() // p.shape[0])
                parts.append(Part(mapper.hf_names(name)[0], 0, rows, 0, cols, slot.offset, cols, bool(p.requires_grad)))
        return parts


def _named(**kw) -> OpenVLAArgs:
    towers = kw.pop("towers")
    a = OpenVLAArgs(**kw)
    a.towers = towers
    return a


_STATS = {"demo": {"action": {"q01": [-1.0, -0.5, 0.0], "q99": [1.0, 0.5, 2.0], "mask": [True, True, False]}}}

ARCHS: Dict[str, OpenVLAArgs] = {
    "tiny-openvla": _named(vocab_size=32064, dim=256, n_layers=2, n_heads=4, n_kv_heads=4, ffn_dim=688, rope_theta=1e4, qkv_bias=False,
                           model_type="openvla", text_model_type="llama", image_token_id=32000, norm_stats=_STATS,
                           action_dim=3,
                           towers=[ViTArgs(embed_dim=64, depth=3, num_heads=2, mlp_dim=128, image_size=56, patch_size=14,
                                           class_token=True, reg_tokens=4, layer_scale=True),
                                   ViTArgs(embed_dim=96, depth=3, num_heads=2, mlp_dim=160, image_size=56, patch_size=14,
                                           class_token=False)]),
    "openvla-7b": _named(vocab_size=32064, dim=4096, n_layers=32, n_heads=32, n_kv_heads=32, ffn_dim=11008, qkv_bias=False,
                         rope_theta=1e4, model_type="openvla", text_model_type="llama", image_token_id=32000,
                         timm_model_ids=["vit_large_patch14_reg4_dinov2.lvd142m", "vit_so400m_patch14_siglip_224"],
                         towers=[ViTArgs(image_size=224, **TIMM_GEOMETRY["vit_large_patch14_reg4_dinov2.lvd142m"]),
                                 ViTArgs(image_size=224, **TIMM_GEOMETRY["vit_so400m_patch14_siglip_224"])]),
}
