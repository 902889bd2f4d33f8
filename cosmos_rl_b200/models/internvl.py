"""Native InternVL: InternViT tiles -> pixel-shuffle projector -> Qwen2 decoder.

The reference carries this family with its own plans and weight map (cosmos_rl/policy/model/internvl/__init__.py:247).
As for :mod:`qwen2_5_vl`, the decoder IS :class:`GPT`; on top of it:

* the vision tower: every image is cut into square tiles by the processor; a tile becomes ``(size / patch)^2`` patch
  embeddings plus a class token with learned positions, and runs through pre-norm blocks (LayerNorm or RMSNorm,
  bidirectional attention, GELU MLP, learned per-channel scales on both residual branches);
* the projector: the class token is dropped, 2 x 2 neighbouring patches are folded into the channel axis ("pixel
  shuffle", ``downsample_ratio`` 0.5), then LayerNorm -> Linear -> GELU -> Linear to the decoder's width;
* the scatter of those tokens into the embedded prompt at the image placeholder id. Positions are ordinary 1-D ones.

``mm_inputs["pixel_values"]`` is ``[tiles, 3, size, size]`` for the whole packed batch, in prompt order.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import ModelRegistry
from .gpt import GPT, GPTArgs, GPTWeightMapper, _linear
from .qwen2_5_vl import _as_dict


@dataclass
class InternViTArgs:
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    image_size: int = 448
    patch_size: int = 14
    num_channels: int = 3
    norm_type: str = "layer_norm"        # or "rms_norm"
    layer_norm_eps: float = 1e-6
    attention_bias: bool = False
    use_qk_norm: bool = False
    layer_scale_init_value: float = 0.1

    @classmethod
    def from_hf(cls, v) -> "InternViTArgs":
        g = (lambda k, d=None: v.get(k, d)) if isinstance(v, dict) else (lambda k, d=None: getattr(v, k, d))
        base = cls()
        kw = {k: (g(k) if g(k) is not None else getattr(base, k)) for k in base.__dataclass_fields__}
        for k in ("image_size", "patch_size"):
            if isinstance(kw[k], (list, tuple)):
                kw[k] = int(kw[k][0])
        return cls(**kw)


@dataclass
class InternVLArgs(GPTArgs):
    vision: InternViTArgs = field(default_factory=InternViTArgs)
    downsample_ratio: float = 0.5
    image_token_id: int = 151667
    text_model_type: str = "qwen2"

    @classmethod
    def from_hf_config(cls, c, **over) -> "InternVLArgs":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        text = _as_dict(g("text_config") or {})
        base = GPTArgs.from_hf_config(dict(text, model_type=text.get("model_type", "qwen2")))
        a = cls(**{k: getattr(base, k) for k in GPTArgs.__dataclass_fields__})
        a.text_model_type = base.model_type
        a.model_type = "internvl"
        a.vision = InternViTArgs.from_hf(g("vision_config") or {})
        a.downsample_ratio = float(g("downsample_ratio", 0.5))
        a.image_token_id = g("image_token_id", 151667)
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
        v = self.vision
        vis = {k: getattr(v, k) for k in v.__dataclass_fields__}
        vis.update(image_size=[v.image_size, v.image_size], patch_size=[v.patch_size, v.patch_size], hidden_act="gelu",
                   model_type="internvl_vision", use_absolute_position_embeddings=True, use_mean_pooling=True)
        return {"architectures": ["InternVLForConditionalGeneration"], "model_type": "internvl", "text_config": text,
                "vision_config": vis, "downsample_ratio": self.downsample_ratio, "image_token_id": self.image_token_id,
                "projector_hidden_act": "gelu", "vision_feature_layer": -1, "vision_feature_select_strategy": "default",
                "vocab_size": self.vocab_size, "hidden_size": self.dim, "torch_dtype": "bfloat16"}


def _norm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    if b is None:
        return F.rms_norm(x, w, eps)[0]
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), w, b, eps)


class InternViTBlock(nn.Module):
    def __init__(self, v: InternViTArgs):
        super().__init__()
        H = v.hidden_size
        self.heads, self.d, self.eps, self.rms = v.num_attention_heads, H // v.num_attention_heads, v.layer_norm_eps, \
            v.norm_type == "rms_norm"
        self.norm1_w = nn.Parameter(torch.ones(H))
        self.norm2_w = nn.Parameter(torch.ones(H))
        self.norm1_b = None if self.rms else nn.Parameter(torch.zeros(H))
        self.norm2_b = None if self.rms else nn.Parameter(torch.zeros(H))
        self.q_proj = nn.Linear(H, H, bias=v.attention_bias)
        self.k_proj = nn.Linear(H, H, bias=v.attention_bias)
        self.v_proj = nn.Linear(H, H, bias=v.attention_bias)
        self.q_norm = nn.Parameter(torch.ones(H)) if v.use_qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(H)) if v.use_qk_norm else None
        self.proj = nn.Linear(H, H, bias=True)
        self.fc1 = nn.Linear(H, v.intermediate_size, bias=True)
        self.fc2 = nn.Linear(v.intermediate_size, H, bias=True)
        self.scale1 = nn.Parameter(torch.full((H,), v.layer_scale_init_value))
        self.scale2 = nn.Parameter(torch.full((H,), v.layer_scale_init_value))

    def forward(self, x: torch.Tensor, cu: torch.Tensor, max_len: int) -> torch.Tensor:
        N = x.shape[0]
        h = _norm(x, self.norm1_w, self.norm1_b, self.eps)
        q = _linear(h, self.q_proj.weight, self.q_proj.bias)
        k = _linear(h, self.k_proj.weight, self.k_proj.bias)
        v = _linear(h, self.v_proj.weight, self.v_proj.bias)
        if self.q_norm is not None:                       # normalised over the whole width, before the head split
            q, k = F.rms_norm(q, self.q_norm, 1e-6)[0], F.rms_norm(k, self.k_norm, 1e-6)[0]
        shp = (N, self.heads, self.d)
        o = F.full_attention(q.view(shp), k.view(shp), v.view(shp), cu, cu, max_len, max_len)
        x = x + self.scale1 * _linear(o.reshape(N, -1), self.proj.weight, self.proj.bias)
        h = _norm(x, self.norm2_w, self.norm2_b, self.eps)
        h = _linear(torch.nn.functional.gelu(_linear(h, self.fc1.weight, self.fc1.bias)), self.fc2.weight, self.fc2.bias)
        return x + self.scale2 * h


class InternViT(nn.Module):
    def __init__(self, v: InternViTArgs, out_dim: int, downsample_ratio: float):
        super().__init__()
        self.v, self.ratio = v, downsample_ratio
        self.grid = v.image_size // v.patch_size
        H = v.hidden_size
        self.patch_embed = nn.Linear(v.num_channels * v.patch_size * v.patch_size, H, bias=True)   # the convolution
        self.cls_token = nn.Parameter(torch.zeros(1, H))
        self.position_embeddings = nn.Parameter(torch.zeros(self.grid * self.grid + 1, H))
        self.blocks = nn.ModuleList([InternViTBlock(v) for _ in range(v.num_hidden_layers)])
        fold = int(round(1 / downsample_ratio)) ** 2
        self.proj_norm_w = nn.Parameter(torch.ones(H * fold))
        self.proj_norm_b = nn.Parameter(torch.zeros(H * fold))
        self.proj_fc1 = nn.Linear(H * fold, out_dim, bias=True)
        self.proj_fc2 = nn.Linear(out_dim, out_dim, bias=True)

    def _positions(self, g: int) -> torch.Tensor:
        """Learned positions for a ``g x g`` patch grid (bicubic resampling when the tiles are not the trained size)."""
        pe = self.position_embeddings
        if g == self.grid:
            return pe
        cls, patch = pe[:1], pe[1:].view(1, self.grid, self.grid, -1).permute(0, 3, 1, 2)
        patch = torch.nn.functional.interpolate(patch.float(), size=(g, g), mode="bicubic", align_corners=False)
        return torch.cat([cls, patch.permute(0, 2, 3, 1).reshape(g * g, -1).to(pe.dtype)])

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels [tiles, C, S, S]`` -> ``[tiles * (S / patch * ratio)^2, out_dim]`` in tile order, row-major."""
        v = self.v
        B, C, S, _ = pixels.shape
        p, g = v.patch_size, S // v.patch_size
        x = pixels.to(self.patch_embed.weight.dtype).view(B, C, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B * g * g, -1)
        x = _linear(x, self.patch_embed.weight, self.patch_embed.bias).view(B, g * g, -1)
        x = torch.cat([self.cls_token.expand(B, 1, -1), x], dim=1) + self._positions(g)[None]
        n = g * g + 1
        x = x.reshape(B * n, -1)
        cu = torch.arange(0, (B + 1) * n, n, dtype=torch.int32, device=x.device)
        for blk in self.blocks:
            x = blk(x, cu, n)
        x = x.view(B, n, -1)[:, 1:].reshape(B, g, g, -1)                       # drop the class token
        # fold 2 x 2 neighbours into the channels (same element order as the checkpoint's projector expects)
        r = self.ratio
        x = x.view(B, g, int(g * r), int(x.shape[-1] / r)).permute(0, 2, 1, 3).contiguous()
        x = x.view(B, int(g * r), int(g * r), int(x.shape[-1] / r)).permute(0, 2, 1, 3).contiguous()
        x = x.view(-1, x.shape[-1])
        x = torch.nn.functional.layer_norm(x, (x.shape[-1],), self.proj_norm_w, self.proj_norm_b, 1e-5)
        x = torch.nn.functional.gelu(_linear(x, self.proj_fc1.weight, self.proj_fc1.bias))
        return _linear(x, self.proj_fc2.weight, self.proj_fc2.bias)


class InternVLWeightMapper(GPTWeightMapper):
    TOWER = {"patch_embed": "embeddings.patch_embeddings.projection", "cls_token": "embeddings.cls_token",
             "position_embeddings": "embeddings.position_embeddings"}
    BLOCK = {"norm1_w": "layernorm_before.weight", "norm1_b": "layernorm_before.bias", "norm2_w": "layernorm_after.weight",
             "norm2_b": "layernorm_after.bias", "q_proj": "attention.q_proj", "k_proj": "attention.k_proj",
             "v_proj": "attention.v_proj", "q_norm": "attention.q_norm.weight", "k_norm": "attention.k_norm.weight",
             "proj": "attention.projection_layer", "fc1": "mlp.fc1", "fc2": "mlp.fc2", "scale1": "lambda_1",
             "scale2": "lambda_2"}
    PROJ = {"proj_norm_w": "layer_norm.weight", "proj_norm_b": "layer_norm.bias", "proj_fc1": "linear_1",
            "proj_fc2": "linear_2"}

    def hf_names(self, local: str) -> List[str]:
        if not local.startswith("visual."):
            return [n if n.startswith("lm_head") else "model.language_model." + n[len("model."):]
                    for n in super().hf_names(local)]
        name = local[len("visual."):]
        head, _, rest = name.partition(".")
        if head in self.PROJ:
            return ["model.multi_modal_projector." + self.PROJ[head] + ("." + rest if rest else "")]
        if head in self.TOWER:
            return ["model.vision_tower." + self.TOWER[head] + ("." + rest if rest else "")]
        idx, _, tail = rest.partition(".")                 # blocks.<i>.<field>[.weight|.bias]
        field_, _, leaf = tail.partition(".")
        return [f"model.vision_tower.encoder.layer.{idx}." + self.BLOCK[field_] + ("." + leaf if leaf else "")]

    def load_param(self, name, p, read, available, tp, r) -> bool:
        from .hf_io import _tp_slice
        hf = self.hf_names(name)
        if not all(h in available for h in hf):
            if name.startswith("lm_head") and "model.language_model.embed_tokens.weight" in available:
                hf = ["model.language_model.embed_tokens.weight"]
            else:
                return False
        cfg = _as_dict(_as_dict(getattr(self, "config", None) or {}).get("text_config") or {})
        parts = []
        for h in hf:
            t = read(h)
            if name.startswith("visual."):
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
        v = InternViTArgs.from_hf(_as_dict(getattr(self, "config", None) or {}).get("vision_config") or {})
        if name == "visual.patch_embed.weight":           # stored as a 2-D convolution
            return t.reshape(t.shape[0], v.num_channels, v.patch_size, v.patch_size)
        if name == "visual.cls_token":
            return t.reshape(1, 1, -1)
        if name == "visual.position_embeddings":
            return t.reshape(1, t.shape[0], t.shape[1])
        return t


@ModelRegistry.register(InternVLWeightMapper)
class InternVL(GPT):
    is_vlm = True
    paged_engine = False     # rollouts re-run the packed forward (no vision prefill in the paged engine)

    def __init__(self, args: InternVLArgs):
        saved, args.model_type = args.model_type, args.text_model_type       # the decoder is built as its own family
        try:
            super().__init__(args)
        finally:
            args.model_type = saved
        self.visual = InternViT(args.vision, args.dim, args.downsample_ratio) if self.is_first_stage else None
        self.mm_inputs: Dict[str, Any] = {}

    @staticmethod
    def supported_model_types():
        return ["internvl"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(InternVLArgs.from_hf_config(hf_config, **kw))

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = super().embed(input_ids)
        px = (self.mm_inputs or {}).get("pixel_values")
        if px is None or px.numel() == 0:
            return h
        feats = self.visual(px.to(h.device))
        mask = input_ids == self.args.image_token_id
        if int(mask.sum()) != feats.shape[0]:
            raise ValueError(f"{int(mask.sum())} placeholder tokens but {feats.shape[0]} vision tokens")
        return h.masked_scatter(mask[:, None], feats.to(h.dtype))

    def shard_parts(self, flat):
        """The decoder's parts plus every vision tensor whole (the tower is replicated over tensor-parallel ranks)."""
        from ..parallel.reshard import Part, gpt_parts
        mapper = InternVLWeightMapper({"model_type": "internvl"})
        mapper.layer_offset, mapper.layer_map = self.layer_offset, self.layer_map
        dec = copy.copy(flat)
        dec.params = [(n, p) for n, p in flat.params if not n.startswith("visual.")]
        parts = gpt_parts(self, dec)
        for name, p in flat.params:
            if name.startswith("visual."):
                slot = flat.by_name[name]
                rows, cols = (1, p.numel()) if p.dim() == 1 else (p.shape[0], p.numel() // p.shape[0])
                parts.append(Part(mapper.hf_names(name)[0], 0, rows, 0, cols, slot.offset, cols, bool(p.requires_grad)))
        return parts


def _named(**kw) -> InternVLArgs:
    vision = kw.pop("vision")
    a = InternVLArgs(**kw)
    a.vision = vision
    return a


ARCHS: Dict[str, InternVLArgs] = {
    "tiny-internvl": _named(vocab_size=32000, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=688, rope_theta=1e6,
                            qkv_bias=True, model_type="internvl", image_token_id=31990,
                            vision=InternViTArgs(hidden_size=64, num_hidden_layers=2, num_attention_heads=2,
                                                 intermediate_size=128, image_size=56, patch_size=14)),
}
