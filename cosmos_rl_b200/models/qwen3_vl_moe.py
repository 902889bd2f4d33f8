"""Native Qwen3-VL-MoE: vision tower with deep-stack taps -> Qwen3-MoE decoder with interleaved multimodal rotary positions.

The reference carries this family natively (cosmos_rl/policy/model/qwen3_vl_moe/__init__.py:356). The decoder IS
:class:`Qwen3MoE` (same router, stacked experts, expert-parallel exchange, weight-sync parts per expert); added here:

* the vision tower: patches -> linear patch embedding (a 3-D convolution in the checkpoint) + learned position table
  resampled bilinearly to the image's grid -> LayerNorm blocks with 2-D rotary attention over whole frames and a
  tanh-GELU MLP -> a merger (LayerNorm per patch, 2 x 2 fold, two linears);
* deep-stack taps: after chosen tower blocks a second kind of merger (2 x 2 fold first, then LayerNorm) produces one
  feature per image token, and the k-th tap is ADDED to the residual stream behind decoder block k at the image
  positions;
* multimodal rotary positions in the interleaved layout (frequencies 1, 4, 7, ... follow height, 2, 5, 8, ... width).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import ModelRegistry
from .gpt import _linear
from .qwen2_5_vl import _as_dict, apply_rotary, mrope_positions
from .qwen3_moe import Qwen3MoE, Qwen3MoEArgs, Qwen3MoEBlock, Qwen3MoEWeightMapper


@dataclass
class Qwen3VisionArgs:
    depth: int = 27
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    out_hidden_size: int = 2048
    patch_size: int = 16
    temporal_patch_size: int = 2
    in_channels: int = 3
    spatial_merge_size: int = 2
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: List[int] = field(default_factory=lambda: [8, 16, 24])

    @classmethod
    def from_hf(cls, v) -> "Qwen3VisionArgs":
        g = (lambda k, d=None: v.get(k, d)) if isinstance(v, dict) else (lambda k, d=None: getattr(v, k, d))
        base = cls()
        return cls(**{k: (g(k) if g(k) is not None else getattr(base, k)) for k in base.__dataclass_fields__})


@dataclass
class Qwen3VLMoEArgs(Qwen3MoEArgs):
    vision: Qwen3VisionArgs = field(default_factory=Qwen3VisionArgs)
    mrope_section: List[int] = field(default_factory=lambda: [24, 20, 20])
    image_token_id: int = 151655
    video_token_id: int = 151656

    @classmethod
    def from_hf_config(cls, c, **over) -> "Qwen3VLMoEArgs":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        text = _as_dict(g("text_config") or {})
        rope = text.get("rope_parameters") or text.get("rope_scaling") or {}
        base = Qwen3MoEArgs.from_hf_config(dict(text, rope_theta=rope.get("rope_theta", text.get("rope_theta", 5e6))))
        a = cls(**{k: getattr(base, k) for k in Qwen3MoEArgs.__dataclass_fields__})
        a.model_type = "qwen3_vl_moe"
        a.norm_topk_prob = True                             # the family always renormalises the top-k weights
        a.vision = Qwen3VisionArgs.from_hf(g("vision_config") or {})
        a.mrope_section = list(rope.get("mrope_section") or [24, 20, 20])
        a.image_token_id, a.video_token_id = g("image_token_id", 151655), g("video_token_id", 151656)
        a.tie_word_embeddings = bool(g("tie_word_embeddings", text.get("tie_word_embeddings", False)))
        for k, v in over.items():
            setattr(a, k, v)
        a.__post_init__()
        return a

    def to_hf_config(self) -> Dict[str, Any]:
        text = Qwen3MoEArgs.to_hf_config(self)
        text.pop("architectures", None)
        text.pop("rope_theta", None)
        text.update(model_type="qwen3_vl_moe_text", decoder_sparse_step=1, mlp_only_layers=[],
                    rope_parameters={"rope_type": "default", "rope_theta": self.rope_theta,
                                     "mrope_section": list(self.mrope_section), "mrope_interleaved": True})
        v = self.vision
        vis = {k: getattr(v, k) for k in v.__dataclass_fields__}
        vis.update(hidden_act="gelu_pytorch_tanh", model_type="qwen3_vl_moe")
        return {"architectures": ["Qwen3VLMoeForConditionalGeneration"], "model_type": "qwen3_vl_moe", "text_config": text,
                "vision_config": vis, "image_token_id": self.image_token_id, "video_token_id": self.video_token_id,
                "tie_word_embeddings": self.tie_word_embeddings, "torch_dtype": "bfloat16"}


def _layer_norm(x, w, b, eps: float = 1e-6):
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), w, b, eps)


class _Merger(nn.Module):
    """Folds 2 x 2 neighbouring patches into one token of the decoder's width. ``post``: normalise after the fold (the
    deep-stack taps) instead of per patch (the final merger)."""

    def __init__(self, v: Qwen3VisionArgs, post: bool):
        super().__init__()
        self.post, self.fold = post, v.hidden_size * v.spatial_merge_size ** 2
        n = self.fold if post else v.hidden_size
        self.norm_w, self.norm_b = nn.Parameter(torch.ones(n)), nn.Parameter(torch.zeros(n))
        self.fc1 = nn.Linear(self.fold, self.fold, bias=True)
        self.fc2 = nn.Linear(self.fold, v.out_hidden_size, bias=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = _layer_norm(x.view(-1, self.fold), self.norm_w, self.norm_b) if self.post else \
            _layer_norm(x, self.norm_w, self.norm_b).view(-1, self.fold)
        return _linear(torch.nn.functional.gelu(_linear(x, self.fc1.weight, self.fc1.bias)), self.fc2.weight, self.fc2.bias)


class Qwen3VisionBlock(nn.Module):
    def __init__(self, v: Qwen3VisionArgs):
        super().__init__()
        H = v.hidden_size
        self.heads, self.d = v.num_heads, H // v.num_heads
        self.norm1_w, self.norm1_b = nn.Parameter(torch.ones(H)), nn.Parameter(torch.zeros(H))
        self.norm2_w, self.norm2_b = nn.Parameter(torch.ones(H)), nn.Parameter(torch.zeros(H))
        self.qkv = nn.Linear(H, 3 * H, bias=True)
        self.proj = nn.Linear(H, H, bias=True)
        self.fc1 = nn.Linear(H, v.intermediate_size, bias=True)
        self.fc2 = nn.Linear(v.intermediate_size, H, bias=True)

    def forward(self, x, cos, sin, cu, max_len: int):
        N = x.shape[0]
        h = _layer_norm(x, self.norm1_w, self.norm1_b)
        q, k, v = _linear(h, self.qkv.weight, self.qkv.bias).view(N, 3, self.heads, self.d).unbind(1)
        q, k = apply_rotary(q, k, cos, sin)
        o = F.full_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, max_len, max_len)
        x = x + _linear(o.reshape(N, -1), self.proj.weight, self.proj.bias)
        h = _layer_norm(x, self.norm2_w, self.norm2_b)
        h = torch.nn.functional.gelu(_linear(h, self.fc1.weight, self.fc1.bias), approximate="tanh")
        return x + _linear(h, self.fc2.weight, self.fc2.bias)


class Qwen3VisionTower(nn.Module):
    def __init__(self, v: Qwen3VisionArgs):
        super().__init__()
        self.v = v
        self.patch_embed = nn.Linear(v.in_channels * v.temporal_patch_size * v.patch_size ** 2, v.hidden_size, bias=True)
        self.pos_embed = nn.Embedding(v.num_position_embeddings, v.hidden_size)
        self.side = int(round(v.num_position_embeddings ** 0.5))
        self.blocks = nn.ModuleList([Qwen3VisionBlock(v) for _ in range(v.depth)])
        self.merger = _Merger(v, post=False)
        self.deepstack = nn.ModuleList([_Merger(v, post=True) for _ in v.deepstack_visual_indexes])

    def _merge_order(self, t: int, h: int, w: int) -> torch.Tensor:
        """Row-major patch indices of one frame grid re-ordered so that 2 x 2 merge groups are contiguous."""
        m = self.v.spatial_merge_size
        idx = torch.arange(h * w).view(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
        return idx

    def _positions(self, grid: List[List[int]], device) -> torch.Tensor:
        """Learned positions for every patch: the trained ``side x side`` table read bilinearly at the grid points."""
        out = []
        tab = self.pos_embed.weight
        for t, h, w in grid:
            ys, xs = torch.linspace(0, self.side - 1, h), torch.linspace(0, self.side - 1, w)
            y0, x0 = ys.int(), xs.int()
            y1, x1 = (y0 + 1).clip(max=self.side - 1), (x0 + 1).clip(max=self.side - 1)
            dy, dx = (ys - y0)[:, None], (xs - x0)[None, :]
            corners = ((y0, x0, (1 - dy) * (1 - dx)), (y0, x1, (1 - dy) * dx), (y1, x0, dy * (1 - dx)), (y1, x1, dy * dx))
            pe = 0
            for yy, xx, wgt in corners:
                ids = (yy[:, None].long() * self.side + xx[None, :].long()).reshape(-1).to(device)
                pe = pe + tab[ids] * wgt.reshape(-1, 1).to(device, tab.dtype)
            pe = pe[self._merge_order(t, h, w).to(device)]
            out.append(pe.repeat(t, 1))
        return torch.cat(out)

    def _rotary(self, grid: List[List[int]], device):
        d_rot = (self.v.hidden_size // self.v.num_heads) // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, d_rot, 2, dtype=torch.float32) / d_rot))
        ang = []
        for t, h, w in grid:
            r = torch.arange(h)[:, None].expand(h, w).reshape(-1)[self._merge_order(t, h, w)].float()
            c = torch.arange(w)[None, :].expand(h, w).reshape(-1)[self._merge_order(t, h, w)].float()
            ang.append(torch.cat([r[:, None] * inv[None], c[:, None] * inv[None]], dim=-1).repeat(t, 1))
        ang = torch.cat(ang).to(device)
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos(), emb.sin()

    def forward(self, pixels: torch.Tensor, grid_thw: torch.Tensor) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        """-> (image tokens ``[N / merge^2, out_hidden]``, one deep-stack feature tensor of that shape per tap)."""
        grid = grid_thw.tolist()
        dev = pixels.device
        x = _linear(pixels.to(self.patch_embed.weight.dtype), self.patch_embed.weight, self.patch_embed.bias)
        x = x + self._positions(grid, dev)
        cos, sin = self._rotary(grid, dev)
        frames = [0]
        for t, h, w in grid:
            for _ in range(t):
                frames.append(frames[-1] + h * w)
        cu = torch.tensor(frames, dtype=torch.int32, device=dev)
        max_len = max(b - a for a, b in zip(frames[:-1], frames[1:]))
        taps = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, cu, max_len)
            if i in self.v.deepstack_visual_indexes:
                taps.append(self.deepstack[self.v.deepstack_visual_indexes.index(i)](x))
        return self.merger(x), taps


class Qwen3VLMoEBlock(Qwen3MoEBlock):
    """A decoder block that adds a deep-stack feature to the residual stream behind it at the image positions."""
    ds_rows: Optional[torch.Tensor] = None
    ds_feats: Optional[torch.Tensor] = None

    def forward(self, h, res, positions, cu_seqlens, max_seqlen, tp=None, recompute: str = "none"):
        h, res = super().forward(h, res, positions, cu_seqlens, max_seqlen, tp, recompute)
        if self.ds_rows is not None:
            h = h.index_add(0, self.ds_rows, self.ds_feats.to(h.dtype))      # stream = h + res: adding to h is enough
        return h, res


class Qwen3VLMoEWeightMapper(Qwen3MoEWeightMapper):
    """Decoder under ``model.language_model.`` with the experts of a block stored as two stacked tensors
    (``mlp.experts.gate_up_proj [E, 2 I, H]``, ``mlp.experts.down_proj [E, H, I]``); tower under ``model.visual.``."""
    BLOCK = {"norm1_w": "norm1.weight", "norm1_b": "norm1.bias", "norm2_w": "norm2.weight", "norm2_b": "norm2.bias",
             "qkv": "attn.qkv", "proj": "attn.proj", "fc1": "mlp.linear_fc1", "fc2": "mlp.linear_fc2"}
    MERGER = {"norm_w": "norm.weight", "norm_b": "norm.bias", "fc1": "linear_fc1", "fc2": "linear_fc2"}

    def _global_layer(self, stem: str) -> str:
        if stem.startswith("layers.") and (self.layer_offset or self.layer_map):
            i, rest = stem[len("layers."):].split(".", 1)
            g = self.layer_map[int(i)] if self.layer_map else int(i) + self.layer_offset
            return f"layers.{g}.{rest}"
        return stem

    def hf_names(self, local: str) -> List[str]:
        if local.startswith("visual."):
            parts = local.split(".")
            if parts[1] == "patch_embed":
                return ["model.visual.patch_embed.proj." + parts[2]]
            if parts[1] == "pos_embed":
                return ["model.visual.pos_embed.weight"]
            if parts[1] == "blocks":
                return [f"model.visual.blocks.{parts[2]}." + self.BLOCK[parts[3]] + ("." + parts[4] if len(parts) > 4 else "")]
            base = "model.visual.merger." if parts[1] == "merger" else f"model.visual.deepstack_merger_list.{parts[2]}."
            tail = parts[2:] if parts[1] == "merger" else parts[3:]
            return [base + self.MERGER[tail[0]] + ("." + tail[1] if len(tail) > 1 else "")]
        if local.endswith("w_gate_up") or local.endswith("w_down"):
            stem = self._global_layer(local.rsplit(".", 1)[0])
            return [f"model.language_model.{stem}.experts." + ("gate_up_proj" if local.endswith("w_gate_up") else "down_proj")]
        return [n if n.startswith("lm_head") else "model.language_model." + n[len("model."):]
                for n in super().hf_names(local)]

    def load_param(self, name, p, read, available, tp, r) -> bool:
        from .hf_io import _tp_slice
        hf = self.hf_names(name)
        if not all(h in available for h in hf):
            if name.startswith("lm_head") and "model.language_model.embed_tokens.weight" in available:
                hf = ["model.language_model.embed_tokens.weight"]
            else:
                return False
        if name.endswith("w_gate_up") or name.endswith("w_down"):
            El = p.shape[0]
            e0 = getattr(self, "ep_rank", 0) * El
            p.copy_(read(hf[0])[e0:e0 + El].to(p.dtype))
            return True
        cfg = _as_dict(_as_dict(getattr(self, "config", None) or {}).get("text_config") or {})
        parts = []
        for h in hf:
            t = read(h)
            parts.append(t.reshape(p.shape) if name.startswith("visual.") else _tp_slice(h, t, tp, r, cfg))
        t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != model shape {tuple(p.shape)}")
        p.copy_(t.to(p.dtype))
        return True

    def export_tensor(self, name: str, t: torch.Tensor) -> torch.Tensor:
        if name == "visual.patch_embed.weight":
            v = Qwen3VisionArgs.from_hf(_as_dict(getattr(self, "config", None) or {}).get("vision_config") or {})
            return t.reshape(t.shape[0], v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)
        return t


@ModelRegistry.register(Qwen3VLMoEWeightMapper)
class Qwen3VLMoE(Qwen3MoE):
    is_vlm = True
    paged_engine = False     # rollouts re-run the packed forward (no vision prefill in the paged engine)

    def __init__(self, args: Qwen3VLMoEArgs):
        super().__init__(args)
        self.layers = nn.ModuleList([Qwen3VLMoEBlock(args) for _ in range(args.n_layers)])
        for layer in self.layers:
            layer.self_attn.mrope_section = list(args.mrope_section)
            layer.self_attn.mrope_interleaved = True
        self.visual = Qwen3VisionTower(args.vision) if self.is_first_stage else None
        self.mm_inputs: Dict[str, Any] = {}

    @staticmethod
    def supported_model_types():
        return ["qwen3_vl_moe"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(Qwen3VLMoEArgs.from_hf_config(hf_config, **kw))

    def _clear_taps(self) -> None:
        for layer in self.layers:
            layer.ds_rows = layer.ds_feats = None

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = super().embed(input_ids)
        self._clear_taps()
        mm = self.mm_inputs or {}
        rows_all, taps_all = [], None
        for px, grid, tok in (("pixel_values", "image_grid_thw", self.args.image_token_id),
                              ("pixel_values_videos", "video_grid_thw", self.args.video_token_id)):
            if mm.get(px) is None or mm.get(grid) is None or not len(mm[grid]):
                continue
            feats, taps = self.visual(mm[px].to(h.device), mm[grid])
            mask = input_ids == tok
            if int(mask.sum()) != feats.shape[0]:
                raise ValueError(f"{int(mask.sum())} placeholder tokens but {feats.shape[0]} vision tokens")
            h = h.masked_scatter(mask[:, None], feats.to(h.dtype))
            rows_all.append(mask.nonzero(as_tuple=True)[0])
            taps_all = taps if taps_all is None else [torch.cat([a, b]) for a, b in zip(taps_all, taps)]
        if rows_all:
            rows = torch.cat(rows_all)
            for k, feats in enumerate(taps_all):
                self.layers[k].ds_rows, self.layers[k].ds_feats = rows, feats
        return h

    def get_position_ids(self, cu_seqlens: torch.Tensor, total: int, input_ids: Optional[torch.Tensor] = None):
        mm = self.mm_inputs or {}
        if input_ids is None or (mm.get("image_grid_thw") is None and mm.get("video_grid_thw") is None):
            return super().get_position_ids(cu_seqlens, total)
        a = self.args
        return mrope_positions(input_ids, cu_seqlens, a.image_token_id, a.video_token_id, mm.get("image_grid_thw"),
                               mm.get("video_grid_thw"), a.vision.spatial_merge_size, 1.0, mm.get("second_per_grid_ts"))

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        mm = self.mm_inputs or {}
        if self.is_first_stage and position_ids.dim() == 1 and (mm.get("image_grid_thw") is not None
                                                                or mm.get("video_grid_thw") is not None):
            position_ids = self.get_position_ids(cu_seqlens, input_ids.shape[0], input_ids)
        try:
            return super().forward(input_ids, position_ids, cu_seqlens, max_seqlen)
        finally:
            self._clear_taps()

    def export_items(self):
        """(checkpoint name, tensor): the stacked experts go out as they are, everything else through the mapper."""
        from .hf_io import _split_fused
        a = self.args
        mapper = Qwen3VLMoEWeightMapper(a.to_hf_config())
        mapper.layer_offset, mapper.layer_map = self.layer_offset, self.layer_map
        out = []
        for name, p in self.named_parameters():
            if name.endswith("w_gate_up") or name.endswith("w_down"):
                out.append((mapper.hf_names(name)[0], p.detach()))
            else:
                out.extend(_split_fused(name, p.detach(), mapper, a.to_hf_config(), a.n_heads // a.tp_size,
                                        max(1, a.n_kv_heads // a.tp_size), a.head_dim))
        return out

    def shard_parts(self, flat):
        """Decoder parts as for Qwen3-MoE (experts: one rectangle per expert inside the stacked checkpoint tensor),
        plus every tower tensor whole."""
        from ..parallel.reshard import Part, gpt_parts
        a = self.args
        mapper = Qwen3VLMoEWeightMapper({"model_type": "qwen3_vl_moe"})
        mapper.layer_offset, mapper.layer_map = self.layer_offset, self.layer_map
        is_expert = lambda n: n.endswith("w_gate_up") or n.endswith("w_down")
        dec = copy.copy(flat)
        dec.params = [(n, p) for n, p in flat.params if not is_expert(n) and not n.startswith("visual.")]
        parts = gpt_parts(self, dec)
        for name, p in flat.params:
            slot = flat.by_name[name]
            tr = bool(p.requires_grad)
            if is_expert(name):
                El, rows, cols = p.shape
                e0 = a.ep_rank * El
                hf = mapper.hf_names(name)[0]
                for i in range(El):             # rows of the checkpoint tensor viewed as [E * rows, cols]
                    parts.append(Part(hf, (e0 + i) * rows, (e0 + i + 1) * rows, 0, cols, slot.offset + i * rows * cols,
                                      cols, tr))
            elif name.startswith("visual."):
                rows, cols = (1, p.numel()) if p.dim() == 1 else (p.shape[0], p.numel() // p.shape[0])
                parts.append(Part(mapper.hf_names(name)[0], 0, rows, 0, cols, slot.offset, cols, tr))
        return parts


def _named(**kw) -> Qwen3VLMoEArgs:
    vision = kw.pop("vision")
    a = Qwen3VLMoEArgs(**kw)
    a.vision = vision
    return a


ARCHS: Dict[str, Qwen3VLMoEArgs] = {
    "tiny-qwen3-vl-moe": _named(vocab_size=32000, dim=256, n_layers=3, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512,
                                rope_theta=5e6, qkv_bias=False, qk_norm=True, model_type="qwen3_vl_moe", n_experts=8,
                                top_k=2, moe_ffn_dim=128, mrope_section=[12, 10, 10], image_token_id=31990,
                                video_token_id=31991,
                                vision=Qwen3VisionArgs(depth=3, hidden_size=64, num_heads=2, intermediate_size=96,
                                                       out_hidden_size=256, num_position_embeddings=64,
                                                       deepstack_visual_indexes=[0, 2])),
}
