"""Native Qwen2.5-VL: windowed vision transformer + Qwen2 decoder with multimodal rotary positions.

The reference ships its own implementation of this family (cosmos_rl/policy/model/qwen2_5_vl/__init__.py:566,
cosmos_rl/policy/model/vision_encoder/) so that the decoder gets its tensor / sequence / pipeline plans and the weight
synchronisation knows every tensor. Here the decoder IS :class:`GPT` (same fused projections, same kernels, same
parallel plans); this file adds what the family has on top of it:

* the vision tower: patches ``[N, C * t * p * p]`` -> linear patch embedding -> blocks of RMSNorm / attention with a
  2-D rotary embedding / gated MLP, where all but a few blocks attend inside 112 x 112 pixel windows and the others over
  the whole image -> a merger that folds 2 x 2 neighbouring patches into one token of the decoder's width;
* the scatter of those tokens into the embedded prompt at the image / video placeholder ids;
* multimodal rotary positions: three position streams (time, height, width); the rotary dimensions are divided
  into sections that each follow one stream. Text tokens carry the same value in all three.

Packed batches: ``forward`` takes the packed ids like :class:`GPT` and reads the pixels of the batch from
``mm_inputs`` (``pixel_values``, ``image_grid_thw``, optionally ``pixel_values_videos``, ``video_grid_thw``,
``second_per_grid_ts``), which the trainer sets before every call.
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


@dataclass
class VisionArgs:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    out_hidden_size: int = 3584
    patch_size: int = 14
    temporal_patch_size: int = 2
    in_channels: int = 3
    spatial_merge_size: int = 2
    window_size: int = 112
    fullatt_block_indexes: List[int] = field(default_factory=lambda: [7, 15, 23, 31])
    tokens_per_second: int = 2
    norm_eps: float = 1e-6

    @classmethod
    def from_hf(cls, v) -> "VisionArgs":
        g = (lambda k, d=None: v.get(k, d)) if isinstance(v, dict) else (lambda k, d=None: getattr(v, k, d))
        base = cls()
        return cls(**{k: (g(k) if g(k) is not None else getattr(base, k)) for k in base.__dataclass_fields__
                      if k != "norm_eps"})


@dataclass
class Qwen25VLArgs(GPTArgs):
    vision: VisionArgs = field(default_factory=VisionArgs)
    mrope_section: List[int] = field(default_factory=lambda: [16, 24, 24])
    image_token_id: int = 151655
    video_token_id: int = 151656

    @classmethod
    def from_hf_config(cls, c, **over) -> "Qwen25VLArgs":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        text = g("text_config") or c
        tg = (lambda k, d=None: text.get(k, d)) if isinstance(text, dict) else (lambda k, d=None: getattr(text, k, d))
        base = GPTArgs.from_hf_config(dict(_as_dict(text), model_type="qwen2"))
        rope = tg("rope_parameters") or tg("rope_scaling") or {}
        a = cls(**{k: getattr(base, k) for k in GPTArgs.__dataclass_fields__})
        a.model_type = "qwen2_5_vl"
        a.qkv_bias = True
        a.vision = VisionArgs.from_hf(g("vision_config") or {})
        a.mrope_section = list(rope.get("mrope_section") or [16, 24, 24])
        if rope.get("rope_theta"):
            a.rope_theta = float(rope["rope_theta"])
        a.image_token_id = g("image_token_id", 151655)
        a.video_token_id = g("video_token_id", 151656)
        a.tie_word_embeddings = bool(g("tie_word_embeddings", tg("tie_word_embeddings", False)))
        for k, v in over.items():
            setattr(a, k, v)
        a.__post_init__()
        return a

    def to_hf_config(self) -> Dict[str, Any]:
        text = GPTArgs.to_hf_config(self)
        text.update(model_type="qwen2_5_vl_text",
                    rope_parameters={"rope_type": "default", "rope_theta": self.rope_theta,
                                     "mrope_section": list(self.mrope_section)})
        text.pop("architectures", None)
        text.pop("rope_theta", None)
        v = self.vision
        vis = {k: getattr(v, k) for k in v.__dataclass_fields__ if k != "norm_eps"}
        vis["hidden_act"] = "silu"
        vis["model_type"] = "qwen2_5_vl"
        return {"architectures": ["Qwen2_5_VLForConditionalGeneration"], "model_type": "qwen2_5_vl",
                "text_config": text, "vision_config": vis, "image_token_id": self.image_token_id,
                "video_token_id": self.video_token_id, "tie_word_embeddings": self.tie_word_embeddings,
                "vocab_size": self.vocab_size, "hidden_size": self.dim, "torch_dtype": "bfloat16"}


def _named(**kw) -> Qwen25VLArgs:
    vision = kw.pop("vision")
    a = Qwen25VLArgs(**kw)
    a.vision = vision
    return a


# random-init architectures (shapes of the public checkpoints; the tiny one is for tests)
ARCHS: Dict[str, Qwen25VLArgs] = {
    "tiny-qwen2.5-vl": _named(vocab_size=32000, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=688, rope_theta=1e6,
                              qkv_bias=True, model_type="qwen2_5_vl", mrope_section=[8, 12, 12], image_token_id=31990,
                              video_token_id=31991,
                              vision=VisionArgs(depth=2, hidden_size=64, num_heads=2, intermediate_size=96,
                                                out_hidden_size=256, window_size=56, fullatt_block_indexes=[1])),
    "qwen2.5-vl-7b": _named(vocab_size=152064, dim=3584, n_layers=28, n_heads=28, n_kv_heads=4, ffn_dim=18944,
                            rope_theta=1e6, qkv_bias=True, model_type="qwen2_5_vl", max_seq_len=128000,
                            vision=VisionArgs()),
}


def _as_dict(c) -> Dict[str, Any]:
    if isinstance(c, dict):
        return c
    return c.to_dict() if hasattr(c, "to_dict") else dict(vars(c))


# ---------------------------------------------------------------------------------------------------
# rotary helpers
# ---------------------------------------------------------------------------------------------------
def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """``q, k [T, heads, d]``, ``cos, sin [T, d]`` (fp32); the rotation runs in fp32."""
    c, s = cos[:, None, :], sin[:, None, :]
    qf, kf = q.float(), k.float()
    return (qf * c + _rotate_half(qf) * s).to(q.dtype), (kf * c + _rotate_half(kf) * s).to(k.dtype)


def mrope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, sections: List[int],
                  interleaved: bool = False):
    """``positions [3, T]`` -> ``cos, sin [T, head_dim]``: rotary frequency ``j`` follows the stream its section belongs
    to (the sections count frequencies: they sum to ``head_dim / 2``). Chunked layout: the first ``sections[0]``
    frequencies follow time, the next height, the rest width. ``interleaved`` (Qwen3-VL): frequencies 1, 4, 7, ... up
    to ``3 sections[1]`` follow height, 2, 5, 8, ... up to ``3 sections[2]`` width, everything else time."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=positions.device) / half))
    if interleaved:
        owner = torch.zeros(half, dtype=torch.int64, device=positions.device)
        owner[1:3 * sections[1]:3] = 1
        owner[2:3 * sections[2]:3] = 2
    else:
        owner = torch.repeat_interleave(torch.arange(len(sections), device=positions.device) % 3,
                                        torch.tensor(sections, device=positions.device))
    pos = positions.to(torch.float32)[owner, :]                  # [half, T]: the stream of every frequency
    freqs = (pos * inv[:, None]).transpose(0, 1)                 # [T, half]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def mrope_positions(input_ids: torch.Tensor, cu_seqlens: torch.Tensor, image_token_id: int, video_token_id: int,
                    image_grid_thw: Optional[torch.Tensor], video_grid_thw: Optional[torch.Tensor],
                    spatial_merge: int, tokens_per_second: float = 2.0,
                    second_per_grid_ts: Optional[List[float]] = None) -> torch.Tensor:
    """``[3, T]`` positions (time, height, width) of a packed batch. Inside every sequence text tokens count up with
    the same value in all three streams; a run of placeholder tokens of one image (or video) of merged grid
    ``t x h x w`` gets ``start + time index * interval``, ``start + row``, ``start + column``, and the text behind it
    continues at ``start + max(t extent, h, w)``."""
    ids = input_ids.tolist()
    cu = cu_seqlens.tolist()
    images = image_grid_thw.tolist() if image_grid_thw is not None else []
    videos = video_grid_thw.tolist() if video_grid_thw is not None else []
    secs = list(second_per_grid_ts) if second_per_grid_ts is not None else [1.0] * len(videos)
    ii = vi = 0
    out = torch.zeros(3, len(ids), dtype=torch.int64)
    for s in range(len(cu) - 1):
        p, pos, end = cu[s], 0, cu[s + 1]
        while p < end:
            tok = ids[p]
            if tok == image_token_id or tok == video_token_id:
                if tok == image_token_id:
                    t, h, w = images[ii]
                    ii += 1
                    interval = 0.0
                else:
                    t, h, w = videos[vi]
                    interval = tokens_per_second * secs[vi]
                    vi += 1
                gh, gw = h // spatial_merge, w // spatial_merge
                n = t * gh * gw
                if p + n > end:
                    raise ValueError("a sequence ends inside the placeholder run of an image")
                tt = (torch.arange(t).repeat_interleave(gh * gw).to(torch.float64) * interval).to(torch.int64)
                hh = torch.arange(gh).repeat_interleave(gw).repeat(t)
                ww = torch.arange(gw).repeat(gh * t)
                out[:, p:p + n] = torch.stack([tt, hh, ww]) + pos
                pos += int(max(int(tt.max()) + 1 if n else 0, gh, gw))
                p += n
            else:
                out[:, p] = pos
                pos += 1
                p += 1
    return out.to(input_ids.device)


# ---------------------------------------------------------------------------------------------------
# vision tower
# ---------------------------------------------------------------------------------------------------
class VisionBlock(nn.Module):
    def __init__(self, v: VisionArgs):
        super().__init__()
        self.heads, self.d, self.eps = v.num_heads, v.hidden_size // v.num_heads, v.norm_eps
        self.norm1 = nn.Parameter(torch.ones(v.hidden_size))
        self.norm2 = nn.Parameter(torch.ones(v.hidden_size))
        self.qkv = nn.Linear(v.hidden_size, 3 * v.hidden_size, bias=True)
        self.proj = nn.Linear(v.hidden_size, v.hidden_size, bias=True)
        self.gate_up_proj = nn.Linear(v.hidden_size, 2 * v.intermediate_size, bias=True)
        self.down_proj = nn.Linear(v.intermediate_size, v.hidden_size, bias=True)

    def forward(self, x, cos, sin, cu, max_len: int):
        N = x.shape[0]
        h = F.rms_norm(x, self.norm1, self.eps)[0]
        q, k, v = _linear(h, self.qkv.weight, self.qkv.bias).view(N, 3, self.heads, self.d).unbind(1)
        q, k = apply_rotary(q, k, cos, sin)
        o = F.full_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, max_len, max_len)
        x = x + _linear(o.reshape(N, -1), self.proj.weight, self.proj.bias)
        h = F.rms_norm(x, self.norm2, self.eps)[0]
        gu = _linear(h, self.gate_up_proj.weight, self.gate_up_proj.bias)
        return x + _linear(F.swiglu(gu), self.down_proj.weight, self.down_proj.bias)


class VisionTower(nn.Module):
    def __init__(self, v: VisionArgs):
        super().__init__()
        self.v = v
        self.unit = v.spatial_merge_size ** 2
        patch_dim = v.in_channels * v.temporal_patch_size * v.patch_size * v.patch_size
        self.patch_embed = nn.Linear(patch_dim, v.hidden_size, bias=False)      # the 3-D convolution as one GEMM
        self.blocks = nn.ModuleList([VisionBlock(v) for _ in range(v.depth)])
        self.merger_norm = nn.Parameter(torch.ones(v.hidden_size))
        self.merger_fc1 = nn.Linear(v.hidden_size * self.unit, v.hidden_size * self.unit, bias=True)
        self.merger_fc2 = nn.Linear(v.hidden_size * self.unit, v.out_hidden_size, bias=True)

    # ---- index arithmetic on the host (grids are small)
    def _patch_positions(self, grid: List[List[int]]) -> torch.Tensor:
        """(row, column) of every patch in the order the processor emits them: 2 x 2 merge groups are contiguous."""
        m = self.v.spatial_merge_size
        out = []
        for t, h, w in grid:
            r = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            c = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack([r, c], dim=-1).repeat(t, 1))
        return torch.cat(out)

    def _windows(self, grid: List[List[int]]) -> Tuple[torch.Tensor, List[int]]:
        """Order of the merged tokens that makes every attention window contiguous, and the window boundaries in
        patches. A window covers ``window_size`` pixels per side; border windows are smaller."""
        v = self.v
        side = v.window_size // v.spatial_merge_size // v.patch_size
        order, bounds, base = [], [0], 0
        for t, h, w in grid:
            gh, gw = h // v.spatial_merge_size, w // v.spatial_merge_size
            idx = torch.arange(t * gh * gw).view(t, gh, gw)
            for f in range(t):
                for r0 in range(0, gh, side):
                    for c0 in range(0, gw, side):
                        win = idx[f, r0:r0 + side, c0:c0 + side].reshape(-1)
                        order.append(win + base)
                        bounds.append(bounds[-1] + win.numel() * self.unit)
            base += t * gh * gw
        return torch.cat(order), bounds

    def forward(self, pixels: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``pixels [N, C * t * p * p]``, ``grid_thw [n_images, 3]`` in patches -> ``[N / merge^2, out_hidden]`` in the
        processor's token order."""
        v = self.v
        grid = grid_thw.tolist()
        dev = pixels.device
        x = _linear(pixels.to(self.patch_embed.weight.dtype), self.patch_embed.weight)
        N = x.shape[0]
        d_rot = (v.hidden_size // v.num_heads) // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, d_rot, 2, dtype=torch.float32) / d_rot))
        pos = self._patch_positions(grid).to(torch.float32)                       # [N, 2]
        ang = torch.cat([pos[:, 0:1] * inv[None, :], pos[:, 1:2] * inv[None, :]], dim=-1)     # [N, d / 2]
        order, win_bounds = self._windows(grid)
        order = order.to(dev)
        x = x.view(N // self.unit, self.unit, -1)[order].reshape(N, -1)
        ang = ang.view(N // self.unit, self.unit, -1)[order.cpu()].reshape(N, -1).to(dev)
        emb = torch.cat((ang, ang), dim=-1)
        cos, sin = emb.cos(), emb.sin()
        cu_win = torch.tensor(win_bounds, dtype=torch.int32, device=dev)
        max_win = max(b - a for a, b in zip(win_bounds[:-1], win_bounds[1:]))
        frames = [0]
        for t, h, w in grid:
            for _ in range(t):
                frames.append(frames[-1] + h * w)
        cu_full = torch.tensor(frames, dtype=torch.int32, device=dev)
        max_full = max(b - a for a, b in zip(frames[:-1], frames[1:]))
        for i, blk in enumerate(self.blocks):
            if i in v.fullatt_block_indexes:
                x = blk(x, cos, sin, cu_full, max_full)
            else:
                x = blk(x, cos, sin, cu_win, max_win)
        x = F.rms_norm(x, self.merger_norm, v.norm_eps)[0].view(N // self.unit, -1)
        x = _linear(torch.nn.functional.gelu(_linear(x, self.merger_fc1.weight, self.merger_fc1.bias)),
                    self.merger_fc2.weight, self.merger_fc2.bias)
        return x[torch.argsort(order)]


# ---------------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------------
class Qwen25VLWeightMapper(GPTWeightMapper):
    """Decoder names as for Qwen2 under ``model.language_model.``; vision names under ``model.visual.``. Checkpoints
    written before that nesting (``model.layers...``, ``visual...``) load through ``alternatives``."""

    VISION = {"merger_norm": "merger.ln_q.weight", "merger_fc1": "merger.mlp.0", "merger_fc2": "merger.mlp.2",
              "patch_embed.weight": "patch_embed.proj.weight"}

    def hf_names(self, local: str) -> List[str]:
        if local.startswith("visual."):
            name = local[len("visual."):]
            for k, v in self.VISION.items():
                if name == k or name.startswith(k + "."):
                    name = v + name[len(k):]
                    break
            name = name.replace(".norm1", ".norm1.weight").replace(".norm2", ".norm2.weight")
            name = name.replace(".qkv.", ".attn.qkv.").replace(".proj.", ".attn.proj.") if ".blocks." in "." + name \
                else name
            name = name.replace("gate_up_proj", "mlp.gate_up_proj").replace(".down_proj", ".mlp.down_proj")
            name = "model.visual." + name
            if "gate_up_proj" in name:
                return [name.replace("gate_up_proj", "gate_proj"), name.replace("gate_up_proj", "up_proj")]
            return [name]
        out = []
        for n in super().hf_names(local):
            out.append(n if n.startswith("lm_head") else "model.language_model." + n[len("model."):])
        return out

    @staticmethod
    def alternatives(name: str) -> List[str]:
        """Other spellings of a checkpoint name, newest layout first."""
        alts = [name]
        if name.startswith("model.language_model."):
            alts.append("model." + name[len("model.language_model."):])
        if name.startswith("model.visual."):
            alts.append(name[len("model."):])
        return alts

    def load_param(self, name, p, read, available, tp, r) -> bool:
        """Vision parameters (replicated over tensor-parallel ranks) and renamed decoder parameters."""
        from .hf_io import _tp_slice
        hf = self.hf_names(name)
        resolved = []
        for h in hf:
            hit = next((a for a in self.alternatives(h) if a in available), None)
            if hit is None:
                if name.startswith("lm_head"):
                    hit = next((a for a in ("model.language_model.embed_tokens.weight", "model.embed_tokens.weight")
                                if a in available), None)
                if hit is None:
                    return False
            resolved.append(hit)
        parts = []
        for h in resolved:
            t = read(h)
            if name == "visual.patch_embed.weight":
                t = t.reshape(t.shape[0], -1)
            parts.append(t if name.startswith("visual.") else _tp_slice(h, t, tp, r, self.cfg_text()))
        t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != model shape {tuple(p.shape)}")
        p.copy_(t.to(p.dtype))
        return True

    def export_tensor(self, name: str, t: torch.Tensor) -> torch.Tensor:
        if name == "visual.patch_embed.weight":     # the checkpoint stores the patch embedding as a 3-D convolution
            v = VisionArgs.from_hf(_as_dict(getattr(self, "config", None) or {}).get("vision_config") or {})
            return t.reshape(t.shape[0], v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)
        return t

    def cfg_text(self) -> Dict[str, Any]:
        c = getattr(self, "config", None) or {}
        c = _as_dict(c)
        return _as_dict(c.get("text_config") or c)


@ModelRegistry.register(Qwen25VLWeightMapper)
class Qwen25VL(GPT):
    is_vlm = True
    paged_engine = False     # rollouts re-run the packed forward (no vision prefill in the paged engine)

    def __init__(self, args: Qwen25VLArgs):
        super().__init__(args)
        self.visual = VisionTower(args.vision) if self.is_first_stage else None
        self.mm_inputs: Dict[str, Any] = {}
        for layer in self.layers:
            layer.self_attn.mrope_section = list(args.mrope_section)

    @staticmethod
    def supported_model_types():
        return ["qwen2_5_vl"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(Qwen25VLArgs.from_hf_config(hf_config, **kw))

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        super().init_weights(seed, std)

    # ------------------------------------------------------------------ inputs
    def vision_tokens(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """(placeholder id, features) pairs of the current batch, images first."""
        mm = self.mm_inputs or {}
        out = []
        dev = self.norm.device if self.norm is not None else next(self.parameters()).device
        for px, grid, tok in (("pixel_values", "image_grid_thw", self.args.image_token_id),
                              ("pixel_values_videos", "video_grid_thw", self.args.video_token_id)):
            if mm.get(px) is not None and mm.get(grid) is not None and len(mm[grid]):
                out.append((tok, self.visual(mm[px].to(dev), mm[grid])))
        return out

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = super().embed(input_ids)
        for tok, feats in self.vision_tokens():
            mask = input_ids == tok
            if int(mask.sum()) != feats.shape[0]:
                raise ValueError(f"{int(mask.sum())} placeholder tokens but {feats.shape[0]} vision tokens")
            h = h.masked_scatter(mask[:, None], feats.to(h.dtype))
        return h

    def get_position_ids(self, cu_seqlens: torch.Tensor, total: int, input_ids: Optional[torch.Tensor] = None):
        """1-D positions without pixels in the batch (or without ids); else ``[3, T]`` multimodal positions."""
        mm = self.mm_inputs or {}
        if input_ids is None or (mm.get("image_grid_thw") is None and mm.get("video_grid_thw") is None):
            return super().get_position_ids(cu_seqlens, total)
        a = self.args
        return mrope_positions(input_ids, cu_seqlens, a.image_token_id, a.video_token_id, mm.get("image_grid_thw"),
                               mm.get("video_grid_thw"), a.vision.spatial_merge_size, a.vision.tokens_per_second,
                               mm.get("second_per_grid_ts"))

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        mm = self.mm_inputs or {}
        if self.is_first_stage and position_ids.dim() == 1 and (mm.get("image_grid_thw") is not None
                                                                or mm.get("video_grid_thw") is not None):
            position_ids = self.get_position_ids(cu_seqlens, input_ids.shape[0], input_ids)
        return super().forward(input_ids, position_ids, cu_seqlens, max_seqlen)

    # ------------------------------------------------------------------ weight synchronisation
    def shard_parts(self, flat):
        """The decoder's parts plus every vision tensor whole (the tower is replicated over tensor-parallel ranks)."""
        from ..parallel.reshard import Part, gpt_parts
        mapper = Qwen25VLWeightMapper({"model_type": "qwen2_5_vl"})
        mapper.layer_offset = self.layer_offset
        mapper.layer_map = self.layer_map
        dec = copy.copy(flat)
        dec.params = [(n, p) for n, p in flat.params if not n.startswith("visual.")]
        parts = gpt_parts(self, dec)
        for name, p in flat.params:
            if not name.startswith("visual."):
                continue
            slot, hf = flat.by_name[name], mapper.hf_names(name)
            if p.dim() == 1:                      # a (possibly fused) vector: the pieces lie side by side
                per, cols = 1, p.shape[0] // len(hf)
            else:                                 # a (possibly fused) matrix: the pieces are stacked by rows
                per, cols = p.shape[0] // len(hf), p.numel() // p.shape[0]
            for i, h in enumerate(hf):
                parts.append(Part(h, 0, per, 0, cols, slot.offset + i * per * cols, cols, bool(p.requires_grad)))
        return parts

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        n, f = super().get_nparams_and_flops(seq_len)
        return n, f
