"""Diffusion transformer for image / video latents: patch embedding, sin-cos position code, timestep embedding that
drives adaLN-zero modulation of every block, bidirectional self-attention over the latent tokens, cross-attention
onto the text embeddings, gated MLP, and an adaLN output head that predicts the flow-matching velocity per patch
(the role of cosmos_rl/policy/model/wfm/networks/minimal_v4_dit.py and of the SD3 / SANA transformers the reference
drives through diffusers, cosmos_rl/policy/model/diffusers/). All sequences of a batch are packed into one token
axis so both attentions run through the same non-causal varlen kernel."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import BaseModel, ModelRegistry, WeightMapper


@dataclass
class DiTArgs:
    in_channels: int = 16
    patch_size: Tuple[int, int, int] = (1, 2, 2)          # (frames, height, width) of one token
    dim: int = 1024
    n_layers: int = 12
    n_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 4096
    text_dim: int = 1024
    freq_dim: int = 256
    norm_eps: float = 1e-6
    model_type: str = "dit"

    @classmethod
    def from_hf_config(cls, c, **over) -> "DiTArgs":
        d = {k: v for k, v in dict(c).items() if k in cls.__dataclass_fields__}
        if "patch_size" in d:
            d["patch_size"] = tuple(d["patch_size"])
        d.update(over)
        return cls(**d)

    def to_hf_config(self) -> Dict[str, Any]:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d["patch_size"] = list(self.patch_size)
        d["architectures"] = ["DiT"]
        return d


ARCHS = {
    "tiny-dit": DiTArgs(in_channels=4, patch_size=(1, 2, 2), dim=128, n_layers=2, n_heads=4, head_dim=32, ffn_dim=256,
                        text_dim=64, freq_dim=64),
    "dit-2b": DiTArgs(in_channels=16, patch_size=(1, 2, 2), dim=2048, n_layers=28, n_heads=16, head_dim=128,
                      ffn_dim=8192, text_dim=1024),
}


def sincos_1d(pos: torch.Tensor, dim: int, base: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freq = torch.exp(-math.log(base) * torch.arange(half, dtype=torch.float32, device=pos.device) / max(half, 1))
    ang = pos.float()[:, None] * freq[None, :]
    out = torch.cat([torch.sin(ang), torch.cos(ang)], dim=-1)
    return torch.nn.functional.pad(out, (0, dim - out.shape[-1]))


def position_code(t: int, h: int, w: int, dim: int, device) -> torch.Tensor:
    """[t*h*w, dim]: the channel axis is split into a frame, a row and a column part."""
    dt = dim // 4 if t > 1 else 0
    dh = (dim - dt) // 2
    dw = dim - dt - dh
    ft, fh, fw = torch.meshgrid(torch.arange(t, device=device), torch.arange(h, device=device),
                                torch.arange(w, device=device), indexing="ij")
    parts = [sincos_1d(fh.flatten(), dh), sincos_1d(fw.flatten(), dw)]
    if dt:
        parts.insert(0, sincos_1d(ft.flatten(), dt))
    return torch.cat(parts, dim=-1)


def _ln(x: torch.Tensor, eps: float) -> torch.Tensor:
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), eps=eps).to(x.dtype)


class DiTBlock(nn.Module):
    def __init__(self, a: DiTArgs):
        super().__init__()
        self.h, self.d, self.eps = a.n_heads, a.head_dim, a.norm_eps
        hd = a.n_heads * a.head_dim
        self.modulation = nn.Linear(a.dim, 6 * a.dim)
        self.qkv = nn.Linear(a.dim, 3 * hd)
        self.q_norm = nn.Parameter(torch.ones(a.head_dim))
        self.k_norm = nn.Parameter(torch.ones(a.head_dim))
        self.attn_out = nn.Linear(hd, a.dim)
        self.cross_q = nn.Linear(a.dim, hd)
        self.cross_kv = nn.Linear(a.text_dim, 2 * hd)
        self.cross_out = nn.Linear(hd, a.dim)
        self.fc1 = nn.Linear(a.dim, a.ffn_dim)
        self.fc2 = nn.Linear(a.ffn_dim, a.dim)

    def forward(self, x, cond, rows, text, cu_x, cu_t, max_x: int, max_t: int):
        """x [N, dim] packed latent tokens, cond [B, dim] timestep embedding, rows [N] sample index of each token,
        text [L, text_dim] packed text tokens."""
        N, h, d = x.shape[0], self.h, self.d
        m = self.modulation(torch.nn.functional.silu(cond))[rows]
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = m.chunk(6, dim=-1)
        y = _ln(x, self.eps) * (1 + sc_a) + sh_a
        q, k, v = self.qkv(y).view(N, 3, h, d).unbind(1)
        q = F.rms_norm(q.reshape(N * h, d), self.q_norm, self.eps)[0].view(N, h, d)
        k = F.rms_norm(k.reshape(N * h, d), self.k_norm, self.eps)[0].view(N, h, d)
        x = x + g_a * self.attn_out(F.full_attention(q, k, v.contiguous(), cu_x, cu_x, max_x, max_x).reshape(N, h * d))
        cq = self.cross_q(_ln(x, self.eps)).view(N, h, d)
        ck, cv = self.cross_kv(text).view(text.shape[0], 2, h, d).unbind(1)
        x = x + self.cross_out(F.full_attention(cq, ck.contiguous(), cv.contiguous(), cu_x, cu_t, max_x, max_t
                                                ).reshape(N, h * d))
        y = _ln(x, self.eps) * (1 + sc_m) + sh_m
        return x + g_m * self.fc2(torch.nn.functional.gelu(self.fc1(y), approximate="tanh"))


class DiTWeightMapper(WeightMapper):
    """Checkpoints of this family are stored under the framework's own parameter names."""

    def hf_names(self, local: str) -> List[str]:
        return [local]


@ModelRegistry.register(DiTWeightMapper)
class DiT(BaseModel):
    paged_engine = False

    def __init__(self, args: DiTArgs):
        super().__init__()
        self.args = a = args
        pt, ph, pw = a.patch_size
        self.patch_dim = a.in_channels * pt * ph * pw
        self.patch_in = nn.Linear(self.patch_dim, a.dim)
        self.time_in = nn.Sequential(nn.Linear(a.freq_dim, a.dim), nn.SiLU(), nn.Linear(a.dim, a.dim))
        self.layers = nn.ModuleList([DiTBlock(a) for _ in range(a.n_layers)])
        self.final_modulation = nn.Linear(a.dim, 2 * a.dim)
        self.patch_out = nn.Linear(a.dim, self.patch_dim)
        self.gradient_checkpointing = False

    @staticmethod
    def supported_model_types():
        return ["dit"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        kw = {k: v for k, v in kw.items() if k in DiTArgs.__dataclass_fields__}
        return cls(DiTArgs.from_hf_config(hf_config, **kw))

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Normal init; the modulation and output projections start at zero (adaLN-zero: every block is the identity
        and the predicted velocity is zero at step 0)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if "modulation" in name or name.startswith("patch_out"):
                    p.zero_()
                elif p.dim() == 1:
                    p.fill_(1.0) if name.endswith("_norm") else p.zero_()
                else:
                    p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std).to(p.dtype))

    init_weights_on_device = init_weights

    def shard_parts(self, flat):
        """Weight-sync parts: every tensor whole (the family runs data parallel only)."""
        from ..parallel.reshard import whole_parts
        return whole_parts(flat)

    # ------------------------------------------------------------------ patches
    def patchify(self, z: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        """[B, C, T, H, W] -> [B, n, C*pt*ph*pw] and the token grid."""
        B, C, T, H, W = z.shape
        pt, ph, pw = self.args.patch_size
        assert T % pt == 0 and H % ph == 0 and W % pw == 0, "latent size must be a multiple of the patch size"
        t, h, w = T // pt, H // ph, W // pw
        x = z.view(B, C, t, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, t * h * w, C * pt * ph * pw), (t, h, w)

    def unpatchify(self, x: torch.Tensor, grid: Tuple[int, int, int]) -> torch.Tensor:
        t, h, w = grid
        pt, ph, pw = self.args.patch_size
        B, C = x.shape[0], self.args.in_channels
        x = x.view(B, t, h, w, C, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return x.reshape(B, C, t * pt, h * ph, w * pw)

    # ------------------------------------------------------------------ forward
    def forward(self, latents: torch.Tensor, timesteps: torch.Tensor, text: torch.Tensor,
                text_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """latents [B, C, T, H, W] (or [B, C, H, W]), timesteps [B] in [0, 1] (1 = pure noise), text [B, L, text_dim]
        with an optional validity mask [B, L]. Returns the velocity (noise - data) with the shape of ``latents``."""
        a = self.args
        image = latents.dim() == 4
        z = latents.unsqueeze(2) if image else latents
        B = z.shape[0]
        tok, grid = self.patchify(z)
        n = tok.shape[1]
        dt = self.patch_in.weight.dtype
        x = self.patch_in(tok.to(dt)) + position_code(*grid, a.dim, z.device).to(dt)[None]
        x = x.reshape(B * n, a.dim)
        cond = self.time_in(sincos_1d(timesteps.float() * 1000.0, a.freq_dim).to(dt))
        rows = torch.arange(B, device=z.device).repeat_interleave(n)
        cu_x = torch.arange(0, (B + 1) * n, n, dtype=torch.int32, device=z.device)
        if text_mask is None:
            L = text.shape[1]
            txt, cu_t, max_t = text.reshape(B * L, -1), torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=z.device), L
        else:
            keep = text_mask.bool()
            lens = keep.sum(1)
            txt = text[keep]
            cu_t = torch.nn.functional.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
            max_t = int(lens.max())
        txt = txt.to(dt)
        for blk in self.layers:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(blk, x, cond, rows, txt, cu_x, cu_t, n, max_t, use_reentrant=False)
            else:
                x = blk(x, cond, rows, txt, cu_x, cu_t, n, max_t)
        shift, scale = self.final_modulation(torch.nn.functional.silu(cond))[rows].chunk(2, dim=-1)
        out = self.patch_out(_ln(x, a.norm_eps) * (1 + scale) + shift).view(B, n, self.patch_dim)
        v = self.unpatchify(out.float(), grid)
        return v.squeeze(2) if image else v

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        n = sum(p.numel() for p in self.parameters())
        a = self.args
        return n, 6 * n + 12 * a.n_layers * a.n_heads * a.head_dim * seq_len
