"""Multimodal diffusion transformer (the SD3 family): two token streams, image latents and text, with separate weights
that meet in ONE joint attention per block.

The reference drives Stable Diffusion 3 through the ``diffusers`` pipeline (cosmos_rl/policy/model/diffusers/sd3_model.py:39-366
around ``SD3Transformer2DModel``); that package is not a dependency here, so the network is written out on this package's
kernels, under the parameter names of the published checkpoints (``transformer_blocks.N.attn.to_q``, ``add_q_proj``,
``norm1.linear``, ``ff.net.0.proj`` ...), so a ``transformer/`` folder of such a checkpoint loads as it is:

* latents ``[B, C, H, W]`` are cut into 2 x 2 patches, embedded, and get a fixed 2-D sin-cos position code cropped from
  the centre of a ``pos_embed_max_size`` grid;
* the conditioning vector is ``MLP(sinusoid(1000 t)) + MLP(pooled text embedding)``; the text tokens go through one
  linear layer into the model width;
* every block modulates both streams from the conditioning vector (adaLN-zero: shift / scale / gate for attention and
  MLP), projects each stream to q, k, v with its own weights (optionally RMS-normalised per head, SD3.5), runs one
  bidirectional attention over the concatenation ``[image tokens; text tokens]`` of each sample through the packed
  non-causal kernel, and sends the two halves back through their own output projections and GELU-tanh MLPs. The LAST
  block only reads the text stream (its text side has no output projection and no MLP);
* an adaLN output layer and a linear map back to patches give the velocity ``noise - data`` at time ``t`` (1 = noise).

Calling convention of the diffusion trainers: ``model(latents, t, text, text_mask)``. The pooled text embedding rides as
row 0 of ``text`` (zero-padded to the text width, always valid in the mask) when ``pooled_dim > 0``; the model splits it
off, so data sets, rollouts and trainers need no extra argument.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import BaseModel, ModelRegistry, WeightMapper
from .dit import _ln


@dataclass
class MMDiTArgs:
    sample_size: int = 128               # latent height / width the position grid is centred for
    patch_size: int = 2
    in_channels: int = 16
    out_channels: int = 16
    num_layers: int = 24
    attention_head_dim: int = 64
    num_attention_heads: int = 24
    joint_attention_dim: int = 4096      # width of the text tokens
    caption_projection_dim: int = 1536   # = model width
    pooled_projection_dim: int = 2048
    pos_embed_max_size: int = 192
    qk_norm: Optional[str] = None        # "rms_norm" (SD3.5) or None
    model_type: str = "mmdit"

    @property
    def dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @property
    def pooled_dim(self) -> int:
        return self.pooled_projection_dim

    @classmethod
    def from_hf_config(cls, c, **over) -> "MMDiTArgs":
        d = {k: v for k, v in dict(c).items() if k in cls.__dataclass_fields__}
        d.update({k: v for k, v in over.items() if k in cls.__dataclass_fields__})
        return cls(**d)

    def to_hf_config(self) -> Dict[str, Any]:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d.update(_class_name="SD3Transformer2DModel", architectures=["SD3Transformer2DModel"])
        return d


def timestep_sinusoid(t: torch.Tensor, dim: int = 256) -> torch.Tensor:
    """``[cos | sin]`` of ``t * exp(-ln(10000) i / half)`` (the ``flip_sin_to_cos`` layout of the published weights)."""
    half = dim // 2
    freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = t.float()[:, None] * freq[None]
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1)


def sincos_2d(dim: int, grid: int, base: int, device) -> torch.Tensor:
    """Position table of a ``grid x grid`` patch grid, scaled as if the grid had ``base`` cells per side:
    ``[grid * grid, dim]``, first half of the channels from the column index, second half from the row index, each as
    ``[sin | cos]`` (the layout of ``get_2d_sincos_pos_embed``)."""
    pos = torch.arange(grid, dtype=torch.float64, device=device) / (grid / base)
    gy, gx = torch.meshgrid(pos, pos, indexing="ij")

    def one(p: torch.Tensor, d: int) -> torch.Tensor:
        omega = 1.0 / 10000 ** (torch.arange(d // 2, dtype=torch.float64, device=device) / (d / 2.0))
        out = p.reshape(-1)[:, None] * omega[None]
        return torch.cat([torch.sin(out), torch.cos(out)], dim=1)

    return torch.cat([one(gx, dim // 2), one(gy, dim // 2)], dim=1).float()


class _MLP(nn.Module):
    """``linear_1 -> SiLU -> linear_2`` (timestep and pooled-text embedders)."""

    def __init__(self, i: int, o: int):
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(i, o), nn.Linear(o, o)

    def forward(self, x):
        return self.linear_2(torch.nn.functional.silu(self.linear_1(x)))


class _TimeText(nn.Module):
    def __init__(self, dim: int, pooled: int):
        super().__init__()
        self.timestep_embedder = _MLP(256, dim)
        self.text_embedder = _MLP(pooled, dim) if pooled > 0 else None


class _Mod(nn.Module):
    def __init__(self, dim: int, n: int):
        super().__init__()
        self.linear = nn.Linear(dim, n * dim)


class _Proj(nn.Module):
    def __init__(self, i: int, o: int):
        super().__init__()
        self.proj = nn.Linear(i, o)


class _FF(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.net = nn.ModuleList([_Proj(dim, 4 * dim), nn.Identity(), nn.Linear(4 * dim, dim)])

    def forward(self, x):
        return self.net[2](torch.nn.functional.gelu(self.net[0].proj(x), approximate="tanh"))


class _JointAttention(nn.Module):
    def __init__(self, a: MMDiTArgs, context_pre_only: bool):
        super().__init__()
        D, self.h, self.d = a.dim, a.num_attention_heads, a.attention_head_dim
        self.to_q, self.to_k, self.to_v = nn.Linear(D, D), nn.Linear(D, D), nn.Linear(D, D)
        self.add_q_proj, self.add_k_proj, self.add_v_proj = nn.Linear(D, D), nn.Linear(D, D), nn.Linear(D, D)
        self.to_out = nn.ModuleList([nn.Linear(D, D)])
        self.to_add_out = None if context_pre_only else nn.Linear(D, D)
        rms = a.qk_norm == "rms_norm"
        self.norm_q = _RMS(self.d) if rms else None
        self.norm_k = _RMS(self.d) if rms else None
        self.norm_added_q = _RMS(self.d) if rms else None
        self.norm_added_k = _RMS(self.d) if rms else None

    def forward(self, x, c, ix, ic, cu, max_len: int):
        """x [Nx, D], c [Nc, D]; ix / ic: positions of the image and text tokens in the joint packed order."""
        h, d = self.h, self.d
        n = x.shape[0] + c.shape[0]

        def joint(px, pc, nx, nc):
            a, b = px(x).view(-1, h, d), pc(c).view(-1, h, d)
            if nx is not None:
                a, b = nx(a), nc(b)
            out = a.new_empty(n, h, d)
            out[ix], out[ic] = a, b
            return out

        q = joint(self.to_q, self.add_q_proj, self.norm_q, self.norm_added_q)
        k = joint(self.to_k, self.add_k_proj, self.norm_k, self.norm_added_k)
        v = joint(self.to_v, self.add_v_proj, None, None)
        o = F.full_attention(q, k, v, cu, cu, max_len, max_len).reshape(n, h * d)
        ox = self.to_out[0](o[ix])
        oc = self.to_add_out(o[ic]) if self.to_add_out is not None else None
        return ox, oc


class _RMS(nn.Module):
    def __init__(self, d: int, eps: float = 1e-6):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), eps

    def forward(self, x):
        return F.rms_norm(x.reshape(-1, x.shape[-1]), self.weight, self.eps)[0].view(x.shape)


class JointBlock(nn.Module):
    def __init__(self, a: MMDiTArgs, context_pre_only: bool):
        super().__init__()
        D = a.dim
        self.pre_only = context_pre_only
        self.norm1 = _Mod(D, 6)
        self.norm1_context = _Mod(D, 2 if context_pre_only else 6)
        self.attn = _JointAttention(a, context_pre_only)
        self.ff = _FF(D)
        self.ff_context = None if context_pre_only else _FF(D)

    def forward(self, x, c, emb, rx, rc, ix, ic, cu, max_len: int):
        """emb [B, D] SiLU-ed conditioning; rx / rc: sample index of every image / text token."""
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = self.norm1.linear(emb)[rx].chunk(6, dim=-1)
        xn = _ln(x, 1e-6) * (1 + sc_a) + sh_a
        if self.pre_only:
            c_scale, c_shift = self.norm1_context.linear(emb)[rc].chunk(2, dim=-1)       # scale first in this layer
            cn = _ln(c, 1e-6) * (1 + c_scale) + c_shift
        else:
            csh_a, csc_a, cg_a, csh_m, csc_m, cg_m = self.norm1_context.linear(emb)[rc].chunk(6, dim=-1)
            cn = _ln(c, 1e-6) * (1 + csc_a) + csh_a
        ox, oc = self.attn(xn, cn, ix, ic, cu, max_len)
        x = x + g_a * ox
        x = x + g_m * self.ff(_ln(x, 1e-6) * (1 + sc_m) + sh_m)
        if self.pre_only:
            return x, c
        c = c + cg_a * oc
        c = c + cg_m * self.ff_context(_ln(c, 1e-6) * (1 + csc_m) + csh_m)
        return x, c


class MMDiTWeightMapper(WeightMapper):
    """Parameter names ARE the published ones; only the patch convolution is stored flattened here."""

    def hf_names(self, local: str) -> List[str]:
        return [local]

    def load_param(self, name, p, read, available, tp, r) -> bool:
        if name not in available:
            return False
        t = read(name)
        p.copy_((t.reshape(p.shape) if t.numel() == p.numel() else t).to(p.dtype))
        return True

    def export_tensor(self, name: str, t: torch.Tensor) -> torch.Tensor:
        if name == "pos_embed.proj.weight":
            cfg = dict(getattr(self, "config", None) or {})
            ps, ch = int(cfg.get("patch_size", 2)), int(cfg.get("in_channels", 16))
            return t.reshape(t.shape[0], ch, ps, ps)
        return t


@ModelRegistry.register(MMDiTWeightMapper)
class MMDiT(BaseModel):
    paged_engine = False

    def __init__(self, args: MMDiTArgs):
        super().__init__()
        self.args = a = args
        D = a.dim
        if a.caption_projection_dim != D:
            raise ValueError("caption_projection_dim must equal heads * head_dim")
        self.pos_embed = _Proj(a.in_channels * a.patch_size * a.patch_size, D)          # the patch convolution
        self.time_text_embed = _TimeText(D, a.pooled_projection_dim)
        self.context_embedder = nn.Linear(a.joint_attention_dim, D)
        self.transformer_blocks = nn.ModuleList([JointBlock(a, i == a.num_layers - 1) for i in range(a.num_layers)])
        self.norm_out = _Mod(D, 2)
        self.proj_out = nn.Linear(D, a.patch_size * a.patch_size * a.out_channels)
        self.gradient_checkpointing = False

    @property
    def layers(self):
        return self.transformer_blocks

    @staticmethod
    def supported_model_types():
        return ["mmdit", "sd3"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        return cls(MMDiTArgs.from_hf_config(hf_config, **kw))

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Normal init; every modulation layer and the output projection start at zero (each block is the identity and
        the predicted velocity is zero at step 0)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if ".norm1" in name or name.startswith(("norm_out", "proj_out")):
                    p.zero_()
                elif p.dim() == 1:
                    p.fill_(1.0) if "norm_" in name and name.endswith("weight") else p.zero_()
                else:
                    p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std).to(p.dtype))

    init_weights_on_device = init_weights

    def shard_parts(self, flat):
        from ..parallel.reshard import whole_parts
        return whole_parts(flat)

    def _positions(self, gh: int, gw: int, device) -> torch.Tensor:
        a = self.args
        m = a.pos_embed_max_size
        if gh > m or gw > m:
            raise ValueError(f"a {gh} x {gw} patch grid exceeds pos_embed_max_size {m}")
        table = sincos_2d(a.dim, m, a.sample_size // a.patch_size, device).view(m, m, a.dim)
        top, left = (m - gh) // 2, (m - gw) // 2
        return table[top:top + gh, left:left + gw].reshape(gh * gw, a.dim)

    def forward(self, latents: torch.Tensor, timesteps: torch.Tensor, text: torch.Tensor,
                text_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """latents [B, C, H, W] (or [B, C, 1, H, W]), timesteps [B] in [0, 1], text [B, L, joint_attention_dim] whose
        row 0 holds the pooled embedding when ``pooled_projection_dim > 0``, optional validity mask [B, L]."""
        a = self.args
        video = latents.dim() == 5
        z = latents.squeeze(2) if video else latents
        B, C, H, W = z.shape
        p = a.patch_size
        gh, gw = H // p, W // p
        n = gh * gw
        dt = self.pos_embed.proj.weight.dtype
        dev = z.device
        tok = z.to(dt).view(B, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(B * n, C * p * p)
        x = self.pos_embed.proj(tok) + self._positions(gh, gw, dev).to(dt).repeat(B, 1)
        emb = self.time_text_embed.timestep_embedder(timestep_sinusoid(timesteps.float() * 1000.0).to(dt))
        if self.time_text_embed.text_embedder is not None:
            pooled = text[:, 0, :a.pooled_projection_dim].to(dt)
            emb = emb + self.time_text_embed.text_embedder(pooled)
            text = text[:, 1:]
            text_mask = text_mask[:, 1:] if text_mask is not None else None
        emb = torch.nn.functional.silu(emb)
        L = text.shape[1]
        if text_mask is None:
            lens = torch.full((B,), L, dtype=torch.long, device=dev)
            ctx = text.reshape(B * L, -1)
        else:
            keep = text_mask.bool()
            lens = keep.sum(1)
            ctx = text[keep]
        c = self.context_embedder(ctx.to(dt))
        # joint packed order per sample: image tokens first, then that sample's text tokens
        tot = lens + n
        cu = torch.nn.functional.pad(tot.cumsum(0), (1, 0)).to(torch.int32)
        start = cu[:-1].long()
        rx = torch.arange(B, device=dev).repeat_interleave(n)
        rc = torch.repeat_interleave(torch.arange(B, device=dev), lens)
        ix = (start[:, None] + torch.arange(n, device=dev)[None]).reshape(-1)
        within = torch.arange(int(lens.sum()), device=dev) - torch.repeat_interleave(
            torch.nn.functional.pad(lens.cumsum(0), (1, 0))[:-1], lens)
        ic = start[rc] + n + within
        max_len = int(tot.max())
        for blk in self.transformer_blocks:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                x, c = checkpoint(blk, x, c, emb, rx, rc, ix, ic, cu, max_len, use_reentrant=False)
            else:
                x, c = blk(x, c, emb, rx, rc, ix, ic, cu, max_len)
        scale, shift = self.norm_out.linear(emb)[rx].chunk(2, dim=-1)
        out = self.proj_out(_ln(x, 1e-6) * (1 + scale) + shift).float()
        oc = a.out_channels
        v = out.view(B, gh, gw, p, p, oc).permute(0, 5, 1, 3, 2, 4).reshape(B, oc, H, W)
        return v.unsqueeze(2) if video else v

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        n = sum(p.numel() for p in self.parameters())
        return n, 6 * n + 12 * self.args.num_layers * self.args.dim * seq_len


ARCHS = {
    "tiny-mmdit": MMDiTArgs(sample_size=8, patch_size=2, in_channels=4, out_channels=4, num_layers=3, attention_head_dim=32,
                            num_attention_heads=4, joint_attention_dim=64, caption_projection_dim=128,
                            pooled_projection_dim=48, pos_embed_max_size=16),
    "sd3-medium": MMDiTArgs(sample_size=128, num_layers=24, attention_head_dim=64, num_attention_heads=24,
                            caption_projection_dim=1536),
    "sd3.5-large": MMDiTArgs(sample_size=128, num_layers=38, attention_head_dim=64, num_attention_heads=38,
                             caption_projection_dim=2432, qk_norm="rms_norm"),
}
