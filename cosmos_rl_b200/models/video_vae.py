"""Causal 3-D convolutional video VAE (the tokenizer in front of the diffusion transformer).

The world-model trainers of the reference encode pixels with the Wan 2.1 / 2.2 VAE
(cosmos_rl/policy/model/wfm/tokenizer/wan2pt1.py:1-1215): a convolutional encoder / decoder whose time axis is causal,
so that the first frame is a picture on its own and a clip of ``1 + 4 k`` frames becomes ``1 + k`` latent frames at 1/8 of
the height and width. This is a network of that family written for this package (channel-wise RMS norm, residual blocks
of causal 3-D convolutions, per-frame spatial attention in the middle, strided causal convolutions for the temporal
steps); it does not load the published Wan weights, whose module tree differs. ``encode`` returns the posterior,
``tokenize`` the normalised latent the DiT trains on (per-channel mean / std as buffers), ``decode`` the pixels.

Causality is what makes long clips tractable: latent frame ``j`` depends on pixel frames ``<= 4 j`` only, so the latent of
a prefix of a clip is the prefix of the clip's latent, and generated frames can be decoded as they come.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as tF


@dataclass
class VideoVAEArgs:
    in_channels: int = 3
    z_dim: int = 16
    base_dim: int = 96
    dim_mult: Tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    temporal_down: Tuple[bool, ...] = (False, True, True)     # per spatial down-sampling stage: halve time too?
    attn_at_middle: bool = True
    model_type: str = "video_vae"

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.dim_mult) - 1)

    @property
    def temporal_factor(self) -> int:
        return 2 ** sum(self.temporal_down)


class CausalConv3d(nn.Conv3d):
    """3-D convolution that pads the time axis in front only (frame t never sees frame t + 1)."""

    def __init__(self, cin: int, cout: int, kernel=3, stride=1):
        k = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
        s = (stride,) * 3 if isinstance(stride, int) else tuple(stride)
        super().__init__(cin, cout, k, s, padding=0)
        self.pad = (k[2] // 2, k[2] // 2, k[1] // 2, k[1] // 2, k[0] - 1, 0)

    def forward(self, x: torch.Tensor, first: bool = True) -> torch.Tensor:
        """``first`` = the clip starts here: the missing past is the first frame repeated (so a still picture stays
        a still picture); otherwise the caller has put the real past frames in front already."""
        pw = self.pad
        if first and pw[4]:
            x = torch.cat([x[:, :, :1].expand(-1, -1, pw[4], -1, -1), x], dim=2)
        return super().forward(tF.pad(x, pw[:4]))


class ChannelRMSNorm(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        w = self.weight.view(1, -1, *([1] * (x.dim() - 2)))
        return tF.normalize(x.float(), dim=1).to(x.dtype) * (x.shape[1] ** 0.5) * w


class ResBlock(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.n1, self.c1 = ChannelRMSNorm(cin), CausalConv3d(cin, cout)
        self.n2, self.c2 = ChannelRMSNorm(cout), CausalConv3d(cout, cout)
        self.skip = CausalConv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.c1(tF.silu(self.n1(x)))
        h = self.c2(tF.silu(self.n2(h)))
        return h + (x if self.skip is None else self.skip(x))


class FrameAttention(nn.Module):
    """Single-head self-attention over the pixels of each frame (no mixing across time: causality is kept)."""

    def __init__(self, dim: int):
        super().__init__()
        self.norm = ChannelRMSNorm(dim)
        self.qkv = nn.Conv2d(dim, 3 * dim, 1)
        self.proj = nn.Conv2d(dim, dim, 1)

    def forward(self, x):
        B, C, T, H, W = x.shape
        y = self.norm(x).permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        q, k, v = self.qkv(y).reshape(B * T, 3, C, H * W).unbind(1)
        o = tF.scaled_dot_product_attention(q.transpose(1, 2)[:, None], k.transpose(1, 2)[:, None], v.transpose(1, 2)[:, None])
        o = self.proj(o[:, 0].transpose(1, 2).reshape(B * T, C, H, W))
        return x + o.reshape(B, T, C, H, W).permute(0, 2, 1, 3, 4)


class Down(nn.Module):
    """Halve height and width; with ``temporal`` also halve time: the first frame stays, and output frame j >= 1 is a
    stride-2 convolution over input frames 2 j - 2, 2 j - 1, 2 j (1 + 2 m frames -> 1 + m, nothing from the future)."""

    def __init__(self, dim: int, temporal: bool):
        super().__init__()
        self.spatial = nn.Conv2d(dim, dim, 3, stride=2, padding=0)
        self.temporal = nn.Conv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1)) if temporal else None

    def forward(self, x):
        B, C, T, H, W = x.shape
        y = tF.pad(x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W), (0, 1, 0, 1))
        y = self.spatial(y)
        x = y.reshape(B, T, C, y.shape[-2], y.shape[-1]).permute(0, 2, 1, 3, 4)
        if self.temporal is not None and x.shape[2] > 1:
            x = torch.cat([x[:, :, :1], self.temporal(x)], dim=2)
        return x


class Up(nn.Module):
    """Double height and width (nearest + convolution); with ``temporal`` also double time after the first frame
    (1 + m frames -> 1 + 2 m) with a causal convolution that emits two frames per input frame."""

    def __init__(self, dim: int, out: int, temporal: bool):
        super().__init__()
        self.spatial = nn.Conv2d(dim, out, 3, padding=1)
        self.temporal = CausalConv3d(dim, 2 * dim, (3, 1, 1)) if temporal else None

    def forward(self, x):
        if self.temporal is not None and x.shape[2] > 1:
            B, C, T, H, W = x.shape
            y = self.temporal(x)[:, :, 1:]                           # [B, 2 C, T - 1, H, W]
            y = y.reshape(B, 2, C, T - 1, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, C, 2 * (T - 1), H, W)
            x = torch.cat([x[:, :, :1], y], dim=2)
        B, C, T, H, W = x.shape
        y = tF.interpolate(x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W), scale_factor=2.0, mode="nearest")
        y = self.spatial(y)
        return y.reshape(B, T, -1, 2 * H, 2 * W).permute(0, 2, 1, 3, 4)


class Encoder(nn.Module):
    def __init__(self, a: VideoVAEArgs):
        super().__init__()
        dims = [a.base_dim * m for m in a.dim_mult]
        self.stem = CausalConv3d(a.in_channels, dims[0])
        blocks: List[nn.Module] = []
        cin = dims[0]
        for i, d in enumerate(dims):
            for _ in range(a.num_res_blocks):
                blocks.append(ResBlock(cin, d))
                cin = d
            if i < len(dims) - 1:
                blocks.append(Down(cin, a.temporal_down[i]))
        self.blocks = nn.ModuleList(blocks)
        self.mid1, self.mid2 = ResBlock(cin, cin), ResBlock(cin, cin)
        self.attn = FrameAttention(cin) if a.attn_at_middle else None
        self.norm, self.head = ChannelRMSNorm(cin), CausalConv3d(cin, 2 * a.z_dim)

    def forward(self, x):
        h = self.stem(x)
        for b in self.blocks:
            h = b(h)
        h = self.mid1(h)
        if self.attn is not None:
            h = self.attn(h)
        h = self.mid2(h)
        return self.head(tF.silu(self.norm(h)))


class Decoder(nn.Module):
    def __init__(self, a: VideoVAEArgs):
        super().__init__()
        dims = [a.base_dim * m for m in reversed(a.dim_mult)]
        self.stem = CausalConv3d(a.z_dim, dims[0])
        self.mid1, self.mid2 = ResBlock(dims[0], dims[0]), ResBlock(dims[0], dims[0])
        self.attn = FrameAttention(dims[0]) if a.attn_at_middle else None
        blocks: List[nn.Module] = []
        cin = dims[0]
        t_up = list(reversed(a.temporal_down))
        for i, d in enumerate(dims):
            for _ in range(a.num_res_blocks + 1):
                blocks.append(ResBlock(cin, d))
                cin = d
            if i < len(dims) - 1:
                blocks.append(Up(cin, cin, t_up[i]))
        self.blocks = nn.ModuleList(blocks)
        self.norm, self.head = ChannelRMSNorm(cin), CausalConv3d(cin, a.in_channels)

    def forward(self, z):
        h = self.mid1(self.stem(z))
        if self.attn is not None:
            h = self.attn(h)
        h = self.mid2(h)
        for b in self.blocks:
            h = b(h)
        return self.head(tF.silu(self.norm(h)))


class VideoVAE(nn.Module):
    def __init__(self, args: Optional[VideoVAEArgs] = None):
        super().__init__()
        self.args = a = args or VideoVAEArgs()
        self.encoder, self.decoder = Encoder(a), Decoder(a)
        self.register_buffer("latent_mean", torch.zeros(a.z_dim))
        self.register_buffer("latent_std", torch.ones(a.z_dim))

    def latent_frames(self, frames: int) -> int:
        return 1 + (frames - 1) // self.args.temporal_factor

    def encode(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``x [B, C, 1 + f k, H, W]`` in [-1, 1] -> (mean, log-variance) ``[B, z, 1 + k, H / s, W / s]``."""
        f = self.args.temporal_factor
        if (x.shape[2] - 1) % f:
            raise ValueError(f"a clip needs 1 + {f} k frames, got {x.shape[2]}")
        mean, logvar = self.encoder(x).chunk(2, dim=1)
        return mean, logvar.clamp(-30.0, 20.0)

    def _norm(self, z):
        shape = (1, -1, 1, 1, 1)
        return (z - self.latent_mean.view(shape)) / self.latent_std.view(shape)

    def tokenize(self, x: torch.Tensor, sample: bool = False, generator=None) -> torch.Tensor:
        """The normalised latent the diffusion transformer is trained on (posterior mean unless ``sample``)."""
        mean, logvar = self.encode(x)
        if sample:
            mean = mean + torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype) * (0.5 * logvar).exp()
        return self._norm(mean)

    def decode(self, z: torch.Tensor, normalized: bool = True) -> torch.Tensor:
        if normalized:
            shape = (1, -1, 1, 1, 1)
            z = z * self.latent_std.view(shape) + self.latent_mean.view(shape)
        return self.decoder(z)

    def loss(self, x: torch.Tensor, kl_weight: float = 1e-6, generator=None) -> Dict[str, torch.Tensor]:
        mean, logvar = self.encode(x)
        z = mean + torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype) * (0.5 * logvar).exp()
        rec = self.decoder(z)
        l_rec = (rec - x).abs().mean()
        l_kl = 0.5 * (mean.pow(2) + logvar.exp() - 1.0 - logvar).mean()
        return {"loss": l_rec + kl_weight * l_kl, "rec": l_rec.detach(), "kl": l_kl.detach()}

    @torch.no_grad()
    def fit_latent_stats(self, clips: List[torch.Tensor]) -> None:
        """Per-channel mean / std of the posterior means over ``clips``: the normalisation ``tokenize`` applies."""
        zs = torch.cat([self.encode(c)[0].transpose(0, 1).reshape(self.args.z_dim, -1) for c in clips], dim=1)
        self.latent_mean.copy_(zs.mean(1))
        self.latent_std.copy_(zs.std(1).clamp_min(1e-6))
