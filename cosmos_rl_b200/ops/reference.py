"""Plain PyTorch fp32 statements of every op in this package.

They serve two purposes: they are the oracle that the CUDA kernels are tested against, and they are the
implementation used for CPU tensors (the CPU/gloo plumbing configuration and the unit tests). They are
never used for CUDA tensors.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """``weight * x * rsqrt(mean(x^2) + eps)`` in fp32 (cosmos_rl/policy/kernel/norm.py:36-41).
    With ``residual`` the norm is applied to ``x + residual`` and that sum is returned as well."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * weight.float()).to(x.dtype)
    return y, (x if residual is not None else None)


def rope_cos_sin(positions: torch.Tensor, d: int, theta: float):
    inv_freq = torch.exp2(-(2.0 * torch.arange(d // 2, dtype=torch.float32, device=positions.device) / d)
                          * math.log2(theta))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def apply_rope(q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor, theta: float,
               backward: bool = False):
    """Rotate-half RoPE on ``q [T, hq, d]`` / ``k [T, hkv, d]`` (cosmos_rl/policy/kernel/rope.py:33-57)."""
    d = q.shape[-1]
    cos, sin = rope_cos_sin(positions, d, theta)
    if backward:
        sin = -sin
    cos, sin = cos[:, None, :], sin[:, None, :]

    def rot(x):
        xf = x.float()
        a, b = xf[..., : d // 2], xf[..., d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)

    return rot(q), (rot(k) if k is not None else None)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` on a fused ``[..., 2I]`` projection (cosmos_rl/policy/kernel/fused.py:31-37)."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0):
    """Per-token log-prob of ``labels`` and entropy of ``softmax(hidden @ weight.T / temperature)``
    (cosmos_rl/utils/util.py:314-366, 899-916). Rows with ``label < 0`` get log-prob 0."""
    logits = (hidden.float() @ weight.float().t()) / temperature
    lse = torch.logsumexp(logits, dim=-1)
    safe = labels.clamp_min(0)
    z = logits.gather(-1, safe[:, None]).squeeze(-1)
    lp = torch.where(labels >= 0, z - lse, torch.zeros_like(z))
    p = torch.softmax(logits, dim=-1)
    ent = lse - (p * logits).sum(-1)
    return lp, ent


def varlen_attention(q, k, v, cu_seqlens, scale: Optional[float] = None, causal: bool = True, cu_k=None,
                     return_lse: bool = False):
    """Packed-sequence causal GQA attention; ``q [Tq, hq, d]``, ``k/v [Tk, hkv, d]``
    (semantics of flash_attn_varlen_func as used at cosmos_rl/policy/model/gpt/__init__.py:264-273).
    With ``cu_k`` the keys of a sequence may be longer than its queries; the queries are then aligned to the END
    of the keys (query i sees keys ``0 .. i + len_k - len_q``)."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    lse = torch.full((hq, T), float("inf"), dtype=torch.float32, device=q.device)
    cs = cu_seqlens.tolist()
    ck = cs if cu_k is None else cu_k.tolist()
    for i in range(len(cs) - 1):
        s, e = cs[i], cs[i + 1]
        ks, ke = ck[i], ck[i + 1]
        if e <= s or ke <= ks:
            continue
        qi = q[s:e].transpose(0, 1).float()                       # [hq, Lq, d]
        ki = k[ks:ke].transpose(0, 1).float().repeat_interleave(g, dim=0)
        vi = v[ks:ke].transpose(0, 1).float().repeat_interleave(g, dim=0)
        sc = (qi @ ki.transpose(-1, -2)) * scale
        if causal:
            Lq, Lk = e - s, ke - ks
            mask = torch.ones(Lq, Lk, dtype=torch.bool, device=q.device).tril(Lk - Lq)
            sc = sc.masked_fill(~mask, float("-inf"))
        out[s:e] = (torch.softmax(sc, dim=-1) @ vi).transpose(0, 1).to(q.dtype)
        if return_lse:
            lse[:, s:e] = torch.logsumexp(sc, dim=-1)
    return (out, lse) if return_lse else out


def paged_decode(q, cache, block_table, seq_lens, scale: Optional[float] = None, v_transposed: bool = False):
    """One-query-per-sequence attention over a paged cache ``[pages, 2, hkv, page_size, d]`` (V slabs stored
    as ``[d, page_size]`` when ``v_transposed``)."""
    B, hq, d = q.shape
    hkv, page_size = cache.shape[2], cache.shape[3]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        n_pages = (L + page_size - 1) // page_size
        pages = block_table[b, :n_pages].long()
        kk = cache[pages, 0].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :L].float()
        if v_transposed:
            vv = cache[pages, 1].reshape(-1, hkv, d, page_size).permute(1, 0, 3, 2).reshape(hkv, -1, d)[:, :L].float()
        else:
            vv = cache[pages, 1].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :L].float()
        kk = kk.repeat_interleave(g, dim=0)
        vv = vv.repeat_interleave(g, dim=0)
        sc = torch.einsum("hd,hld->hl", q[b].float(), kk) * scale
        out[b] = torch.einsum("hl,hld->hd", torch.softmax(sc, dim=-1), vv).to(q.dtype)
    return out


def kv_append(k, v, cache, slot_mapping, v_transposed: bool = False):
    page_size = cache.shape[3]
    hkv, d = k.shape[1], k.shape[2]
    for t in range(k.shape[0]):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        page, off = divmod(slot, page_size)
        cache[page, 0, :, off] = k[t]
        if v_transposed:
            cache[page, 1].view(hkv, d, page_size)[:, :, off] = v[t]
        else:
            cache[page, 1, :, off] = v[t]


def sample(logits, temperature, top_p, top_k, generator: Optional[torch.Generator] = None):
    """Temperature / top-k / top-p sampling; returns tokens and their log-prob under softmax(logits / T)."""
    B, V = logits.shape
    toks = torch.empty(B, dtype=torch.long, device=logits.device)
    lps = torch.empty(B, dtype=torch.float32, device=logits.device)
    for b in range(B):
        t = float(temperature[b]) if temperature is not None else 1.0
        x = logits[b].float()
        if t <= 0:
            lsm = torch.log_softmax(x, -1)
            toks[b] = int(x.argmax())
            lps[b] = lsm[toks[b]]
            continue
        x = x / t
        lsm = torch.log_softmax(x, -1)
        p = lsm.exp()
        keep = torch.ones(V, dtype=torch.bool, device=logits.device)
        k = int(top_k[b]) if top_k is not None else -1
        if 0 < k < V:
            kth = torch.topk(p, k).values[-1]
            keep &= p >= kth
        tp = float(top_p[b]) if top_p is not None else 1.0
        if tp < 1.0:
            pk = torch.where(keep, p, torch.zeros_like(p))
            sp, si = torch.sort(pk, descending=True)
            cum = sp.cumsum(0)
            cutoff = int((cum < tp * pk.sum()).sum()) + 1
            k2 = torch.zeros(V, dtype=torch.bool, device=logits.device)
            k2[si[:cutoff]] = True
            keep &= k2
        pk = torch.where(keep, p, torch.zeros_like(p))
        toks[b] = int(torch.multinomial(pk / pk.sum(), 1, generator=generator))
        lps[b] = lsm[toks[b]]
    return toks, lps


E4M3_MAX = 448.0


def quant_fp8_block(w: torch.Tensor, block_rows: int = 128, block_cols: int = 128):
    """bf16 -> e4m3 with one fp32 scale per ``block_rows x block_cols`` block; returns (q, scales)."""
    R, C = w.shape
    nr, nc = (R + block_rows - 1) // block_rows, (C + block_cols - 1) // block_cols
    pad = torch.zeros(nr * block_rows, nc * block_cols, dtype=torch.float32, device=w.device)
    pad[:R, :C] = w.float()
    blocks = pad.view(nr, block_rows, nc, block_cols)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scales = amax / E4M3_MAX
    q = (blocks / scales[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).view(nr * block_rows, nc * block_cols)[:R, :C]
    return q.to(torch.float8_e4m3fn), scales


def dequant_fp8_block(q: torch.Tensor, scales: torch.Tensor, block_rows: int = 128, block_cols: int = 128):
    R, C = q.shape
    s = scales.repeat_interleave(block_rows, 0)[:R].repeat_interleave(block_cols, 1)[:, :C]
    return q.float() * s


def adamw_step(master, m, v, grad, lr, beta1, beta2, eps, weight_decay, step, grad_scale: float = 1.0):
    """Decoupled-weight-decay Adam on fp32 master weights (torch.optim.AdamW semantics,
    cosmos_rl/policy/trainer/optm/__init__.py:365-400)."""
    g = grad.float() * grad_scale
    master.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bias1 = 1.0 - beta1 ** step
    bias2 = 1.0 - beta2 ** step
    denom = v.sqrt() / math.sqrt(bias2) + eps
    master.addcdiv_(m, denom, value=-lr / bias1)


# ---------------------------------------------------------------------------------------------- microscaling fp4
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def mxfp4_sf_index(R: int, n_cb: int, swizzle: bool, device=None) -> torch.Tensor:
    """Byte offset of the scale of (row, 32-element block) for every pair, ``[R, n_cb]`` int64."""
    r = torch.arange(R, device=device)[:, None]
    cb = torch.arange(n_cb, device=device)[None, :]
    if not swizzle:
        return r * n_cb + cb
    tiles_c = (n_cb + 3) // 4
    rr = r % 128
    return ((r // 128) * tiles_c + cb // 4) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + cb % 4


def quant_mxfp4(w: torch.Tensor, swizzle: bool = False):
    """bf16/fp32 ``[R, C]`` (C % 32 == 0) -> (packed E2M1 ``[R, C/2]`` uint8, E8M0 scales uint8). Scale exponent
    ``floor(log2(amax)) - 2`` per 32 elements, elements rounded to nearest (ties to the even code), saturating at 6."""
    R, C = w.shape
    n_cb = C // 32
    x = w.float().view(R, n_cb, 32)
    amax = x.abs().amax(-1)
    ex = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp_min(1e-45))) - 2, torch.full_like(amax, -127.0))
    ex = ex.clamp(-127, 127)
    a = (x.double() * torch.exp2(-ex.double())[..., None]).abs()
    code = ((a > 0.25).int() + (a >= 0.75).int() + (a > 1.25).int() + (a >= 1.75).int() + (a > 2.5).int()
            + (a >= 3.5).int() + (a > 5.0).int())
    code = code | ((x < 0).int() << 3)
    code = code.view(R, C)
    q = (code[:, 0::2] | (code[:, 1::2] << 4)).to(torch.uint8)
    n_sf = ((R + 127) // 128) * ((n_cb + 3) // 4) * 512 if swizzle else R * n_cb
    sf = torch.zeros(n_sf, dtype=torch.uint8, device=w.device)
    sf[mxfp4_sf_index(R, n_cb, swizzle, w.device).flatten()] = (ex + 127).to(torch.uint8).flatten()
    return q, sf


def dequant_mxfp4(q: torch.Tensor, sf: torch.Tensor, swizzle: bool = False) -> torch.Tensor:
    R, C = q.shape[0], q.shape[1] * 2
    n_cb = C // 32
    lut = torch.tensor(_E2M1, dtype=torch.float32, device=q.device)
    code = torch.stack([q & 0xF, q >> 4], dim=-1).view(R, C).long()
    val = lut[code & 7] * torch.where((code & 8) > 0, -1.0, 1.0)
    ex = sf[mxfp4_sf_index(R, n_cb, swizzle, q.device)].float() - 127.0
    return (val.view(R, n_cb, 32) * torch.exp2(ex)[..., None]).view(R, C)
