"""LoRA adapters for the policy model: inject low-rank ``A``/``B`` pairs next to selected linear weights,
train only those, and merge them into the base weight before a weight sync (and unmerge afterwards), so the
rollout engine always receives plain dense weights (cosmos_rl/policy/lora/plugin.py:29-459; merge before P2R
cosmos_rl/policy/worker/rl_worker.py:455-466, 548-551)."""
from __future__ import annotations

import math
import re
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as tF


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, r: int, alpha: float, dropout: float = 0.0, use_rslora: bool = False):
        super().__init__()
        self.base = base
        self.r = r
        self.scaling = alpha / math.sqrt(r) if use_rslora else alpha / r
        self.lora_A = nn.Parameter(torch.empty(r, base.in_features, dtype=base.weight.dtype, device=base.weight.device))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, r, dtype=base.weight.dtype, device=base.weight.device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.merged = False
        base.weight.requires_grad_(False)
        if base.bias is not None:
            base.bias.requires_grad_(False)

    # expose the wrapped layer's attributes so model code that reads ``.weight`` keeps working
    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def delta(self) -> torch.Tensor:
        return (self.lora_B.float() @ self.lora_A.float() * self.scaling).to(self.base.weight.dtype)

    def forward(self, x):
        y = tF.linear(x, self.base.weight, self.base.bias)
        if self.merged:
            return y
        return y + tF.linear(tF.linear(self.dropout(x), self.lora_A), self.lora_B) * self.scaling

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged:
            self.base.weight.add_(self.delta())
            self.merged = True

    @torch.no_grad()
    def unmerge(self) -> None:
        if self.merged:
            self.base.weight.sub_(self.delta())
            self.merged = False


def _matches(name: str, targets) -> bool:
    if targets in ("all-linear", ["all-linear"]):
        return True
    if isinstance(targets, str):
        return re.search(targets, name) is not None
    leaf = name.rsplit(".", 1)[-1]
    return any(t == leaf or name.endswith(t) for t in targets)


def inject_lora(model: nn.Module, cfg) -> List[str]:
    """Wrap every ``nn.Linear`` whose name matches ``cfg.target_modules``. Returns the wrapped module names.
    Everything that is not an adapter (or listed in ``modules_to_save``) is frozen."""
    wrapped = []
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if isinstance(child, nn.Linear) and _matches(full, cfg.target_modules) and "lm_head" not in full:
                r = (cfg.r_pattern or {}).get(child_name, cfg.r)
                alpha = (cfg.alpha_pattern or {}).get(child_name, cfg.lora_alpha)
                setattr(mod, child_name, LoRALinear(child, r, alpha, cfg.lora_dropout, cfg.use_rslora))
                wrapped.append(full)
    keep = set(cfg.modules_to_save or [])
    for name, p in model.named_parameters():
        if "lora_A" in name or "lora_B" in name:
            p.requires_grad_(True)
        elif not any(k in name for k in keep):
            p.requires_grad_(False)
    return wrapped


def lora_modules(model: nn.Module) -> Iterable[LoRALinear]:
    return (m for m in model.modules() if isinstance(m, LoRALinear))


def merge_lora(model: nn.Module) -> None:
    for m in lora_modules(model):
        m.merge()


def unmerge_lora(model: nn.Module) -> None:
    for m in lora_modules(model):
        m.unmerge()


def adapter_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """PEFT-style names (``base_model.model.<path>.lora_A.weight``) for ``adapter_model.safetensors``."""
    out = {}
    for name, m in model.named_modules():
        if isinstance(m, LoRALinear):
            out[f"base_model.model.{name}.lora_A.weight"] = m.lora_A.detach().cpu()
            out[f"base_model.model.{name}.lora_B.weight"] = m.lora_B.detach().cpu()
    return out


def adapter_config(cfg, wrapped: List[str]) -> Dict:
    return {"peft_type": "LORA", "r": cfg.r, "lora_alpha": cfg.lora_alpha, "lora_dropout": cfg.lora_dropout,
            "target_modules": sorted({w.rsplit(".", 1)[-1] for w in wrapped}), "use_rslora": cfg.use_rslora,
            "bias": "none", "task_type": "CAUSAL_LM"}


# ---------------------------------------------------------------------------------------------- native models
# The native model families call their projections functionally (``_linear(x, module.weight, module.bias)`` on
# fused qkv / gate_up weights), so adapters are attached to the projection module as two extra parameters and found
# through a reference hung on the weight tensor; module wrapping (above) serves models that call ``module(x)``.
_FUSED_ALIASES = {"q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj", "gate_proj": "gate_up_proj",
                  "up_proj": "gate_up_proj"}


class LoraRef:
    """What ``_linear`` needs to add the low-rank path of one projection."""

    def __init__(self, module: nn.Module, scaling: float):
        self.module, self.scaling, self.merged, self.enabled = module, scaling, False, True

    def apply(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if self.merged or not self.enabled:
            return y
        m = self.module
        B = m.lora_B if m.lora_row_mask is None else m.lora_B * m.lora_row_mask
        return y + tF.linear(tF.linear(x, m.lora_A), B) * self.scaling

    def delta(self) -> torch.Tensor:
        m = self.module
        B = m.lora_B if m.lora_row_mask is None else m.lora_B * m.lora_row_mask
        return (B.float() @ m.lora_A.float() * self.scaling).to(m.weight.dtype)


def _fused_row_mask(module: nn.Linear, leaf: str, wanted: List[str], model_args) -> Optional[torch.Tensor]:
    """Adapters on a fused projection cover only the requested parts (e.g. q and v of qkv): rows of the others get a
    zero mask so their weights never move."""
    parts = [k for k, v in _FUSED_ALIASES.items() if v == leaf]
    if not parts or all(p in wanted for p in parts):
        return None
    out = module.out_features
    if leaf == "qkv_proj":
        d = model_args.head_dim
        hq = model_args.n_heads // max(1, model_args.tp_size)
        hkv = max(1, model_args.n_kv_heads // max(1, model_args.tp_size))
        sizes = [hq * d, hkv * d, hkv * d]
    else:
        sizes = [out // 2, out // 2]
    mask = torch.cat([torch.full((s,), 1.0 if p in wanted else 0.0) for p, s in zip(parts, sizes)])
    return mask[:, None]


def attach_lora(model: nn.Module, cfg) -> List[str]:
    """Give every targeted projection of a native model ``lora_A [r, in]`` / ``lora_B [out, r]`` parameters (call
    before the flat parameter buffer is built, so they live in it) and freeze everything else."""
    targets = cfg.target_modules
    all_linear = targets in ("all-linear", ["all-linear"])
    names = [] if all_linear or isinstance(targets, str) else list(targets)
    wanted_leaves = {_FUSED_ALIASES.get(t, t) for t in names}
    attached = []
    for full, mod in model.named_modules():
        if not isinstance(mod, nn.Linear) or "lm_head" in full:
            continue
        leaf = full.rsplit(".", 1)[-1]
        hit = all_linear or (re.search(targets, full) is not None if isinstance(targets, str) else leaf in wanted_leaves)
        if not hit:
            continue
        r = (cfg.r_pattern or {}).get(leaf, cfg.r)
        alpha = (cfg.alpha_pattern or {}).get(leaf, cfg.lora_alpha)
        dev, dt = mod.weight.device, mod.weight.dtype
        mod.lora_A = nn.Parameter(torch.empty(r, mod.in_features, device=dev, dtype=dt))
        mod.lora_B = nn.Parameter(torch.empty(mod.out_features, r, device=dev, dtype=dt))
        mod.lora_scaling = alpha / math.sqrt(r) if cfg.use_rslora else alpha / r
        mask = None if (all_linear or isinstance(targets, str)) else _fused_row_mask(mod, leaf, names, getattr(model, "args", None))
        mod.lora_row_mask = mask
        attached.append(full)
    if not attached:
        raise ValueError(f"policy.lora.target_modules={targets!r} matches no projection of {type(model).__name__}")
    keep = set(cfg.modules_to_save or [])
    for name, p in model.named_parameters():
        p.requires_grad_(".lora_" in name or any(k in name for k in keep))
    return attached


def bind_lora(model: nn.Module) -> int:
    """After the parameters were materialised: hang the adapter reference on each targeted weight, move the row masks
    to the parameters' device. Returns the number of adapted projections."""
    n = 0
    for mod in model.modules():
        if isinstance(mod, nn.Linear) and hasattr(mod, "lora_A"):
            if mod.lora_row_mask is not None:
                mod.lora_row_mask = mod.lora_row_mask.to(mod.weight.device, mod.weight.dtype)
            mod.weight._lora = LoraRef(mod, mod.lora_scaling)
            n += 1
    return n


@torch.no_grad()
def reset_lora_parameters(model: nn.Module, seed: int = 0, init=True) -> None:
    """``init`` follows PEFT's ``init_lora_weights``: True = A Kaiming-uniform, B = 0 (the adapted model starts as the
    base model); "gaussian" = A ~ N(0, 1/r), B = 0; False = both random (debugging: the adapter is not a no-op)."""
    if init not in (True, False, "gaussian"):
        raise NotImplementedError(f"init_lora_weights = {init!r}: supported are true, false and \"gaussian\"")
    g = torch.Generator(device="cpu").manual_seed(seed)
    for mod in model.modules():
        if isinstance(mod, nn.Linear) and hasattr(mod, "lora_A"):
            if init == "gaussian":
                a = torch.randn(mod.lora_A.shape, generator=g) / mod.lora_A.shape[0]
            else:
                bound = 1.0 / math.sqrt(mod.in_features)        # kaiming_uniform with a = sqrt(5)
                a = (torch.rand(mod.lora_A.shape, generator=g) * 2 - 1) * bound
            mod.lora_A.copy_(a.to(mod.lora_A.dtype))
            if init is False:
                bound_b = 1.0 / math.sqrt(mod.lora_B.shape[1])
                mod.lora_B.copy_(((torch.rand(mod.lora_B.shape, generator=g) * 2 - 1) * bound_b).to(mod.lora_B.dtype))
            else:
                mod.lora_B.zero_()


def lora_refs(model: nn.Module) -> List[LoraRef]:
    return [m.weight._lora for m in model.modules()
            if isinstance(m, nn.Linear) and hasattr(m, "lora_A") and getattr(m.weight, "_lora", None) is not None]


@torch.no_grad()
def merge_native(model: nn.Module) -> None:
    """W += B A (before a weight sync or an export of dense weights)."""
    for ref in lora_refs(model):
        if not ref.merged:
            ref.module.weight.add_(ref.delta())
            ref.merged = True


@torch.no_grad()
def unmerge_native(model: nn.Module) -> None:
    for ref in lora_refs(model):
        if ref.merged:
            ref.module.weight.sub_(ref.delta())
            ref.merged = False


class adapters_disabled:
    """Context: run the base model (the KL reference of a LoRA policy is the policy without its adapters)."""

    def __init__(self, model: nn.Module):
        self.refs = lora_refs(model)

    def __enter__(self):
        self.prev = [r.enabled for r in self.refs]
        for r in self.refs:
            r.enabled = False

    def __exit__(self, *exc):
        for r, p in zip(self.refs, self.prev):
            r.enabled = p


def native_adapter_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """PEFT-named adapter tensors; adapters on fused projections are split back (the parts share ``lora_A`` and own
    their rows of ``lora_B``, which is exactly what the fused product represents)."""
    out: Dict[str, torch.Tensor] = {}
    a = getattr(model, "args", None)
    for full, mod in model.named_modules():
        if not (isinstance(mod, nn.Linear) and hasattr(mod, "lora_A")):
            continue
        leaf = full.rsplit(".", 1)[-1]
        stem = full[: -len(leaf)]
        parts = [k for k, v in _FUSED_ALIASES.items() if v == leaf]
        A, B = mod.lora_A.detach().cpu(), mod.lora_B.detach().cpu()
        if mod.lora_row_mask is not None:
            B = B * mod.lora_row_mask.cpu()
        if not parts:
            pieces = [(leaf, B)]
        elif leaf == "qkv_proj":
            d, hq, hkv = a.head_dim, a.n_heads // max(1, a.tp_size), max(1, a.n_kv_heads // max(1, a.tp_size))
            pieces = list(zip(parts, B.split([hq * d, hkv * d, hkv * d], dim=0)))
        else:
            pieces = list(zip(parts, B.chunk(2, dim=0)))
        for name, b in pieces:
            if mod.lora_row_mask is not None and not bool(b.any()) and bool(B.any()):
                continue                                     # a part that was not targeted
            out[f"base_model.model.model.{stem}{name}.lora_A.weight"] = A.clone()
            out[f"base_model.model.model.{stem}{name}.lora_B.weight"] = b.contiguous()
    return out
