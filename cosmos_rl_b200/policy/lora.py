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
