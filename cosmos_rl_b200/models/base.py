"""Model registry and the base interface every policy model implements
(cosmos_rl/policy/model/base.py:59-545 for BaseModel, :798-1070 for WeightMapper,
cosmos_rl/policy/model/__init__.py:39-136 for the registry)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple, Type

import torch
import torch.nn as nn


class WeightMapper:
    """Translates between this framework's parameter names/layouts and the HF checkpoint's."""

    def __init__(self, hf_config: Any):
        self.config = hf_config

    # local (fused) name -> list of (hf_name, row_slice) it is assembled from
    def local_to_hf(self, name: str, shape: Tuple[int, ...]) -> List[Tuple[str, Optional[Tuple[int, int]]]]:
        return [(name, None)]

    def policy_map_local_key_to_hf_key(self, name: str) -> str:
        return name

    def rollout_map_local_key_to_hf_key(self, name: str) -> str:
        return name


class IdentityWeightMapper(WeightMapper):
    """For families whose checkpoints are stored under the framework's own parameter names (custom policies of
    non-language workloads): every tensor maps to itself."""

    def hf_names(self, local: str) -> List[str]:
        return [local]


class ModelRegistry:
    _models: Dict[str, Type["BaseModel"]] = {}
    _mappers: Dict[str, Type[WeightMapper]] = {}

    @classmethod
    def register(cls, mapper_cls: Type[WeightMapper] = WeightMapper, default: bool = False):
        def deco(model_cls):
            for mt in model_cls.supported_model_types():
                cls._models[mt] = model_cls
                cls._mappers[mt] = mapper_cls
            if default:
                cls._models["hfmodel"] = model_cls
                cls._mappers["hfmodel"] = mapper_cls
            return model_cls
        return deco

    @classmethod
    def get(cls, model_type: str) -> Type["BaseModel"]:
        if model_type in cls._models:
            return cls._models[model_type]
        if "hfmodel" in cls._models:
            return cls._models["hfmodel"]
        raise KeyError(f"no model registered for type {model_type!r}; known: {sorted(cls._models)}")

    @classmethod
    def mapper(cls, model_type: str) -> Type[WeightMapper]:
        return cls._mappers.get(model_type, WeightMapper)

    @classmethod
    def supported(cls) -> List[str]:
        return sorted(cls._models)

    @classmethod
    def build_model(cls, hf_config, force_hf: bool = False, **kw) -> "BaseModel":
        """``force_hf`` (``train.force_use_hf``): the generic transformers wrapper even where a native model exists."""
        mt = getattr(hf_config, "model_type", None) or hf_config.get("model_type")
        if force_hf and "hfmodel" in cls._models:
            return cls._models["hfmodel"].from_hf_config(hf_config, **kw)
        return cls.get(mt).from_hf_config(hf_config, **kw)


class BaseModel(nn.Module):
    @staticmethod
    def supported_model_types() -> List[str]:
        raise NotImplementedError

    @classmethod
    def from_hf_config(cls, hf_config, **kw) -> "BaseModel":
        raise NotImplementedError

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        raise NotImplementedError

    def get_position_ids(self, **kw):
        raise NotImplementedError

    def check_tp_compatible(self, tp_size: int) -> None:
        pass

    def check_cp_compatible(self, cp_size: int, tp_size: int) -> None:
        pass

    @property
    def weight_sync_transforms(self) -> List[Tuple[str, Callable[[], torch.Tensor]]]:
        """(rollout-side name, zero-arg callable returning the tensor view to ship) for every parameter."""
        return [(n, (lambda p=p: p.data)) for n, p in self.named_parameters()]
