"""Rollout backend registry and interface (cosmos_rl/rollout/rollout_base.py:29-274)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Type


@dataclass
class RolloutResult:
    prompt: Any
    completions: List[Any]
    completion_token_ids: Optional[List[List[int]]] = None
    completion_logprobs: Optional[List[List[float]]] = None
    cumulative_logprob: Optional[List[float]] = None
    completed_conversations: Optional[List[Any]] = None
    extra_info: Optional[Dict[str, Any]] = None


class RolloutRegistry:
    _backends: Dict[str, Type["RolloutBase"]] = {}

    @classmethod
    def register(cls, backend: str):
        def deco(c):
            cls._backends[backend] = c
            return c
        return deco

    @classmethod
    def get(cls, backend: str) -> Type["RolloutBase"]:
        if backend not in cls._backends:
            raise KeyError(f"unknown rollout backend {backend!r}; known: {sorted(cls._backends)}")
        return cls._backends[backend]

    @classmethod
    def known(cls) -> List[str]:
        return sorted(cls._backends)


class RolloutBase:
    def __init__(self, config, parallel_dims, device, **kw):
        self.config, self.parallel_dims, self.device = config, parallel_dims, device

    def init_engine(self, load_format: str = "dummy", **kw) -> None:
        raise NotImplementedError

    def rollout_generation(self, payloads, data_packer, data_fetcher, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        raise NotImplementedError

    def get_underlying_model(self):
        raise NotImplementedError

    def model_param_map(self) -> Dict[str, Any]:
        return dict(self.get_underlying_model().named_parameters())

    def pre_get_params_for_sync_hook(self, **kw) -> None:
        pass

    def post_get_params_for_sync_hook(self, **kw) -> None:
        pass
